"""CPU-side checks of the drop-in boundary: the shared library loads, exports every symbol the
header declares, and rejects bad arguments on the host before anything touches a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from candle_b200.csrc import build as b
    b.build()
    from candle_b200 import _lib
    return _lib


def _declared_symbols():
    src = open(os.path.join(ROOT, "include", "candle_moe.h")).read()
    return sorted(set(re.findall(r"CANDLE_MOE_API\s+[\w\s\*]+?\b(candle_moe_\w+)\s*\(", src)))


def test_header_symbols_are_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 12
    handle = C.CDLL(lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in include/candle_moe.h but not exported"
    assert set(names) == set(lib.SYMBOLS), "ctypes prototypes and header disagree"
    assert lib.load().candle_moe_version().startswith(b"candle_moe_sm100")


def _weights(lib, **kw):
    w = lib.MoeWeightsC()
    w.d_model, w.d_ff, w.n_experts, w.top_k, w.renorm = 4096, 14336, 8, 2, 1
    w.dtype_w13, w.dtype_w2 = 12, 14
    for k, v in kw.items():
        setattr(w, k, v)
    return w


def test_workspace_query_is_host_only_and_monotonic(lib):
    L = lib.load()
    out = C.c_size_t(0)
    sizes = []
    for T in (0, 1, 8, 32, 2048):
        assert L.candle_moe_workspace_bytes(C.byref(_weights(lib)), T, C.byref(out)) == 0
        sizes.append(out.value)
    assert sizes == sorted(sizes) and sizes[-1] > 2048 * 2 * 14336 * 4
    # hidden f32 + its int8 copy dominate: [T*k, ff] * 5 bytes; two K-split slots of [T*k, d] f32
    assert sizes[-1] < 2048 * 2 * (14336 * 6 + 4096 * 20) + (1 << 20)


@pytest.mark.parametrize("field,value,code", [
    ("d_model", 4000, -2),        # not a multiple of 256 for Q4K
    ("d_ff", 100, -2),
    ("n_experts", 129, -2),
    ("top_k", 9, -2),
    ("top_k", 0, -2),
    ("dtype_w13", 2, -3),         # Q4_0 is not on this path
    ("dtype_w2", 15, -3),
])
def test_bad_shapes_and_dtypes_are_rejected(lib, field, value, code):
    out = C.c_size_t(0)
    assert lib.load().candle_moe_workspace_bytes(C.byref(_weights(lib, **{field: value})), 8, C.byref(out)) == code


def test_null_pointers_are_rejected_before_any_launch(lib):
    L = lib.load()
    w = _weights(lib)
    assert L.candle_moe_forward(None, C.byref(w), None, 4, None, None, 0) == -1
    assert L.candle_moe_router_topk(None, None, None, None, 4, 4096, 8, 2, 1, None, None) == -1
    assert L.candle_moe_permute(None, None, 4, 2, 8, None, None, None, None) == -1
    assert L.candle_moe_quantize_act(None, None, 4, 4096, 12, None, None, None) == -1
    assert L.candle_moe_combine(None, None, None, None, None, 4, 2, 4096, None, None, None, None) == -1
    assert L.candle_moe_quantize_weights(None, 12, None, 256, None) == -1
    assert L.candle_moe_workspace_bytes(None, 4, C.byref(C.c_size_t())) == -1
    # zero rows is a no-op, like an empty tensor through Module::forward
    one = C.c_float(0)
    w.router = C.cast(C.byref(one), C.c_void_p)
    assert L.candle_moe_forward(None, C.byref(w), C.byref(one), 0, C.byref(one), None, 0) == 0


def test_error_type_carries_status(lib):
    with pytest.raises(lib.CandleMoeError) as ei:
        lib.check("candle_moe_forward", -4)
    assert ei.value.status == -4 and "WORKSPACE" in str(ei.value)


def test_host_mirror_rejects_cpu_tensors(lib):
    import torch
    from candle_b200 import GgmlDType, QTensor
    with pytest.raises(ValueError):
        QTensor(torch.zeros(144, dtype=torch.uint8), GgmlDType.Q4K, (1, 256))
    assert GgmlDType.Q4K.type_size() == 144 and GgmlDType.Q6K.type_size() == 210 and GgmlDType.Q8_0.type_size() == 34


def test_tuning_switches_round_trip(lib):
    L = lib.load()
    v = C.c_int64(-1)
    assert L.candle_moe_get_tuning(lib.TUNE_GEMM_MIN_ROWS, C.byref(v)) == 0
    old = v.value
    assert L.candle_moe_set_tuning(lib.TUNE_GEMM_MIN_ROWS, 77) == 0
    assert L.candle_moe_get_tuning(lib.TUNE_GEMM_MIN_ROWS, C.byref(v)) == 0 and v.value == 77
    assert L.candle_moe_set_tuning(lib.TUNE_GEMM_MIN_ROWS, old) == 0
    assert L.candle_moe_set_tuning(99, 1) == -2 and L.candle_moe_get_tuning(99, C.byref(v)) == -2


def _ep_cfg(lib, **kw):
    cfg = lib.EpConfigC()
    cfg.rank, cfg.world, cfg.n_experts_global, cfg.top_k, cfg.renorm, cfg.max_tokens = 0, 2, 8, 2, 1, 32
    one = C.c_float(0)
    cfg.router = C.cast(C.pointer(one), C.c_void_p)
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg, one


def test_expert_parallel_geometry_is_host_only(lib):
    """Form and workspace of candle_moe_ep_forward follow from the configuration alone (no device, no NCCL)."""
    L = lib.load()
    local = _weights(lib, n_experts=4)
    form, cap, need = C.c_int32(0), C.c_int64(0), C.c_size_t(0)
    cfg, keep = _ep_cfg(lib)
    assert L.candle_moe_ep_forward_form(C.byref(cfg), C.byref(local), C.byref(form), C.byref(cap)) == 0
    assert (form.value, cap.value) == (1, 64)  # decode-sized step: slots of max_tokens * min(k, local experts) rows
    assert L.candle_moe_ep_forward_workspace_bytes(C.byref(cfg), C.byref(local), C.byref(need)) == 0 and need.value > 0
    from candle_b200.expert_parallel import choose_form
    for world, tokens, d in ((2, 32, 4096), (8, 32, 4096), (2, 4096, 6144), (4, 2048, 6144), (8, 1024, 4096)):
        cfg, keep = _ep_cfg(lib, world=world, max_tokens=tokens)
        local = _weights(lib, n_experts=8 // world, top_k=min(2, 8 // world), d_model=d, d_ff=16384)
        assert L.candle_moe_ep_forward_form(C.byref(cfg), C.byref(local), C.byref(form), C.byref(cap)) == 0
        assert form.value == choose_form(world, tokens, 2, 8 // world, d)[0]
    # ranks must divide the experts; Q8_0 experts have no expert-parallel form; a missing communicator is refused
    cfg, keep = _ep_cfg(lib, world=3)
    assert L.candle_moe_ep_forward_form(C.byref(cfg), C.byref(_weights(lib, n_experts=4)), C.byref(form), None) == -2
    cfg, keep = _ep_cfg(lib)
    assert L.candle_moe_ep_forward_form(C.byref(cfg), C.byref(_weights(lib, n_experts=4, dtype_w13=8, d_model=4096)),
                                        C.byref(form), None) == -3
