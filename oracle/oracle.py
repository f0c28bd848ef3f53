"""ctypes binding of the CPU oracle (``oracle/candle_moe_oracle.cpp``).

TEST INFRASTRUCTURE ONLY.  Imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU
legs of ``bench.py``; the shipped package ``candle_b200`` never imports it.  All arrays are numpy,
all arithmetic happens in the C++ restatement of the reference's CPU path.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcandle_moe_oracle.so")

# GgmlDType::to_u32, candle-core/src/quantized/mod.rs:176-195
Q4_0, Q8_0, Q4K, Q6K, Q8K = 2, 8, 12, 14, 15
ORDER_SIMD, ORDER_LANES, ORDER_UNOPT = 0, 1, 2
DTYPE_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4K: "Q4K", Q6K: "Q6K", Q8K: "Q8K"}


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the shared object is missing or stale."""
    src = os.path.join(HERE, "candle_moe_oracle.cpp")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B"], check=True, stdout=subprocess.DEVNULL)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        L.orc_block_bytes.restype = C.c_size_t
        L.orc_block_bytes.argtypes = [C.c_int]
        L.orc_block_elems.restype = C.c_int
        L.orc_block_elems.argtypes = [C.c_int]
        L.orc_vec_dot_dtype.restype = C.c_int
        L.orc_vec_dot_dtype.argtypes = [C.c_int]
        L.orc_vec_dot.restype = C.c_float
        L.orc_vec_dot.argtypes = [C.c_int, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_quantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_quantize_rows.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.orc_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_matmul.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_softmax_last_dim.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.orc_silu.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_sigmoid.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_index_add_dim0.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_ggml_like_vector.argtypes = [C.c_float, C.c_size_t, C.c_void_p]
        L.orc_router_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                      C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_moe_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p]
        L.orc_mlp_forward.argtypes = [C.c_int, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def block_bytes(dtype: int) -> int:
    return lib().orc_block_bytes(dtype)


def block_elems(dtype: int) -> int:
    return lib().orc_block_elems(dtype)


def row_bytes(dtype: int, k: int) -> int:
    assert k % block_elems(dtype) == 0
    return k // block_elems(dtype) * block_bytes(dtype)


def max_threads() -> int:
    return lib().orc_max_threads()


def set_threads(n: int) -> None:
    lib().orc_set_threads(n)


def quantize(dtype: int, x) -> np.ndarray:
    """``QTensor::quantize``: f32 [rows, k] (or [k]) -> raw block bytes, row-major."""
    x = _f32(x)
    k = x.shape[-1]
    rows = x.size // k
    out = np.zeros(rows * row_bytes(dtype, k), dtype=np.uint8)
    rc = lib().orc_quantize_rows(dtype, _p(x), rows, k, _p(out))
    assert rc == 0, rc
    return out


def dequantize(dtype: int, blocks: np.ndarray, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    rc = lib().orc_dequantize(dtype, _p(blocks), n, _p(out))
    assert rc == 0, rc
    return out


def vec_dot(dtype: int, n: int, w: np.ndarray, act: np.ndarray, order: int = ORDER_SIMD) -> float:
    return float(lib().orc_vec_dot(dtype, n, _p(w), _p(act), order))


def matmul(dtype: int, lhs, rhs_blocks: np.ndarray, n: int, order: int = ORDER_SIMD) -> np.ndarray:
    """``k_quants::matmul``: lhs f32 [m, k] times the transposed quantized [n, k] -> f32 [m, n]."""
    lhs = _f32(lhs)
    m, k = lhs.shape
    dst = np.empty((m, n), dtype=np.float32)
    rc = lib().orc_matmul(dtype, m, k, n, _p(lhs), _p(rhs_blocks), _p(dst), order)
    assert rc == 0, rc
    return dst


def softmax_last_dim(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_softmax_last_dim(_p(x), x.size // x.shape[-1], x.shape[-1], _p(out))
    return out


def silu(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_silu(_p(x), x.size, _p(out))
    return out


def sigmoid(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_sigmoid(_p(x), x.size, _p(out))
    return out


def index_add_dim0(dst, ids, src) -> np.ndarray:
    dst = _f32(dst).copy()
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    src = _f32(src)
    rc = lib().orc_index_add_dim0(_p(dst), dst.shape[0], dst.shape[1], _p(ids), ids.size, _p(src))
    assert rc == 0, rc
    return dst


def ggml_like_vector(offset: float, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_ggml_like_vector(offset, n, _p(out))
    return out


def router_topk(x, wg, k: int, renorm: bool = True, bias=None):
    x, wg = _f32(x), _f32(wg)
    T, d = x.shape
    E = wg.shape[0]
    bias = None if bias is None else _f32(bias)
    probs = np.empty((T, E), dtype=np.float32)
    ids = np.empty((T, k), dtype=np.uint32)
    w = np.empty((T, k), dtype=np.float32)
    rc = lib().orc_router_topk(_p(x), _p(wg), _p(bias), T, d, E, k, int(renorm), _p(probs), _p(ids), _p(w))
    assert rc == 0, rc
    return probs, ids, w


class _MoeWeightsC(C.Structure):
    _fields_ = [
        ("d_model", C.c_int32), ("d_ff", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
        ("renorm", C.c_int32), ("dtype_w13", C.c_int32), ("dtype_w2", C.c_int32), ("d_ff_shared", C.c_int32),
        ("dtype_shared13", C.c_int32), ("dtype_shared2", C.c_int32), ("order", C.c_int32), ("_pad", C.c_int32),
        ("router", C.c_void_p), ("router_bias", C.c_void_p),
        ("w1", C.POINTER(C.c_void_p)), ("w3", C.POINTER(C.c_void_p)), ("w2", C.POINTER(C.c_void_p)),
        ("sw1", C.c_void_p), ("sw3", C.c_void_p), ("sw2", C.c_void_p), ("shared_gate", C.c_void_p),
    ]


@dataclass
class MoeWeights:
    """Host-side weights of one block: raw GGUF block bytes per expert, f32 router."""
    d_model: int
    d_ff: int
    top_k: int
    dtype_w13: int
    dtype_w2: int
    router: np.ndarray                      # [E, d] f32
    w1: List[np.ndarray]                    # E x bytes of [ff, d]
    w3: List[np.ndarray]
    w2: List[np.ndarray]                    # E x bytes of [d, ff]
    renorm: bool = True
    router_bias: Optional[np.ndarray] = None
    d_ff_shared: int = 0
    dtype_shared13: int = Q8_0
    dtype_shared2: int = Q8_0
    sw1: Optional[np.ndarray] = None
    sw3: Optional[np.ndarray] = None
    sw2: Optional[np.ndarray] = None
    shared_gate: Optional[np.ndarray] = None  # [d] f32
    _keep: list = field(default_factory=list, repr=False)

    @property
    def n_experts(self) -> int:
        return len(self.w1)


@dataclass
class MoeResult:
    y: np.ndarray               # [T, d]
    topk_ids: np.ndarray        # [T, k] rank order
    topk_w: np.ndarray          # [T, k]
    expert_counts: np.ndarray   # [E]
    expert_rows: np.ndarray     # [T*k] token ids grouped by expert (ascending inside an expert)


def moe_forward(w: MoeWeights, x, order: int = ORDER_SIMD) -> MoeResult:
    """The whole block as the reference's CPU path computes it."""
    x = _f32(x)
    T, d = x.shape
    assert d == w.d_model
    E, k = w.n_experts, w.top_k
    arr = C.c_void_p * E
    cw = _MoeWeightsC(
        w.d_model, w.d_ff, E, k, int(w.renorm), w.dtype_w13, w.dtype_w2, w.d_ff_shared, w.dtype_shared13,
        w.dtype_shared2, order, 0,
        _p(w.router), _p(w.router_bias),
        arr(*[a.ctypes.data for a in w.w1]), arr(*[a.ctypes.data for a in w.w3]), arr(*[a.ctypes.data for a in w.w2]),
        _p(w.sw1), _p(w.sw3), _p(w.sw2), _p(w.shared_gate),
    )
    y = np.empty((T, d), dtype=np.float32)
    ids = np.empty((T, k), dtype=np.uint32)
    tw = np.empty((T, k), dtype=np.float32)
    counts = np.zeros(E, dtype=np.uint32)
    rows = np.zeros(T * k, dtype=np.uint32)
    rc = lib().orc_moe_forward(C.byref(cw), _p(x), T, _p(y), _p(ids), _p(tw), _p(counts), _p(rows))
    assert rc == 0, rc
    return MoeResult(y, ids, tw, counts, rows)


def rms_norm(x, alpha, eps: float):
    """``candle_nn::ops::rms_norm`` on the CPU (ops.rs:504-514)."""
    x, alpha = _f32(x), _f32(alpha)
    rows, d = x.shape
    out = np.empty_like(x)
    L = lib()
    L.orc_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_size_t, C.c_void_p]
    rc = L.orc_rms_norm(_p(x), _p(alpha), C.c_float(eps), rows, d, _p(out))
    assert rc == 0, rc
    return out


def mlp_forward(dt13: int, dt2: int, x, w1, w3, w2, ff: int, order: int = ORDER_SIMD):
    """One expert (``Mlp::forward``): returns (out [rows, d], hidden [rows, ff])."""
    x = _f32(x)
    rows, d = x.shape
    out = np.empty((rows, d), dtype=np.float32)
    hid = np.empty((rows, ff), dtype=np.float32)
    rc = lib().orc_mlp_forward(dt13, dt2, rows, d, ff, _p(x), _p(w1), _p(w3), _p(w2), _p(out), _p(hid), order)
    assert rc == 0, rc
    return out, hid


def make_moe_weights(seed: int, d: int, ff: int, E: int, k: int, dt13: int, dt2: int, *, renorm: bool = True,
                     std: float = 0.02, router_bias=None, ff_shared: int = 0, dt_shared13: int = Q8_0,
                     dt_shared2: int = Q8_0) -> MoeWeights:
    """Seeded synthetic block: weights ~ N(0, std) quantized with the reference's quantizer,
    router f32 ~ N(0, std).  Tensor order router, e0.w1, e0.w3, e0.w2, e1..., shared, gate."""
    rng = np.random.default_rng(seed)
    nrm = lambda *s: (rng.standard_normal(s, dtype=np.float32) * np.float32(std))
    router = nrm(E, d)
    w1, w3, w2 = [], [], []
    for _ in range(E):
        w1.append(quantize(dt13, nrm(ff, d)))
        w3.append(quantize(dt13, nrm(ff, d)))
        w2.append(quantize(dt2, nrm(d, ff)))
    mw = MoeWeights(d, ff, k, dt13, dt2, router, w1, w3, w2, renorm=renorm,
                    router_bias=None if router_bias is None else _f32(router_bias))
    if ff_shared:
        mw.d_ff_shared, mw.dtype_shared13, mw.dtype_shared2 = ff_shared, dt_shared13, dt_shared2
        mw.sw1 = quantize(dt_shared13, nrm(ff_shared, d))
        mw.sw3 = quantize(dt_shared13, nrm(ff_shared, d))
        mw.sw2 = quantize(dt_shared2, nrm(d, ff_shared))
        mw.shared_gate = nrm(d)
    return mw


def make_activations(seed: int, T: int, d: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((T, d), dtype=np.float32)
