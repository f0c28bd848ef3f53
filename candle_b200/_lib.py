"""Loads libcandle_moe_sm100.so (the C ABI declared in include/candle_moe.h) through ctypes.

There is no fallback: if the library is missing or a call returns a nonzero status the caller gets
an exception.  The library is built in-tree by ``python candle_b200/csrc/build.py``.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libcandle_moe_sm100.so")

MAX_EXPERTS = 128
MAX_TOPK = 8

ERROR_NAMES = {
    -1: "CANDLE_MOE_E_NULL (a required pointer is NULL)",
    -2: "CANDLE_MOE_E_SHAPE (bad dimension)",
    -3: "CANDLE_MOE_E_DTYPE (unsupported weight dtype)",
    -4: "CANDLE_MOE_E_WORKSPACE (workspace too small)",
    -5: "CANDLE_MOE_E_ALIGN (pointer alignment)",
    -6: "CANDLE_MOE_E_NO_DEVICE",
    -7: "CANDLE_MOE_E_STATIC_SCRATCH (needs more than the built-in 16 MiB scratch)",
    -8: "CANDLE_MOE_E_NCCL (libnccl missing or an NCCL call failed)",
    -9: "CANDLE_MOE_E_EP_MISMATCH (the ranks' exchange metadata disagree; nothing was exchanged)",
}

# candle_moe_set_tuning keys
TUNE_GEMM_ENABLED, TUNE_GEMM_MIN_ROWS, TUNE_STREAM_MAX_ROWS, TUNE_FORCE_ROWS, TUNE_MID_ENABLED = range(5)


class CandleMoeError(RuntimeError):
    """Mirrors candle's `Error::Cuda`: a launcher returned a nonzero status."""

    def __init__(self, fn: str, status: int):
        self.status = status
        what = ERROR_NAMES.get(status, f"cudaError_t {status}" if status > 0 else f"status {status}")
        super().__init__(f"{fn} failed: {what}")


class MoeWeightsC(C.Structure):
    """candle_moe_weights_t"""
    _fields_ = [
        ("d_model", C.c_int32), ("d_ff", C.c_int32), ("n_experts", C.c_int32), ("top_k", C.c_int32),
        ("renorm", C.c_int32), ("dtype_w13", C.c_int32), ("dtype_w2", C.c_int32), ("d_ff_shared", C.c_int32),
        ("dtype_shared13", C.c_int32), ("dtype_shared2", C.c_int32),
        ("router", C.c_void_p), ("router_bias", C.c_void_p),
        ("w1", C.POINTER(C.c_void_p)), ("w3", C.POINTER(C.c_void_p)), ("w2", C.POINTER(C.c_void_p)),
        ("shared_w1", C.c_void_p), ("shared_w3", C.c_void_p), ("shared_w2", C.c_void_p),
        ("shared_gate", C.c_void_p),
        ("w1_prepacked", C.POINTER(C.c_void_p)), ("w3_prepacked", C.POINTER(C.c_void_p)),
        ("w2_prepacked", C.POINTER(C.c_void_p)),
        ("shared_w1_prepacked", C.c_void_p), ("shared_w3_prepacked", C.c_void_p), ("shared_w2_prepacked", C.c_void_p),
    ]


class EpConfigC(C.Structure):
    """candle_moe_ep_config_t"""
    _fields_ = [
        ("rank", C.c_int32), ("world", C.c_int32), ("n_experts_global", C.c_int32), ("top_k", C.c_int32),
        ("renorm", C.c_int32), ("max_tokens", C.c_int32), ("force_form", C.c_int32),
        ("inject_count_mismatch", C.c_int32), ("max_recv_rows", C.c_int64),
        ("router", C.c_void_p), ("router_bias", C.c_void_p),
    ]


# every symbol include/candle_moe.h declares: name -> (restype, argtypes)
_P, _I32, _I64, _SZ = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
_PP = C.POINTER(C.c_void_p)
SYMBOLS = {
    "candle_moe_version": (C.c_char_p, []),
    "candle_moe_set_tuning": (C.c_int, [C.c_int32, C.c_int64]),
    "candle_moe_get_tuning": (C.c_int, [C.c_int32, C.POINTER(C.c_int64)]),
    "candle_moe_workspace_bytes": (C.c_int, [C.POINTER(MoeWeightsC), _I64, C.POINTER(_SZ)]),
    "candle_moe_router_topk": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _I32, _I32, _I32, _P, _P]),
    "candle_moe_permute": (C.c_int, [_P, _P, _I64, _I32, _I32, _P, _P, _P, _P]),
    "candle_moe_quantize_act": (C.c_int, [_P, _P, _I64, _I32, _I32, _P, _P, _P]),
    "candle_moe_combine": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _P, _P, _P, _P]),
    "candle_moe_grouped_gate_up": (C.c_int, [_P, _PP, _PP, _I32, _I32, _I32, _I32, _P, _P, _I64, _P, _P, _P, _P]),
    "candle_moe_grouped_down": (C.c_int, [_P, _PP, _I32, _I32, _I32, _I32, _P, _I64, _P, _P, _P, _P]),
    "candle_moe_forward": (C.c_int, [_P, C.POINTER(MoeWeightsC), _P, _I64, _P, _P, _SZ]),
    "candle_moe_ffn_layer_workspace_bytes": (C.c_int, [C.POINTER(MoeWeightsC), _I64, C.POINTER(_SZ)]),
    "candle_moe_ffn_layer": (C.c_int, [_P, C.POINTER(MoeWeightsC), _P, C.c_float, _P, _I64, _P, _P, _SZ]),
    "candle_moe_forward_timed": (C.c_int, [_P, C.POINTER(MoeWeightsC), _P, _I64, _P, _P, _SZ, _P]),
    "candle_moe_forward_static": (C.c_int, [_P, C.POINTER(MoeWeightsC), _P, _I64, _P]),
    "candle_moe_workspace_views": (C.c_int, [C.POINTER(MoeWeightsC), _I64, _P, _PP, _PP, _PP, _PP]),
    "candle_moe_prepacked_bytes": (C.c_int, [_I32, _I64, _I32, C.POINTER(_SZ)]),
    "candle_moe_prepack": (C.c_int, [_P, _I32, _P, _I64, _I32, _P]),
    "candle_moe_grouped_gate_up_prepacked": (C.c_int, [_P, _PP, _PP, _I32, _I32, _I32, _I32, _P, _P, _I64, _P, _P, _P, _P]),
    "candle_moe_grouped_down_prepacked": (C.c_int, [_P, _PP, _I32, _I32, _I32, _I32, _P, _I64, _P, _P, _P, _P]),
    "candle_moe_device_status": (C.c_int, [C.POINTER(C.c_int32)]),
    "candle_moe_device_status_reset": (C.c_int, []),
    "candle_moe_selftest_bounded_wait": (C.c_int, [_P, _I32]),
    "candle_moe_ep_unique_id": (C.c_int, [_P]),
    "candle_moe_ep_comm_init": (C.c_int, [_P, _I32, _I32, C.POINTER(C.c_void_p)]),
    "candle_moe_ep_comm_from_nccl": (C.c_int, [_P, C.POINTER(C.c_void_p)]),
    "candle_moe_ep_comm_destroy": (C.c_int, [_P]),
    "candle_moe_ep_last_error": (C.c_char_p, []),
    "candle_moe_ep_forward_workspace_bytes": (C.c_int, [C.POINTER(EpConfigC), C.POINTER(MoeWeightsC), C.POINTER(_SZ)]),
    "candle_moe_ep_forward_form": (C.c_int, [C.POINTER(EpConfigC), C.POINTER(MoeWeightsC), C.POINTER(C.c_int32),
                                             C.POINTER(C.c_int64)]),
    "candle_moe_ep_forward": (C.c_int, [_P, _P, C.POINTER(EpConfigC), C.POINTER(MoeWeightsC), _P, _I64, _P, _P, _SZ]),
    "candle_moe_ep_forward_timed": (C.c_int, [_P, _P, C.POINTER(EpConfigC), C.POINTER(MoeWeightsC), _P, _I64, _P, _P, _SZ,
                                              _P, _P]),
    "candle_moe_ep_row_bytes": (C.c_int, [_I32, C.POINTER(C.c_size_t)]),
    "candle_moe_ep_pack": (C.c_int, [_P, _P, _I64, _I32, _P, _P, _P, _P]),
    "candle_moe_ep_workspace_bytes": (C.c_int, [C.POINTER(MoeWeightsC), _I64, C.POINTER(C.c_size_t)]),
    "candle_moe_ep_experts": (C.c_int, [_P, C.POINTER(MoeWeightsC), _P, _P, _I32, _I64, _I64, _P, _P, C.c_size_t]),
    "candle_moe_qmatmul_workspace_bytes": (C.c_int, [_I32, _I64, _I32, _I32, C.POINTER(_SZ)]),
    "candle_moe_qmatmul": (C.c_int, [_P, _P, _P, _I32, _I32, _I32, _P, _I64, _P, _P, _SZ]),
    "candle_moe_rmsnorm": (C.c_int, [_P, _P, _P, C.c_float, _I64, _I32, _P]),
    "candle_moe_rope_kv_append": (C.c_int, [_P, _P, _I64, _P, _P, _I32, _I32, _I32, _I32, _I64, _I32, _P, _P, _P]),
    "candle_moe_decode_attention_workspace_bytes": (C.c_int, [_I32, _I32, _I32, _I32, C.POINTER(_SZ)]),
    "candle_moe_decode_attention": (C.c_int, [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _I64, _I32, _P, _P, _SZ]),
    "candle_moe_quantize_weights": (C.c_int, [_P, _I32, _P, _I64, _P]),
    "candle_moe_dequantize": (C.c_int, [_P, _I32, _P, _I64, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library or raises; never substitutes another implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python candle_b200/csrc/build.py` "
                "(there is no CPU or PyTorch fallback for this path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        raise CandleMoeError(fn, status)
