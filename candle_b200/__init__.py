"""B200-native quantized mixture-of-experts feed-forward block for candle's quantized_llama.

The package is a thin host-side mirror (`GgmlDType`, `QTensor`, `QMatMul`, `Mlp`, `MlpOrMoe`) over
the C ABI of `libcandle_moe_sm100.so` (include/candle_moe.h); all arithmetic runs in hand-written
CUDA kernels for sm_100a.  Importing the package loads the library and raises if it is missing.
"""
from . import _lib

_lib.load()  # fail loudly: there is no fallback implementation

from ._lib import CandleMoeError  # noqa: E402
from .quantized import GgmlDType, QMatMul, QTensor  # noqa: E402
from .moe import Mlp, MlpOrMoe  # noqa: E402
from .expert_parallel import ExpertParallelMoe  # noqa: E402

__all__ = ["CandleMoeError", "GgmlDType", "QMatMul", "QTensor", "Mlp", "MlpOrMoe", "ExpertParallelMoe"]
