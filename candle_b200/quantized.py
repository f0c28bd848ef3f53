"""Host-side mirror of candle's quantized tensor types for the MoE feed-forward path.

Names and meaning follow candle-core/src/quantized/mod.rs: `GgmlDType` (:134-253), `QTensor`
(:35-38, :286-398) and `QMatMul` (:400-556).  A `QTensor` here owns a CUDA buffer holding the raw
GGUF blocks, row-major `[n][k / block]`, exactly the bytes `QCudaStorage` keeps
(candle-core/src/quantized/cuda.rs:597-616).  Device memory and streams come from torch.
"""
from __future__ import annotations

import enum
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib


class GgmlDType(enum.IntEnum):
    """GGML ids as returned by `GgmlDType::to_u32` (candle-core/src/quantized/mod.rs:176-195)."""
    F32 = 0
    Q8_0 = 8
    Q4K = 12
    Q6K = 14

    def block_size(self) -> int:
        """`GgmlDType::block_size` (mod.rs:232-252)."""
        return {GgmlDType.F32: 1, GgmlDType.Q8_0: 32, GgmlDType.Q4K: 256, GgmlDType.Q6K: 256}[self]

    def type_size(self) -> int:
        """`GgmlDType::type_size` (mod.rs:208-229): bytes per block."""
        return {GgmlDType.F32: 4, GgmlDType.Q8_0: 34, GgmlDType.Q4K: 144, GgmlDType.Q6K: 210}[self]


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class QTensor:
    """A quantized `[n, k]` matrix on a CUDA device (`QTensor`, mod.rs:35-38)."""

    def __init__(self, data: torch.Tensor, dtype: GgmlDType, shape: Tuple[int, int]):
        if not data.is_cuda or data.dtype != torch.uint8:
            raise ValueError("QTensor storage must be a CUDA uint8 tensor")
        n, k = shape
        if k % dtype.block_size():
            raise ValueError(f"last dim {k} is not a multiple of the {dtype.name} block size")
        if data.numel() != n * (k // dtype.block_size()) * dtype.type_size():
            raise ValueError("storage size does not match shape and dtype")
        self.data, self._dtype, self._shape = data, GgmlDType(dtype), (int(n), int(k))

    # -- constructors -----------------------------------------------------------------------------
    @classmethod
    def from_blocks(cls, blocks, dtype: GgmlDType, shape: Tuple[int, int], device="cuda") -> "QTensor":
        """Upload raw GGUF block bytes (what `qtensor_from_ggml` + `load_quantized` do,
        candle-core/src/quantized/ggml_file.rs:138-189, cuda.rs:597-616)."""
        if isinstance(blocks, np.ndarray):
            blocks = torch.from_numpy(np.ascontiguousarray(blocks).view(np.uint8))
        return cls(blocks.to(device=device, dtype=torch.uint8).contiguous(), dtype, shape)

    @classmethod
    def quantize(cls, src: torch.Tensor, dtype: GgmlDType) -> "QTensor":
        """`QTensor::quantize` (mod.rs:288-318), on the device and bit-exact with the CPU quantizer."""
        if src.dim() != 2 or not src.is_cuda:
            raise ValueError("quantize expects a 2-D CUDA tensor")
        src = src.to(torch.float32).contiguous()
        n, k = src.shape
        dtype = GgmlDType(dtype)
        if k % dtype.block_size():
            raise ValueError(f"last dim {k} is not a multiple of the {dtype.name} block size")
        out = torch.empty(n * (k // dtype.block_size()) * dtype.type_size(), dtype=torch.uint8, device=src.device)
        with torch.cuda.device(src.device):
            st = _lib.load().candle_moe_quantize_weights(_stream_ptr(src.device), int(dtype), src.data_ptr(),
                                                          src.numel(), out.data_ptr())
        _lib.check("candle_moe_quantize_weights", st)
        return cls(out, dtype, (n, k))

    # -- accessors ---------------------------------------------------------------------------------
    def dtype(self) -> GgmlDType:
        return self._dtype

    def shape(self) -> Tuple[int, int]:
        return self._shape

    def device(self) -> torch.device:
        return self.data.device

    def storage_size_in_bytes(self) -> int:
        return self.data.numel()

    def device_ptr(self) -> int:
        return self.data.data_ptr()

    def prepack(self) -> torch.Tensor:
        """Decode-path copy in register-fragment order (`candle_moe_prepack`); cached on the tensor."""
        if getattr(self, "_prepacked", None) is None:
            import ctypes as C
            n, k = self._shape
            need = C.c_size_t(0)
            _lib.check("candle_moe_prepacked_bytes",
                       _lib.load().candle_moe_prepacked_bytes(int(self._dtype), n, k, C.byref(need)))
            out = torch.empty(need.value, dtype=torch.uint8, device=self.data.device)
            with torch.cuda.device(self.data.device):
                st = _lib.load().candle_moe_prepack(_stream_ptr(self.data.device), int(self._dtype), self.data.data_ptr(),
                                                    n, k, out.data_ptr())
            _lib.check("candle_moe_prepack", st)
            self._prepacked = out
        return self._prepacked

    def dequantize(self) -> torch.Tensor:
        """`QTensor::dequantize` (mod.rs:349-353)."""
        n, k = self._shape
        out = torch.empty((n, k), dtype=torch.float32, device=self.data.device)
        with torch.cuda.device(self.data.device):
            st = _lib.load().candle_moe_dequantize(_stream_ptr(self.data.device), int(self._dtype),
                                                   self.data.data_ptr(), n * k, out.data_ptr())
        _lib.check("candle_moe_dequantize", st)
        return out


class QMatMul:
    """`QMatMul::QTensor` (mod.rs:400-404): `forward(xs)` computes `xs . W^T` with the k-quant
    arithmetic of `k_quants::matmul` (activations quantized per row, integer block dots)."""

    def __init__(self, qtensor: QTensor):
        self.inner = qtensor
        self._ws: Optional[torch.Tensor] = None
        self._ws_rows = 0
        self._prepacked: Optional[torch.Tensor] = None

    @classmethod
    def from_qtensor(cls, qtensor: QTensor) -> "QMatMul":
        return cls(qtensor)

    def prepack(self) -> "QMatMul":
        """Make the decode-path copy of the matrix (one-time; Q4_K / Q6_K whose shape the repack takes)."""
        n, k = self.inner.shape()
        dt = self.inner.dtype()
        if dt in (GgmlDType.Q4K, GgmlDType.Q6K) and n % 16 == 0 and k % 256 == 0 and (dt == GgmlDType.Q4K or (k // 256) % 2 == 0):
            self._prepacked = self.inner.prepack()
        elif dt == GgmlDType.Q8_0:
            self._prepacked = self.inner.prepack()
        return self

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        """`QMatMul::forward` (mod.rs:533-537) through `candle_moe_qmatmul`."""
        import ctypes as C
        lib = _lib.load()
        n, k = self.inner.shape()
        if xs.shape[-1] != k:
            raise ValueError(f"shape mismatch in qmatmul: {tuple(xs.shape)} x ({n}, {k})^T")
        if not xs.is_cuda or xs.dtype != torch.float32:
            raise ValueError("QMatMul.forward expects a CUDA f32 tensor")
        lead = xs.shape[:-1]
        x2 = xs.reshape(-1, k).contiguous()
        rows = x2.shape[0]
        dev, dt = x2.device, int(self.inner.dtype())
        out = torch.empty((rows, n), dtype=torch.float32, device=dev)
        if rows == 0:
            return out.reshape(*lead, n)
        if self._ws is None or rows > self._ws_rows:
            need = C.c_size_t(0)
            cap = max(rows, 2 * self._ws_rows)
            _lib.check("candle_moe_qmatmul_workspace_bytes", lib.candle_moe_qmatmul_workspace_bytes(dt, cap, n, k, C.byref(need)))
            # rows <= 64 and rows > 64 lay the scratch out differently: hold the larger of the two
            small = C.c_size_t(0)
            _lib.check("candle_moe_qmatmul_workspace_bytes",
                       lib.candle_moe_qmatmul_workspace_bytes(dt, min(cap, 64), n, k, C.byref(small)))
            self._ws = torch.empty(max(need.value, small.value) + 256, dtype=torch.uint8, device=dev)
            self._ws_rows = cap
        ws_ptr = (self._ws.data_ptr() + 255) // 256 * 256
        pp = None if self._prepacked is None else self._prepacked.data_ptr()
        with torch.cuda.device(dev):
            _lib.check("candle_moe_qmatmul",
                       lib.candle_moe_qmatmul(_stream_ptr(dev), self.inner.device_ptr(), pp, dt, n, k, x2.data_ptr(), rows,
                                              out.data_ptr(), ws_ptr, self._ws.numel() - 256))
        return out.reshape(*lead, n)

    __call__ = forward
