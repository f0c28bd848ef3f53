"""GGUF container: reading the expert tensors of a MoE layer into device `QTensor`s, and writing files.

Follows candle-core/src/quantized/gguf_file.rs: `VersionedMagic` (:27-48), `Value` / `ValueType`
(:152-438), `Content::read` (:441-516), `TensorInfo::read_from_mmap` (:92-125), `write` (:534-582).
The layer loader follows the tensor names of candle-transformers/src/models/quantized_llama.rs:544-579
(`blk.{l}.ffn_{gate,down,up}.{i}.weight`, `blk.{l}.ffn_gate_inp.weight`, `blk.{l}.ffn_norm.weight`) and
also accepts the merged form newer converters write (`blk.{l}.ffn_{gate,down,up}_exps.weight`, one
`[E, n, k]` tensor per matrix kind), which the reference does not read.

Parsing needs no device: `Content.read` and `TensorInfo.raw` work on bytes (a `bytes`, `mmap` or
numpy buffer); only `TensorInfo.read` / `Content.tensor` / `load_moe_layer` upload.  The block bytes are
uploaded as they lie in the file, which is the layout the kernels read (cuda.rs:597-616 does the same).
"""
from __future__ import annotations

import enum
import mmap as _mmap
import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

DEFAULT_ALIGNMENT = 32  # gguf_file.rs:9
_MAGICS = (0x46554747, 0x47475546)  # gguf_file.rs:20


class GgufError(ValueError):
    """Any malformed-file or wrong-type condition the reference reports through `crate::bail!`."""


class ValueType(enum.IntEnum):
    """`ValueType::from_u32` / `to_u32` (gguf_file.rs:400-438)."""
    U8 = 0
    I8 = 1
    U16 = 2
    I16 = 3
    U32 = 4
    I32 = 5
    F32 = 6
    BOOL = 7
    STRING = 8
    ARRAY = 9
    U64 = 10
    I64 = 11
    F64 = 12


_SCALAR_FMT = {ValueType.U8: "<B", ValueType.I8: "<b", ValueType.U16: "<H", ValueType.I16: "<h", ValueType.U32: "<I",
               ValueType.I32: "<i", ValueType.F32: "<f", ValueType.U64: "<Q", ValueType.I64: "<q", ValueType.F64: "<d"}


@dataclass(frozen=True)
class Value:
    """A typed metadata value (`Value`, gguf_file.rs:182-196).  Arrays hold `Value`s."""
    type: ValueType
    v: Any

    # constructors for the common cases
    @classmethod
    def u32(cls, v: int) -> "Value":
        return cls(ValueType.U32, int(v))

    @classmethod
    def f32(cls, v: float) -> "Value":
        return cls(ValueType.F32, float(np.float32(v)))

    @classmethod
    def string(cls, v: str) -> "Value":
        return cls(ValueType.STRING, str(v))

    @classmethod
    def array(cls, vs: Sequence["Value"]) -> "Value":
        return cls(ValueType.ARRAY, list(vs))

    def _as(self, t: ValueType, what: str):
        if self.type != t:
            raise GgufError(f"not a {what} {self!r}")
        return self.v

    # the accessors of gguf_file.rs:218-324; only to_u64 upcasts
    def to_u8(self):
        return self._as(ValueType.U8, "u8")

    def to_i8(self):
        return self._as(ValueType.I8, "i8")

    def to_u16(self):
        return self._as(ValueType.U16, "u16")

    def to_i16(self):
        return self._as(ValueType.I16, "i16")

    def to_u32(self):
        return self._as(ValueType.U32, "u32")

    def to_i32(self):
        return self._as(ValueType.I32, "i32")

    def to_u64(self):
        if self.type in (ValueType.U64, ValueType.U8, ValueType.U16, ValueType.U32, ValueType.BOOL):
            return int(self.v)
        raise GgufError(f"not a u64 or upcastable to u64 {self!r}")

    def to_i64(self):
        return self._as(ValueType.I64, "i64")

    def to_f32(self):
        return self._as(ValueType.F32, "f32")

    def to_f64(self):
        return self._as(ValueType.F64, "f64")

    def to_bool(self):
        return self._as(ValueType.BOOL, "bool")

    def to_vec(self):
        return self._as(ValueType.ARRAY, "vec")

    def to_string(self):
        return self._as(ValueType.STRING, "string")

    def py(self):
        """Plain Python value (arrays become lists), for comparisons in tests."""
        return [e.py() for e in self.v] if self.type == ValueType.ARRAY else self.v


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = memoryview(buf), 0

    def take(self, n: int) -> memoryview:
        if n < 0 or self.pos + n > len(self.buf):
            raise GgufError("failed to fill whole buffer")  # what read_exact reports at end of file
        out = self.buf[self.pos:self.pos + n]
        self.pos += n
        return out

    def unpack(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]


def _read_len(c: _Cursor, version: int) -> int:
    return c.unpack("<I") if version == 1 else c.unpack("<Q")


def _read_string(c: _Cursor, version: int) -> str:
    """gguf_file.rs:135-150: length-prefixed, trailing NULs dropped, invalid UTF-8 replaced."""
    raw = bytes(c.take(_read_len(c, version)))
    return raw.rstrip(b"\0").decode("utf-8", errors="replace")


def _value_type(u: int) -> ValueType:
    try:
        return ValueType(u)
    except ValueError:
        raise GgufError(f"unrecognized value-type {u:#08x}") from None


def _read_value(c: _Cursor, t: ValueType, version: int) -> Value:
    """`Value::read` (gguf_file.rs:326-361)."""
    if t in _SCALAR_FMT:
        return Value(t, c.unpack(_SCALAR_FMT[t]))
    if t == ValueType.BOOL:
        b = c.unpack("<B")
        if b > 1:
            raise GgufError(f"unexpected bool value {b}")
        return Value(t, bool(b))
    if t == ValueType.STRING:
        return Value(t, _read_string(c, version))
    et = _value_type(c.unpack("<I"))
    n = _read_len(c, version)
    return Value(t, [_read_value(c, et, version) for _ in range(n)])


# GGML dtype ids (candle-core/src/quantized/mod.rs:153-195) with (block elements, block bytes) (:208-252)
_GGML = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
         7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2K", 256, 84), 11: ("Q3K", 256, 110),
         12: ("Q4K", 256, 144), 13: ("Q5K", 256, 176), 14: ("Q6K", 256, 210), 15: ("Q8K", 256, 292), 30: ("BF16", 1, 2)}


def ggml_dtype_name(u: int) -> str:
    return _GGML[u][0]


@dataclass
class TensorInfo:
    """`TensorInfo` (gguf_file.rs:50-55): `shape` is outermost first (the file stores it reversed)."""
    ggml_dtype: int
    shape: Tuple[int, ...]
    offset: int

    def size_in_bytes(self) -> int:
        _, bs, ts = _GGML[self.ggml_dtype]
        n = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        if n % bs:
            raise GgufError(f"the number of elements {n} is not divisible by the block size {bs}")
        return n // bs * ts

    def raw(self, data, tensor_data_offset: int) -> np.ndarray:
        """The tensor's bytes as a view of `data` (`read_from_mmap`, gguf_file.rs:92-125)."""
        size = self.size_in_bytes()
        start = tensor_data_offset + self.offset
        if start + size > len(data):
            raise GgufError(f"tensor data extends beyond file boundary: offset={start}, size={size}, file_len={len(data)}")
        return np.frombuffer(data, dtype=np.uint8, count=size, offset=start)

    def read(self, data, tensor_data_offset: int, device="cuda"):
        """Upload.  Block formats the kernels read come back as a `QTensor` (2-D) or, for a merged expert
        tensor `[E, n, k]`, as a list of E `QTensor`s over one device buffer; F32 / F16 / BF16 tensors come
        back as f32 torch tensors (what `QMatMul::from_arc` makes of them, mod.rs:430-436)."""
        import torch
        from .quantized import GgmlDType, QTensor
        raw = self.raw(data, tensor_data_offset)
        name = _GGML[self.ggml_dtype][0]
        if name in ("F32", "F16", "BF16"):
            if name == "F32":
                t = torch.from_numpy(raw.view(np.float32).copy())
            elif name == "F16":
                t = torch.from_numpy(raw.view(np.float16).copy()).to(torch.float32)
            else:
                t = torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).to(torch.float32)
            return t.reshape(self.shape).to(device)
        try:
            dt = GgmlDType(self.ggml_dtype)
        except ValueError:
            raise GgufError(f"{name} tensors are not read by this path (Q4K, Q6K, Q8_0 and float types are)") from None
        dev_bytes = torch.from_numpy(raw.copy()).to(device)
        if len(self.shape) == 2:
            return QTensor(dev_bytes, dt, (self.shape[0], self.shape[1]))
        if len(self.shape) != 3:
            raise GgufError(f"a quantized tensor of rank {len(self.shape)} is not read by this path")
        E, n, k = self.shape
        per = len(raw) // E
        # every expert matrix must start where the kernels' bulk copies may start
        parts = [dev_bytes[e * per:(e + 1) * per] for e in range(E)]
        if per % 256:
            parts = [p.clone() for p in parts]
        return [QTensor(p, dt, (n, k)) for p in parts]


@dataclass
class Content:
    """`Content` (gguf_file.rs:127-133)."""
    version: int
    metadata: Dict[str, Value]
    tensor_infos: Dict[str, TensorInfo]
    tensor_data_offset: int

    @classmethod
    def read(cls, data) -> "Content":
        """`Content::read` (gguf_file.rs:441-516) over the file's bytes."""
        c = _Cursor(data)
        magic = c.unpack("<I")
        if magic not in _MAGICS:
            raise GgufError(f"unknown magic 0x{magic:08x}")
        version = c.unpack("<I")
        if version not in (1, 2, 3):
            raise GgufError(f"gguf: unsupported magic/version Gguf/{version}")
        n_tensors = _read_len(c, version)
        n_kv = _read_len(c, version)
        metadata: Dict[str, Value] = {}
        for _ in range(n_kv):
            key = _read_string(c, version)
            metadata[key] = _read_value(c, _value_type(c.unpack("<I")), version)
        infos: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = _read_string(c, version)
            nd = c.unpack("<I")
            dims = [c.unpack("<I") if version == 1 else c.unpack("<Q") for _ in range(nd)]
            u = c.unpack("<I")
            if u not in _GGML:
                raise GgufError(f"unknown dtype for tensor {u}")
            infos[name] = TensorInfo(u, tuple(reversed(dims)), c.unpack("<Q"))
        al = metadata.get("general.alignment")
        alignment = DEFAULT_ALIGNMENT
        if al is not None and al.type in (ValueType.U8, ValueType.U16, ValueType.U32, ValueType.I8, ValueType.I16,
                                          ValueType.I32) and al.v >= 0:
            alignment = al.v
        if alignment == 0:
            raise GgufError("general.alignment is zero")  # the reference divides by it
        return cls(version, metadata, infos, -(-c.pos // alignment) * alignment)

    def info(self, name: str) -> TensorInfo:
        if name not in self.tensor_infos:
            raise GgufError(f"cannot find tensor info for {name}")
        return self.tensor_infos[name]

    def tensor(self, data, name: str, device="cuda"):
        """`Content::tensor` (gguf_file.rs:518-529)."""
        return self.info(name).read(data, self.tensor_data_offset, device)

    def md_get(self, key: str) -> Value:
        if key not in self.metadata:
            raise GgufError(f"cannot find {key} in metadata")
        return self.metadata[key]


def open_mmap(path: str):
    """Map a file read-only; returns (mmap, Content).  The mapping must outlive `TensorInfo.raw` views."""
    with open(path, "rb") as f:
        mm = _mmap.mmap(f.fileno(), 0, access=_mmap.ACCESS_READ)
    return mm, Content.read(mm)


# ---- writing -------------------------------------------------------------------------------------

def _write_string(w: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    w.write(struct.pack("<Q", len(b)))
    w.write(b)


def _write_value(w: BinaryIO, val: Value) -> None:
    """`Value::write` (gguf_file.rs:363-397)."""
    t = val.type
    if t in _SCALAR_FMT:
        w.write(struct.pack(_SCALAR_FMT[t], val.v))
    elif t == ValueType.BOOL:
        w.write(struct.pack("<B", 1 if val.v else 0))
    elif t == ValueType.STRING:
        _write_string(w, val.v)
    else:
        kinds = {e.type for e in val.v}
        if len(kinds) > 1:
            raise GgufError(f"multiple value-types in the same array {sorted(k.name for k in kinds)}")
        et = kinds.pop() if kinds else ValueType.U32
        w.write(struct.pack("<IQ", int(et), len(val.v)))
        for e in val.v:
            _write_value(w, e)


def _pad32(n: int) -> int:
    return 31 - (31 + n) % 32


def write(w: BinaryIO, metadata: Sequence[Tuple[str, Value]],
          tensors: Sequence[Tuple[str, int, Tuple[int, ...], Union[bytes, np.ndarray]]]) -> None:
    """`gguf_file::write` (gguf_file.rs:534-582): a version-2 file, tensor data padded to 32 bytes.
    A tensor is (name, ggml dtype id, shape outermost first, block bytes)."""
    start = w.tell()
    w.write(struct.pack("<IIQQ", 0x46554747, 2, len(tensors), len(metadata)))
    for name, val in metadata:
        _write_string(w, name)
        w.write(struct.pack("<I", int(val.type)))
        _write_value(w, val)
    offset = 0
    blobs: List[bytes] = []
    for name, dt, shape, data in tensors:
        blob = data.tobytes() if isinstance(data, np.ndarray) else bytes(data)
        if TensorInfo(dt, tuple(shape), 0).size_in_bytes() != len(blob):
            raise GgufError(f"tensor {name}: {len(blob)} bytes do not match shape {tuple(shape)} of {ggml_dtype_name(dt)}")
        _write_string(w, name)
        w.write(struct.pack("<I", len(shape)))
        for dim in reversed(shape):
            w.write(struct.pack("<Q", dim))
        w.write(struct.pack("<IQ", dt, offset))
        blobs.append(blob)
        offset += len(blob) + _pad32(len(blob))
    w.write(b"\0" * _pad32(w.tell() - start))
    for blob in blobs:
        w.write(blob)
        w.write(b"\0" * _pad32(len(blob)))


# ---- the MoE layer -------------------------------------------------------------------------------

@dataclass
class MoeLayerTensors:
    """Names of one layer's FFN tensors, resolved against a file."""
    gate_inp: str
    ffn_norm: str
    merged: bool
    w1: List[str]  # per expert, or one merged name
    w2: List[str]
    w3: List[str]


def moe_layer_names(ct: Content, layer_idx: int, n_expert: int) -> MoeLayerTensors:
    """The tensor names quantized_llama.rs:544-579 reads for layer `layer_idx`; the merged `_exps` form is used
    when the per-expert names are absent."""
    p = f"blk.{layer_idx}"
    per = [[f"{p}.ffn_{kind}.{i}.weight" for i in range(n_expert)] for kind in ("gate", "down", "up")]
    merged = [f"{p}.ffn_{kind}_exps.weight" for kind in ("gate", "down", "up")]
    if all(n in ct.tensor_infos for names in per for n in names):
        return MoeLayerTensors(f"{p}.ffn_gate_inp.weight", f"{p}.ffn_norm.weight", False, per[0], per[1], per[2])
    if all(n in ct.tensor_infos for n in merged):
        for n in merged:
            shp = ct.tensor_infos[n].shape
            if len(shp) != 3 or shp[0] != n_expert:
                raise GgufError(f"{n}: shape {shp} does not hold {n_expert} expert matrices")
        return MoeLayerTensors(f"{p}.ffn_gate_inp.weight", f"{p}.ffn_norm.weight", True, [merged[0]], [merged[1]], [merged[2]])
    # report the first name the reference would have failed on
    missing = next(n for names in zip(*per) for n in names if n not in ct.tensor_infos)
    raise GgufError(f"cannot find tensor info for {missing}")


def load_moe_layer(ct: Content, data, layer_idx: int, device="cuda", *, arch: str = "llama", prepack: bool = False):
    """Build the MoE block of layer `layer_idx` from a GGUF file, as `ModelWeights::from_gguf` does for its
    `mlp_or_moe` (quantized_llama.rs:496-579).  Returns (block, ffn_norm weight [d] f32 on the device, rms eps)."""
    from .moe import Mlp, MlpOrMoe
    from .quantized import QMatMul, QTensor
    n_expert = ct.md_get(f"{arch}.expert_count").to_u32()
    n_used = ct.md_get(f"{arch}.expert_used_count").to_u32()
    eps = ct.md_get(f"{arch}.attention.layer_norm_rms_epsilon").to_f32()
    if n_expert <= 1:
        raise GgufError("not a mixture-of-experts file (expert_count <= 1)")
    names = moe_layer_names(ct, layer_idx, n_expert)
    gate_inp = ct.tensor(data, names.gate_inp, device)
    if isinstance(gate_inp, QTensor):
        gate_inp = gate_inp.dequantize()  # a quantized router: the reference multiplies by it as a QMatMul
    ffn_norm = ct.tensor(data, names.ffn_norm, device)
    if names.merged:
        w1, w2, w3 = (ct.tensor(data, n[0], device) for n in (names.w1, names.w2, names.w3))
    else:
        w1, w2, w3 = ([ct.tensor(data, n, device) for n in ns] for ns in (names.w1, names.w2, names.w3))
    experts = [Mlp(QMatMul.from_qtensor(a), QMatMul.from_qtensor(b), QMatMul.from_qtensor(c)) for a, b, c in zip(w1, w2, w3)]
    block = MlpOrMoe.moe(n_used, gate_inp, experts)
    if prepack:
        block.prepack()
    return block, ffn_norm.reshape(-1), float(eps)
