"""GGUF reading and writing (candle-core/src/quantized/gguf_file.rs) and the MoE layer loader
(candle-transformers/src/models/quantized_llama.rs:496-579).

The reference's own test of this code is a write -> read round trip
(candle-pyo3/tests/native/test_utils.py:26-52); the cases here add files assembled byte by byte in the
test (independent of the writer) as known answers for the reader, and the error cases the reader has."""
import io
import struct

import numpy as np
import pytest

from candle_b200 import gguf
from candle_b200.gguf import Content, GgufError, Value, ValueType


def _s(text: bytes, v1=False) -> bytes:
    return struct.pack("<I" if v1 else "<Q", len(text)) + text


def _handmade_v3() -> bytes:
    """magic, version 3, 2 tensors, 5 key/values, padded to general.alignment = 64."""
    b = struct.pack("<IIQQ", 0x46554747, 3, 2, 5)
    b += _s(b"general.alignment") + struct.pack("<II", 4, 64)
    b += _s(b"llama.expert_count\0\0") + struct.pack("<II", 4, 8)            # trailing NULs are dropped
    b += _s(b"name") + struct.pack("<I", 8) + _s(b"tiny")
    b += _s(b"flags") + struct.pack("<IIQ", 9, 7, 3) + bytes([1, 0, 1])       # array of 3 bools
    b += _s(b"nested") + struct.pack("<IIQ", 9, 9, 2) + struct.pack("<IQhh", 3, 2, -1, 2) + struct.pack("<IQ", 3, 0)
    b += _s(b"a.weight") + struct.pack("<IQQIQ", 2, 256, 3, 12, 0)            # file order: innermost first
    b += _s(b"b.weight") + struct.pack("<IQIQ", 1, 4, 0, 448)
    pad = -len(b) % 64
    data = bytes(range(256)) * 2
    return b + b"\0" * pad + data[:432] + b"\0" * 16 + struct.pack("<4f", 1.0, -2.0, 0.5, 3.0)


def test_reader_known_answer_v3():
    raw = _handmade_v3()
    ct = Content.read(raw)
    assert ct.version == 3
    assert ct.tensor_data_offset % 64 == 0 and raw[ct.tensor_data_offset:ct.tensor_data_offset + 3] == bytes([0, 1, 2])
    assert ct.md_get("llama.expert_count").to_u32() == 8
    assert ct.md_get("name").to_string() == "tiny"
    assert ct.md_get("flags").py() == [True, False, True]
    assert ct.md_get("nested").py() == [[-1, 2], []]
    a = ct.info("a.weight")
    assert a.shape == (3, 256) and gguf.ggml_dtype_name(a.ggml_dtype) == "Q4K" and a.size_in_bytes() == 3 * 144
    assert bytes(a.raw(raw, ct.tensor_data_offset)) == (bytes(range(256)) * 2)[:432]
    b = ct.info("b.weight")
    assert b.shape == (4,) and b.raw(raw, ct.tensor_data_offset).view(np.float32).tolist() == [1.0, -2.0, 0.5, 3.0]
    with pytest.raises(GgufError, match="cannot find tensor info for c.weight"):
        ct.info("c.weight")
    with pytest.raises(GgufError, match="cannot find nope in metadata"):
        ct.md_get("nope")


def test_reader_known_answer_v1_uses_32_bit_lengths():
    b = struct.pack("<IIII", 0x46554747, 1, 1, 1)
    b += _s(b"k", True) + struct.pack("<IIIff", 9, 6, 2, 1.5, -0.25)
    b += _s(b"t", True) + struct.pack("<IIIIQ", 2, 32, 2, 8, 0)
    b += b"\0" * (-len(b) % 32) + bytes(68)
    ct = Content.read(b)
    assert ct.version == 1 and ct.md_get("k").py() == [1.5, -0.25]
    assert ct.info("t").shape == (2, 32) and ct.info("t").size_in_bytes() == 68
    assert ct.tensor_data_offset % 32 == 0


def test_byte_swapped_magic_is_accepted_like_the_reference():
    b = struct.pack("<IIQQ", 0x47475546, 2, 0, 0)
    assert Content.read(b).tensor_data_offset == 32


@pytest.mark.parametrize("raw,msg", [
    (struct.pack("<IIQQ", 0x12345678, 3, 0, 0), "unknown magic 0x12345678"),
    (struct.pack("<IIQQ", 0x46554747, 4, 0, 0), "unsupported magic/version"),
    (struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _s(b"k") + struct.pack("<IB", 7, 2), "unexpected bool value 2"),
    (struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _s(b"k") + struct.pack("<I", 13), "unrecognized value-type"),
    (struct.pack("<IIQQ", 0x46554747, 3, 1, 0) + _s(b"t") + struct.pack("<IQIQ", 1, 32, 99, 0), "unknown dtype for tensor 99"),
    (struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + _s(b"k") + struct.pack("<I", 4), "failed to fill whole buffer"),
    (struct.pack("<IIQ", 0x46554747, 3, 0), "failed to fill whole buffer"),
])
def test_reader_errors(raw, msg):
    with pytest.raises(GgufError, match=msg):
        Content.read(raw)


def test_tensor_size_errors():
    b = struct.pack("<IIQQ", 0x46554747, 3, 2, 0)
    b += _s(b"odd") + struct.pack("<IQIQ", 1, 100, 12, 0)        # 100 elements of a 256-element block format
    b += _s(b"far") + struct.pack("<IQIQ", 1, 256, 12, 1 << 20)
    b += b"\0" * (-len(b) % 32) + bytes(144)
    ct = Content.read(b)
    with pytest.raises(GgufError, match="100 is not divisible by the block size 256"):
        ct.info("odd").raw(b, ct.tensor_data_offset)
    with pytest.raises(GgufError, match="extends beyond file boundary"):
        ct.info("far").raw(b, ct.tensor_data_offset)


def test_value_accessors_follow_the_reference():
    assert Value(ValueType.U8, 7).to_u64() == 7 and Value(ValueType.BOOL, True).to_u64() == 1
    with pytest.raises(GgufError, match="not a u64"):
        Value(ValueType.I32, 7).to_u64()
    with pytest.raises(GgufError, match="not a u32"):   # only to_u64 upcasts
        Value(ValueType.U8, 7).to_u32()
    with pytest.raises(GgufError, match="not a f32"):
        Value(ValueType.F64, 1.0).to_f32()


def test_write_read_round_trip_and_layout():
    rng = np.random.default_rng(3)
    q4 = rng.integers(0, 256, 16 * 144, dtype=np.uint8)           # [16, 256] of Q4K: 2304 bytes (a multiple of 32)
    q8 = rng.integers(0, 256, 3 * 34, dtype=np.uint8)             # [3, 32] of Q8_0: 102 bytes (padded to 128)
    f = rng.standard_normal((16, 16)).astype(np.float32)
    md = [("a", Value(ValueType.I64, 1)), ("b", Value.string("foo")),
          ("c", Value.array([Value.u32(1), Value.u32(2), Value.u32(3)])),
          ("d", Value.array([Value.array([Value.u32(1), Value.u32(2)]), Value.array([Value.u32(3), Value.u32(4)])])),
          ("e", Value.array([])), ("f", Value(ValueType.BOOL, True)), ("g", Value(ValueType.F64, 0.1))]
    w = io.BytesIO()
    gguf.write(w, md, [("q8", 8, (3, 32), q8), ("q4", 12, (16, 256), q4), ("f", 0, (16, 16), f)])
    raw = w.getvalue()
    assert raw[:8] == struct.pack("<II", 0x46554747, 2) and len(raw) % 32 == 0
    ct = Content.read(raw)
    assert ct.version == 2 and ct.tensor_data_offset % 32 == 0
    assert {k: v.py() for k, v in ct.metadata.items()} == {"a": 1, "b": "foo", "c": [1, 2, 3], "d": [[1, 2], [3, 4]], "e": [],
                                                            "f": True, "g": 0.1}
    assert ct.md_get("e").type == ValueType.ARRAY
    assert [ct.info(n).offset for n in ("q8", "q4", "f")] == [0, 128, 128 + 2304]
    assert np.array_equal(ct.info("q8").raw(raw, ct.tensor_data_offset), q8)
    assert np.array_equal(ct.info("q4").raw(raw, ct.tensor_data_offset), q4)
    assert np.array_equal(ct.info("f").raw(raw, ct.tensor_data_offset).view(np.float32).reshape(16, 16), f)
    with pytest.raises(GgufError, match="multiple value-types in the same array"):
        gguf.write(io.BytesIO(), [("x", Value.array([Value.u32(1), Value.f32(1.0)]))], [])
    with pytest.raises(GgufError, match="do not match shape"):
        gguf.write(io.BytesIO(), [], [("t", 12, (2, 256), q4)])


def _layer_file(orc, mw, merged: bool, layer=1, eps=1e-5) -> bytes:
    """A one-layer Mixtral-style file holding the oracle-side weights `mw`."""
    d, ff, E = mw.d_model, mw.d_ff, mw.n_experts
    md = [("general.architecture", Value.string("llama")), ("llama.expert_count", Value.u32(E)),
          ("llama.expert_used_count", Value.u32(mw.top_k)), ("llama.embedding_length", Value.u32(d)),
          ("llama.attention.layer_norm_rms_epsilon", Value.f32(eps))]
    p = f"blk.{layer}"
    norm = (1.0 + 0.05 * np.random.default_rng(9).standard_normal(d)).astype(np.float32)
    ts = [(f"{p}.ffn_gate_inp.weight", 0, (E, d), mw.router), (f"{p}.ffn_norm.weight", 0, (d,), norm)]
    kinds = (("gate", mw.w1, mw.dtype_w13, (ff, d)), ("down", mw.w2, mw.dtype_w2, (d, ff)), ("up", mw.w3, mw.dtype_w13, (ff, d)))
    for kind, ws, dt, shp in kinds:
        if merged:
            ts.append((f"{p}.ffn_{kind}_exps.weight", dt, (E,) + shp, np.concatenate([np.asarray(w).view(np.uint8).ravel() for w in ws])))
        else:
            ts += [(f"{p}.ffn_{kind}.{i}.weight", dt, shp, np.asarray(ws[i]).view(np.uint8).ravel()) for i in range(E)]
    w = io.BytesIO()
    gguf.write(w, md, ts)
    return w.getvalue(), norm


@pytest.mark.parametrize("merged", [False, True])
def test_moe_layer_names_and_bytes(orc, merged):
    mw = orc.make_moe_weights(21, 256, 512, 4, 2, orc.Q4K, orc.Q6K)
    raw, _ = _layer_file(orc, mw, merged)
    ct = Content.read(raw)
    names = gguf.moe_layer_names(ct, 1, 4)
    assert names.merged == merged and len(names.w1) == (1 if merged else 4)
    for e in range(4):
        for lst, ws in ((names.w1, mw.w1), (names.w2, mw.w2), (names.w3, mw.w3)):
            got = ct.info(lst[0] if merged else lst[e]).raw(raw, ct.tensor_data_offset)
            want = np.asarray(ws[e]).view(np.uint8).ravel()
            if merged:
                got = got[e * len(want):(e + 1) * len(want)]
            assert np.array_equal(got, want)
    with pytest.raises(GgufError, match=r"cannot find tensor info for blk.0.ffn_gate.0.weight"):
        gguf.moe_layer_names(ct, 0, 4)
    if merged:
        with pytest.raises(GgufError, match="does not hold 8 expert matrices"):
            gguf.moe_layer_names(ct, 1, 8)


@pytest.mark.gpu
@pytest.mark.parametrize("merged,prepack", [(False, False), (True, True)])
def test_layer_loaded_from_a_file_equals_the_layer_built_from_the_same_bytes(orc, torch_cuda, tmp_path, merged, prepack):
    from tests import helpers as H
    torch = torch_cuda
    mw = orc.make_moe_weights(22, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    raw, norm = _layer_file(orc, mw, merged, eps=1e-6)
    path = tmp_path / "layer.gguf"
    path.write_bytes(raw)
    mm, ct = gguf.open_mmap(str(path))
    blk, ffn_norm, eps = gguf.load_moe_layer(ct, mm, 1, "cuda", prepack=prepack)
    assert eps == float(np.float32(1e-6)) and torch.equal(ffn_norm.cpu(), torch.from_numpy(norm))
    assert blk.n_expert_used == 2 and blk.n_experts == 8
    direct = H.device_block(orc, mw)
    if prepack:
        direct.prepack()
    x = torch.from_numpy(orc.make_activations(5, 40, 512)).cuda()
    assert torch.equal(blk.forward(x), direct.forward(x))
    y = blk.forward_layer(x, ffn_norm, eps)
    assert torch.equal(y, direct.forward_layer(x, torch.from_numpy(norm), eps))
    want = orc.moe_forward(mw, orc.rms_norm(x.cpu().numpy(), norm, eps)).y + x.cpu().numpy()
    assert H.rel_l2(y.cpu().numpy(), want) < 5e-4
