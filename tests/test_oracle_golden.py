"""Pins the CPU oracle against the known-answer values of the reference's own tests.

Each test names the reference test it mirrors (candle-core/tests/quantized_tests.rs unless noted).
"""
import numpy as np
import pytest

from tests.golden import reference_known_answers as KA


def _round3(v):
    return np.round(1000.0 * v.astype(np.float64)) / 1000.0


@pytest.mark.parametrize("name", ["Q4K", "Q6K", "Q8K"])
def test_ramp_roundtrip_spot_values(orc, name):
    """quantize_q4k / quantize_q6k / quantize_q8k (:566-752): ramp -> quantize -> dequantize."""
    dt = {"Q4K": orc.Q4K, "Q6K": orc.Q6K, "Q8K": orc.Q8K}[name]
    tol, spots, tol_big = KA.RAMP_ROUNDTRIP[name]
    src = KA.ramp(0.5, 1024)
    assert [float(src[i]) for i in KA.SPOT_INDICES] == [np.float32(v) for v in KA.RAMP_SRC_SPOTS]
    dst = orc.dequantize(dt, orc.quantize(dt, src), 1024)
    assert np.max(np.abs(dst - src)) < tol
    got = _round3(dst)[KA.SPOT_INDICES]
    assert [float(g) for g in got] == [float(s) for s in spots]
    big = KA.ramp(128.0, 1024)
    dst_big = orc.dequantize(dt, orc.quantize(dt, big), 1024)
    assert np.max(np.abs(dst_big - big)) < tol_big


@pytest.mark.parametrize("name", ["Q4K", "Q6K", "Q8K", "Q8_0", "Q4_0"])
def test_ggml_quantization_rmse(orc, name):
    """ggml_quantization_error_test (:440-469): sqrt(sum sq)/n of 0.1 + 2cos(i) under 0.002."""
    dt = getattr(orc, name)
    src = orc.ggml_like_vector(0.0, KA.GGML_TEST_SIZE)
    dst = orc.dequantize(dt, orc.quantize(dt, src), src.size)
    err = np.float32(np.sqrt(np.sum((src - dst).astype(np.float32) ** 2, dtype=np.float32))) / src.size
    assert err <= KA.GGML_MAX_QUANTIZATION_TOTAL_ERROR


def test_q4_0_roundtrip_exact(orc):
    """quantize_q4_0 (:262-292)."""
    src = np.arange(128, dtype=np.float32)
    dst = orc.dequantize(orc.Q4_0, orc.quantize(orc.Q4_0, src), 128)
    assert dst.tolist() == KA.Q4_0_ROUNDTRIP_0_127


@pytest.mark.parametrize("name", ["Q4K", "Q6K", "Q8_0", "Q4_0"])
def test_ggml_matmul_error(orc, name):
    """ggml_matmul_error_test (:846-911): opt vs unopt vec_dot, matmul vs vec_dot, error vs f32."""
    dt = getattr(orc, name)
    adt = orc.lib().orc_vec_dot_dtype(dt)
    n = KA.GGML_TEST_SIZE
    ramp = (np.arange(n, dtype=np.float32) / np.float32(n)).astype(np.float32)
    cases = [(orc.ggml_like_vector(0.0, n), orc.ggml_like_vector(1.0, n), 1.0), (ramp, ramp, 2.0)]
    for a, b, err_m in cases:
        aq = orc.quantize(dt, a)
        bq = orc.quantize(adt, b)
        simd = orc.vec_dot(dt, n, aq, bq, orc.ORDER_SIMD)
        lanes = orc.vec_dot(dt, n, aq, bq, orc.ORDER_LANES)
        unopt = orc.vec_dot(dt, n, aq, bq, orc.ORDER_UNOPT)
        assert simd == lanes, "intrinsics and their scalar lane restatement must agree bit for bit"
        assert abs(simd - unopt) / n <= 1e-6
        mm = float(orc.matmul(dt, b[None, :], aq, 1)[0, 0])
        assert abs(mm - simd) / n <= 1e-6
        ref = np.float32(0.0)
        for p in (a * b):  # sequential f32 sum like vec_dot_reference
            ref = np.float32(ref + p)
        for r in (simd, mm, unopt):
            err = abs(r - float(ref)) / n
            assert np.isfinite(err) and err <= KA.GGML_MAX_DOT_PRODUCT_ERROR
            assert err - KA.ERROR_LENIENCY <= KA.GGML_REFERENCE_MATMUL_ERROR[name] * err_m


def test_q4_0_matmul_exact_cpu_values(orc):
    """quantized_matmul / quantized_matmul_neg (:89-207): exact CPU results of k_quants::matmul.
    Validates the matmul driver and the Q8_0 activation quantizer end to end."""
    m, k, n = 3, 64, 4
    lhs = np.arange(m * k, dtype=np.float32).reshape(m, k)
    rhs = np.arange(k * n, dtype=np.float32)
    for order in (orc.ORDER_SIMD, orc.ORDER_UNOPT):
        dst = orc.matmul(orc.Q4_0, lhs, orc.quantize(orc.Q4_0, rhs.reshape(n, k)), n, order)
        assert np.round(dst.reshape(-1)).tolist() == KA.Q4_0_MATMUL_RAMP_CPU
    lhs = (np.arange(m * k, dtype=np.float32) - np.float32(m * k / 2.0)).reshape(m, k)
    rhs = np.arange(k * n, dtype=np.float32) - np.float32(k * n) / np.float32(3.0)
    dst = orc.matmul(orc.Q4_0, lhs, orc.quantize(orc.Q4_0, rhs.reshape(n, k)), n)
    assert np.round(dst.reshape(-1)).tolist() == KA.Q4_0_MATMUL_NEG_CPU


@pytest.mark.parametrize("name", ["Q4K", "Q6K", "Q8_0"])
def test_row_independence(orc, name):
    """qmm_batch (:221-256): the same row gives bit-identical outputs wherever it sits in a batch."""
    dt = getattr(orc, name)
    rng = np.random.default_rng(5)
    lhs = rng.standard_normal((2, 256), dtype=np.float32)
    w = orc.quantize(dt, rng.standard_normal((6, 256), dtype=np.float32))
    mm = orc.matmul(dt, lhs, w, 6)
    mm3 = orc.matmul(dt, np.concatenate([lhs, lhs, lhs]), w, 6)
    assert np.array_equal(mm3[0:2], mm) and np.array_equal(mm3[2:4], mm) and np.array_equal(mm3[4:6], mm)


def test_softmax_known_answers(orc):
    """candle-nn/tests/ops.rs:9-53."""
    data = np.array(KA.SOFTMAX_DATA, dtype=np.float32)
    out = orc.softmax_last_dim(np.log(data).astype(np.float32))
    assert np.round(out.astype(np.float64), 4).tolist() == KA.SOFTMAX_LAST_DIM_OF_LOG


def test_silu_known_answers(orc):
    """candle-core/tests/tensor_tests.rs:222-255."""
    out = orc.silu(np.array(KA.SILU_IN, dtype=np.float32))
    assert np.round(out.astype(np.float64), 4).tolist() == KA.SILU_OUT


def test_index_add_known_answers(orc):
    """candle-core/tests/tensor_tests.rs:1008-1023."""
    t = np.arange(12, dtype=np.float32).reshape(4, 3)
    out = orc.index_add_dim0(np.zeros((6, 3), np.float32), KA.INDEX_ADD_IDS, t)
    assert out.tolist() == KA.INDEX_ADD_OUT


def test_dequantized_matmul_agrees_with_quantized_dot(orc):
    """Sanity on seeded N(0, 0.02) weights: the integer dot against Q8K activations equals the
    float dot of the two dequantized vectors up to f32 summation error."""
    rng = np.random.default_rng(11)
    k = 1024
    for dt in (orc.Q4K, orc.Q6K, orc.Q8_0):
        adt = orc.lib().orc_vec_dot_dtype(dt)
        w = rng.standard_normal(k, dtype=np.float32) * np.float32(0.02)
        x = rng.standard_normal(k, dtype=np.float32)
        wq, xq = orc.quantize(dt, w), orc.quantize(adt, x)
        got = orc.vec_dot(dt, k, wq, xq)
        want = float(np.dot(orc.dequantize(dt, wq, k).astype(np.float64), orc.dequantize(adt, xq, k).astype(np.float64)))
        assert abs(got - want) <= 1e-5 * max(1.0, abs(want))


def test_router_topk_semantics(orc):
    """quantized_llama.rs:162-179: stable descending order, ties keep the lower expert first,
    weights renormalised over the selected pair in rank order."""
    d, E = 32, 8
    wg = np.zeros((E, d), np.float32)
    wg[2, 0] = 1.0
    wg[5, 0] = 1.0          # experts 2 and 5 tie exactly
    wg[7, 1] = 0.5
    x = np.zeros((3, d), np.float32)
    x[0, 0] = 2.0           # 2 and 5 tie at the top -> [2, 5]
    x[1, 1] = 4.0           # 7 wins, all others tie -> [7, 0]
    probs, ids, w = orc.router_topk(x, wg, 2)
    assert ids[0].tolist() == [2, 5] and ids[1].tolist() == [7, 0] and ids[2].tolist() == [0, 1]
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
    s = np.float32(probs[1, 7] + probs[1, 0])
    assert w[1, 0] == np.float32(probs[1, 7] / s)
    _, ids_nr, w_nr = orc.router_topk(x, wg, 2, renorm=False)
    assert np.array_equal(ids_nr, ids) and w_nr[1, 0] == probs[1, 7]


def test_moe_block_matches_composition(orc):
    """The fused oracle block equals its own primitives composed as quantized_llama.rs:143-210."""
    d, ff, E, k, T = 256, 512, 4, 2, 9
    mw = orc.make_moe_weights(3, d, ff, E, k, orc.Q4K, orc.Q6K)
    x = orc.make_activations(4, T, d)
    res = orc.moe_forward(mw, x)
    _, ids, tw = orc.router_topk(x, mw.router, k)
    assert np.array_equal(ids, res.topk_ids) and np.array_equal(tw, res.topk_w)
    y = np.zeros((T, d), np.float32)
    rows_cat = []
    for e in range(E):
        sel = [(t, r) for t in range(T) for r in range(k) if ids[t, r] == e]
        rows = [t for t, _ in sel]
        rows_cat += rows
        assert res.expert_counts[e] == len(rows)
        if not rows:
            continue
        out, _ = orc.mlp_forward(orc.Q4K, orc.Q6K, x[rows], mw.w1[e], mw.w3[e], mw.w2[e], ff)
        scaled = out * np.array([tw[t, r] for t, r in sel], np.float32)[:, None]
        y = orc.index_add_dim0(y, rows, scaled)
    assert res.expert_rows.tolist() == rows_cat
    assert np.array_equal(y, res.y)


def test_rms_norm_known_answers(orc):
    """candle-nn/tests/ops.rs:55-66."""
    x = np.array(KA.RMS_NORM_DATA, dtype=np.float32).reshape(-1, 3)
    got = orc.rms_norm(x, np.array(KA.RMS_NORM_ALPHA, dtype=np.float32), KA.RMS_NORM_EPS)
    assert np.array_equal(np.round(got.astype(np.float64), 4), np.array(KA.RMS_NORM_EXPECTED).reshape(-1, 3))
