"""Full-size parity: the block at the sizes the benchmarks run, compared with the CPU oracle.

The whole batch runs on the GPU.  The oracle then gets (a) every row's routing -- the router product is
cheap, so ids and per-expert token lists are compared for the WHOLE batch -- and (b) a sample of at
least 256 rows for the expert arithmetic: rows of the block are independent of one another
(candle-transformers/src/models/quantized_llama.rs:185-203 processes a row's experts from that row
alone), so the oracle on the sample is the oracle on the batch.  The sample always holds rows of the
busiest and of the emptiest expert.  Weights are quantized on the device (bit-exact with the reference
quantizer, tests/test_gpu_parity.py) and the same bytes are handed to the oracle.

Also here: rows that hold NaN or infinities (the reference sorts with `total_cmp`, quantized_llama.rs:166,
so its selection is total; the CUDA path must select the same in-range experts).
"""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

SHAPES = {
    # Mixtral-8x7B layer; fine-grained experts with a shared expert, all Q8_0; Mixtral-8x22B layer with skewed routing
    "mixtral_8x7b": dict(d=4096, ff=14336, E=8, k=2, dt13=12, dt2=14, renorm=True, ff_shared=0, zipf=False),
    "fine_grained_q8_0": dict(d=2048, ff=1408, E=60, k=4, dt13=8, dt2=8, renorm=False, ff_shared=5632, zipf=False),
    "mixtral_8x22b_skewed": dict(d=6144, ff=16384, E=8, k=2, dt13=12, dt2=14, renorm=True, ff_shared=0, zipf=True),
}


def _sample_rows(ids: np.ndarray, counts: np.ndarray, n: int, rng) -> np.ndarray:
    """n row indices: up to n/4 rows of the busiest expert, up to n/4 of the emptiest one that has rows, the rest random."""
    T = ids.shape[0]
    busy = int(np.argmax(counts))
    nz = np.where(counts > 0)[0]
    idle = int(nz[np.argmin(counts[nz])])
    pick = []
    for e in (busy, idle):
        rows = np.where((ids == e).any(axis=1))[0]
        pick.append(rows[: n // 4])
    chosen = np.unique(np.concatenate(pick))
    rest = np.setdiff1d(np.arange(T), chosen)
    extra = rng.choice(rest, size=min(len(rest), n - len(chosen)), replace=False)
    return np.sort(np.concatenate([chosen, extra]))


def _full_size_case(orc, torch, name, T, prepack, seed):
    cfg = SHAPES[name]
    blk, mw = H.random_device_block(orc, torch, cfg, seed)
    if prepack:
        blk.prepack()
    g = torch.Generator(device="cuda").manual_seed(seed + 100)
    x = torch.randn((T, cfg["d"]), generator=g, device="cuda", dtype=torch.float32)
    y = blk.forward(x)
    ids, tw, counts, perm = blk.last_routing(T)
    ids, counts, perm = ids.numpy().astype(np.uint32), counts.numpy(), perm.numpy()
    xh = x.cpu().numpy()

    # (a) routing of the whole batch
    probs, ids_ref, w_ref = orc.router_topk(xh, mw.router, cfg["k"], cfg["renorm"], mw.router_bias)
    n_tie = H.check_routing(probs, ids_ref, ids)
    assert n_tie <= max(1, T // 500), f"{n_tie} near-ties in {T} rows"
    assert int(counts.sum()) == T * cfg["k"]
    # per-expert token lists: the stable grouping of the ids the device selected (== the oracle's wherever ids agree)
    order = np.argsort(ids.reshape(-1).astype(np.int64), kind="stable")
    assert np.array_equal(perm, order // cfg["k"])
    assert np.array_equal(counts, np.bincount(ids.reshape(-1), minlength=cfg["E"]))
    if n_tie == 0:
        order_ref = np.argsort(ids_ref.reshape(-1).astype(np.int64), kind="stable")
        assert np.array_equal(perm, order_ref // cfg["k"])

    # (b) expert arithmetic on a sample of rows
    rows = _sample_rows(ids, counts, 256, np.random.default_rng(seed))
    assert len(rows) >= min(256, T)
    ref = orc.moe_forward(mw, xh[rows])
    same = (ref.topk_ids == ids[rows]).all(axis=1)
    assert same.sum() >= len(rows) - n_tie
    got = y[torch.from_numpy(rows).cuda()].cpu().numpy()
    mr, l2 = H.max_rel(got[same], ref.y[same]), H.rel_l2(got[same], ref.y[same])
    assert mr <= H.MAX_REL_TOL and l2 <= H.REL_L2_TOL, f"{name} T={T}: max-rel {mr:.3e} rel-L2 {l2:.3e}"
    v = C.c_int32(-1)
    from candle_b200 import _lib
    assert _lib.load().candle_moe_device_status(C.byref(v)) == 0 and v.value == 0
    return counts


@pytest.mark.parametrize("prepack", [True, False])
def test_mixtral_8x7b_prefill_2048_rows(orc, torch_cuda, prepack):
    """d=4096, ff=14336, 8 experts, top-2, w1/w3 Q4_K, w2 Q6_K at 2048 rows: the tensor-core grouped GEMM with
    K = 4096 / 14336, 56-block Q6_K rows and position tiles filled by real routing (with the repacked copies the
    Q6_K down product takes the GEMM too; without them the streaming form)."""
    _full_size_case(orc, torch_cuda, "mixtral_8x7b", 2048, prepack, seed=3)


@pytest.mark.parametrize("T", [64, 128, 256])
def test_mixtral_8x7b_mid_sized_batches(orc, torch_cuda, T):
    """The batch sizes between the decode kernels and the large-batch GEMM (about T/4 rows per expert)."""
    _full_size_case(orc, torch_cuda, "mixtral_8x7b", T, True, seed=4)


@pytest.mark.parametrize("prepack", [True, False])
def test_fine_grained_q8_0_4096_rows(orc, torch_cuda, prepack):
    """d=2048, 60 routed experts of ff=1408, top-4 without renormalisation, shared expert ff=5632 gated by
    sigmoid(x.g), all Q8_0, 4096 rows (qwen2_moe.rs:261-323).  With the repacked copies the products take the
    tensor-core GEMM (gate_up with exact two-part fp16 operands, down with the scales folded into fp16 operands: the
    one path whose float side is not the reference's per-block f32 scaling, held to the same bounds); without them
    the int8 tile kernel."""
    _full_size_case(orc, torch_cuda, "fine_grained_q8_0", 4096, prepack, seed=5)


def test_mixtral_8x22b_skewed_routing_1024_rows(orc, torch_cuda):
    """d=6144, ff=16384, 8 experts, top-2, router bias log(1/(i+1)): Zipf-like load, expert 0 busiest."""
    counts = _full_size_case(orc, torch_cuda, "mixtral_8x22b_skewed", 1024, True, seed=6)
    assert counts[0] == counts.max() and counts.max() > 2 * counts.min()


@pytest.mark.parametrize("dt13,dt2,ff", [(8, 8, 1408), (12, 14, 1536), (14, 14, 1536), (12, 12, 1536)])
@pytest.mark.parametrize("T,prepack", [(1024, True), (150, True), (32, True), (32, False), (300, False)])
def test_repeated_forwards_are_bit_identical(orc, torch_cuda, dt13, dt2, ff, T, prepack):
    """The same rows through the same block eight times: every kernel adds in a fixed order, so the outputs are equal
    bit for bit.  (A difference here is a race: a stage of a copy ring handed back before its reader is done.)
    T = 1024 fills several position tiles per expert and several tiles per CTA; T = 150 takes the narrow tiles; T = 32
    the decode kernels (with the repacked copies) or the streaming kernels (without); T = 300 without the copies the
    forms that read the GGUF blocks."""
    torch = torch_cuda
    # the all-Q8_0 block also carries a shared expert (its products take the same tensor-core forms)
    cfg = dict(d=2048, ff=ff, E=4, k=2, dt13=dt13, dt2=dt2, renorm=True, ff_shared=2816 if dt13 == 8 else 0, zipf=False)
    blk, _ = H.random_device_block(orc, torch, cfg, seed=11)
    if prepack:
        blk.prepack()
    g = torch.Generator(device="cuda").manual_seed(12)
    x = torch.randn((T, cfg["d"]), generator=g, device="cuda", dtype=torch.float32)
    ys = []
    for _ in range(8):
        ys.append(blk.forward(x).clone())
        torch.cuda.synchronize()
    assert all(torch.equal(ys[0], y) for y in ys[1:]), [int((ys[0] != y).sum()) for y in ys[1:]]


# ------------------------------------------------------------------------------------------------
# rows holding NaN / infinities
# ------------------------------------------------------------------------------------------------
def _nonfinite_rows(T, d, rng):
    x = rng.standard_normal((T, d), dtype=np.float32)
    x[1, 7] = np.nan
    x[3, 0] = np.inf
    x[4, d - 1] = -np.inf
    x[6, 5], x[6, 9] = np.inf, -np.inf
    x[8, :] = np.nan
    return x, [1, 3, 4, 6, 8]


@pytest.mark.parametrize("E,k", [(8, 2), (60, 4), (128, 8)])
def test_router_selection_is_total_on_nonfinite_rows(orc, torch_cuda, E, k):
    """Only the router entry point: it writes ids and weights and indexes nothing with them."""
    torch = torch_cuda
    from candle_b200 import _lib
    T, d = 12, 512
    rng = np.random.default_rng(E)
    x, bad = _nonfinite_rows(T, d, rng)
    wg = rng.standard_normal((E, d), dtype=np.float32) * np.float32(0.02)
    _, ids_ref, w_ref = orc.router_topk(x, wg, k, True, None)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(wg).cuda()
    ids = torch.full((T, k), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros((T, k), dtype=torch.float32, device="cuda")
    st = _lib.load().candle_moe_router_topk(torch.cuda.current_stream().cuda_stream, xd.data_ptr(), wd.data_ptr(), None,
                                            T, d, E, k, 1, ids.data_ptr(), w.data_ptr())
    assert st == 0
    torch.cuda.synchronize()
    got = ids.cpu().numpy()
    assert (got >= 0).all() and (got < E).all()
    assert np.array_equal(got.astype(np.uint32), ids_ref)
    wn = w.cpu().numpy()
    for t in bad:
        assert np.isnan(wn[t]).all() and np.isnan(w_ref[t]).all()
    good = [t for t in range(T) if t not in bad]
    assert np.allclose(wn[good], w_ref[good], rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("T,prepack", [(12, True), (12, False), (1, True), (200, True)])
def test_block_with_nonfinite_rows(orc, torch_cuda, T, prepack):
    """A row holding a NaN comes out NaN (as the reference's does) and the other rows are what they are without it."""
    torch = torch_cuda
    mw = orc.make_moe_weights(41, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk = H.device_block(orc, mw)
    if prepack:
        blk.prepack()
    rng = np.random.default_rng(T)
    if T >= 12:
        x, bad = _nonfinite_rows(T, 512, rng)
    else:
        x, bad = np.full((1, 512), np.nan, np.float32), [0]
    clean = x.copy()
    clean[bad] = 0.0
    y = blk.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ids, _, counts, perm = blk.last_routing(T)
    assert (ids.numpy() >= 0).all() and (ids.numpy() < 8).all() and int(counts.sum()) == 2 * T
    y_clean = blk.forward(torch.from_numpy(clean).cuda()).cpu().numpy()
    good = [t for t in range(T) if t not in bad]
    for t in bad:
        assert np.isnan(y[t]).all()
    if good:
        assert np.isfinite(y[good]).all()
        # the other rows may share their experts' kernels with different neighbours: same integers, f32 order only
        assert H.rel_l2(y[good], y_clean[good]) < 1e-5
        ref = orc.moe_forward(mw, x[good])
        assert H.rel_l2(y[good], ref.y) <= H.REL_L2_TOL and H.max_rel(y[good], ref.y) <= H.MAX_REL_TOL
