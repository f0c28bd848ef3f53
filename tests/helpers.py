"""Shared helpers for the GPU parity tests: build the device block from oracle-side weights and
compare outputs with the metrics the acceptance bounds are stated in."""
from __future__ import annotations

import numpy as np

# acceptance bounds of the block output against the reference's CPU path
MAX_REL_TOL = 2e-3   # max |a - b| / max |b|
REL_L2_TOL = 1e-3    # ||a - b||_2 / ||b||_2
NEAR_TIE_GAP = 1e-6  # a routing mismatch is tolerated only when the probabilities differ by less


def max_rel(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.max(np.abs(a.astype(np.float64) - b.astype(np.float64))) / max(np.max(np.abs(b)), 1e-30))


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    return float(np.linalg.norm(a64 - b64) / max(np.linalg.norm(b64), 1e-30))


def device_block(orc, mw, device="cuda"):
    """candle_b200.MlpOrMoe holding the same bytes as the oracle-side `MoeWeights`."""
    import torch
    from candle_b200 import GgmlDType, Mlp, MlpOrMoe, QMatMul, QTensor

    d, ff = mw.d_model, mw.d_ff
    dt13, dt2 = GgmlDType(mw.dtype_w13), GgmlDType(mw.dtype_w2)

    def qm(blocks, dt, shape):
        return QMatMul.from_qtensor(QTensor.from_blocks(blocks, dt, shape, device))

    experts = [Mlp(qm(mw.w1[e], dt13, (ff, d)), qm(mw.w2[e], dt2, (d, ff)), qm(mw.w3[e], dt13, (ff, d)))
               for e in range(mw.n_experts)]
    kw = {}
    if mw.d_ff_shared:
        fs = mw.d_ff_shared
        s13, s2 = GgmlDType(mw.dtype_shared13), GgmlDType(mw.dtype_shared2)
        kw["shared_expert"] = Mlp(qm(mw.sw1, s13, (fs, d)), qm(mw.sw2, s2, (d, fs)), qm(mw.sw3, s13, (fs, d)))
        kw["shared_expert_gate"] = torch.from_numpy(mw.shared_gate)
    bias = None if mw.router_bias is None else torch.from_numpy(mw.router_bias)
    return MlpOrMoe.moe(mw.top_k, torch.from_numpy(mw.router).to(device), experts, norm_topk_prob=mw.renorm,
                        router_bias=bias, **kw)


def check_routing(orc_probs, ids_ref, ids_got, near_ties_out=None):
    """ids must match exactly; a mismatch is accepted only for a documented near-tie (gap < 1e-6 in
    softmax probability between the experts that swapped)."""
    bad = np.argwhere(ids_ref != ids_got)
    n_tie = 0
    for t in sorted(set(int(r[0]) for r in bad)):
        a, b = set(ids_ref[t].tolist()), set(ids_got[t].tolist())
        p = orc_probs[t]
        diff = (a ^ b) or a  # same set in different order: compare the reordered members
        vals = sorted(float(p[e]) for e in diff)
        assert vals[-1] - vals[0] < NEAR_TIE_GAP, f"token {t}: routing differs beyond a near-tie: {ids_ref[t]} vs {ids_got[t]}"
        n_tie += 1
    if near_ties_out is not None:
        near_ties_out.append(n_tie)
    return n_tie


def q8k_planar(orc, blocks: np.ndarray, rows: int, k: int):
    """Split oracle BlockQ8K bytes into (qs int8 [rows,k], d f32 [rows,k/256], bsums i16 [rows,k/16])."""
    nb = rows * k // 256
    b = blocks.reshape(nb, 292)
    d = b[:, 0:4].copy().view(np.float32).reshape(rows, k // 256)
    qs = b[:, 4:260].copy().view(np.int8).reshape(rows, k)
    bs = b[:, 260:292].copy().view(np.int16).reshape(rows, k // 16)
    return qs, d, bs


def q8_0_planar(orc, blocks: np.ndarray, rows: int, k: int):
    nb = rows * k // 32
    b = blocks.reshape(nb, 34)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(rows, k // 32)
    qs = b[:, 2:34].copy().view(np.int8).reshape(rows, k)
    return qs, d


def random_device_block(orc, torch, cfg, seed=0, device="cuda"):
    """A block of the given shape with N(0, 0.02) weights generated and quantized ON THE DEVICE, and the oracle-side
    `MoeWeights` holding the same bytes.  cfg: d, ff, E, k, dt13, dt2, renorm, ff_shared, zipf (router bias
    log(1/(i+1)))."""
    from candle_b200 import GgmlDType, Mlp, MlpOrMoe, QMatMul, QTensor
    d, ff, E = cfg["d"], cfg["ff"], cfg["E"]
    g = torch.Generator(device=device).manual_seed(seed)

    def q(shape, dt):
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
        return QMatMul(QTensor.quantize(w, GgmlDType(dt)))

    host = lambda qm: qm.inner.data.cpu().numpy()
    experts = [Mlp(q((ff, d), cfg["dt13"]), q((d, ff), cfg["dt2"]), q((ff, d), cfg["dt13"])) for _ in range(E)]
    router = torch.randn((E, d), generator=g, device=device, dtype=torch.float32) * 0.02
    bias = np.log(1.0 / (np.arange(E) + 1.0)).astype(np.float32) if cfg.get("zipf") else None
    kw = {}
    if cfg.get("ff_shared"):
        fs = cfg["ff_shared"]
        kw["shared_expert"] = Mlp(q((fs, d), cfg["dt13"]), q((d, fs), cfg["dt2"]), q((fs, d), cfg["dt13"]))
        kw["shared_expert_gate"] = torch.randn(d, generator=g, device=device, dtype=torch.float32) * 0.02
    blk = MlpOrMoe.moe(cfg["k"], router, experts, norm_topk_prob=cfg["renorm"],
                       router_bias=None if bias is None else torch.from_numpy(bias), **kw)
    mw = orc.MoeWeights(d, ff, cfg["k"], cfg["dt13"], cfg["dt2"], router.cpu().numpy(),
                        [host(m.feed_forward_w1) for m in experts], [host(m.feed_forward_w3) for m in experts],
                        [host(m.feed_forward_w2) for m in experts], renorm=cfg["renorm"], router_bias=bias)
    if cfg.get("ff_shared"):
        s = kw["shared_expert"]
        mw.d_ff_shared, mw.dtype_shared13, mw.dtype_shared2 = cfg["ff_shared"], cfg["dt13"], cfg["dt2"]
        mw.sw1, mw.sw3, mw.sw2 = host(s.feed_forward_w1), host(s.feed_forward_w3), host(s.feed_forward_w2)
        mw.shared_gate = kw["shared_expert_gate"].cpu().numpy()
    return blk, mw
