"""The decode-step harness (candle_b200/llama_decode.py) against a CPU restatement of the same step built from the
oracle's pieces: `QMatMul::forward` as the oracle's quantized matmul, RmsNorm, the whole MoE block, and numpy for the
attention glue, following `ModelWeights::forward` (candle-transformers/src/models/quantized_llama.rs:869-898) and
`forward_attn` (:264-345) for one new token per sequence.  Reduced sizes (2 layers, 8 heads of 64, context 24)."""
import math

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _host(qm):
    return qm.inner.data.cpu().numpy()


def _cpu_step(orc, model, tokens, index_pos, k_cache, v_cache, stages=None):
    """Logits of the step; `stages`, if a list, receives (layer, "attention" | "ffn", input, output) per half layer."""
    cfg = model.cfg
    B, hd, nh, nkv = model.batch, cfg.head_dim, cfg.n_head, cfg.n_kv_head
    x = model.tok_embeddings.cpu().numpy()[tokens]
    cos, sin = model.cos.cpu().numpy()[index_pos], model.sin.cpu().numpy()[index_pos]

    def rope(t):  # [B, H, hd]
        out = np.empty_like(t)
        out[..., 0::2] = t[..., 0::2] * cos - t[..., 1::2] * sin
        out[..., 1::2] = t[..., 0::2] * sin + t[..., 1::2] * cos
        return out

    for li in range(cfg.n_layer):
        lw = model.sets[model.layer_set[li]]
        h = orc.rms_norm(x, lw.attention_norm.cpu().numpy(), cfg.rms_eps)
        q = orc.matmul(cfg.dt_attn, h, _host(lw.attention_wq), nh * hd).reshape(B, nh, hd)
        k = orc.matmul(cfg.dt_attn, h, _host(lw.attention_wk), nkv * hd).reshape(B, nkv, hd)
        v = orc.matmul(cfg.dt_attn, h, _host(lw.attention_wv), nkv * hd).reshape(B, nkv, hd)
        q, k = rope(q), rope(k)
        kc, vc = k_cache[li], v_cache[li]
        kc[:, :, index_pos], vc[:, :, index_pos] = k, v
        n = index_pos + 1
        g = nh // nkv
        y = np.empty((B, nh, hd), np.float32)
        for b in range(B):
            for hq in range(nh):
                kk, vv = kc[b, hq // g, :n], vc[b, hq // g, :n]
                att = (kk @ q[b, hq]) / np.float32(math.sqrt(hd))
                att = np.exp(att - att.max())
                att = att / att.sum()
                y[b, hq] = att @ vv
        x_in = x
        x = orc.matmul(cfg.dt_attn, y.reshape(B, nh * hd), _host(lw.attention_wo), cfg.d_model) + x
        if stages is not None:
            stages.append((li, "attention", x_in, x))
        mw = orc.MoeWeights(cfg.d_model, cfg.d_ff, cfg.n_expert_used, cfg.dt_w13, cfg.dt_w2, lw.router.cpu().numpy(),
                            [_host(m.feed_forward_w1) for m in lw.experts], [_host(m.feed_forward_w3) for m in lw.experts],
                            [_host(m.feed_forward_w2) for m in lw.experts])
        hn = orc.rms_norm(x, lw.ffn_norm.cpu().numpy(), cfg.rms_eps)
        x_in = x
        x = orc.moe_forward(mw, hn).y + x
        if stages is not None:
            stages.append((li, "ffn", x_in, x))
    x = orc.rms_norm(x, model.norm.cpu().numpy(), cfg.rms_eps)
    return orc.matmul(cfg.dt_output, x, _host(model.output), cfg.vocab)


@pytest.mark.parametrize("attention", ["library", "pytorch"])
@pytest.mark.parametrize("prepack", [True, False])
def test_decode_step_matches_the_cpu_restatement(orc, torch_cuda, prepack, attention):
    torch = torch_cuda
    from candle_b200.llama_decode import DecodeConfig, DecodeStep
    cfg = DecodeConfig(vocab=512, d_model=512, n_head=8, n_kv_head=2, head_dim=64, n_layer=2, n_expert=8, n_expert_used=2,
                       d_ff=1024, max_seq=32)
    B, index_pos = 5, 23
    model = DecodeStep(cfg, B, torch.device("cuda"), n_distinct=2, seed=3, prepack=prepack, attention=attention)
    tokens = torch.randint(0, cfg.vocab, (B,), generator=torch.Generator(device="cuda").manual_seed(1), device="cuda")
    k0 = [t.cpu().numpy().copy() for t in model.k_cache]
    v0 = [t.cpu().numpy().copy() for t in model.v_cache]
    logits = model.forward(tokens, index_pos).cpu().numpy()
    stages = []
    ref = _cpu_step(orc, model, tokens.cpu().numpy(), index_pos, k0, v0, stages)
    assert np.isfinite(logits).all()
    # every half layer on the CPU's own input: the per-block bounds hold for each (the attention half adds a softmax
    # over f32 scores and two more quantized products)
    for li, what, x_in, x_out in stages:
        xd = torch.from_numpy(x_in).cuda()
        got = (model.attention(li, xd, index_pos) if what == "attention" else model.ffn(li, xd)).cpu().numpy()
        mr, l2 = H.max_rel(got, x_out), H.rel_l2(got, x_out)
        assert mr <= H.MAX_REL_TOL and l2 <= H.REL_L2_TOL, f"layer {li} {what}: max-rel {mr:.3e} rel-L2 {l2:.3e}"
    # the whole step: differences of the order of one int8 step in a re-quantized activation row (1 / 128 of the
    # row's largest value) are amplified by the following layers at these small widths (d = 512: two blocks per row)
    assert H.rel_l2(logits, ref) <= 2e-2, (H.rel_l2(logits, ref), H.max_rel(logits, ref))
    # the cache holds the new position, and nothing else changed
    for li in range(cfg.n_layer):
        kc = model.k_cache[li].cpu().numpy()
        assert np.array_equal(kc[:, :, :index_pos], k0[li][:, :, :index_pos])
        assert H.rel_l2(kc[:, :, index_pos], k0[li][:, :, index_pos]) <= 1e-3
    # determinism, and replay from a CUDA graph gives the same logits
    again = model.forward(tokens, index_pos).cpu().numpy()
    assert np.array_equal(again, logits)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.forward(tokens, index_pos)
    graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), logits)


@pytest.mark.parametrize("B,n_head,n_kv,hd,max_seq,n_ctx", [(3, 32, 8, 128, 1100, 1037), (2, 8, 8, 128, 64, 1), (5, 8, 2, 64, 600, 513),
                                                              (1, 16, 2, 128, 512, 512)])
def test_decode_attention_matches_a_plain_softmax(torch_cuda, B, n_head, n_kv, hd, max_seq, n_ctx):
    """The chunked kernel against the one-pass f32 formula of `standard_attention` (quantized_llama.rs:303-317)."""
    import ctypes as C
    torch = torch_cuda
    from candle_b200 import _lib
    L = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(n_ctx)
    q = torch.randn((B, n_head, hd), generator=g, device="cuda")
    kc = torch.randn((B, n_kv, max_seq, hd), generator=g, device="cuda")
    vc = torch.randn((B, n_kv, max_seq, hd), generator=g, device="cuda")
    kc[:, :, n_ctx:] = float("nan")  # positions past the context must never be read
    vc[:, :, n_ctx:] = float("nan")
    need = C.c_size_t(0)
    assert L.candle_moe_decode_attention_workspace_bytes(B, n_head, hd, n_ctx, C.byref(need)) == 0
    ws = torch.empty(need.value + 16, dtype=torch.uint8, device="cuda")
    y = torch.full((B, n_head * hd), float("nan"), device="cuda")
    st = L.candle_moe_decode_attention(torch.cuda.current_stream().cuda_stream, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, n_head,
                                       n_kv, hd, max_seq, n_ctx, y.data_ptr(), ws.data_ptr(), ws.numel())
    assert st == 0
    grp = n_head // n_kv
    qd = q.double().reshape(B, n_kv, grp, hd)
    att = torch.softmax(qd @ kc[:, :, :n_ctx].double().transpose(-1, -2) / math.sqrt(hd), dim=-1)
    ref = (att @ vc[:, :, :n_ctx].double()).reshape(B, n_head * hd)
    got = y.double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-6
    # shapes outside the supported set are refused, not mis-computed
    assert L.candle_moe_decode_attention(None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, 6, 2, 128, max_seq, n_ctx,
                                         y.data_ptr(), ws.data_ptr(), ws.numel()) in (-2, -4)
