"""A decode step of the model the MoE block sits in: `ModelWeights::forward` of candle-transformers'
quantized_llama (quantized_llama.rs:869-898) for one new token per sequence.

This is a HARNESS around the block, so that its share of a whole decode step can be measured; it is not a model
runtime.  What runs where:

* this library (C ABI): every quantized product -- wq / wk / wv (as one product over their concatenated rows) / wo and
  the lm head through `QMatMul.forward` (`candle_moe_qmatmul`) --, and with `attention="library"` the rest of the
  attention half: `attention_norm` (`candle_moe_rmsnorm`), rotary embedding + cache append
  (`candle_moe_rope_kv_append`), the attention over the cache (`candle_moe_decode_attention`); the FFN half of each layer (`ffn_norm` -> MoE block -> `+ residual`) as one call
  (`candle_moe_ffn_layer`), or, with the experts sharded over ranks, `ExpertParallelMoe.forward` between a PyTorch
  RmsNorm and residual add;
* stock PyTorch ops, with the reference's arithmetic: token embedding lookup, the final norm, the residual add of the
  attention half, and, with `attention="pytorch"`, the whole glue of the attention half: RmsNorm
  (candle-nn/src/ops.rs:504-514), interleaved rotary embedding (`rope_i`, candle-nn/src/rotary_emb.rs:53-66, tables of
  quantized_llama.rs:410-427), the f32 KV cache append (candle-nn/src/kv_cache.rs:143-164) and the attention itself as
  the reference's `standard_attention` (quantized_llama.rs:303-317: q k^T / sqrt(head_dim), softmax, times v, grouped
  heads instead of a materialised `repeat_kv`).

One layer's quantized bytes may be shared by several layers (`n_distinct` sets of weights rotate over the layers):
a random-init 32-layer model does not need 32 different random layers to be timed, only enough distinct bytes that
nothing stays in L2 from one layer to the next.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from .moe import Mlp, MlpOrMoe
from .quantized import GgmlDType, QMatMul, QTensor


@dataclass
class DecodeConfig:
    """Mixtral-8x7B by default (GGUF metadata names in quantized_llama.rs:468-490)."""
    vocab: int = 32000
    d_model: int = 4096
    n_head: int = 32
    n_kv_head: int = 8
    head_dim: int = 128
    rope_theta: float = 1e6
    rms_eps: float = 1e-5
    n_layer: int = 32
    n_expert: int = 8
    n_expert_used: int = 2
    d_ff: int = 14336
    dt_attn: int = int(GgmlDType.Q4K)
    dt_w13: int = int(GgmlDType.Q4K)
    dt_w2: int = int(GgmlDType.Q6K)
    dt_output: int = int(GgmlDType.Q6K)
    max_seq: int = 4096


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """candle_nn::ops::rms_norm in f32 (ops.rs:504-514): x / sqrt(mean(x^2) + eps) * weight."""
    m = torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x / m * weight


def rope_tables(head_dim: int, theta: float, max_seq: int, device) -> tuple:
    """`precomput_freqs_cis` (quantized_llama.rs:410-427): cos / sin of pos * theta^(-i / head_dim), i even."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(max_seq, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """`rope_i` (rotary_emb.rs:53-66): pairs (x[2i], x[2i+1]) rotated by the angle of (position, i).
    x [B, H, S, D]; cos / sin [S, D / 2]."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * cos - x1 * sin
    out[..., 1::2] = x0 * sin + x1 * cos
    return out


class LayerWeights:
    """The tensors of one `LayerWeights` (quantized_llama.rs:214-232) that a decode step reads."""

    def __init__(self, cfg: DecodeConfig, device, gen: torch.Generator, n_local_experts: Optional[int] = None,
                 first_expert: int = 0, prepack: bool = True):
        d, hd = cfg.d_model, cfg.head_dim

        def q(shape, dt, g=gen):
            w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
            m = QMatMul(QTensor.quantize(w, GgmlDType(dt)))
            return m.prepack() if prepack else m

        self.attention_wq = q((cfg.n_head * hd, d), cfg.dt_attn)
        self.attention_wk = q((cfg.n_kv_head * hd, d), cfg.dt_attn)
        self.attention_wv = q((cfg.n_kv_head * hd, d), cfg.dt_attn)
        self.attention_wo = q((d, cfg.n_head * hd), cfg.dt_attn)
        # the three projections as ONE product over the concatenated rows wq | wk | wv (a row's result does not depend on
        # which other rows the matrix holds, so this is the same arithmetic in one launch sequence instead of three)
        qkv = torch.cat([self.attention_wq.inner.data, self.attention_wk.inner.data, self.attention_wv.inner.data])
        self.attention_wqkv = QMatMul(QTensor(qkv, GgmlDType(cfg.dt_attn), ((cfg.n_head + 2 * cfg.n_kv_head) * hd, d)))
        if prepack:
            self.attention_wqkv.prepack()
        self.attention_norm = 1.0 + 0.1 * torch.randn(d, generator=gen, device=device)
        self.ffn_norm = 1.0 + 0.1 * torch.randn(d, generator=gen, device=device)
        self.router = torch.randn((cfg.n_expert, d), generator=gen, device=device, dtype=torch.float32) * 0.02
        n_loc = cfg.n_expert if n_local_experts is None else n_local_experts
        base_seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen, device=device))
        self.experts: List[Mlp] = []
        for e in range(first_expert, first_expert + n_loc):
            ge = torch.Generator(device=device).manual_seed(base_seed + e)  # expert e is the same bytes on any rank layout
            mk = lambda shape, dt: QMatMul(QTensor.quantize(torch.randn(shape, generator=ge, device=device) * 0.02, GgmlDType(dt)))
            self.experts.append(Mlp(mk((cfg.d_ff, d), cfg.dt_w13), mk((d, cfg.d_ff), cfg.dt_w2), mk((cfg.d_ff, d), cfg.dt_w13)))
        self.mlp_or_moe: Optional[MlpOrMoe] = None
        if n_local_experts is None:
            self.mlp_or_moe = MlpOrMoe.moe(cfg.n_expert_used, self.router, self.experts)
            if prepack:
                self.mlp_or_moe.prepack()


class DecodeStep:
    """One new token for each of `batch` sequences whose first `index_pos` positions are in the KV cache."""

    def __init__(self, cfg: DecodeConfig, batch: int, device, *, n_distinct: int = 4, seed: int = 0, prepack: bool = True,
                 expert_parallel=None, kv_fill: float = 0.5, attention: str = "library"):
        """`expert_parallel`: None, or {"world", "rank", "make": layer_weights -> ExpertParallelMoe} for the sharded form.
        `attention`: "library" (the attention half through this library: candle_moe_rmsnorm, one product over wq | wk | wv,
        candle_moe_rope_kv_append, candle_moe_decode_attention) or "pytorch" (three products, PyTorch ops for the rest)."""
        self.cfg, self.batch, self.device = cfg, batch, device
        self.attention_impl = attention
        self._att_ws = None
        g = torch.Generator(device=device).manual_seed(seed)
        self.tok_embeddings = torch.randn((cfg.vocab, cfg.d_model), generator=g, device=device, dtype=torch.float32) * 0.02
        self.norm = 1.0 + 0.1 * torch.randn(cfg.d_model, generator=g, device=device)
        w = torch.randn((cfg.vocab, cfg.d_model), generator=g, device=device, dtype=torch.float32) * 0.02
        self.output = QMatMul(QTensor.quantize(w, GgmlDType(cfg.dt_output)))
        if prepack:
            self.output.prepack()
        del w
        n_distinct = max(1, min(n_distinct, cfg.n_layer))
        self.ep = None
        if expert_parallel is None:
            self.sets = [LayerWeights(cfg, device, g, prepack=prepack) for _ in range(n_distinct)]
        else:
            world, rank = expert_parallel["world"], expert_parallel["rank"]
            n_loc = cfg.n_expert // world
            self.sets = [LayerWeights(cfg, device, g, n_loc, rank * n_loc, prepack) for _ in range(n_distinct)]
            self.ep = [expert_parallel["make"](s) for s in self.sets]
        self.layer_set = [i % n_distinct for i in range(cfg.n_layer)]
        self.cos, self.sin = rope_tables(cfg.head_dim, cfg.rope_theta, cfg.max_seq, device)
        # f32 KV cache [layer][B, n_kv_head, max_seq, head_dim], as `KvCache::new(2, max_seq)` holds it
        shape = (batch, cfg.n_kv_head, cfg.max_seq, cfg.head_dim)
        self.k_cache = [torch.randn(shape, generator=g, device=device, dtype=torch.float32) * kv_fill for _ in range(cfg.n_layer)]
        self.v_cache = [torch.randn(shape, generator=g, device=device, dtype=torch.float32) * kv_fill for _ in range(cfg.n_layer)]

    # -- pieces (timed separately by the benchmark) -----------------------------------------------------
    def attention(self, li: int, x: torch.Tensor, index_pos: int) -> torch.Tensor:
        """`attention_norm` + `forward_attn` + residual (quantized_llama.rs:880-883, 264-345) for seq_len = 1."""
        cfg, B = self.cfg, self.batch
        lw = self.sets[self.layer_set[li]]
        kc, vc = self.k_cache[li], self.v_cache[li]
        n = index_pos + 1
        if self.attention_impl == "library":
            import ctypes as C
            from . import _lib
            from .quantized import _stream_ptr
            L, st = _lib.load(), _stream_ptr(self.device)
            x = x.contiguous()
            h = torch.empty_like(x)
            with torch.cuda.device(self.device):
                _lib.check("candle_moe_rmsnorm", L.candle_moe_rmsnorm(st, x.data_ptr(), lw.attention_norm.data_ptr(), cfg.rms_eps, B,
                                                                      cfg.d_model, h.data_ptr()))
                qkv = lw.attention_wqkv.forward(h)
                q = torch.empty((B, cfg.n_head, cfg.head_dim), dtype=torch.float32, device=self.device)
                _lib.check("candle_moe_rope_kv_append",
                           L.candle_moe_rope_kv_append(st, qkv.data_ptr(), qkv.shape[1], self.cos[index_pos].data_ptr(),
                                                       self.sin[index_pos].data_ptr(), B, cfg.n_head, cfg.n_kv_head, cfg.head_dim,
                                                       cfg.max_seq, index_pos, q.data_ptr(), kc.data_ptr(), vc.data_ptr()))
            y = self._library_attention(q, kc, vc, n)
            return lw.attention_wo.forward(y) + x
        h = rms_norm(x, lw.attention_norm, cfg.rms_eps)
        q = lw.attention_wq.forward(h).view(B, 1, cfg.n_head, cfg.head_dim).transpose(1, 2)
        k = lw.attention_wk.forward(h).view(B, 1, cfg.n_kv_head, cfg.head_dim).transpose(1, 2)
        v = lw.attention_wv.forward(h).view(B, 1, cfg.n_kv_head, cfg.head_dim).transpose(1, 2)
        cos, sin = self.cos[index_pos:index_pos + 1], self.sin[index_pos:index_pos + 1]
        q, k = rope_interleaved(q, cos, sin), rope_interleaved(k, cos, sin)
        kc[:, :, index_pos:index_pos + 1] = k
        vc[:, :, index_pos:index_pos + 1] = v
        g = cfg.n_head // cfg.n_kv_head
        qg = q.reshape(B, cfg.n_kv_head, g, cfg.head_dim)              # the g query heads that share a kv head
        att = torch.matmul(qg, kc[:, :, :n].transpose(-1, -2)) / math.sqrt(cfg.head_dim)
        att = torch.softmax(att, dim=-1)
        y = torch.matmul(att, vc[:, :, :n]).reshape(B, cfg.n_head * cfg.head_dim)
        return lw.attention_wo.forward(y) + x

    def _library_attention(self, q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, n: int) -> torch.Tensor:
        import ctypes as C
        from . import _lib
        from .quantized import _stream_ptr
        cfg, B = self.cfg, self.batch
        L = _lib.load()
        if self._att_ws is None:
            need = C.c_size_t(0)
            _lib.check("candle_moe_decode_attention_workspace_bytes",
                       L.candle_moe_decode_attention_workspace_bytes(B, cfg.n_head, cfg.head_dim, cfg.max_seq, C.byref(need)))
            self._att_ws = torch.empty(need.value + 16, dtype=torch.uint8, device=self.device)
        qc = q.reshape(B, cfg.n_head, cfg.head_dim).contiguous()
        y = torch.empty((B, cfg.n_head * cfg.head_dim), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            st = L.candle_moe_decode_attention(_stream_ptr(self.device), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, cfg.n_head,
                                               cfg.n_kv_head, cfg.head_dim, cfg.max_seq, n, y.data_ptr(), self._att_ws.data_ptr(),
                                               self._att_ws.numel())
        _lib.check("candle_moe_decode_attention", st)
        return y

    def ffn(self, li: int, x: torch.Tensor) -> torch.Tensor:
        """`ffn_norm` -> `mlp_or_moe` -> `+ residual` (quantized_llama.rs:886-891)."""
        si = self.layer_set[li]
        lw = self.sets[si]
        if self.ep is None:
            return lw.mlp_or_moe.forward_layer(x, lw.ffn_norm, self.cfg.rms_eps)
        return self.ep[si].forward(rms_norm(x, lw.ffn_norm, self.cfg.rms_eps)) + x

    def forward(self, tokens: torch.Tensor, index_pos: int) -> torch.Tensor:
        """tokens [B] int64 -> logits [B, vocab]."""
        x = torch.nn.functional.embedding(tokens, self.tok_embeddings)
        for li in range(self.cfg.n_layer):
            x = self.attention(li, x, index_pos)
            x = self.ffn(li, x)
        x = rms_norm(x, self.norm, self.cfg.rms_eps)
        return self.output.forward(x)

    # -- accounting ----------------------------------------------------------------------------------------
    def bytes_per_step(self, index_pos: int) -> dict:
        """Bytes a decode step must read from HBM: every layer's quantized matrices (all experts, as a batch of 32
        rows selects them all), the KV cache up to the current position, the lm head."""
        cfg = self.cfg
        blk = {int(GgmlDType.Q4K): (256, 144), int(GgmlDType.Q6K): (256, 210), int(GgmlDType.Q8_0): (32, 34)}
        mb = lambda dt, n, k: n * (k // blk[dt][0]) * blk[dt][1]
        d, hd = cfg.d_model, cfg.head_dim
        attn = 2 * mb(cfg.dt_attn, cfg.n_head * hd, d) + 2 * mb(cfg.dt_attn, cfg.n_kv_head * hd, d)
        moe = cfg.n_expert * (2 * mb(cfg.dt_w13, cfg.d_ff, d) + mb(cfg.dt_w2, d, cfg.d_ff))
        kv = 2 * self.batch * cfg.n_kv_head * (index_pos + 1) * hd * 4
        return {"attention_weights": cfg.n_layer * attn, "moe_weights": cfg.n_layer * moe, "kv_cache": cfg.n_layer * kv,
                "lm_head": mb(cfg.dt_output, cfg.vocab, d)}
