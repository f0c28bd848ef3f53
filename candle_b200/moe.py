"""Host-side mirror of the quantized MoE feed-forward block of candle-transformers'
quantized_llama (`Mlp` :117-131, `MlpOrMoe` :133-211).

`MlpOrMoe.moe(...)` holds the same things the reference enum variant holds (`n_expert_used`,
`feed_forward_gate_inp`, `experts: Vec<Mlp>`) and `forward(xs)` has `Module::forward`'s contract:
`xs` f32 `[b, seq, d]` on the device, result of the same shape.  The whole block is ONE call into
the C ABI (`candle_moe_forward`): no host synchronisation, no per-expert uploads.  The optional
shared expert follows `SparseMoeBlock` of qwen2_moe.rs:226-323.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib
from .quantized import GgmlDType, QMatMul, QTensor, _stream_ptr


@dataclass
class Mlp:
    """`Mlp` (quantized_llama.rs:117-122): w1/w3 are `[d_ff, d]`, w2 is `[d, d_ff]`."""
    feed_forward_w1: QMatMul
    feed_forward_w2: QMatMul
    feed_forward_w3: QMatMul

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        """`Mlp::forward` (:124-131) for a dense (non-MoE) layer: one group holding every row."""
        blk = MlpOrMoe(n_expert_used=1, feed_forward_gate_inp=None, experts=[self], _dense=True)
        return blk.forward(xs)


class MlpOrMoe:
    """`MlpOrMoe::MoE` (quantized_llama.rs:134-141)."""

    def __init__(self, n_expert_used: int, feed_forward_gate_inp: Optional[torch.Tensor], experts: List[Mlp], *,
                 norm_topk_prob: bool = True, router_bias: Optional[torch.Tensor] = None,
                 shared_expert: Optional[Mlp] = None, shared_expert_gate: Optional[torch.Tensor] = None,
                 _dense: bool = False):
        if not experts:
            raise ValueError("at least one expert is required")
        w1 = experts[0].feed_forward_w1.inner
        w2 = experts[0].feed_forward_w2.inner
        self.d_ff, self.d_model = w1.shape()
        self.device = w1.device()
        self.experts = experts
        self.n_expert_used = int(n_expert_used)
        self.norm_topk_prob = bool(norm_topk_prob)
        for m in experts:
            for q, shp, dt in ((m.feed_forward_w1.inner, (self.d_ff, self.d_model), w1.dtype()),
                               (m.feed_forward_w3.inner, (self.d_ff, self.d_model), w1.dtype()),
                               (m.feed_forward_w2.inner, (self.d_model, self.d_ff), w2.dtype())):
                if q.shape() != shp or q.dtype() != dt:
                    raise ValueError("all experts must share shapes and dtypes")
        if _dense:
            # a dense Mlp is the block with one expert that every row selects with weight 1
            feed_forward_gate_inp = torch.zeros((1, self.d_model), dtype=torch.float32, device=self.device)
        if feed_forward_gate_inp is None:
            raise ValueError("feed_forward_gate_inp is required")
        # The fused path takes an f32 router only (GGUF Mixtral files keep ffn_gate_inp in F32;
        # QMatMul::from_arc dequantizes F32/F16/BF16 gates to a dense tensor, mod.rs:430-436).
        if feed_forward_gate_inp.dtype != torch.float32:
            raise ValueError("the fused MoE path needs an f32 router (feed_forward_gate_inp)")
        self.feed_forward_gate_inp = feed_forward_gate_inp.to(self.device).contiguous()
        if tuple(self.feed_forward_gate_inp.shape) != (len(experts), self.d_model):
            raise ValueError("router must be [n_experts, d_model]")
        self.router_bias = None if router_bias is None else router_bias.to(self.device, torch.float32).contiguous()
        self.shared_expert = shared_expert
        self.shared_expert_gate = None
        if shared_expert is not None:
            if shared_expert_gate is None:
                raise ValueError("shared_expert needs shared_expert_gate")
            self.shared_expert_gate = shared_expert_gate.to(self.device, torch.float32).reshape(-1).contiguous()

        E = len(experts)
        self._arr = C.c_void_p * E
        self._w1 = self._arr(*[m.feed_forward_w1.inner.device_ptr() for m in experts])
        self._w3 = self._arr(*[m.feed_forward_w3.inner.device_ptr() for m in experts])
        self._w2 = self._arr(*[m.feed_forward_w2.inner.device_ptr() for m in experts])
        cw = _lib.MoeWeightsC()
        cw.d_model, cw.d_ff, cw.n_experts, cw.top_k = self.d_model, self.d_ff, E, self.n_expert_used
        cw.renorm = int(self.norm_topk_prob)
        cw.dtype_w13, cw.dtype_w2 = int(w1.dtype()), int(w2.dtype())
        cw.router = self.feed_forward_gate_inp.data_ptr()
        cw.router_bias = None if self.router_bias is None else self.router_bias.data_ptr()
        cw.w1, cw.w3, cw.w2 = self._w1, self._w3, self._w2
        if shared_expert is not None:
            s1, s2 = shared_expert.feed_forward_w1.inner, shared_expert.feed_forward_w2.inner
            cw.d_ff_shared = s1.shape()[0]
            cw.dtype_shared13, cw.dtype_shared2 = int(s1.dtype()), int(s2.dtype())
            cw.shared_w1 = s1.device_ptr()
            cw.shared_w3 = shared_expert.feed_forward_w3.inner.device_ptr()
            cw.shared_w2 = s2.device_ptr()
            cw.shared_gate = self.shared_expert_gate.data_ptr()
        self._cw = cw
        self._ws: Optional[torch.Tensor] = None
        self._ws_tokens = 0

    # quantized_llama.rs constructs the variant from GGUF tensors; this is the same from QTensors
    @classmethod
    def moe(cls, n_expert_used: int, feed_forward_gate_inp: torch.Tensor, experts: List[Mlp], **kw) -> "MlpOrMoe":
        return cls(n_expert_used, feed_forward_gate_inp, experts, **kw)

    def prepack(self) -> "MlpOrMoe":
        """Make the optional repacked copies of every expert matrix (one-time, doubles the weight memory of this
        block): k-quants for the decode kernels (batches of up to 96 rows) and Q6_K in the large-batch GEMM, Q8_0 for
        the large-batch GEMM."""
        def copies(mats):
            # every matrix of the family or none: a shape the repack does not take (CANDLE_MOE_E_SHAPE, e.g. Q6_K rows
            # with an odd number of 256-blocks) leaves the family on its GGUF blocks
            try:
                return [m.inner.prepack() for m in mats]
            except _lib.CandleMoeError as e:
                if e.status != -2:  # CANDLE_MOE_E_SHAPE
                    raise
                return None

        w13 = copies([m.feed_forward_w1 for m in self.experts] + [m.feed_forward_w3 for m in self.experts])
        w2 = copies([m.feed_forward_w2 for m in self.experts])
        E = len(self.experts)
        if w13 is not None:
            self._p1 = self._arr(*[t.data_ptr() for t in w13[:E]])
            self._p3 = self._arr(*[t.data_ptr() for t in w13[E:]])
            self._cw.w1_prepacked, self._cw.w3_prepacked = self._p1, self._p3
        if w2 is not None:
            self._p2 = self._arr(*[t.data_ptr() for t in w2])
            self._cw.w2_prepacked = self._p2
        if self.shared_expert is not None and self.shared_expert.feed_forward_w1.inner.dtype() == GgmlDType.Q8_0:
            s = self.shared_expert
            sh = copies([s.feed_forward_w1, s.feed_forward_w3, s.feed_forward_w2])
            if sh is not None:
                self._cw.shared_w1_prepacked, self._cw.shared_w3_prepacked, self._cw.shared_w2_prepacked = (
                    t.data_ptr() for t in sh)
        return self

    @property
    def n_experts(self) -> int:
        return len(self.experts)

    def workspace_bytes(self, tokens: int) -> int:
        out = C.c_size_t(0)
        _lib.check("candle_moe_workspace_bytes",
                   _lib.load().candle_moe_workspace_bytes(C.byref(self._cw), tokens, C.byref(out)))
        return out.value

    def reserve(self, tokens: int) -> None:
        """Allocate the scratch for up to `tokens` rows once (the C ABI itself never allocates)."""
        if self._ws is None or tokens > self._ws_tokens:
            self._ws = torch.empty(self.workspace_bytes(tokens) + 256, dtype=torch.uint8, device=self.device)
            self._ws_tokens = tokens

    def _ws_ptr(self) -> int:
        return (self._ws.data_ptr() + 255) // 256 * 256

    def forward(self, xs: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`Module::forward` (quantized_llama.rs:143-210)."""
        if not xs.is_cuda:
            raise ValueError("MlpOrMoe.forward has no CPU path: xs must be on the CUDA device")
        if xs.dtype != torch.float32 or xs.shape[-1] != self.d_model:
            raise ValueError(f"expected f32 [.., {self.d_model}], got {xs.dtype} {tuple(xs.shape)}")
        x2 = xs.reshape(-1, self.d_model).contiguous()
        T = x2.shape[0]
        self.reserve(max(T, 1))
        y = out if out is not None else torch.empty_like(x2)
        with torch.cuda.device(self.device):
            st = _lib.load().candle_moe_forward(_stream_ptr(self.device), C.byref(self._cw), x2.data_ptr(), T,
                                                y.data_ptr(), self._ws_ptr(), self._ws.numel() - 256)
        _lib.check("candle_moe_forward", st)
        return y.reshape(xs.shape)

    __call__ = forward

    def forward_layer(self, xs: torch.Tensor, ffn_norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
        """The FFN half of a decoder layer: `xs + self.forward(rms_norm(xs, ffn_norm_weight, eps))`
        (quantized_llama.rs:887-891), one call into the C ABI."""
        if not xs.is_cuda or xs.dtype != torch.float32 or xs.shape[-1] != self.d_model:
            raise ValueError(f"expected a CUDA f32 [.., {self.d_model}] tensor")
        x2 = xs.reshape(-1, self.d_model).contiguous()
        T = x2.shape[0]
        nw = ffn_norm_weight.to(self.device, torch.float32).contiguous()
        need = C.c_size_t(0)
        L = _lib.load()
        _lib.check("candle_moe_ffn_layer_workspace_bytes", L.candle_moe_ffn_layer_workspace_bytes(C.byref(self._cw), max(T, 1),
                                                                                             C.byref(need)))
        if self._ws is None or self._ws.numel() - 256 < need.value:
            self._ws = torch.empty(need.value + 256, dtype=torch.uint8, device=self.device)
            self._ws_tokens = T
        y = torch.empty_like(x2)
        with torch.cuda.device(self.device):
            st = L.candle_moe_ffn_layer(_stream_ptr(self.device), C.byref(self._cw), nw.data_ptr(), float(eps), x2.data_ptr(), T,
                                        y.data_ptr(), self._ws_ptr(), self._ws.numel() - 256)
        _lib.check("candle_moe_ffn_layer", st)
        return y.reshape(xs.shape)

    STAGES = ("router_topk", "permute", "quantize_x", "gate_up", "quantize_h", "down", "shared_expert", "combine")

    def forward_timed(self, xs: torch.Tensor):
        """One forward with CUDA events between its launches: (y, {stage: milliseconds})."""
        x2 = xs.reshape(-1, self.d_model).contiguous()
        T = x2.shape[0]
        self.reserve(max(T, 1))
        y = torch.empty_like(x2)
        ms = (C.c_float * 8)()
        with torch.cuda.device(self.device):
            st = _lib.load().candle_moe_forward_timed(_stream_ptr(self.device), C.byref(self._cw), x2.data_ptr(), T,
                                                      y.data_ptr(), self._ws_ptr(), self._ws.numel() - 256, ms)
        _lib.check("candle_moe_forward_timed", st)
        return y.reshape(xs.shape), {n: float(ms[i]) for i, n in enumerate(self.STAGES)}

    def last_routing(self, T: int):
        """Routing of the last forward over T rows, read back for tests and expert-parallel callers:
        (topk_ids [T,k] i64, topk_w [T,k] f32, expert_counts [E] i64, perm_token [T*k] i64)."""
        ids, tw, cnt, perm = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        _lib.check("candle_moe_workspace_views",
                   _lib.load().candle_moe_workspace_views(C.byref(self._cw), T, self._ws_ptr(), C.byref(ids),
                                                          C.byref(tw), C.byref(cnt), C.byref(perm)))
        base, k, E = self._ws_ptr(), self.n_expert_used, self.n_experts
        raw = self._ws[base - self._ws.data_ptr():]

        def view(ptr, n, dt):
            off = ptr.value - base
            return raw[off:off + 4 * n].view(dt)

        torch.cuda.current_stream(self.device).synchronize()
        return (view(ids, T * k, torch.int32).reshape(T, k).long().cpu(),
                view(tw, T * k, torch.float32).reshape(T, k).cpu(),
                view(cnt, E, torch.int32).long().cpu(),
                view(perm, T * k, torch.int32).long().cpu())
