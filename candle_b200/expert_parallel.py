"""Expert-parallel form of the quantized MoE block: the experts of `MlpOrMoe::MoE`
(candle-transformers/src/models/quantized_llama.rs:134-211) sharded over the ranks of a
`torch.distributed` process group, one process per GPU.

Rank r owns experts [r * E/N, (r + 1) * E/N) and routes its own tokens.  A step is

    route + quantize + group by expert            (local, as on one device)
    all-to-all of the per-expert row counts       (N * E/N integers)
    all-to-all of the packed quantized rows       (grouped order is already destination order)
    the local experts over the received rows      (candle_moe_ep_experts)
    all-to-all of the expert outputs back
    weighted combine                              (local, as on one device)

The reference has no multi-device form of the block; the results here are those of the single-device
block bit for bit, because a row's expert products do not depend on which other rows share the call and
what travels is the quantized row the receiving matmul would have produced itself.

The exchange logic lives in this class and only needs the four device steps of `ops`, so the same code
runs over NCCL with the CUDA library and, in the CPU tests, over gloo with a stand-in for the device steps.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from . import _lib
from .moe import Mlp, MlpOrMoe
from .quantized import _stream_ptr


@dataclass
class Routed:
    """What the local routing step leaves for the later steps (device tensors)."""
    T: int
    topk_ids: torch.Tensor   # [T, k] int32
    topk_w: torch.Tensor     # [T, k] f32
    counts: torch.Tensor     # [E] int32, rows per GLOBAL expert
    perm_token: torch.Tensor  # [T*k] int32
    pair_pos: torch.Tensor   # [T*k] int32
    extra: Any = None        # backend-private (quantized rows)


class CudaOps:
    """The four device steps over the C ABI."""

    def __init__(self, n_experts_global: int, top_k: int, router: torch.Tensor, router_bias: Optional[torch.Tensor],
                 renorm: bool, local_block: MlpOrMoe):
        self.E, self.k, self.router, self.bias, self.renorm = n_experts_global, top_k, router, router_bias, renorm
        self.local = local_block
        self.d = local_block.d_model
        self.dev = local_block.device
        self.L = _lib.load()
        rb = C.c_size_t(0)
        _lib.check("candle_moe_ep_row_bytes", self.L.candle_moe_ep_row_bytes(self.d, C.byref(rb)))
        self.row_bytes = rb.value
        self._ws: Optional[torch.Tensor] = None
        self._ws_rows = 0

    def route(self, x: torch.Tensor) -> Routed:
        T, d, E, k, L, dev = x.shape[0], self.d, self.E, self.k, self.L, self.dev
        i32, f32 = torch.int32, torch.float32
        ids = torch.empty((T, k), dtype=i32, device=dev)
        tw = torch.empty((T, k), dtype=f32, device=dev)
        counts = torch.empty(E, dtype=i32, device=dev)
        offsets = torch.empty(E + 1, dtype=i32, device=dev)
        perm = torch.empty(T * k, dtype=i32, device=dev)
        pos = torch.empty(T * k, dtype=i32, device=dev)
        xq = torch.empty((T, d), dtype=torch.int8, device=dev)
        xs = torch.empty((T, d // 256), dtype=f32, device=dev)
        xb = torch.empty((T, d // 16), dtype=torch.int16, device=dev)
        st = _stream_ptr(dev)
        bias = None if self.bias is None else self.bias.data_ptr()
        _lib.check("candle_moe_router_topk", L.candle_moe_router_topk(st, x.data_ptr(), self.router.data_ptr(), bias, T, d, E, k,
                                                                      int(self.renorm), ids.data_ptr(), tw.data_ptr()))
        _lib.check("candle_moe_quantize_act", L.candle_moe_quantize_act(st, x.data_ptr(), T, d, int(self.local._cw.dtype_w13),
                                                                        xq.data_ptr(), xs.data_ptr(), xb.data_ptr()))
        _lib.check("candle_moe_permute", L.candle_moe_permute(st, ids.data_ptr(), T, k, E, counts.data_ptr(), offsets.data_ptr(),
                                                              perm.data_ptr(), pos.data_ptr()))
        return Routed(T, ids, tw, counts, perm, pos, (xq, xs, xb))

    def pack(self, r: Routed) -> torch.Tensor:
        n = r.T * self.k
        send = torch.empty((n, self.row_bytes), dtype=torch.uint8, device=self.dev)
        xq, xs, xb = r.extra
        _lib.check("candle_moe_ep_pack", self.L.candle_moe_ep_pack(_stream_ptr(self.dev), r.perm_token.data_ptr(), n, self.d,
                                                                   xq.data_ptr(), xs.data_ptr(), xb.data_ptr(), send.data_ptr()))
        return send

    def empty_rows(self, n: int) -> torch.Tensor:
        return torch.empty((n, self.row_bytes), dtype=torch.uint8, device=self.dev)

    def empty_out(self, n: int) -> torch.Tensor:
        return torch.empty((n, self.d), dtype=torch.float32, device=self.dev)

    def experts(self, recv_rows: torch.Tensor, recv_counts: torch.Tensor, n_rows: int, max_rows: int) -> torch.Tensor:
        out = self.empty_out(n_rows)
        if n_rows == 0:
            return out
        if self._ws is None or n_rows > self._ws_rows:
            need = C.c_size_t(0)
            cap = max(n_rows, 2 * self._ws_rows)
            _lib.check("candle_moe_ep_workspace_bytes",
                       self.L.candle_moe_ep_workspace_bytes(C.byref(self.local._cw), cap, C.byref(need)))
            self._ws = torch.empty(need.value + 256, dtype=torch.uint8, device=self.dev)
            self._ws_rows = cap
        ws_ptr = (self._ws.data_ptr() + 255) // 256 * 256
        n_src = recv_counts.shape[0]
        _lib.check("candle_moe_ep_experts",
                   self.L.candle_moe_ep_experts(_stream_ptr(self.dev), C.byref(self.local._cw), recv_rows.data_ptr(),
                                                recv_counts.data_ptr(), n_src, n_rows, max_rows, out.data_ptr(), ws_ptr,
                                                self._ws.numel() - 256))
        return out

    def combine(self, r: Routed, ret_rows: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        y = torch.empty_like(x)
        _lib.check("candle_moe_combine",
                   self.L.candle_moe_combine(_stream_ptr(self.dev), ret_rows.data_ptr(), r.topk_ids.data_ptr(),
                                             r.topk_w.data_ptr(), r.pair_pos.data_ptr(), r.T, self.k, self.d, None,
                                             x.data_ptr(), None, y.data_ptr()))
        return y


class ExpertParallelMoe:
    """`MlpOrMoe::MoE` over a process group.  `local_experts` are this rank's E/N experts (global expert id =
    rank * E/N + local index); `feed_forward_gate_inp` is the full `[E, d]` router, replicated."""

    def __init__(self, n_expert_used: int, feed_forward_gate_inp: torch.Tensor, local_experts: List[Mlp], *,
                 group: Optional[dist.ProcessGroup] = None, norm_topk_prob: bool = True,
                 router_bias: Optional[torch.Tensor] = None, prepack: bool = False, ops: Any = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k = int(n_expert_used)
        E = feed_forward_gate_inp.shape[0]
        if E % self.world:
            raise ValueError(f"{E} experts do not divide over {self.world} ranks")
        self.E, self.E_local = E, E // self.world
        if ops is None:
            if len(local_experts) != self.E_local:
                raise ValueError(f"this rank holds {len(local_experts)} experts, expected {self.E_local}")
            dev = local_experts[0].feed_forward_w1.inner.device()
            router = feed_forward_gate_inp.to(dev, torch.float32).contiguous()
            lo = self.rank * self.E_local
            # the local block only describes this rank's expert matrices to the C ABI (its router and top-k are not
            # used there); a rank may hold fewer experts than a token selects
            local = MlpOrMoe(min(self.k, self.E_local), router[lo:lo + self.E_local].contiguous(), local_experts,
                             norm_topk_prob=norm_topk_prob)
            if prepack:
                local.prepack()
            bias = None if router_bias is None else router_bias.to(dev, torch.float32).contiguous()
            ops = CudaOps(E, self.k, router, bias, norm_topk_prob, local)
        self.ops = ops
        self.d_model = ops.d

    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_split=None, in_split=None) -> None:
        if not dist.is_initialized():
            out.copy_(inp)
            return
        dist.all_to_all_single(out, inp, out_split, in_split, group=self.group)

    PHASES = ("route_pack", "exchange_rows", "experts", "exchange_results", "combine")

    def forward(self, xs: torch.Tensor, mark=None) -> torch.Tensor:
        """One step.  `mark`, if given, is called after each of PHASES (for per-phase timing)."""
        mark = mark or (lambda: None)
        x2 = xs.reshape(-1, self.d_model).contiguous()
        N, El = self.world, self.E_local
        r = self.ops.route(x2)
        send_rows = self.ops.pack(r)
        mark()
        # rows per (destination rank, its local expert) -> rows per (source rank, my local expert)
        recv_counts = torch.empty((N, El), dtype=r.counts.dtype, device=r.counts.device)
        self._a2a(recv_counts.view(-1), r.counts.view(-1))
        both = torch.stack([r.counts.view(N, El), recv_counts]).cpu()  # the one host synchronisation of the step
        send_split = [int(v) for v in both[0].sum(1)]
        recv_split = [int(v) for v in both[1].sum(1)]
        n_rows = sum(recv_split)
        max_rows = int(both[1].sum(0).max()) if n_rows else 0
        recv_rows = self.ops.empty_rows(n_rows)
        self._a2a(recv_rows, send_rows, recv_split, send_split)
        mark()
        out_rows = self.ops.experts(recv_rows, recv_counts, n_rows, max_rows)
        mark()
        ret_rows = self.ops.empty_out(r.T * self.k)
        self._a2a(ret_rows, out_rows, send_split, recv_split)
        mark()
        y = self.ops.combine(r, ret_rows, x2)
        mark()
        self.last_rows, self.last_max_rows = n_rows, max_rows
        return y.reshape(xs.shape)

    __call__ = forward
