"""Expert-parallel form of the quantized MoE block: the experts of `MlpOrMoe::MoE`
(candle-transformers/src/models/quantized_llama.rs:134-211) sharded over ranks, one process per GPU.

Rank r owns experts [r * E/N, (r + 1) * E/N) and routes its own tokens.  A step is

    route + quantize + group by expert            (local, as on one device)
    all-to-all of the packed quantized rows       (grouped order is already destination order)
    the local experts over the received rows
    all-to-all of the expert outputs back
    weighted combine                              (local, as on one device)

On CUDA the whole step is ONE call into the C ABI (`candle_moe_ep_forward`, candle_b200/csrc/ep_nccl.cu): the
library owns the NCCL calls, Python only makes the communicator -- rank 0 creates the NCCL id and hands it to the
others through `torch.distributed`, the way candle's multi-process example does with a file
(candle-examples/examples/llama_multiprocess/main.rs:148-173).

The reference has no multi-device form of the block; the results here are those of the single-device block,
because a row's expert products do not depend on which other rows share the call and what travels is the
quantized row the receiving matmul would have produced itself.

`ExpertParallelMoe(..., ops=...)` runs the SAME exchange protocol in Python over any `torch.distributed` backend
with the device steps supplied by `ops`: the CPU tests run it over gloo with the oracle standing in for the
kernels, which covers the protocol's index arithmetic, its two forms and its failure handling without a GPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from .moe import Mlp, MlpOrMoe
from .quantized import GgmlDType, _stream_ptr

EP_MAGIC = 0x45504D43
SLOT_FORM_MAX_BYTES = 24 << 20  # per direction and rank; above it the exact form runs (candle_b200/csrc/ep_nccl.cu)
FORM_SLOTS, FORM_EXACT = 1, 2


class EpMismatchError(RuntimeError):
    """The ranks' exchange metadata disagree.  Raised on EVERY rank, before any row is exchanged."""


@dataclass
class Routed:
    """What the local routing step leaves for the later steps."""
    T: int
    topk_ids: torch.Tensor   # [T, k] int32
    topk_w: torch.Tensor     # [T, k] f32
    counts: torch.Tensor     # [E] int32, rows per GLOBAL expert
    perm_token: torch.Tensor  # [T*k] int32
    pair_pos: torch.Tensor   # [T*k] int32
    extra: Any = None        # backend-private (quantized rows)


class CudaOps:
    """The device steps over the C ABI, one call each, for a host that drives the exchange itself."""

    def __init__(self, n_experts_global: int, top_k: int, router: torch.Tensor, router_bias: Optional[torch.Tensor],
                 renorm: bool, local_block: MlpOrMoe):
        for dt in (local_block._cw.dtype_w13, local_block._cw.dtype_w2):
            if dt == int(GgmlDType.Q8_0):
                raise ValueError("expert parallelism takes k-quant experts (Q4_K / Q6_K): the travelling row is a Q8K row")
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


def choose_form(world: int, max_tokens: int, top_k: int, n_local: int, d_model: int, force_form: int = 0):
    """(form, slot capacity in rows): the rule of candle_moe_ep_forward, from the configuration alone."""
    cap = max_tokens * min(top_k, n_local)
    row_bytes = -(-(d_model + d_model // 8 + d_model // 64) // 16) * 16
    hdr = -(-(16 + 4 * n_local) // 16) * 16
    fwd, back = world * (hdr + cap * row_bytes), world * cap * d_model * 4
    form = FORM_SLOTS if max(fwd, back) <= SLOT_FORM_MAX_BYTES else FORM_EXACT
    return (force_form or form), cap


class ExpertParallelMoe:
    """`MlpOrMoe::MoE` over ranks.  `local_experts` are this rank's E/N experts (global expert id =
    rank * E/N + local index); `feed_forward_gate_inp` is the full `[E, d]` router, replicated.

    `max_tokens` bounds the rows ANY rank routes in one step and must be the same on every rank (it sizes the
    slots of the small-step form); when omitted it is agreed once, at the first forward, as the largest row count
    among the ranks of that step."""

    PHASES = ("route_pack", "exchange_rows", "experts", "exchange_results", "combine")

    def __init__(self, n_expert_used: int, feed_forward_gate_inp: torch.Tensor, local_experts: List[Mlp], *,
                 group: Optional[dist.ProcessGroup] = None, norm_topk_prob: bool = True,
                 router_bias: Optional[torch.Tensor] = None, prepack: bool = False, ops: Any = None,
                 max_tokens: Optional[int] = None, force_form: int = 0, max_recv_rows: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k = int(n_expert_used)
        E = feed_forward_gate_inp.shape[0]
        if E % self.world:
            raise ValueError(f"{E} experts do not divide over {self.world} ranks")
        self.E, self.E_local = E, E // self.world
        self.max_tokens, self.force_form, self.max_recv_rows = max_tokens, int(force_form), int(max_recv_rows)
        self.inject_count_mismatch = False  # tests: this rank reports a bad count table in its next exact-form step
        self.last_rows = self.last_max_rows = -1
        self.ops = ops
        self._comm = C.c_void_p(None)
        self._ws: Optional[torch.Tensor] = None
        self._ws_key = None
        if ops is not None:
            self.d_model = ops.d
            return
        if len(local_experts) != self.E_local:
            raise ValueError(f"this rank holds {len(local_experts)} experts, expected {self.E_local}")
        w1 = local_experts[0].feed_forward_w1.inner
        w2 = local_experts[0].feed_forward_w2.inner
        if GgmlDType.Q8_0 in (w1.dtype(), w2.dtype()):
            raise ValueError("expert parallelism takes k-quant experts (Q4_K / Q6_K): the travelling row is a Q8K row")
        dev = w1.device()
        self.device = dev
        self.router = feed_forward_gate_inp.to(dev, torch.float32).contiguous()
        self.router_bias = None if router_bias is None else router_bias.to(dev, torch.float32).contiguous()
        self.renorm = bool(norm_topk_prob)
        lo = self.rank * self.E_local
        # the local block only describes this rank's expert matrices to the C ABI (its router and top-k are not
        # used there); a rank may hold fewer experts than a token selects
        self.local = MlpOrMoe(min(self.k, self.E_local), self.router[lo:lo + self.E_local].contiguous(), local_experts,
                              norm_topk_prob=norm_topk_prob)
        if prepack:
            self.local.prepack()
        self.d_model = self.local.d_model
        self.L = _lib.load()

    # ---- communicator ------------------------------------------------------------------------------------
    def _communicator(self):
        if self.world == 1 or self._comm:
            return self._comm
        nbytes = 128
        on_gpu = dist.get_backend(self.group) == "nccl"
        buf = torch.zeros(nbytes, dtype=torch.uint8)
        if self.rank == 0:
            raw = (C.c_uint8 * nbytes)()
            _lib.check("candle_moe_ep_unique_id", self.L.candle_moe_ep_unique_id(raw))
            buf = torch.tensor(list(raw), dtype=torch.uint8)
        if on_gpu:
            buf = buf.to(self.device)
        src = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        dist.broadcast(buf, src, group=self.group)
        raw = (C.c_uint8 * nbytes)(*buf.cpu().tolist())
        with torch.cuda.device(self.device):
            st = self.L.candle_moe_ep_comm_init(raw, self.rank, self.world, C.byref(self._comm))
        self._check("candle_moe_ep_comm_init", st)
        return self._comm

    def close(self) -> None:
        if self._comm:
            _lib.load().candle_moe_ep_comm_destroy(self._comm)
            self._comm = C.c_void_p(None)

    def _check(self, fn: str, status: int) -> None:
        if status == -9:
            raise EpMismatchError(self.L.candle_moe_ep_last_error().decode())
        if status == -8:
            raise _lib.CandleMoeError(fn + " [" + self.L.candle_moe_ep_last_error().decode() + "]", status)
        _lib.check(fn, status)

    def _agree_max_tokens(self, T: int) -> None:
        if self.max_tokens is None:
            m = torch.tensor([T], dtype=torch.int64)
            if dist.is_initialized():
                if dist.get_backend(self.group) == "nccl":
                    m = m.cuda()
                dist.all_reduce(m, op=dist.ReduceOp.MAX, group=self.group)
            self.max_tokens = max(int(m.item()), 1)
        if T > self.max_tokens:
            raise ValueError(f"{T} rows in a step, but this block was set up for at most {self.max_tokens} per rank")

    def _config(self) -> "_lib.EpConfigC":
        cfg = _lib.EpConfigC()
        cfg.rank, cfg.world, cfg.n_experts_global, cfg.top_k = self.rank, self.world, self.E, self.k
        cfg.renorm, cfg.max_tokens, cfg.force_form = int(self.renorm), int(self.max_tokens), self.force_form
        cfg.inject_count_mismatch = int(self.inject_count_mismatch)
        cfg.max_recv_rows = self.max_recv_rows
        cfg.router = self.router.data_ptr()
        cfg.router_bias = None if self.router_bias is None else self.router_bias.data_ptr()
        return cfg

    def form(self) -> int:
        """1 = slots, 2 = exact: which form a step takes with the current configuration."""
        if self.ops is not None:
            return choose_form(self.world, self.max_tokens, self.k, self.E_local, self.d_model, self.force_form)[0]
        f = C.c_int32(0)
        cfg = self._config()
        _lib.check("candle_moe_ep_forward_form", self.L.candle_moe_ep_forward_form(C.byref(cfg), C.byref(self.local._cw), C.byref(f), None))
        return f.value

    # ---- the step ------------------------------------------------------------------------------------------
    def forward(self, xs: torch.Tensor, out: Optional[torch.Tensor] = None, timed: bool = False):
        """One step.  With `timed` returns (y, {phase: ms}) measured with CUDA events between the phases."""
        x2 = xs.reshape(-1, self.d_model).contiguous()
        T = x2.shape[0]
        self._agree_max_tokens(T)
        if self.ops is not None:
            y = self._forward_protocol(x2)
            return y.reshape(xs.shape)
        if not x2.is_cuda or x2.dtype != torch.float32:
            raise ValueError("ExpertParallelMoe.forward expects a CUDA f32 tensor")
        cfg = self._config()
        key = (self.max_tokens, self.force_form, self.max_recv_rows)
        if self._ws is None or self._ws_key != key:
            need = C.c_size_t(0)
            _lib.check("candle_moe_ep_forward_workspace_bytes",
                       self.L.candle_moe_ep_forward_workspace_bytes(C.byref(cfg), C.byref(self.local._cw), C.byref(need)))
            self._ws = torch.empty(need.value + 256, dtype=torch.uint8, device=self.device)
            self._ws_key = key
        ws_ptr = (self._ws.data_ptr() + 255) // 256 * 256
        y = out if out is not None else torch.empty_like(x2)
        comm = self._communicator()
        with torch.cuda.device(self.device):
            if timed:
                ms = (C.c_float * 5)()
                info = (C.c_int64 * 2)()
                st = self.L.candle_moe_ep_forward_timed(_stream_ptr(self.device), comm, C.byref(cfg), C.byref(self.local._cw),
                                                        x2.data_ptr(), T, y.data_ptr(), ws_ptr, self._ws.numel() - 256, ms, info)
                self._check("candle_moe_ep_forward_timed", st)
                self.last_rows, self.last_max_rows = int(info[0]), int(info[1])
                return y.reshape(xs.shape), {n: float(ms[i]) for i, n in enumerate(self.PHASES)}
            st = self.L.candle_moe_ep_forward(_stream_ptr(self.device), comm, C.byref(cfg), C.byref(self.local._cw),
                                              x2.data_ptr(), T, y.data_ptr(), ws_ptr, self._ws.numel() - 256)
        self._check("candle_moe_ep_forward", st)
        return y.reshape(xs.shape)

    __call__ = forward

    # ---- the same protocol in Python over any backend (device steps from `ops`) -------------------------
    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_split=None, in_split=None) -> None:
        if not dist.is_initialized():
            out.copy_(inp)
            return
        dist.all_to_all_single(out, inp, out_split, in_split, group=self.group)

    def _forward_protocol(self, x2: torch.Tensor) -> torch.Tensor:
        N, El, k, ops = self.world, self.E_local, self.k, self.ops
        form, cap = choose_form(N, self.max_tokens, k, El, self.d_model, self.force_form)
        r = ops.route(x2)
        rows = ops.pack(r)                              # [T*k, row] in grouped (= destination) order
        true_counts = r.counts.view(N, El).to(torch.int64).cpu()
        counts = true_counts.clone()
        if self.inject_count_mismatch:  # the table this rank announces no longer describes the rows it holds
            counts[0, 0] += 1
        send_split = [int(v) for v in true_counts.sum(1)]
        if form == FORM_SLOTS:
            return self._protocol_slots(x2, r, rows, counts, send_split, cap)
        # ---- exact form: counts first, checked everywhere, verdict agreed before any row moves ----
        msg = torch.zeros((N, El + 2), dtype=torch.int64)
        msg[:, :El] = counts
        msg[:, El], msg[:, El + 1] = EP_MAGIC, r.T
        got = torch.empty_like(msg)
        self._a2a(got.view(-1), msg.view(-1))
        recv_counts = got[:, :El]
        ok = bool((got[:, El] == EP_MAGIC).all()) and bool((got[:, El + 1] <= self.max_tokens).all())
        ok = ok and bool((recv_counts <= got[:, El + 1:El + 2]).all()) and int(counts.sum()) == r.T * k
        n_rows = int(recv_counts.sum())
        limit = self.max_recv_rows or N * cap
        ok = ok and n_rows <= limit
        verdict = torch.tensor([1 if ok else 0], dtype=torch.int64)
        if dist.is_initialized():
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        if int(verdict) == 0:
            raise EpMismatchError("expert-parallel count tables disagree between ranks (or exceed the configured capacity)")
        recv_split = [int(v) for v in recv_counts.sum(1)]
        max_rows = int(recv_counts.sum(0).max()) if n_rows else 0
        recv_rows = ops.empty_rows(n_rows)
        self._a2a(recv_rows, rows, recv_split, send_split)
        out_rows = ops.experts(recv_rows, recv_counts.to(r.counts.dtype), n_rows, max_rows)
        ret_rows = ops.empty_out(r.T * k)
        self._a2a(ret_rows, out_rows, send_split, recv_split)
        self.last_rows, self.last_max_rows = n_rows, max_rows
        return ops.combine(r, ret_rows, x2)

    def _protocol_slots(self, x2, r, rows, counts, send_split, cap) -> torch.Tensor:
        """Fixed-capacity slots with the counts in a header; nothing here depends on a data-dependent size."""
        N, El, k, ops = self.world, self.E_local, self.k, self.ops
        hdr = torch.zeros((N, 4 + El), dtype=torch.int64)
        hdr[:, 0], hdr[:, 1], hdr[:, 2] = EP_MAGIC, r.T, torch.tensor(send_split, dtype=torch.int64)
        hdr[:, 4:] = counts
        slots = rows.new_zeros((N, cap) + tuple(rows.shape[1:]))
        base = np.concatenate([[0], np.cumsum(send_split)])
        for dst in range(N):
            slots[dst, :send_split[dst]] = rows[base[dst]:base[dst + 1]]
        got_hdr, got = torch.empty_like(hdr), torch.empty_like(slots)
        self._a2a(got_hdr.view(-1), hdr.view(-1))
        self._a2a(got.view(N, -1), slots.view(N, -1))
        # the receiver's plan: a header that fails a check counts as an empty slot (the device kernel raises a flag)
        self.bad_slots = []
        cnt = got_hdr[:, 4:].clone()
        for src in range(N):
            h = got_hdr[src]
            good = int(h[0]) == EP_MAGIC and int(h[1]) <= self.max_tokens and int(h[2]) <= cap
            good = good and int(cnt[src].sum()) == int(h[2]) and bool((cnt[src] <= h[1]).all())
            if not good:
                cnt[src] = 0
                self.bad_slots.append(src)
        n_src_rows = [int(v) for v in cnt.sum(1)]
        n_rows = sum(n_src_rows)
        compact = torch.cat([got[src, :n_src_rows[src]] for src in range(N)]) if n_rows else ops.empty_rows(0)
        max_rows = int(cnt.sum(0).max()) if n_rows else 0
        out_rows = ops.experts(compact, cnt.to(r.counts.dtype), n_rows, max_rows)
        back = out_rows.new_zeros((N, cap, self.d_model))
        b2 = np.concatenate([[0], np.cumsum(n_src_rows)])
        for src in range(N):
            back[src, :n_src_rows[src]] = out_rows[b2[src]:b2[src + 1]]
        ret = torch.empty_like(back)
        self._a2a(ret.view(N, -1), back.view(N, -1))
        # where pair (t, rank) finds its result: slot of the owner rank, position inside that rank's rows
        pos = r.pair_pos.to(torch.int64).cpu().numpy()
        owner = np.searchsorted(base[1:], pos, side="right")
        slot_pos = owner * cap + (pos - base[owner])
        r2 = Routed(r.T, r.topk_ids, r.topk_w, r.counts, r.perm_token, torch.from_numpy(slot_pos.astype(np.int32)), r.extra)
        self.last_rows, self.last_max_rows = n_rows, max_rows
        return ops.combine(r2, ret.view(N * cap, self.d_model), x2)
