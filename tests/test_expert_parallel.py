"""Expert parallelism.

CPU part (world size 2, gloo): `ExpertParallelMoe(..., ops=...)` runs the exchange protocol of
candle_moe_ep_forward in Python with the oracle standing in for the device steps, so what is tested is the
protocol -- both forms (fixed-capacity slots with in-band counts; exact sizes after a checked count exchange),
their index arithmetic, and their failure handling: a count table that does not describe the rows is rejected on
EVERY rank before any row moves; a rank that leaves between steps ends the others' next step with an error
inside the process group's timeout.  Every rank's result must equal the oracle's single-process block on that
rank's tokens bit for bit.

GPU part: the C ABI path (`candle_moe_ep_forward`, NCCL inside the library).  One GPU: world size 1 (both forms,
the exchanges are device copies), replay from a CUDA graph, the local phase of a rank that holds one expert, a slot
header that fails its check (dropped on the device, reported through the health word), a bounded wait that runs out.
Two or more GPUs (skipped when the box has one): child processes, one per GPU, compare every rank's output with
the oracle, exercise the rejected count table and the replay of the slot form from a CUDA graph.  A rank that leaves
between steps is a CPU (gloo) test only: the library's raw NCCL communicator has no watchdog, so the GPUs of the
remaining ranks would wait without limit.
"""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import helpers as H


class OracleOps:
    """The device steps of ExpertParallelMoe computed on the CPU by the oracle (f32 rows travel)."""

    def __init__(self, orc, mw, rank, world):
        self.orc, self.mw = orc, mw
        self.d, self.k, self.E = mw.d_model, mw.top_k, mw.n_experts
        self.El = self.E // world
        self.lo = rank * self.El
        self.expert_calls = 0

    def route(self, x):
        from candle_b200.expert_parallel import Routed
        xn = x.numpy()
        T = xn.shape[0]
        _, ids, tw = self.orc.router_topk(xn, self.mw.router, self.k, self.mw.renorm, self.mw.router_bias)
        ids = np.asarray(ids).astype(np.int64).reshape(T, self.k)
        flat = ids.reshape(-1)
        order = np.argsort(flat, kind="stable")            # by expert, tokens ascending inside an expert
        perm_token = (order // self.k).astype(np.int32)
        pair_pos = np.empty(T * self.k, dtype=np.int32)
        pair_pos[order] = np.arange(T * self.k, dtype=np.int32)
        counts = np.bincount(flat, minlength=self.E).astype(np.int32)
        return Routed(T, torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(np.asarray(tw, np.float32).reshape(T, self.k)),
                      torch.from_numpy(counts), torch.from_numpy(perm_token), torch.from_numpy(pair_pos), xn)

    def pack(self, r):
        return torch.from_numpy(r.extra[r.perm_token.numpy()].copy())

    def empty_rows(self, n):
        return torch.empty((n, self.d), dtype=torch.float32)

    empty_out = empty_rows

    def experts(self, recv_rows, recv_counts, n_rows, max_rows):
        self.expert_calls += 1
        rows, cnt = recv_rows.numpy(), recv_counts.numpy()
        assert cnt.sum() == n_rows and (n_rows == 0 or cnt.sum(0).max() <= max_rows)
        out = np.zeros((n_rows, self.d), dtype=np.float32)
        base = np.concatenate([[0], np.cumsum(cnt.reshape(-1))])  # arrival order: source-major, expert-minor
        for e in range(self.El):
            idx = np.concatenate([np.arange(base[s * self.El + e], base[s * self.El + e + 1]) for s in range(cnt.shape[0])])
            if len(idx) == 0:
                continue
            g = self.lo + e
            o, _ = self.orc.mlp_forward(self.mw.dtype_w13, self.mw.dtype_w2, rows[idx], self.mw.w1[g], self.mw.w3[g],
                                        self.mw.w2[g], self.mw.d_ff)
            out[idx] = o
        return torch.from_numpy(out)

    def combine(self, r, ret_rows, x):
        ret, ids, tw, pos = ret_rows.numpy(), r.topk_ids.numpy(), r.topk_w.numpy(), r.pair_pos.numpy().reshape(r.T, self.k)
        y = np.zeros((r.T, self.d), dtype=np.float32)
        for t in range(r.T):
            for j in np.argsort(ids[t], kind="stable"):  # ascending expert id, product rounded before the add
                y[t] = y[t] + np.float32(tw[t, j]) * ret[pos[t, j]]
        return torch.from_numpy(y)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _paths():
    here = os.path.dirname(os.path.abspath(__file__))
    for p in (here, os.path.dirname(here)):
        if p not in sys.path:
            sys.path.insert(0, p)


def _cpu_weights(orc):
    return orc.make_moe_weights(3, 256, 512, 8, 2, orc.Q4K, orc.Q6K,
                                router_bias=np.log(1.0 / (np.arange(8) + 1)).astype(np.float32))  # skewed load


def _cpu_rank(rank, world, port, tokens, form, fail):
    try:
        _paths()
        from oracle import oracle as orc
        from candle_b200.expert_parallel import ExpertParallelMoe
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        mw = _cpu_weights(orc)
        x = orc.make_activations(100 + rank, tokens[rank], 256)
        blk = ExpertParallelMoe(2, torch.from_numpy(mw.router), [], ops=OracleOps(orc, mw, rank, world), force_form=form)
        y = blk.forward(torch.from_numpy(x)).numpy()
        assert blk.form() == form and blk.max_tokens == max(max(tokens), 1)
        ref = orc.moe_forward(mw, x)
        assert np.array_equal(y, ref.y), f"rank {rank}: max diff {np.abs(y - ref.y).max()}"
        # a second step with other sizes reuses the object (within the agreed bound)
        T2 = min(5 + 3 * rank, blk.max_tokens)
        x2 = orc.make_activations(200 + rank, T2, 256)
        assert np.array_equal(blk.forward(torch.from_numpy(x2)).numpy(), orc.moe_forward(mw, x2).y)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        fail.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


def _run_ranks(target, world, args, timeout=240):
    ctx = mp.get_context("spawn")
    fail = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port) + tuple(args) + (fail,)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    msgs = []
    while not fail.empty():
        msgs.append(fail.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            msgs.append("a rank did not finish")
    return msgs, [p.exitcode for p in procs]


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("tokens", [(37, 12), (1, 0)])
def test_exchange_protocol_two_ranks_gloo(tokens, form):
    msgs, codes = _run_ranks(_cpu_rank, 2, (tokens, form))
    assert not msgs and all(c == 0 for c in codes), msgs


def _cpu_rank_bad_table(rank, world, port, form, fail):
    """Rank 1 announces a count table that does not describe its rows."""
    try:
        _paths()
        from oracle import oracle as orc
        from candle_b200.expert_parallel import EpMismatchError, ExpertParallelMoe
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        mw = _cpu_weights(orc)
        ops = OracleOps(orc, mw, rank, world)
        blk = ExpertParallelMoe(2, torch.from_numpy(mw.router), [], ops=ops, force_form=form, max_tokens=16)
        x = orc.make_activations(300 + rank, 9 + rank, 256)
        blk.inject_count_mismatch = rank == 1
        if form == 2:
            # exact form: every rank -- also the one whose own tables are fine -- refuses, before any device step
            with pytest.raises(EpMismatchError):
                blk.forward(torch.from_numpy(x))
            assert ops.expert_calls == 0
        else:
            # slot form: the receiver of the bad slot (rank 0 owns the corrupted entry) drops that slot and says so
            blk.forward(torch.from_numpy(x))
            assert blk.bad_slots == ([1] if rank == 0 else [])
        # the group is still usable: the next step, with honest tables, is right again
        blk.inject_count_mismatch = False
        y = blk.forward(torch.from_numpy(x)).numpy()
        assert np.array_equal(y, orc.moe_forward(mw, x).y)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        fail.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


@pytest.mark.parametrize("form", [1, 2])
def test_count_table_that_disagrees_is_rejected_on_every_rank_gloo(form):
    msgs, codes = _run_ranks(_cpu_rank_bad_table, 2, (form,))
    assert not msgs and all(c == 0 for c in codes), msgs


def _cpu_rank_leaves(rank, world, port, fail):
    """Rank 1 leaves after the first step; rank 0's next step must end with an error, not hang."""
    try:
        import datetime
        import time
        _paths()
        from oracle import oracle as orc
        from candle_b200.expert_parallel import ExpertParallelMoe
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=10))
        mw = _cpu_weights(orc)
        blk = ExpertParallelMoe(2, torch.from_numpy(mw.router), [], ops=OracleOps(orc, mw, rank, world), max_tokens=8)
        x = torch.from_numpy(orc.make_activations(400 + rank, 6, 256))
        blk.forward(x)
        if rank == 1:
            os._exit(0)  # gone between steps, nothing in flight; no clean-up, like a process that died
        t0 = time.time()
        try:
            blk.forward(x)
        except Exception as e:  # noqa: BLE001  (gloo reports a closed connection or its timeout as RuntimeError)
            assert time.time() - t0 < 60, "the error took longer than the timeout allows"
            os._exit(0)  # the group is broken: skip its destructors, which may wait for the peer
        raise AssertionError("the step after a rank left did not fail")
    except Exception as e:  # noqa: BLE001
        fail.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


def test_rank_that_leaves_between_steps_ends_the_others_gloo():
    msgs, codes = _run_ranks(_cpu_rank_leaves, 2, (), timeout=120)
    assert not msgs and all(c == 0 for c in codes), msgs


def test_constructor_refuses_q8_0_experts():
    """The travelling row is a Q8K row: Q8_0 experts (activations quantized per 32) have no expert-parallel form."""
    from candle_b200.expert_parallel import CudaOps

    class FakeCw:
        dtype_w13, dtype_w2 = 8, 8

    class FakeBlock:
        _cw, d_model, device = FakeCw(), 256, "cpu"

    with pytest.raises(ValueError, match="k-quant"):
        CudaOps(8, 2, torch.zeros(8, 256), None, True, FakeBlock())


def test_form_rule_matches_the_sizes():
    from candle_b200.expert_parallel import FORM_EXACT, FORM_SLOTS, choose_form
    assert choose_form(8, 32, 2, 1, 4096) == (FORM_SLOTS, 32)       # decode over 8 ranks: 8 x 32 rows x 16 KB back
    assert choose_form(2, 32, 2, 4, 4096) == (FORM_SLOTS, 64)
    assert choose_form(2, 4096, 2, 4, 6144)[0] == FORM_EXACT         # prefill-sized steps
    assert choose_form(2, 4096, 2, 4, 6144, force_form=1)[0] == FORM_SLOTS


# ------------------------------------------------------------------------------------------------
# one GPU
# ------------------------------------------------------------------------------------------------
def _device_block_and_ep(orc, torch, mw, prepack, **kw):
    from candle_b200 import ExpertParallelMoe
    blk = H.device_block(orc, mw)
    if prepack:
        blk.prepack()
    ep = ExpertParallelMoe(mw.top_k, blk.feed_forward_gate_inp, blk.experts, norm_topk_prob=mw.renorm, prepack=prepack, **kw)
    return blk, ep


@pytest.mark.gpu
@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("T,prepack", [(1, True), (19, False), (19, True), (96, True), (110, True), (300, True)])
def test_single_rank_equals_the_single_device_block(orc, torch_cuda, T, prepack, form):
    torch = torch_cuda
    mw = orc.make_moe_weights(21, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    x = orc.make_activations(40 + T, T, 512)
    blk, ep = _device_block_and_ep(orc, torch, mw, prepack, force_form=form)
    xd = torch.from_numpy(x).cuda()
    y_ep, ms = ep.forward(xd, timed=True)
    assert ep.form() == form and ep.last_rows == T * 2
    y_ep = y_ep.cpu().numpy()
    y_one = blk.forward(xd).cpu().numpy()
    ref = orc.moe_forward(mw, x)
    assert H.rel_l2(y_ep, ref.y) <= H.REL_L2_TOL and H.max_rel(y_ep, ref.y) <= H.MAX_REL_TOL
    # the same quantized rows reach the same weights; the two paths may pick different kernel forms for a given
    # row count (the local phase knows the rows per expert, the single-device block only the bound T), which
    # changes f32 summation order and flips a few re-quantized hidden values by one step
    assert H.rel_l2(y_ep, y_one) < 3e-4
    assert np.array_equal(ep.forward(xd).cpu().numpy(), y_ep)  # untimed call, and determinism
    v = C.c_int32(-1)
    from candle_b200 import _lib
    assert _lib.load().candle_moe_device_status(C.byref(v)) == 0 and v.value == 0


@pytest.mark.gpu
def test_single_rank_steps_of_different_sizes_and_no_rows(orc, torch_cuda):
    torch = torch_cuda
    mw = orc.make_moe_weights(22, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk, ep = _device_block_and_ep(orc, torch, mw, True, max_tokens=64)
    for T in (64, 3, 0, 17):
        x = orc.make_activations(77 + T, T, 512)
        y = ep.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        if T:
            ref = orc.moe_forward(mw, x)
            assert H.rel_l2(y, ref.y) <= H.REL_L2_TOL and H.max_rel(y, ref.y) <= H.MAX_REL_TOL
    with pytest.raises(ValueError, match="at most 64"):
        ep.forward(torch.zeros((65, 512), device="cuda"))


@pytest.mark.gpu
def test_slot_form_replays_from_a_cuda_graph(orc, torch_cuda):
    """No host synchronisation and no data-dependent size in the slot form: a captured step replays over new inputs."""
    torch = torch_cuda
    mw = orc.make_moe_weights(24, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk, ep = _device_block_and_ep(orc, torch, mw, True, force_form=1, max_tokens=40)
    x = torch.from_numpy(orc.make_activations(5, 40, 512)).cuda()
    ep.forward(x)
    torch.cuda.synchronize()
    y = torch.zeros_like(x)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ep.forward(x, out=y)
    for seed in (6, 7):
        xn = orc.make_activations(seed, 40, 512)
        x.copy_(torch.from_numpy(xn))
        graph.replay()
        torch.cuda.synchronize()
        ref = orc.moe_forward(mw, xn)
        assert H.rel_l2(y.cpu().numpy(), ref.y) <= H.REL_L2_TOL and H.max_rel(y.cpu().numpy(), ref.y) <= H.MAX_REL_TOL
        assert torch.equal(y, ep.forward(x))


@pytest.mark.gpu
def test_slot_header_that_fails_its_check_is_dropped_and_reported(orc, torch_cuda):
    """The receiving side checks every slot header on the device; a bad one counts as an empty slot (nothing is indexed
    with numbers that cannot be trusted) and raises bit 2 of the health word.  The next, honest step is right again."""
    torch = torch_cuda
    from candle_b200 import _lib
    L = _lib.load()
    mw = orc.make_moe_weights(25, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk, ep = _device_block_and_ep(orc, torch, mw, True, force_form=1, max_tokens=16)
    xn = orc.make_activations(8, 16, 512)
    x = torch.from_numpy(xn).cuda()
    assert L.candle_moe_device_status_reset() == 0
    ep.inject_count_mismatch = True
    ep.forward(x)
    v = C.c_int32(-1)
    assert L.candle_moe_device_status(C.byref(v)) == 0 and v.value == 4
    assert ep.forward(x, timed=True) is not None and ep.last_rows == 0   # the rows of the bad slot were not processed
    assert L.candle_moe_device_status_reset() == 0
    ep.inject_count_mismatch = False
    y = ep.forward(x).cpu().numpy()
    ref = orc.moe_forward(mw, xn)
    assert H.rel_l2(y, ref.y) <= H.REL_L2_TOL
    assert L.candle_moe_device_status(C.byref(v)) == 0 and v.value == 0


@pytest.mark.gpu
def test_rank_holding_fewer_experts_than_top_k(orc, torch_cuda):
    """8 experts over 8 ranks with top-2: every rank holds ONE expert.  The local phase of one such rank runs on a
    single GPU through the step-by-step entry points; the rows come from eight made-up sources."""
    torch = torch_cuda
    from candle_b200 import MlpOrMoe
    from candle_b200.expert_parallel import CudaOps
    mw = orc.make_moe_weights(23, 512, 1024, 8, 2, orc.Q4K, orc.Q6K)
    blk = H.device_block(orc, mw)
    rank = 5
    local = MlpOrMoe(1, blk.feed_forward_gate_inp[rank:rank + 1].contiguous(), [blk.experts[rank]]).prepack()
    ops = CudaOps(8, 2, blk.feed_forward_gate_inp, None, True, local)
    # rows "received" from 8 sources: quantize + pack them here, as a sender would
    counts = [3, 0, 7, 1, 0, 12, 5, 2]
    n = sum(counts)
    x = orc.make_activations(9, n, 512)
    xd = torch.from_numpy(x).cuda()
    r = ops.route(xd)  # only its quantized rows are used
    r.perm_token = torch.arange(n, dtype=torch.int32, device="cuda")
    r.T, ops_k = n, ops.k
    ops.k = 1
    send = ops.pack(r)
    ops.k = ops_k
    recv_counts = torch.tensor(counts, dtype=torch.int32, device="cuda").reshape(8, 1)
    out = ops.experts(send, recv_counts, n, n).cpu().numpy()
    ref, _ = orc.mlp_forward(mw.dtype_w13, mw.dtype_w2, x, mw.w1[rank], mw.w3[rank], mw.w2[rank], mw.d_ff)
    assert H.rel_l2(out, ref) <= H.REL_L2_TOL and H.max_rel(out, ref) <= H.MAX_REL_TOL


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_reports(torch_cuda):
    """A wait that nothing ever satisfies: the kernel gives up after its poll limit, raises bit 0 of the health word
    and returns; the context stays usable."""
    torch = torch_cuda
    from candle_b200 import _lib
    L = _lib.load()
    assert L.candle_moe_device_status_reset() == 0
    v = C.c_int32(-1)
    assert L.candle_moe_device_status(C.byref(v)) == 0 and v.value == 0
    assert L.candle_moe_selftest_bounded_wait(torch.cuda.current_stream().cuda_stream, 2000) == 0
    assert L.candle_moe_device_status(C.byref(v)) == 0 and v.value == 1
    assert L.candle_moe_device_status_reset() == 0
    assert L.candle_moe_device_status(C.byref(v)) == 0 and v.value == 0
    assert float(torch.ones(8, device="cuda").sum()) == 8.0  # the device still answers


# ------------------------------------------------------------------------------------------------
# two or more GPUs: one child process per GPU, NCCL inside the library
# ------------------------------------------------------------------------------------------------
def _gpu_rank(rank, world, port, mode, fail):
    try:
        import datetime
        _paths()
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        from oracle import oracle as orc
        from candle_b200 import ExpertParallelMoe, _lib
        from candle_b200.expert_parallel import EpMismatchError
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=20))
        mw = orc.make_moe_weights(21, 512, 1024, 8, 2, orc.Q4K, orc.Q6K,
                                  router_bias=np.log(1.0 / (np.arange(8) + 1)).astype(np.float32))
        blk = H.device_block(orc, mw, device=f"cuda:{rank}")
        El = 8 // world
        mine = blk.experts[rank * El:(rank + 1) * El]
        if mode == "parity":
            for form, tokens in ((1, 24), (2, 24), (2, 700), (1, 1)):
                ep = ExpertParallelMoe(2, blk.feed_forward_gate_inp, mine, prepack=True, force_form=form,
                                       router_bias=torch.from_numpy(mw.router_bias))
                T = tokens + 3 * rank if tokens > 1 else (1 if rank == 0 else 0)
                x = orc.make_activations(500 + 10 * form + rank, T, 512)
                y = ep.forward(torch.from_numpy(x).cuda()).cpu().numpy()
                if T:
                    ref = orc.moe_forward(mw, x)
                    assert H.rel_l2(y, ref.y) <= H.REL_L2_TOL and H.max_rel(y, ref.y) <= H.MAX_REL_TOL, (form, tokens)
                v = C.c_int32(-1)
                assert _lib.load().candle_moe_device_status(C.byref(v)) == 0 and v.value == 0
                ep.close()
        elif mode == "bad_table":
            ep = ExpertParallelMoe(2, blk.feed_forward_gate_inp, mine, prepack=True, force_form=2, max_tokens=32,
                                   router_bias=torch.from_numpy(mw.router_bias))
            x = torch.from_numpy(orc.make_activations(600 + rank, 20, 512)).cuda()
            ep.inject_count_mismatch = rank == world - 1
            with pytest.raises(EpMismatchError):
                ep.forward(x)
            ep.inject_count_mismatch = False
            y = ep.forward(x).cpu().numpy()
            ref = orc.moe_forward(mw, x.cpu().numpy())
            assert H.rel_l2(y, ref.y) <= H.REL_L2_TOL
            ep.close()
        elif mode == "graph":
            # the slot form is a fixed sequence of launches and NCCL calls: it replays from a CUDA graph
            ep = ExpertParallelMoe(2, blk.feed_forward_gate_inp, mine, prepack=True, force_form=1, max_tokens=32,
                                   router_bias=torch.from_numpy(mw.router_bias))
            x = torch.from_numpy(orc.make_activations(700 + rank, 32 - rank, 512)).cuda()
            y_eager = ep.forward(x).clone()          # also makes the communicator, the workspace and NCCL's connections
            ep.forward(x)
            torch.cuda.synchronize()
            y_graph = torch.zeros_like(x)
            ok, graph = 1, torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    ep.forward(x, out=y_graph)
            except Exception as exc:  # noqa: BLE001
                ok, why = 0, f"{type(exc).__name__}: {exc}"
            # every rank must have captured before any rank replays (a replay holds collectives)
            flag = torch.tensor([ok], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            assert int(flag) == 1, "capture failed on a rank" + (": " + why if not ok else "")
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y_graph, y_eager)
            ref = orc.moe_forward(mw, x.cpu().numpy())
            assert H.rel_l2(y_graph.cpu().numpy(), ref.y) <= H.REL_L2_TOL
            del graph
            ep.close()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # noqa: BLE001
        fail.put(f"rank {rank}: {type(e).__name__}: {e}")
        raise


def _gpu_world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return 4 if n >= 4 else (2 if n >= 2 else 0)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["parity", "bad_table", "graph"])
def test_multi_gpu_ranks_match_the_oracle(orc, torch_cuda, mode):
    world = _gpu_world()
    if world == 0:
        pytest.skip("needs two or more GPUs")
    msgs, codes = _run_ranks(_gpu_rank, world, (mode,), timeout=300)
    assert not msgs and all(c == 0 for c in codes), msgs
