#!/usr/bin/env python
"""Benchmark of the quantized MoE feed-forward block (candle quantized_llama MlpOrMoe::MoE).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--workload c2|c1|c4|c5|c3|proj]
    python bench.py --impl reference ...      # the CPU restatement of candle's path, same workload

Workload (default, "c2"): a Mixtral-8x7B-shaped layer (d=4096, ff=14336, 8 experts, top-2, w1/w3 Q4_K, w2 Q6_K,
f32 router) at T = 32 decode rows per GPU.  Weights are N(0, 0.02) quantized with the reference's quantizer
arithmetic, activations N(0, 1); everything synthetic.  One "step" is one forward of the block over the T rows.
With N > 1 the experts are sharded over the ranks (expert parallelism, one process per GPU): every rank routes
its own T rows, the packed quantized rows and the expert outputs cross NVLink in two NCCL all-to-alls issued
inside the library (weak scaling: `value` = N T / step time).  "c1" is the CPU-runnable shape, "c4" the
fine-grained Q8_0 layer with a shared expert, "c5" the Mixtral-8x22B-shaped layer with skewed routing, "c3" a
32-layer decode step around the block, "proj" the dense projections.

Timing: W warm-up steps, then batches of exactly K steps, each bracketed by a barrier + synchronize and a pair of
CUDA events; batches repeat until a second of device time has been measured and the MEDIAN batch is reported
(max over ranks).  GPU clocks are sampled with nvidia-smi while those batches run.

Output: ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: d, ff, E, k, dt13, dt2, renorm, ff_shared, default T
    "c1": dict(d=1024, ff=3584, E=8, k=2, dt13=12, dt2=12, renorm=True, ff_shared=0, T=256),
    "c2": dict(d=4096, ff=14336, E=8, k=2, dt13=12, dt2=14, renorm=True, ff_shared=0, T=32),
    "c4": dict(d=2048, ff=1408, E=60, k=4, dt13=8, dt2=8, renorm=False, ff_shared=5632, T=4096),
    "c5": dict(d=6144, ff=16384, E=8, k=2, dt13=12, dt2=14, renorm=True, ff_shared=0, T=8192),
}
BLOCK = {8: (32, 34), 12: (256, 144), 14: (256, 210)}
DT_NAME = {8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}


def mat_bytes(dt, n, k):
    be, bb = BLOCK[dt]
    return n * (k // be) * bb


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peaks():
    """(sustained, burst) dense bf16/fp16 TFLOP/s of this pool's B200s and where the numbers come from."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), float(j["bf16_tflops"]), "measured"
    return 1400.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except (ValueError, IndexError):
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle (C++ restatement of candle's CPU path) on host cores
# --------------------------------------------------------------------------------------------
def cpu_weights(cfg, seed=0):
    """Seeded N(0, 0.02) weights quantized by the oracle's restatement of candle's quantizer;
    matrices are generated on all host threads (one numpy generator per matrix)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as orc
    d, ff, E = cfg["d"], cfg["ff"], cfg["E"]
    jobs = []
    for e in range(E):
        jobs += [(e, "w1", cfg["dt13"], (ff, d)), (e, "w3", cfg["dt13"], (ff, d)), (e, "w2", cfg["dt2"], (d, ff))]
    fs = cfg["ff_shared"]
    if fs:
        jobs += [(E, "sw1", cfg["dt13"], (fs, d)), (E, "sw3", cfg["dt13"], (fs, d)), (E, "sw2", cfg["dt2"], (d, fs))]

    def make(job):
        e, name, dt, shape = job
        rng = np.random.default_rng([seed, e, {"w1": 1, "w3": 3, "w2": 2, "sw1": 4, "sw3": 5, "sw2": 6}[name]])
        return (e, name), rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02), dt

    out = {}
    with ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 1)) as ex:
        for key, w, dt in ex.map(make, jobs):
            out[key] = orc.quantize(dt, w)
    rng = np.random.default_rng([seed, 999])
    router = rng.standard_normal((E, d), dtype=np.float32) * np.float32(0.02)
    bias = None
    if cfg.get("zipf_bias"):
        bias = np.log(1.0 / (np.arange(E) + 1.0)).astype(np.float32)
    mw = orc.MoeWeights(d, ff, cfg["k"], cfg["dt13"], cfg["dt2"], router, [out[(e, "w1")] for e in range(E)],
                        [out[(e, "w3")] for e in range(E)], [out[(e, "w2")] for e in range(E)], renorm=cfg["renorm"],
                        router_bias=bias)
    if fs:
        mw.d_ff_shared, mw.dtype_shared13, mw.dtype_shared2 = fs, cfg["dt13"], cfg["dt2"]
        mw.sw1, mw.sw3, mw.sw2 = out[(E, "sw1")], out[(E, "sw3")], out[(E, "sw2")]
        mw.shared_gate = rng.standard_normal(d, dtype=np.float32) * np.float32(0.02)
    return mw


def use_all_host_threads(orc):
    """OpenMP threads = host cores, whatever OMP_NUM_THREADS says (torch.distributed.run sets it to 1)."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0)) or n
    except (AttributeError, OSError):
        pass
    orc.set_threads(n)
    return orc.max_threads()


def time_oracle(mw, x, steps, warmup):
    from oracle import oracle as orc
    for _ in range(warmup):
        orc.moe_forward(mw, x)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.moe_forward(mw, x)
    return (time.perf_counter() - t0) / max(steps, 1)


def run_reference(args, cfg):
    """`--impl reference`: candle's CPU quantized path, as restated in oracle/ (the reference is Rust
    and no Rust toolchain exists here), on all host threads, same workload, metric and unit."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    orc.build()
    cores = use_all_host_threads(orc)
    T = args.tokens
    # a step is bounded to a sample of the workload's rows so that K steps stay within minutes
    ops_per_row = 2.0 * cfg["k"] * 3 * cfg["d"] * cfg["ff"] + 2.0 * 3 * cfg["d"] * cfg["ff_shared"]
    max_rows = max(1, int(1.0e11 * 1.5 / ops_per_row))  # ~1.5 s per step at ~100 GOP/s
    Ts = min(T, max_rows)
    mw = cpu_weights(cfg)
    x = np.random.default_rng([1, 7]).standard_normal((Ts, cfg["d"]), dtype=np.float32)
    sec = time_oracle(mw, x, args.steps, args.warmup)
    val = Ts / sec
    sample = f"{Ts} of {T} rows per step, all {cfg['E']} experts resident, {cores} OpenMP threads"
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot / f32 accumulate",
        "data": "synthetic", "config": config_dict(args, cfg),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def config_dict(args, cfg):
    return {
        "workload": f"{args.workload}: MoE FFN layer d={cfg['d']} ff={cfg['ff']} E={cfg['E']} top{cfg['k']} "
                    f"w1/w3 {DT_NAME[cfg['dt13']]} w2 {DT_NAME[cfg['dt2']]}"
                    + (f" + shared ff={cfg['ff_shared']}" if cfg["ff_shared"] else "")
                    + f", T={args.tokens} rows per step per GPU",
        "tokens_per_step_per_gpu": args.tokens,
        "l2_policy": "inputs larger than L2: the expert weights streamed each step exceed the 126 MB L2"
        if weights_bytes(cfg) > 200e6 else "L2 flushed between steps by writing a 256 MB buffer",
        "decode_weights": "GGUF blocks" if args.no_prepack else
        "prepacked copies made once at load (candle_moe_prepack; Q4_K +2.8 % bytes, Q6_K same size); "
        "roofline bytes are the GGUF bytes",
        "parallelism": "single GPU" if args.gpus == 1 else
        f"ep{args.gpus}: {cfg['E'] // args.gpus} expert(s) per rank, every rank routes its own {args.tokens} rows; "
        "NCCL all-to-all of the packed quantized rows and of the expert outputs",
    }


def weights_bytes(cfg):
    per = 2 * mat_bytes(cfg["dt13"], cfg["ff"], cfg["d"]) + mat_bytes(cfg["dt2"], cfg["d"], cfg["ff"])
    return per * cfg["E"]


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def build_ep_block(torch, cfg, device, rank, world, prepack=True, max_tokens=None):
    """Expert-parallel block: this rank's E/world experts (expert e is seeded by e, whatever the rank count) and
    the replicated router."""
    from candle_b200 import ExpertParallelMoe, GgmlDType, Mlp, QMatMul, QTensor
    d, ff, E = cfg["d"], cfg["ff"], cfg["E"]
    El = E // world

    def q(g, shape, dt):
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
        return QMatMul(QTensor.quantize(w, GgmlDType(dt)))

    experts = []
    for e in range(rank * El, (rank + 1) * El):
        g = torch.Generator(device=device).manual_seed(1000 + e)
        experts.append(Mlp(q(g, (ff, d), cfg["dt13"]), q(g, (d, ff), cfg["dt2"]), q(g, (ff, d), cfg["dt13"])))
    g = torch.Generator(device=device).manual_seed(999)
    router = torch.randn((E, d), generator=g, device=device, dtype=torch.float32) * 0.02
    bias = torch.log(1.0 / (torch.arange(E, dtype=torch.float32) + 1.0)) if cfg.get("zipf_bias") else None
    return ExpertParallelMoe(cfg["k"], router, experts, norm_topk_prob=cfg["renorm"], router_bias=bias, prepack=prepack,
                             max_tokens=max_tokens)


def build_block(torch, cfg, device, seed=0, prepack=True):
    from candle_b200 import GgmlDType, Mlp, MlpOrMoe, QMatMul, QTensor
    g = torch.Generator(device=device).manual_seed(seed)
    d, ff, E = cfg["d"], cfg["ff"], cfg["E"]

    def q(shape, dt):
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
        return QMatMul(QTensor.quantize(w, GgmlDType(dt)))

    experts = [Mlp(q((ff, d), cfg["dt13"]), q((d, ff), cfg["dt2"]), q((ff, d), cfg["dt13"])) for _ in range(E)]
    router = torch.randn((E, d), generator=g, device=device, dtype=torch.float32) * 0.02
    kw = {}
    if cfg["ff_shared"]:
        fs = cfg["ff_shared"]
        kw["shared_expert"] = Mlp(q((fs, d), cfg["dt13"]), q((d, fs), cfg["dt2"]), q((fs, d), cfg["dt13"]))
        kw["shared_expert_gate"] = torch.randn(d, generator=g, device=device) * 0.02
    if cfg.get("zipf_bias"):
        kw["router_bias"] = torch.log(1.0 / (torch.arange(E, dtype=torch.float32) + 1.0))
    blk = MlpOrMoe.moe(cfg["k"], router, experts, norm_topk_prob=cfg["renorm"], **kw)
    if prepack:
        blk.prepack()
    return blk


def oracle_view(torch, blk, cfg):
    """The same block for the oracle: the device bytes copied to the host."""
    from oracle import oracle as orc
    host = lambda qm: qm.inner.data.cpu().numpy()
    mw = orc.MoeWeights(cfg["d"], cfg["ff"], cfg["k"], cfg["dt13"], cfg["dt2"],
                        blk.feed_forward_gate_inp.cpu().numpy(), [host(m.feed_forward_w1) for m in blk.experts],
                        [host(m.feed_forward_w3) for m in blk.experts], [host(m.feed_forward_w2) for m in blk.experts],
                        renorm=cfg["renorm"],
                        router_bias=None if blk.router_bias is None else blk.router_bias.cpu().numpy())
    if blk.shared_expert is not None:
        s = blk.shared_expert
        mw.d_ff_shared, mw.dtype_shared13, mw.dtype_shared2 = cfg["ff_shared"], cfg["dt13"], cfg["dt2"]
        mw.sw1, mw.sw3, mw.sw2 = host(s.feed_forward_w1), host(s.feed_forward_w3), host(s.feed_forward_w2)
        mw.shared_gate = blk.shared_expert_gate.cpu().numpy()
    return mw


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the dominant kernel, from one
# `ncu --set full` capture of this same command line (the default workload); other workloads: null.
NCU_TRAFFIC_BYTES = {("c2", 32, "gate_up"): 551.5e6, ("c2", 32, "down"): 396.8e6}

MIN_TIMED_SECONDS = 1.0   # batches of K steps repeat until this much device time has been measured
MAX_BATCHES = 400


def time_stages(torch, blk, x, steps):
    """Per-kernel device times of the block: the forward itself with CUDA events recorded on the
    launching stream between its launches (candle_moe_forward_timed), averaged over `steps`."""
    acc = None
    for it in range(steps + 2):
        _, ms = blk.forward_timed(x)
        if it >= 2:
            acc = ms if acc is None else {k: acc[k] + v for k, v in ms.items()}
    _, _, counts, _ = blk.last_routing(x.shape[0])
    return {k: v / steps for k, v in acc.items()}, int((counts > 0).sum())


def timed_batches(torch, step, steps, barrier, flush=None, min_seconds=MIN_TIMED_SECONDS, agree=None):
    """Batches of exactly `steps` steps, each between a barrier + synchronize on both sides and timed with CUDA
    events on the launching stream.  Returns (list of batch milliseconds, wall seconds of the whole region).
    With `flush` every step is timed on its own so that the L2 flush stays outside the timed region.
    `agree(n)`: makes every rank run the same number of batches (the steps may hold collectives)."""
    out = []
    t0 = time.perf_counter()
    n_batches = None
    while True:
        barrier()
        if flush is not None:
            tot = 0.0
            for _ in range(steps):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                torch.cuda.synchronize()
                tot += e0.elapsed_time(e1)
            out.append(tot)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step()
            e1.record()
            barrier()
            out.append(e0.elapsed_time(e1))
        if n_batches is None:
            # after the first batch: how many batches make up the minimum region (at least 3), agreed between ranks
            want = 1 if min_seconds <= 0 else max(3, min(MAX_BATCHES, int(min_seconds * 1e3 / max(out[0], 1e-3)) + 1))
            n_batches = agree(want) if agree else want
        if len(out) >= n_batches:
            break
    barrier()
    return out, time.perf_counter() - t0


def parity_vs_oracle(orc, mw, x_rows, y_rows, ids_rows):
    """GPU rows against the CPU oracle on the same rows: ids exact (near-ties apart), max-rel and rel-L2 of y."""
    ref = orc.moe_forward(mw, x_rows)
    same = (ref.topk_ids == ids_rows).all(axis=1) if ids_rows is not None else np.ones(len(x_rows), bool)
    a, b = y_rows[same].astype(np.float64), ref.y[same].astype(np.float64)
    return {"rows": int(len(x_rows)), "ids_exact": bool(same.all()), "ids_mismatched_rows": int((~same).sum()),
            "rel_l2": float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)),
            "max_rel": float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)),
            "bounds": {"rel_l2": 1e-3, "max_rel": 2e-3}}


def block_launches(cfg, T, prepacked, gemm_min_rows):
    """Kernels one forward of the block launches (the library's own, counted from its launch sequence)."""
    q8 = cfg["dt13"] == 8
    pairs = T * cfg["k"]
    n = 1 + (0 if T == 1 else (3 if pairs > 2048 else 1)) + (1 if q8 else 0)  # router (+ x quantization fused unless Q8_0), dispatch
    maps = lambda E: (2 * E + 15) // 16                                        # tensor-map copies, 16 maps per launch
    gemm = T > gemm_min_rows
    def product(dt, E, takes_gemm):
        if gemm and takes_gemm:
            return 1 + (maps(E) if dt in (12, 8) else 0) + 1                    # operand preparation, maps, GEMM
        return 1
    k13 = cfg["dt13"] == 12 or (prepacked and cfg["dt13"] in (14, 8))
    k2 = cfg["dt2"] == 12 or (prepacked and cfg["dt2"] in (14, 8))
    n += product(cfg["dt13"], cfg["E"], k13) + 1 + product(cfg["dt2"], cfg["E"], k2) + 1  # gate_up, quantize h, down, combine
    if cfg["ff_shared"]:
        sh = prepacked and q8
        n += 1 + (0 if q8 else 1) + product(cfg["dt13"], 1, sh) + 1 + product(cfg["dt2"], 1, sh)  # offsets, (x), gate_up, quantize, down
    return n


def tensor_roofline(cfg, T_rows, ms, what, flops, prepacked=True):
    sus, burst, kind = tensor_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    note = f"{kind} cuBLAS bf16, sustained (burst {burst:.0f})"
    if cfg["dt13"] == 8 and prepacked:
        note += ("; Q8_0 gate_up runs three fp16 MMAs per K step (exact two-part operands), counted once: "
                 "tensor-pipe utilisation is about three times this fraction")
    elif cfg["dt13"] == 8:
        note += "; the Q8_0 products run on int8 tensor-core MMAs (mma.sync), quoted against the measured bf16 figure"
    return {"bound": "tensor", "kernel": what, "achieved": tf, "peak": sus, "unit": "TFLOP/s", "frac": tf / sus,
            "traffic": None, "peak_source": note, "algorithmic_flops_per_launch": flops, "kernel_ms": ms}


def run_ours(args, cfg):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback "
                         "(use --impl reference for the CPU restatement)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        # a rank that falls out of step must end the run with an error, not hang it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    import candle_b200  # noqa: F401  loads libcandle_moe_sm100.so or raises
    if args.gemm_min_rows:
        from candle_b200 import _lib
        _lib.check("candle_moe_set_tuning", _lib.load().candle_moe_set_tuning(_lib.TUNE_GEMM_MIN_ROWS, args.gemm_min_rows))

    T, d = args.tokens, cfg["d"]
    if world > 1:
        return run_ep(args, cfg, torch, dist, rank, world, local, dev)
    if args.ep_local:
        return run_ep_local(args, cfg, torch, dev)
    blk = build_block(torch, cfg, dev, seed=0, prepack=not args.no_prepack)
    blk.reserve(T)
    gx = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn((T, d), generator=gx, device=dev, dtype=torch.float32)
    y = torch.empty_like(x)
    small = weights_bytes(cfg) <= 200e6
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if small else None

    def barrier():
        torch.cuda.synchronize(dev)

    # ---- device-resident timing ----
    for _ in range(args.warmup):
        blk.forward(x, out=y)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    batches, region_s = timed_batches(torch, lambda: blk.forward(x, out=y), args.steps, barrier, flush, args.min_seconds)
    clocks = sampler.stop()
    ms_total = statistics.median(batches)

    # ---- end to end through the public API with host buffers: H2D of x, forward, D2H of y ----
    hx = torch.randn((T, d), dtype=torch.float32).pin_memory()
    hy = torch.empty((T, d), dtype=torch.float32).pin_memory()

    def e2e_step():
        x.copy_(hx, non_blocking=True)
        blk.forward(x, out=y)
        hy.copy_(y, non_blocking=True)

    for _ in range(min(args.warmup, 3)):
        e2e_step()
    e2e_batches, _ = timed_batches(torch, e2e_step, args.steps, barrier, None, min(0.3, args.min_seconds))
    ms_e2e = statistics.median(e2e_batches)

    x.copy_(torch.randn((T, d), generator=torch.Generator().manual_seed(1), dtype=torch.float32))
    stage_ms, active = time_stages(torch, blk, x, max(min(args.steps, 50), 10))
    per_expert13 = 2 * mat_bytes(cfg["dt13"], cfg["ff"], cfg["d"])
    per_expert2 = mat_bytes(cfg["dt2"], cfg["d"], cfg["ff"])
    # algorithmic bytes of the block: active experts' blocks + router + x read + y write
    block_bytes = active * (per_expert13 + per_expert2) + cfg["E"] * d * 4 + 2 * T * d * 4
    if cfg["ff_shared"]:
        block_bytes += 2 * mat_bytes(cfg["dt13"], cfg["ff_shared"], d) + mat_bytes(cfg["dt2"], d, cfg["ff_shared"]) + 4 * d
    block_ops = 2.0 * T * cfg["k"] * 3 * d * cfg["ff"] + 2.0 * T * d * cfg["E"] + 2.0 * T * 3 * d * cfg["ff_shared"]
    peak, peak_kind = peaks()
    top = max(("gate_up", "down"), key=lambda n: stage_ms[n])
    top_bytes = active * (per_expert13 if top == "gate_up" else per_expert2)
    ach = top_bytes / (stage_ms[top] * 1e-3) / 1e9
    ms_step = ms_total / args.steps
    blk_gbs = block_bytes / (ms_step * 1e-3) / 1e9

    # CPU baseline on the same weights (device bytes copied to the host) and the parity of the timed workload
    from oracle import oracle as orc
    orc.build()
    cores = use_all_host_threads(orc)
    mw = oracle_view(torch, blk, cfg)
    ops_per_row = 2.0 * cfg["k"] * 3 * d * cfg["ff"] + 2.0 * 3 * d * cfg["ff_shared"]
    Ts = max(1, min(T, int(1.5e11 / ops_per_row)))
    xh = x[:Ts].cpu().numpy()
    n_cpu = 5 if Ts * ops_per_row < 5e10 else 2
    sec = time_oracle(mw, xh, n_cpu, 1)
    got = blk.forward(x).cpu().numpy()
    ids = blk.last_routing(T)[0].numpy().astype(np.uint32)
    parity = parity_vs_oracle(orc, mw, xh, got[:Ts], ids[:Ts])

    roof = {"bound": "hbm", "kernel": top, "achieved": ach, "peak": peak, "unit": "GB/s",
            "frac": ach / peak, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, T, top)),
            "peak_source": f"{peak_kind} copy bandwidth",
            "algorithmic_bytes_per_launch": top_bytes, "kernel_ms": stage_ms[top]}
    from candle_b200 import _lib as _cm
    gmin = C.c_int64(96)
    _cm.load().candle_moe_get_tuning(_cm.TUNE_GEMM_MIN_ROWS, C.byref(gmin))
    if T > gmin.value:
        # large batches run tensor-core grouped products: the bound is the tensor pipe.  Algorithmic flops of the
        # dominant product (the second multiply of every Q6_K slab is not counted).
        flops = 2.0 * T * cfg["k"] * d * cfg["ff"] * (2 if top == "gate_up" else 1)
        roof = tensor_roofline(cfg, T, stage_ms[top], top, flops, prepacked=not args.no_prepack)
    line = {
        "metric": "moe_layer_tokens_per_s", "value": T * world / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 dot / f32 accumulate", "data": "synthetic", "config": config_dict(args, cfg),
        "roofline": roof,
        "block_roofline": {"bound": "hbm", "algorithmic_bytes": block_bytes, "achieved": blk_gbs,
                           "frac": blk_gbs / peak, "frac_of_nominal_8TBps": blk_gbs / 8000.0,
                           "active_experts": active, "tensor_ops": block_ops,
                           "achieved_tops": block_ops / (ms_step * 1e-3) / 1e12,
                           "frac_of_tensor_peak": block_ops / (ms_step * 1e-3) / 1e12 / tensor_peaks()[0]},
        "stage_ms": stage_ms,
        "timing": {"batches": len(batches), "steps_per_batch": args.steps, "timed_region_s": region_s,
                   "batch_ms_median": ms_total, "batch_ms_min": min(batches), "batch_ms_max": max(batches)},
        "parity": parity,
        "cpu_baseline": {"value": Ts / sec, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{Ts} of {T} rows, same weights and inputs as the GPU step, {n_cpu} timed passes"},
        "e2e": {"value": T * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": T * d * 4, "d2h_bytes_per_step": T * d * 4,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": block_launches(cfg, T, not args.no_prepack, gmin.value) * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))


def ep_oracle_weights(torch, cfg, device):
    """All E experts of the expert-parallel workload rebuilt on one device (expert e is seeded by e alone, whatever
    the rank count) and copied to the host for the oracle."""
    from candle_b200 import GgmlDType, QTensor
    from oracle import oracle as orc
    d, ff, E = cfg["d"], cfg["ff"], cfg["E"]
    w = {"w1": [], "w3": [], "w2": []}
    for e in range(E):
        g = torch.Generator(device=device).manual_seed(1000 + e)
        for name, shape, dt in (("w1", (ff, d), cfg["dt13"]), ("w2", (d, ff), cfg["dt2"]), ("w3", (ff, d), cfg["dt13"])):
            t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
            w[name].append(QTensor.quantize(t, GgmlDType(dt)).data.cpu().numpy())
            del t
    g = torch.Generator(device=device).manual_seed(999)
    router = (torch.randn((E, d), generator=g, device=device, dtype=torch.float32) * 0.02).cpu().numpy()
    bias = np.log(1.0 / (np.arange(E) + 1.0)).astype(np.float32) if cfg.get("zipf_bias") else None
    return orc.MoeWeights(d, ff, cfg["k"], cfg["dt13"], cfg["dt2"], router, w["w1"], w["w3"], w["w2"], renorm=cfg["renorm"],
                          router_bias=bias)


def ep_measure(args, cfg, torch, dist, rank, world, dev, T, steps, warmup, min_seconds, parity_rows, sampler=None):
    """One expert-parallel workload: T rows per rank per step.  Returns the record (rank 0) or None."""
    d = cfg["d"]
    blk = build_ep_block(torch, cfg, dev, rank, world, prepack=not args.no_prepack, max_tokens=T)
    gx = torch.Generator(device=dev).manual_seed(1 + rank)
    x = torch.randn((T, d), generator=gx, device=dev, dtype=torch.float32)
    y = torch.empty_like(x)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize(dev)

    def agree(n):
        t = torch.tensor([n if rank == 0 else 0], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t)

    for _ in range(warmup):
        blk.forward(x, out=y)
    barrier()
    if sampler is not None:
        sampler.start()
    batches, region_s = timed_batches(torch, lambda: blk.forward(x, out=y), steps, barrier, None, min_seconds, agree)
    clocks = sampler.stop() if sampler is not None else None

    hx = torch.randn((T, d), dtype=torch.float32).pin_memory()
    hy = torch.empty((T, d), dtype=torch.float32).pin_memory()

    def e2e_step():
        x.copy_(hx, non_blocking=True)
        blk.forward(x, out=y)
        hy.copy_(y, non_blocking=True)

    for _ in range(3):
        e2e_step()
    e2e_batches, _ = timed_batches(torch, e2e_step, steps, barrier, None, min(0.3, min_seconds), agree)

    # per-phase device times (events between the phases of a step), outside the timed regions above
    x.copy_(torch.randn((T, d), generator=torch.Generator(device=dev).manual_seed(1 + rank), device=dev))
    n_ph = len(blk.PHASES)
    acc = [0.0] * n_ph
    reps = max(min(steps, 20), 3)
    for _ in range(reps):
        _, ms = blk.forward(x, out=y, timed=True)
        for i, n in enumerate(blk.PHASES):
            acc[i] += ms[n] / reps
    form = blk.form()
    t = torch.tensor([statistics.median(batches), statistics.median(e2e_batches)] + acc +
                     [float(blk.last_max_rows), float(blk.last_rows)], dtype=torch.float64, device=dev)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    rows_all = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(rows_all, torch.tensor([blk.last_rows], dtype=torch.int64, device=dev))
    rows_per_rank = [int(v) for v in rows_all]

    # the parity forward is a step like any other: every rank takes part, rank 0 compares its own rows
    yy = blk.forward(x, out=y).cpu().numpy()
    parity = None
    if rank == 0 and parity_rows > 0:
        from oracle import oracle as orc
        orc.build()
        use_all_host_threads(orc)
        mw = ep_oracle_weights(torch, cfg, dev)
        n = min(parity_rows, T)
        parity = parity_vs_oracle(orc, mw, x[:n].cpu().numpy(), yy[:n], None)
        parity["note"] = "rank 0's rows; the oracle holds all experts, rebuilt from their seeds"
        del mw
    blk.close()
    if rank != 0:
        return None
    ms_step = float(tmax[0]) / steps
    ms_e2e = float(tmax[1]) / steps
    phase_ms = {n: float(tmax[2 + i]) for i, n in enumerate(blk.PHASES)}
    rows_expert_max, rows_max = int(tmax[-2]), int(tmax[-1])
    El = cfg["E"] // world
    per13, per2 = 2 * mat_bytes(cfg["dt13"], cfg["ff"], d), mat_bytes(cfg["dt2"], d, cfg["ff"])
    ex_ms = phase_ms["experts"]
    if rows_expert_max > 64:  # tensor-core form
        roof = tensor_roofline(cfg, rows_max, ex_ms, "local experts (gate_up + down) on the busiest rank",
                               2.0 * rows_max * 3 * d * cfg["ff"])
    else:
        peak, peak_kind = peaks()
        byts = El * (per13 + per2)
        gbs = byts / (ex_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "local experts (gate_up + down)", "achieved": gbs, "peak": peak,
                "unit": "GB/s", "frac": gbs / peak, "traffic": None, "peak_source": f"{peak_kind} copy bandwidth",
                "algorithmic_bytes_per_launch": byts, "kernel_ms": ex_ms}
    row_b = d + d // 8 + d // 64
    mean_rows = sum(rows_per_rank) / world
    return {
        "value": T * world / (ms_step * 1e-3), "unit": "tokens/s", "ms_per_step": ms_step,
        "tokens_per_step_per_gpu": T, "form": {1: "slots (no host synchronisation)", 2: "exact (counts checked on the host)"}[form],
        "roofline": roof, "stage_ms": phase_ms,
        "timing": {"batches": len(batches), "steps_per_batch": steps, "timed_region_s": region_s,
                   "batch_ms_median": float(tmax[0])},
        "exchange": {"rows_sent_per_rank": T * cfg["k"], "row_bytes_forward": row_b, "row_bytes_back": 4 * d,
                     "rows_received_per_rank": rows_per_rank, "busiest_over_mean": max(rows_per_rank) / max(mean_rows, 1e-9),
                     "rows_of_busiest_expert": rows_expert_max},
        "parity": parity,
        "e2e": {"value": T * world / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * d * 4,
                "d2h_bytes_per_step": T * d * 4, "ms_per_step": ms_e2e},
        "clocks": clocks,
    }


def run_ep_local(args, cfg, torch, dev):
    """`--ep-local`: the expert-parallel step on ONE GPU (world size 1: both exchanges are device copies), so that
    its pack / plan / regroup / scatter kernels can be timed and profiled without a second GPU.  `--ep-form` picks the
    slot form (1) or the exact form (2)."""
    T, d = args.tokens, cfg["d"]
    blk = build_ep_block(torch, cfg, dev, 0, 1, prepack=not args.no_prepack, max_tokens=T)
    blk.force_form = args.ep_form
    x = torch.randn((T, d), generator=torch.Generator(device=dev).manual_seed(1), device=dev, dtype=torch.float32)
    y = torch.empty_like(x)
    for _ in range(args.warmup):
        blk.forward(x, out=y)
    torch.cuda.synchronize()
    batches, region_s = timed_batches(torch, lambda: blk.forward(x, out=y), args.steps, torch.cuda.synchronize, None, min(0.3, args.min_seconds))
    acc = {n: 0.0 for n in blk.PHASES}
    for _ in range(5):
        _, ms = blk.forward(x, out=y, timed=True)
        for n in acc:
            acc[n] += ms[n] / 5
    ms_step = statistics.median(batches) / args.steps
    print(json.dumps({"metric": "moe_layer_tokens_per_s", "value": T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                      "data": "synthetic", "config": dict(config_dict(args, cfg), parallelism="expert-parallel step on one GPU "
                                                          "(exchanges are device copies)", form=blk.form()),
                      "stage_ms": acc, "rows_received": blk.last_rows}))


def run_ep(args, cfg, torch, dist, rank, world, local, dev):
    """N > 1: expert parallelism.  Every rank holds E / N experts and routes its own T rows per step."""
    if cfg["E"] % world or cfg["dt13"] == 8 or cfg["ff_shared"]:
        raise SystemExit(f"workload {args.workload} has no expert-parallel form over {world} ranks")
    T = args.tokens
    sampler = ClockSampler(local) if rank == 0 else None
    rec = ep_measure(args, cfg, torch, dist, rank, world, dev, T, args.steps, args.warmup, args.min_seconds,
                     parity_rows=min(T, 64), sampler=sampler)
    c5 = None
    if args.workload == "c2" and not args.no_c5:
        # the Mixtral-8x22B-shaped layer with skewed routing, 8192 rows per step split over the ranks
        cfg5 = dict(WORKLOADS["c5"], zipf_bias=True)
        torch.cuda.empty_cache()
        c5 = ep_measure(args, cfg5, torch, dist, rank, world, dev, 8192 // world, 5, 3, 0.2, parity_rows=64)
    if rank == 0:
        line = {
            "metric": "moe_layer_tokens_per_s", "value": rec["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 dot / f32 accumulate", "data": "synthetic", "config": config_dict(args, cfg),
            "roofline": rec["roofline"], "stage_ms": rec["stage_ms"], "timing": rec["timing"], "form": rec["form"],
            "exchange": rec["exchange"], "parity": rec["parity"], "e2e": rec["e2e"],
            "gpu_launches": 10 * args.steps, "clocks": rec["clocks"],
        }
        if c5 is not None:
            c5["workload"] = (f"c5: MoE FFN layer d=6144 ff=16384 E=8 top2 w1/w3 Q4_K w2 Q6_K, router bias log(1/(i+1)), "
                              f"8192 rows per step = {8192 // world} per GPU over {world} GPUs")
            line["c5"] = c5
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


PROJECTIONS = {
    # the dense matrices of the model the block sits in (quantized_llama.rs:275-277, 345, 897), Mixtral-8x7B shapes
    "attn_q": (4096, 4096, 12), "attn_k": (1024, 4096, 12), "attn_output": (4096, 4096, 12), "output": (32000, 4096, 14),
}


def run_projections(args):
    """`--workload proj`: QMatMul::forward of each dense projection at --tokens rows (default 1), device-timed,
    weights rotated over copies that together exceed L2.  One JSON line; not the headline metric."""
    import torch
    from candle_b200 import GgmlDType, QMatMul, QTensor
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    T = args.tokens or 1
    hbm, src = peaks()
    rows = {}
    g = torch.Generator(device=dev).manual_seed(0)
    for name, (n, k, dt) in PROJECTIONS.items():
        nbytes = mat_bytes(dt, n, k)
        copies = max(2, -(-400_000_000 // nbytes))
        w = torch.randn((n, k), generator=g, device=dev) * 0.02
        base = QTensor.quantize(w, GgmlDType(dt))
        mats = []
        for _ in range(copies):
            m = QMatMul.from_qtensor(QTensor(base.data.clone(), GgmlDType(dt), (n, k)))
            if not args.no_prepack:
                m.prepack()
            mats.append(m)
        x = torch.randn((T, k), generator=g, device=dev)
        for i in range(max(args.warmup, 3, copies)):  # every copy once: its scratch is allocated on first use
            mats[i % copies].forward(x)
        torch.cuda.synchronize()
        # the calls of the timed region are replayed from one CUDA graph, so that the figure is the device's time
        # and not the host's launch rate (a call is four short launches)
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(args.steps):
                    mats[i % copies].forward(x)
            graph.replay()
        except Exception as exc:  # noqa: BLE001
            print(f"# graph capture failed ({exc}); timing eager calls", file=sys.stderr)
            graph = None
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(args.steps):
                mats[i % copies].forward(x)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        gbs = nbytes / (us * 1e-6) / 1e9
        rows[name] = {"n": n, "k": k, "dtype": DT_NAME[dt], "us": round(us, 2), "weight_GBps": round(gbs, 1),
                      "frac_of_hbm_peak": round(gbs / hbm, 3), "TFLOPs": round(2.0 * T * n * k / (us * 1e-6) / 1e12, 2), "timed": "graph" if graph is not None else "eager"}
        del mats, graph
    print(json.dumps({"metric": "qmatmul_us", "unit": "us per call (quantize rows + product)", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "tokens": T, "data": "synthetic", "peak_GBps": hbm, "peak_source": src,
                      "config": {"workload": "dense projections of a Mixtral-8x7B layer + lm head", "l2": "weights rotated over > 400 MB of copies",
                                 "prepacked": not args.no_prepack}, "projections": rows}))


def run_c3(args):
    """`--workload c3`: one decode step of a 32-layer Mixtral-8x7B-shaped model at batch 32 with a 4096-token context
    (candle_b200/llama_decode.py: quantized products and the FFN half of every layer through this library, attention
    and the other glue as stock PyTorch ops).  tokens/s = batch / step time."""
    import torch
    import torch.distributed as dist
    from candle_b200.llama_decode import DecodeConfig, DecodeStep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    import candle_b200  # noqa: F401
    cfg = DecodeConfig()
    if args.layers:
        cfg.n_layer = args.layers
    B = args.tokens or 32
    ctx = min(args.context, cfg.max_seq)
    index_pos = ctx - 1
    ep = None
    if world > 1:
        from candle_b200 import ExpertParallelMoe
        ep = {"world": world, "rank": rank,
              "make": lambda lw: ExpertParallelMoe(cfg.n_expert_used, lw.router, lw.experts, prepack=not args.no_prepack,
                                                   max_tokens=B)}
    model = DecodeStep(cfg, B, dev, n_distinct=4, seed=0, prepack=not args.no_prepack, expert_parallel=ep,
                       attention=args.attention)
    tokens = torch.randint(0, cfg.vocab, (B,), generator=torch.Generator(device=dev).manual_seed(5 + rank), device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def agree(n):
        if world == 1:
            return n
        t = torch.tensor([n if rank == 0 else 0], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t)

    logits = model.forward(tokens, index_pos)  # also allocates every scratch buffer
    for _ in range(max(args.warmup, 3) - 1):
        logits = model.forward(tokens, index_pos)
    barrier()
    # the step replays from one CUDA graph where that is possible (single GPU): the host then adds nothing
    graph = None
    step = lambda: model.forward(tokens, index_pos)
    if world == 1 and not args.eager:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                g_logits = model.forward(tokens, index_pos)
            graph.replay()
            torch.cuda.synchronize()
            step = graph.replay
        except Exception as exc:  # noqa: BLE001
            print(f"# graph capture failed ({type(exc).__name__}: {exc}); timing eager steps", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    batches, region_s = timed_batches(torch, step, args.steps, barrier, None, args.min_seconds, agree)
    clocks = sampler.stop() if sampler else None
    ms_step = statistics.median(batches) / args.steps

    # shares: the same layers' attention halves alone and FFN halves alone (eager, events around each loop)
    x = torch.randn((B, cfg.d_model), device=dev)
    def loop_ms(fn, reps=3):
        best = []
        for _ in range(reps):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for li in range(cfg.n_layer):
                fn(li)
            e1.record()
            barrier()
            best.append(e0.elapsed_time(e1))
        return min(best)
    ms_attn = loop_ms(lambda li: model.attention(li, x, index_pos))
    ms_ffn = loop_ms(lambda li: model.ffn(li, x))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(5):
        model.output.forward(x)
    e1.record()
    barrier()
    ms_head = e0.elapsed_time(e1) / 5

    # end to end: token ids from pinned host memory, logits back to pinned host memory
    h_tok = tokens.cpu().pin_memory()
    h_logits = torch.empty((B, cfg.vocab), dtype=torch.float32).pin_memory()
    src = g_logits if graph is not None else None

    def e2e_step():
        tokens.copy_(h_tok, non_blocking=True)
        if graph is not None:
            graph.replay()
            h_logits.copy_(src, non_blocking=True)
        else:
            h_logits.copy_(model.forward(tokens, index_pos), non_blocking=True)

    e2e_batches, _ = timed_batches(torch, e2e_step, args.steps, barrier, None, min(0.3, args.min_seconds), agree)
    ms_e2e = statistics.median(e2e_batches) / args.steps
    t = torch.tensor([ms_step, ms_e2e, ms_attn, ms_ffn], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, ms_e2e, ms_attn, ms_ffn = (float(v) for v in t)
    if rank == 0:
        byts = model.bytes_per_step(index_pos)
        if world > 1:
            byts["moe_weights"] //= world
        total = sum(byts.values())
        peak, peak_kind = peaks()
        line = {
            "metric": "decode_tokens_per_s", "value": B * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 dot / f32 accumulate (quantized products), f32 (attention)",
            "data": "synthetic",
            "config": {"workload": f"c3: {cfg.n_layer}-layer Mixtral-8x7B-shaped decode step, batch {B} per GPU, context {ctx}, "
                                   f"d={cfg.d_model} heads {cfg.n_head}/{cfg.n_kv_head} x {cfg.head_dim}, {cfg.n_expert} experts "
                                   f"top-{cfg.n_expert_used} ff={cfg.d_ff}, vocab {cfg.vocab}",
                       "weights": "4 distinct random layers rotate over the layers (attention Q4_K, w1/w3 Q4_K, w2 Q6_K, lm head Q6_K)",
                       "library_parts": "wq/wk/wv/wo, lm head (candle_moe_qmatmul); ffn_norm + MoE block + residual (candle_moe_ffn_layer"
                                        + (", experts sharded: candle_moe_ep_forward)" if world > 1 else ")")
                                        + ("; attention_norm, rotary embedding + cache append, attention over the f32 KV cache (candle_moe_rmsnorm, "
                                           "candle_moe_rope_kv_append, candle_moe_decode_attention)" if args.attention == "library" else ""),
                       "pytorch_parts": "embedding, final norm, residual add of the attention half"
                                        + ("" if args.attention == "library" else ", attention_norm, interleaved RoPE, f32 KV cache append, "
                                           "attention (q k^T, softmax, v as batched f32 matmuls)"),
                       "l2_policy": "a step reads tens of GB: nothing survives in the 126 MB L2 between steps",
                       "timed": "CUDA graph replay" if graph is not None else "eager launches",
                       "parallelism": "single GPU" if world == 1 else f"ep{world}: experts sharded, attention replicated, "
                                      f"every rank decodes its own {B} sequences"},
            "roofline": {"bound": "hbm", "kernel": "whole decode step", "achieved": total / (ms_step * 1e-3) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": total / (ms_step * 1e-3) / 1e9 / peak, "traffic": None,
                         "peak_source": f"{peak_kind} copy bandwidth", "algorithmic_bytes_per_launch": total,
                         "bytes": byts, "ms_at_peak": total / (peak * 1e9) * 1e3},
            "shares": {"attention_half_ms": ms_attn, "ffn_half_ms": ms_ffn, "lm_head_ms": ms_head,
                       "ffn_share_of_step": ms_ffn / ms_step,
                       "note": "halves timed alone over all layers with eager launches; the step itself may replay from a graph"},
            "timing": {"batches": len(batches), "steps_per_batch": args.steps, "timed_region_s": region_s},
            "cpu_baseline": None,
            "e2e": {"value": B * world / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * 8,
                    "d2h_bytes_per_step": B * cfg.vocab * 4, "ms_per_step": ms_e2e},
            "gpu_launches": cfg.n_layer * (1 + 6 + 1 + 2 + 6 + 7) * args.steps,
            "finite": bool(torch.isfinite(logits).all()),
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["proj", "c3"])
    ap.add_argument("--layers", type=int, default=0, help="c3: number of layers (default 32)")
    ap.add_argument("--context", type=int, default=4096, help="c3: tokens in the context, the new one included")
    ap.add_argument("--eager", action="store_true", help="c3: time eager launches instead of a CUDA graph replay")
    ap.add_argument("--attention", default="library", choices=["library", "pytorch"],
                    help="c3: attention over the KV cache by this library's kernel or by PyTorch's batched matmuls")
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="device time the timed batches must add up to (0: a single batch, for profiler runs)")
    ap.add_argument("--gemm-min-rows", type=int, default=0,
                    help="bound on an expert's rows above which the tensor-core GEMM runs (default: the library's)")
    ap.add_argument("--ep-local", action="store_true", help="N = 1: run the expert-parallel step on one GPU (profiling aid)")
    ap.add_argument("--ep-form", type=int, default=0, choices=[0, 1, 2], help="--ep-local: 1 = slot form, 2 = exact form")
    ap.add_argument("--no-c5", action="store_true",
                    help="N > 1: skip the Mixtral-8x22B-shaped sub-record that accompanies the default workload")
    ap.add_argument("--no-prepack", action="store_true",
                    help="decode straight from the GGUF blocks instead of the one-time prepacked copies")
    args = ap.parse_args()
    if args.workload == "proj":
        return run_projections(args)
    if args.workload == "c3":
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the CPU restatement covers the MoE block, not attention: "
                                                                      "no CPU arm for the whole decode step"}))
            return
        return run_c3(args)
    cfg = dict(WORKLOADS[args.workload])
    if args.workload == "c5":
        cfg["zipf_bias"] = True
    if args.tokens is None:
        args.tokens = cfg["T"]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
