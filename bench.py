#!/usr/bin/env python
"""Benchmark of the weight-quantised matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline line (one JSON object on stdout, printed by rank 0): tokens/s of the
Q4 SwiGLU MLP block of BASELINE.json configs[4] (hidden 4096, intermediate
14336, M = 256 tokens per step), tensor parallel over N GPUs (gate/up sharded by
hidden unit, down by the same rows; the ranks' f32 partials are summed, rounded and
added to the residual stream by one kernel of this library over NVLink peer memory,
or with `--collective nccl` by an NCCL all-reduce and a finishing pass).  A step
is one Mlp::accumulate pass over one synthetic batch.  Total work is fixed as N
grows ("strong" scaling).  Between steps the weights rotate over enough distinct
device copies to exceed twice the L2, so every step streams its weights from HBM.

`--impl reference` times the CPU oracle (the C restatement of the reference's
portable scalar path; the reference itself is Rust and cannot be built here) on
the host cores with the same metric, on a bounded row sample of the same batch.

`value` is device time (CUDA events, max over ranks) with the inputs resident in
HBM.  `e2e` is the same step through the same public call with host buffers: every
step copies its tokens from pinned host memory and its result back to pinned host
memory inside the timed region, the copies running on their own streams with two
buffers each way so that they overlap the neighbouring steps' compute (at N > 1 every rank
copies the tokens in and returns its 1 / N of the rows of the replicated result, so the N
ranks together return all of it; the byte counts in the line are the totals).  `roofline`
is the gate/up projection's GEMM timed alone against the measured tensor peak.

The extra "kernels" list reports the single-kernel configs of BASELINE.json
(Q4 / 2-bit / 1-bit decode GEMV in GB/s, Q4 prefill GEMM in TFLOP/s) measured on
rank 0 at N = 1 (`--no-kernels` skips it).  `--profile-case NAME` runs six plain
launches of one kernel and exits, for profiler captures; `--tokens M` changes the
batch (BASELINE.json also names M = 1).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, BLOCK = 4096, 14336, 32
L2_BYTES = 126 * 1024 * 1024


GATE_UP_DRAM_BYTES_M256 = 71.28e6   # dram__bytes_read.sum + dram__bytes_write.sum, one launch


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                clk, cmax, power = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            mx.append(cmax)
            if power < 250.0:        # idle sample (before / after the loaded section)
                continue
            sm.append(clk)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- synthetic weights

def mlp_weights_f32(seed: int):
    """W_gate, W_up [INTER][HIDDEN], W_down [HIDDEN][INTER] ~ N(0, 0.02), f32 (seeded)."""
    rng = np.random.default_rng(seed)
    wg = (rng.standard_normal((INTER, HIDDEN), dtype=np.float32) * np.float32(0.02))
    wu = (rng.standard_normal((INTER, HIDDEN), dtype=np.float32) * np.float32(0.02))
    wd = (rng.standard_normal((HIDDEN, INTER), dtype=np.float32) * np.float32(0.02))
    return wg, wu, wd


# --------------------------------------------------------------------------- reference arm (CPU oracle)

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as orc
    cores = orc.max_threads()
    orc.set_threads(cores)
    m = args.m
    rows = max(1, min(m, args.ref_rows))
    rng = np.random.default_rng(1)
    # synthetic codes / scales with the value distribution of quantised N(0, 0.02) weights
    wg, wu, wd = mlp_weights_f32(5)
    import sme_gemm_b200 as sg
    both = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, INTER, HIDDEN)
    guq, gus, _ = orc.q4_quantize(both, 1, 2 * INTER, HIDDEN)
    dq, ds, _ = orc.q4_quantize(wd, 0, HIDDEN, INTER)
    del wg, wu, wd, both
    x = rng.standard_normal((m, HIDDEN)).astype(np.float16)
    y = np.zeros((m, HIDDEN), np.float32)

    def step():
        orc.mlp_accumulate(x, y, m, HIDDEN, INTER, guq, gus, dq, ds, BLOCK, 3, 0, rows)

    def step_one():
        orc.mlp_accumulate(x, y, m, HIDDEN, INTER, guq, gus, dq, ds, BLOCK, 3, 0, 1)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    # one row per call is nearly all dequant: the per-call dequant of both weight sets and the per-row cost follow from
    # the two timings, and a whole batch costs the dequant once plus m rows
    t0 = time.perf_counter()
    for _ in range(max(1, args.steps // 2)):
        step_one()
    dt1 = (time.perf_counter() - t0) / max(1, args.steps // 2)
    per_row = max((dt - dt1) / max(rows - 1, 1), 1e-9) if rows > 1 else dt
    t_dequant = max(dt1 - per_row, 0.0) if rows > 1 else 0.0
    value = m / (t_dequant + per_row * m)
    value_no_dequant = 1.0 / per_row
    sample = (f"{rows} of {m} rows per step through the whole block, and 1 row per step to separate the per-call dequant of both "
              f"weight sets ({t_dequant * 1e3:.1f} ms) from the per-row cost ({per_row * 1e3:.2f} ms): tokens/s = m / (dequant + m * per_row); "
              f"with the dequant excluded {value_no_dequant:.1f} tokens/s")
    dt_batch = (t_dequant + per_row * m)
    line = {"impl": "reference", "metric": "q4_mlp_block_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args, None),
            "ms_per_batch_projected": dt_batch * 1e3,
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
                             "value_dequant_excluded": value_no_dequant},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, sets):
    return {"workload": f"Q4 SwiGLU MLP block (BASELINE.json configs[4]): hidden {HIDDEN}, intermediate {INTER}, Q4_0 block {BLOCK}, "
                        f"M={args.m} tokens per step, f16 activations, f32 residual",
            "tokens_per_step": args.m, "parallelism": f"tp{args.gpus}",
            **({"collective": "sum + f16 rounding + residual add in one kernel of this library over NVLink peer memory"
                if getattr(args, "collective", "peer") == "peer" else "NCCL all-reduce + finishing pass"} if args.gpus > 1 else {}),
            "l2": "weights rotate over enough distinct device copies per rank to exceed twice the L2 between steps"}


# --------------------------------------------------------------------------- our arm

def graph_time_us(torch, fn, n_items, reps=20):
    """Average device time of fn(i), i over n_items rotating inputs, measured by
    replaying a CUDA graph of one pass (removes host launch overhead)."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(n_items):
            fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(n_items):
            fn(i)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * n_items)


def kernel_cases(torch, sg, orc):
    """BASELINE.json configs[0..3] as single device-resident kernel calls.  Each entry builds
    lazily and returns (fn(i), number of rotating weight sets, description dict)."""
    rng = np.random.default_rng(7)
    k = 4096

    def sets_for(bytes_per_set):
        return max(2, int(np.ceil(2.2 * L2_BYTES / bytes_per_set)))

    def q4_gemv():
        n = 4096
        w = (rng.standard_normal(n * k) * 0.02).astype(np.float32)
        q, s, _ = orc_quant(sg, w, 0, n, k)
        ws = [sg.Q4Weights.new(q, s, n, k) for _ in range(sets_for(9.4e6))]
        a = torch.randn(1, k, device="cuda", dtype=torch.float16)
        c = torch.zeros(1, n, device="cuda", dtype=torch.float16)
        return (lambda i: sg.matmul_q4(a, ws[i], c, 1)), len(ws), {"config": "q4_gemv_1x4096x4096", "bytes": 9453568}

    def q2_gemv():
        n = 11008
        two = rng.integers(0, 3, k * n).astype(np.uint8)
        codes = (two[0::4] | (two[1::4] << 2) | (two[2::4] << 4) | (two[3::4] << 6)).astype(np.uint8)
        sc = rng.uniform(0.01, 0.05, n * (k // 256)).astype(np.float16).view(np.uint16)
        ws = [sg.Q2Weights.new(codes, sc, n, k) for _ in range(sets_for(11.6e6))]
        a = torch.randn(1, k, device="cuda", dtype=torch.float16)
        c = torch.zeros(1, n, device="cuda", dtype=torch.float16)
        return (lambda i: sg.matmul_q2(a, ws[i], c, 1)), len(ws), {"config": "q2_ternary_gemv_1x4096x11008", "bytes": 11654656}

    def q1_gemv():
        n = 14336
        signs = rng.integers(0, 256, k * n // 8).astype(np.uint8)
        sc = rng.uniform(0.005, 0.03, n * (k // 128)).astype(np.float16).view(np.uint16)
        ws = [sg.Q1Weights.new(signs, sc, sg.WeightLayout.OutIn, n, k, 128) for _ in range(sets_for(8.6e6))]
        a8 = torch.randn(8, k, device="cuda", dtype=torch.float16)
        c8 = torch.zeros(8, n, device="cuda", dtype=torch.float16)
        sv = torch.empty(n, device="cuda", dtype=torch.float16).uniform_(0.5, 1.5)
        bv = torch.randn(n, device="cuda", dtype=torch.float16) * 0.1
        ep = sg.Epilogue().mul_col(sv).add_col(bv)
        return (lambda i: sg.matmul_q1_ep(a8, ws[i], c8, 8, ep)), len(ws), {"config": "q1_gemv_8x4096x14336_mulcol_addcol", "bytes": 8609792}

    def q4_prefill():
        n = 14336
        w = (rng.standard_normal(n * k) * 0.02).astype(np.float32)
        q, s, _ = orc_quant(sg, w, 0, n, k)
        ws = [sg.Q4Weights.new(q, s, n, k) for _ in range(sets_for(33e6))]
        ab = torch.randn(512, k, device="cuda", dtype=torch.bfloat16)
        cb = torch.zeros(512, n, device="cuda", dtype=torch.bfloat16)
        bias = (torch.randn(n, device="cuda") * 0.1).to(torch.bfloat16)
        ep4 = sg.Epilogue("bf16").add_col(bias).silu().clamp(-6.0, 6.0)
        return ((lambda i: sg.matmul_q4_bf16_ep(ab, ws[i], cb, 512, ep4)), len(ws),
                {"config": "q4_prefill_gemm_bf16_512x4096x14336_addcol_silu_clamp", "flops": 2.0 * 512 * k * n})

    def q1_prefill():
        # the int8-activation path at prompt size: 1-bit weights, 512 rows (exact int32 block sums on the f16 tensor-core
        # path, ordered f32 fold); operations = 2 m n k, against the measured f16/bf16 tensor peak
        n = 14336
        signs = rng.integers(0, 256, k * n // 8).astype(np.uint8)
        sc = rng.uniform(0.005, 0.03, n * (k // 128)).astype(np.float16).view(np.uint16)
        ws = [sg.Q1Weights.new(signs, sc, sg.WeightLayout.OutIn, n, k, 128) for _ in range(4)]
        a = torch.randn(512, k, device="cuda", dtype=torch.float16)
        c = torch.zeros(512, n, device="cuda", dtype=torch.float16)
        return ((lambda i: sg.matmul_q1(a, ws[i], c, 512)), len(ws),
                {"config": "q1_int8act_prefill_512x4096x14336", "flops": 2.0 * 512 * k * n,
                 "note": "activation int8 quantisation pass included; 4 weight sets of 7.3 MB rotate (tokens and output exceed the L2 share)"})

    return {"q4_gemv": q4_gemv, "q2_gemv": q2_gemv, "q1_gemv": q1_gemv, "q4_prefill": q4_prefill, "q1_prefill": q1_prefill}


def kernel_configs(torch, sg, orc, peaks):
    """The single-kernel configs on one GPU, timed by CUDA-graph replay."""
    out = []
    for name, build in kernel_cases(torch, sg, orc).items():
        fn, nsets, d = build()
        us = graph_time_us(torch, fn, nsets, reps=10 if "flops" in d else 20)
        if "bytes" in d:
            gbs = d["bytes"] / us / 1e3
            out.append({"config": d["config"], "us": us, "value": gbs, "unit": "GB/s", "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                        "frac_of_nominal_8000": gbs / 8000.0, "algorithmic_bytes": d["bytes"]})
        else:
            tf = d["flops"] / us / 1e6
            out.append({"config": d["config"], "us": us, "value": tf, "unit": "TFLOP/s",
                        "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"], "frac_of_nominal_2250": tf / 2250.0,
                        "algorithmic_flops": d["flops"], **({"note": d["note"]} if "note" in d else {})})
        del fn
    return out


def run_profile_case(args):
    """A few plain launches of one kernel, for a profiler to capture (`--profile-case NAME`):
    three untimed launches, then three more.  Prints no benchmark number."""
    import torch
    import oracle as orc          # input generation only
    import sme_gemm_b200 as sg
    torch.cuda.set_device(0)
    name = args.profile_case
    if name in ("mlp_gate_up", "mlp_down"):
        m = args.m
        wg, wu, wd = mlp_weights_f32(5)
        if name == "mlp_gate_up":
            both = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, INTER, HIDDEN)
            q, s, _ = orc_quant(sg, both, 1, 2 * INTER, HIDDEN)
            n, k = 2 * INTER, HIDDEN
        else:
            q, s, _ = orc_quant(sg, wd, 0, HIDDEN, INTER)
            n, k = HIDDEN, INTER
        ws = [sg.Q4Weights.new(q, s, n, k) for _ in range(3)]
        a = torch.randn(m, k, device="cuda", dtype=torch.float16)
        c = torch.zeros(m, n, device="cuda", dtype=torch.float16)
        fn, nsets = (lambda i: sg.matmul_q4(a, ws[i], c, m)), 3
    else:
        fn, nsets, _ = kernel_cases(torch, sg, orc)[name]()
    for i in range(6):
        fn(i % nsets)
    torch.cuda.synchronize()
    if sg.last_status() != 0:
        raise SystemExit("a kernel abandoned a bounded wait")
    print(json.dumps({"profile_case": name, "launches": 6}), flush=True)


def run_ours(args):
    import torch
    import oracle as orc          # checker / CPU baseline only
    import sme_gemm_b200 as sg

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert world == args.gpus or world == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    peaks = measured_peaks()
    m = args.m

    # ---- weights: this rank's shard, quantised once, uploaded as several distinct copies ----
    from sme_gemm_b200.tp import TpMlp, shard_bounds
    wg, wu, wd = mlp_weights_f32(5)
    lo, hi = shard_bounds(INTER, rank, world)
    fl = hi - lo
    both = sg.interleave_gate_up(wg[lo:hi], wu[lo:hi], sg.WeightLayout.OutIn, fl, HIDDEN)
    guq, gus, _ = orc_quant(sg, both, 1, 2 * fl, HIDDEN)
    dq, ds, _ = orc_quant(sg, np.ascontiguousarray(wd[:, lo:hi]), 0, HIDDEN, fl)
    del wg, wu, wd, both
    bytes_per_set = (2 * fl * HIDDEN + HIDDEN * fl) * 0.5625
    nsets = max(2, int(np.ceil(2.2 * L2_BYTES / bytes_per_set)))
    mlps = []
    for _ in range(nsets):
        up = sg.GatedLinear(sg.Linear(sg.Q4Weights.new(guq, gus, 2 * fl, HIDDEN)), sg.Gate.Silu)
        down = sg.Linear(sg.Q4Weights.new(dq, ds, HIDDEN, fl))
        mlps.append(sg.Mlp.gated(up, down))

    gen = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(m, HIDDEN, device="cuda", dtype=torch.float16, generator=gen)
    y = torch.zeros(m, HIDDEN, device="cuda", dtype=torch.float32)
    partial = torch.zeros(m, HIDDEN, device="cuda", dtype=torch.float32)
    # N > 1: the ranks' partials are summed, rounded and added to the residual stream by one kernel of this
    # library over peer memory (--collective peer, the default), or by an NCCL all-reduce plus the finishing pass
    peer = None
    if world > 1 and args.collective == "peer":
        from sme_gemm_b200.tp import PeerReduce
        try:
            peer = PeerReduce(m, HIDDEN)
        except Exception as e:           # no peer mapping on this box: say so and time the NCCL form
            print(f"rank {rank}: peer memory unavailable ({type(e).__name__}: {e})", file=sys.stderr, flush=True)
            peer = None
        agreed = torch.tensor([1 if peer is not None else 0], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            peer = None
            args.collective = "nccl"
    x_host = x.cpu().pin_memory()
    y_host = torch.zeros(m, HIDDEN, dtype=torch.float32).pin_memory()

    tps = [TpMlp(mm, world, None, peer) for mm in mlps] if (world > 1 and peer is not None) else None

    def step(i, xb=None, yb=None):
        mlp = mlps[i % nsets]
        xb = x if xb is None else xb
        yb = y if yb is None else yb
        if world == 1:
            mlp.accumulate(xb, yb, m)
        else:
            if peer is not None:
                tps[i % nsets].accumulate(xb, yb, m)   # pushes the partial rows to their owners when it can
            else:
                mlp.partial(xb, partial, m)
                dist.all_reduce(partial)
                sg.Mlp.finish(yb, partial)

    def sync():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, tail=None):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # device time of the steps: a short spin kernel ahead of the first event gives the host a head start, so that the
        # interval between the events is the steps' own device time and not the host's launch pace
        torch.cuda._sleep(2_000_000)
        e0.record()
        for i in range(steps):
            fn(i)
        if tail:
            tail()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if dist:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # the timed region is milliseconds long while nvidia-smi samples every 100 ms: sample from
    # before the warm-up until after the end-to-end region and keep the samples taken under load
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()

    def preload(seconds):
        """The same steps for about `seconds`, so that the clock samples are taken under load.
        Every rank runs the same number of steps (rank 0's estimate), as the steps hold collectives."""
        for i in range(4):
            step(i)
        sync()
        t0 = time.perf_counter()
        for i in range(8):
            step(i)
        sync()
        per = max((time.perf_counter() - t0) / 8, 1e-6)
        count = torch.tensor([int(min(20000, max(8, seconds / per)))], device="cuda", dtype=torch.int64)
        if dist:
            dist.broadcast(count, 0)
        for i in range(int(count.item())):
            step(i)
        sync()

    preload(1.0)
    for i in range(args.warmup):
        step(i)
    ms = timed(step, args.steps)
    value = m * args.steps / (ms * 1e-3)

    # ---- end to end: host buffers in and out every step ----
    # Every step copies its input from pinned host memory and its result back to pinned host memory.  The copies
    # run on their own streams with two device buffers each way, so step i+1's input travels while step i computes
    # and step i's result travels while step i+1 computes (two residual streams y take alternate steps).
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    xs, ys = [x, x.clone()], [y, torch.zeros_like(y)]
    yh = [y_host, torch.zeros(m, HIDDEN, dtype=torch.float32).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for e in ev_done + ev_out:
        e.record(cur)

    row_lo, row_hi = rank * m // world, (rank + 1) * m // world

    def e2e_step(i):
        b = i & 1
        s_in.wait_event(ev_done[b])                 # the step two back has finished reading xs[b]
        with torch.cuda.stream(s_in):
            xs[b].copy_(x_host, non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        cur.wait_event(ev_out[b])                   # ys[b]'s previous read-back is complete before it changes
        step(i, xs[b], ys[b])
        ev_done[b].record(cur)
        # y is replicated: every rank returns its 1 / N of the rows to its pinned host buffer, together they return all of it
        s_out.wait_event(ev_done[b])
        with torch.cuda.stream(s_out):
            yh[b][row_lo:row_hi].copy_(ys[b][row_lo:row_hi], non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_tail():
        cur.wait_stream(s_out)                      # the last result has reached the host inside the timed region
        cur.wait_stream(s_in)

    for i in range(4):
        e2e_step(i)
    ms_e2e = timed(e2e_step, args.steps, e2e_tail)
    e2e_value = m * args.steps / (ms_e2e * 1e-3)
    preload(0.5)
    clocks = sampler.stop() if sampler else None

    status = sg.last_status()
    if status != 0:
        raise SystemExit(f"a kernel abandoned a bounded wait (status {status}); numbers are void")

    # ---- N > 1: the tensor-parallel result itself, outside every timed region ----
    tp_check = None
    exchange_us = None
    if world > 1:
        yz = torch.zeros_like(y)
        step(0, x, yz)
        sync()
        # every rank must hold the same bits
        mine = yz.view(torch.int32).to(torch.int64)
        chk = torch.stack([mine.sum(), (mine * (torch.arange(mine.numel(), device="cuda").view_as(mine) % 1021 + 1)).sum()])
        lo_c, hi_c = chk.clone(), chk.clone()
        dist.all_reduce(lo_c, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_c, op=dist.ReduceOp.MAX)
        same = bool(torch.equal(lo_c, hi_c))
        max_rel = None
        if rank == 0:
            # sampled rows against the CPU oracle of the unsharded block (checker only)
            wg_, wu_, wd_ = mlp_weights_f32(5)
            bothf_ = sg.interleave_gate_up(wg_, wu_, sg.WeightLayout.OutIn, INTER, HIDDEN)
            cq, cs, _ = orc.q4_quantize(bothf_, 1, 2 * INTER, HIDDEN)
            cdq, cds, _ = orc.q4_quantize(wd_, 0, HIDDEN, INTER)
            del wg_, wu_, wd_, bothf_
            rows_chk = sorted({0, m // 2, m - 1})
            xs_ = x_host.numpy()[rows_chk]
            want = np.zeros((len(rows_chk), HIDDEN), np.float32)
            orc.set_threads(orc.max_threads())
            orc.mlp_accumulate(xs_, want, len(rows_chk), HIDDEN, INTER, cq, cs, cdq, cds, BLOCK, 3, 0, len(rows_chk))
            got = yz[rows_chk].cpu().numpy()
            max_rel = float(np.max(np.abs(got - want) / (1.0 + np.abs(want))))
        tp_check = {"ranks_bit_identical": same, "max_rel_vs_oracle": max_rel, "rows_checked": 3, "bar": 1e-2}
        ok_flag = torch.tensor([1 if (same and (max_rel is None or max_rel <= 1e-2)) else 0], device="cuda")
        dist.all_reduce(ok_flag, op=dist.ReduceOp.MIN)
        if int(ok_flag.item()) == 0:
            if rank == 0:
                print(json.dumps({"tp_check": tp_check, "error": "tensor-parallel result failed its check"}), flush=True)
            raise SystemExit(3)
        if peer is not None:
            # the exchange alone: sum + rounding + residual add over peer memory, partial buffers as they stand
            def only_finish(i):
                peer.finish(y, pushed=peer.push)
            for i in range(5):
                only_finish(i)
            exchange_us = timed(only_finish, 20) * 1e3 / 20

    # ---- the rank's two projections alone (CUDA-graph replay over the rotating weight copies) ----
    hid_buf = torch.randn(m, fl, device="cuda", dtype=torch.float16) * 0.1
    out_buf = torch.zeros(m, HIDDEN, device="cuda", dtype=torch.float16)
    dn = [mm.down.q4 for mm in mlps]
    us_down = graph_time_us(torch, lambda i: sg.matmul_q4(hid_buf, dn[i], out_buf, m), nsets, reps=10)
    us_down_t = torch.tensor([us_down], device="cuda")
    if dist:
        dist.all_reduce(us_down_t, op=dist.ReduceOp.MAX)
    us_down = float(us_down_t.item())

    # ---- the same block at M = 1 (the decode half of BASELINE.json configs[4]) ----
    m1 = None
    if m != 1 and not args.no_m1:
        x1 = x[:1].contiguous()
        y1 = torch.zeros(1, HIDDEN, device="cuda", dtype=torch.float32)
        part1 = torch.zeros(1, HIDDEN, device="cuda", dtype=torch.float32)
        peer1 = None
        if world > 1 and peer is not None:
            from sme_gemm_b200.tp import PeerReduce
            peer1 = PeerReduce(1, HIDDEN)
        x1_host = x1.cpu().pin_memory()
        y1_host = torch.zeros(1, HIDDEN, dtype=torch.float32).pin_memory()

        def step1(i):
            mlp = mlps[i % nsets]
            if world == 1:
                mlp.accumulate(x1, y1, 1)
            elif peer1 is not None:
                mlp.partial(x1, peer1.partial, 1)
                peer1.finish(y1)
            else:
                mlp.partial(x1, part1, 1)
                dist.all_reduce(part1)
                sg.Mlp.finish(y1, part1)

        def e2e_step1(i):
            x1.copy_(x1_host, non_blocking=True)
            step1(i)
            if rank == 0:
                y1_host.copy_(y1, non_blocking=True)

        for i in range(10):
            step1(i)
        n1 = 200
        ms1 = timed(step1, n1)
        for i in range(5):
            e2e_step1(i)
        ms1_e2e = timed(e2e_step1, n1)
        m1 = {"tokens_per_step": 1, "steps": n1, "ms_per_step": ms1 / n1, "value": n1 / (ms1 * 1e-3), "unit": "tokens/s",
              "e2e": {"value": n1 / (ms1_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms1_e2e / n1,
                      "h2d_bytes_per_step": HIDDEN * 2, "d2h_bytes_per_step": HIDDEN * 4}}
        if rank == 0:
            gu1 = [mm.up.inner.q4 for mm in mlps]
            both1 = torch.zeros(1, 2 * fl, device="cuda", dtype=torch.float16)
            us1 = graph_time_us(torch, lambda i: sg.matmul_q4(x1, gu1[i], both1, 1), nsets, reps=10)
            bytes1 = HIDDEN * 2 * fl * 0.5625 + HIDDEN * 2 + 2 * fl * 2
            m1["roofline"] = {"kernel": "gate/up projection at one row (this rank's shard)", "bound": "hbm", "achieved": bytes1 / us1 / 1e3,
                              "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": bytes1 / us1 / 1e3 / peaks["hbm_gbs"],
                              "us_per_launch": us1, "algorithmic_bytes": bytes1, "traffic": None}
        sync()

    # ---- the same step through the host-pointer C ABI (what a drop-in caller of the reference's FFI hits) ----
    e2e_abi = None
    if world == 1 and rank == 0:
        xh, yh_abi = x_host.numpy(), np.zeros((m, HIDDEN), np.float32)
        for i in range(3):
            mlps[i % nsets].accumulate(xh, yh_abi, m)
        t0 = time.perf_counter()
        for i in range(args.steps):
            mlps[i % nsets].accumulate(xh, yh_abi, m)
        dt_abi = (time.perf_counter() - t0) / args.steps
        e2e_abi = {"value": m / dt_abi, "unit": "tokens/s", "ms_per_step": dt_abi * 1e3,
                   "call": "smeg_mlp_accumulate (host pointers, pageable numpy buffers, wall clock around the blocking call)"}

    if rank != 0:
        if dist:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel: the gate/up projection (tensor bound), timed alone ----
    both_out = torch.zeros(m, 2 * fl, device="cuda", dtype=torch.float16)
    gu = [mm.up.inner.q4 for mm in mlps]
    us_gu = graph_time_us(torch, lambda i: sg.matmul_q4(x, gu[i], both_out, m), nsets, reps=10)
    flops_gu = 2.0 * m * HIDDEN * 2 * fl
    ach = flops_gu / us_gu / 1e6
    # DRAM bytes per launch: read + written bytes of one profiler capture of this kernel on the whole matrix at M = 256
    # (a constant of that capture, not measured by this run); a rank's shard moves its share of the columns
    traffic = GATE_UP_DRAM_BYTES_M256 / world if m == 256 else None
    roofline = {"kernel": "gemm_tc_kernel (gate/up projection, this rank's shard)", "bound": "tensor", "achieved": ach,
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                "peak_source": peaks["source"] + " (burst: kernel timed alone)", "us_per_launch": us_gu, "traffic": traffic,
                "algorithmic_flops": flops_gu}
    if m <= 16:
        # decode-sized steps run the gate/up projection on the decode kernels, which stream the packed weights
        # once: codes + one f16 scale per 32-deep block and column, the activations and the output, each once
        bytes_gu = HIDDEN * 2 * fl * 0.5625 + m * HIDDEN * 2 + m * 2 * fl * 2
        gbs = bytes_gu / us_gu / 1e3
        roofline = {"kernel": "q4_gemv_stream_kernel / q4_gemv_kernel (gate/up projection, this rank's shard)", "bound": "hbm",
                    "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                    "peak_source": peaks["source"], "us_per_launch": us_gu, "traffic": None, "algorithmic_bytes": bytes_gu}

    # ---- CPU baseline beside it: the oracle block on a bounded row sample, all host cores ----
    cores = orc.max_threads()
    orc.set_threads(cores)
    rows = max(1, min(m, args.ref_rows))
    wg, wu, wd = mlp_weights_f32(5)
    bothf = sg.interleave_gate_up(wg, wu, sg.WeightLayout.OutIn, INTER, HIDDEN)
    fguq, fgus, _ = orc.q4_quantize(bothf, 1, 2 * INTER, HIDDEN)
    fdq, fds, _ = orc.q4_quantize(wd, 0, HIDDEN, INTER)
    del wg, wu, wd, bothf
    xs = x_host.numpy()
    yc = np.zeros((m, HIDDEN), np.float32)
    orc.mlp_accumulate(xs, yc, m, HIDDEN, INTER, fguq, fgus, fdq, fds, BLOCK, 3, 0, 1)   # warm
    t0 = time.perf_counter()
    orc.mlp_accumulate(xs, yc, m, HIDDEN, INTER, fguq, fgus, fdq, fds, BLOCK, 3, 0, 1)
    cpu_dt1 = time.perf_counter() - t0
    t0 = time.perf_counter()
    orc.mlp_accumulate(xs, yc, m, HIDDEN, INTER, fguq, fgus, fdq, fds, BLOCK, 3, 0, rows)
    cpu_dt = time.perf_counter() - t0
    per_row = max((cpu_dt - cpu_dt1) / max(rows - 1, 1), 1e-9) if rows > 1 else cpu_dt
    t_deq = max(cpu_dt1 - per_row, 0.0) if rows > 1 else 0.0
    cpu = {"value": m / (t_deq + per_row * m), "unit": "tokens/s", "cores": cores, "kind": "port",
           "value_dequant_excluded": 1.0 / per_row,
           "sample": f"{rows} rows and 1 row of the {m}-row batch through the whole block once each: per-call dequant {t_deq * 1e3:.1f} ms, "
                     f"per row {per_row * 1e3:.2f} ms; tokens/s = m / (dequant + m * per_row)"}

    kernels = kernel_configs(torch, sg, orc, peaks) if (world == 1 and not args.no_kernels) else None
    # kernels of this library per step: above 64 rows the block is two GEMMs (gated product and residual add
    # fused into their stores), else GEMV, gate, GEMV, add; tensor-parallel steps add the finishing pass
    # (above 64 rows: gate/up GEMM, down GEMM and the down projection's depth-split reduce; a rank's shard adds the finish
    # kernel, and one more reduce launch where the planner also splits the gate/up shard's depth -- not counted here)
    launches_per_step = (3 if m > 64 else (2 if m <= 4 else 4)) if world == 1 else (3 if m > 64 else (2 if m <= 4 else 3)) + 1

    line = {"metric": "q4_mlp_block_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(args, nsets),
            "clocks": clocks, "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                                      "d2h_bytes_per_step": m * HIDDEN * 4, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches_per_step * args.steps, "roofline": roofline, "cpu_baseline": cpu}
    line["projections"] = {"gate_up_us": us_gu, "down_us": us_down, "what": "this rank's two GEMMs timed alone (graph replay, max over ranks for down)"}
    if tp_check is not None:
        line["tp_check"] = tp_check
    if exchange_us is not None:
        line["exchange_us"] = exchange_us
    if m1 is not None:
        line["m1"] = m1
    if e2e_abi is not None:
        line["e2e_abi"] = e2e_abi
    if kernels is not None:
        line["kernels"] = kernels
    print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def orc_quant(sg, w, layout, n, k):
    """Quantise with the library's own host quantiser (the product path never calls the oracle)."""
    import ctypes as C
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    nbk = -(-k // BLOCK)
    q = np.zeros((k * n + 1) // 2, np.uint8)
    s = np.zeros(n * nbk, np.uint16)
    rc = sg.lib().smeg_host_q4_quantize(w.ctypes.data, layout, n, k, BLOCK, q.ctypes.data, s.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"smeg_host_q4_quantize returned {rc}")
    return q, s, None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", dest="m", type=int, default=256, help="tokens per step (BASELINE.json: 1 or 256)")
    ap.add_argument("--ref-rows", type=int, default=32, help="rows of the batch the CPU arm computes per step")
    ap.add_argument("--no-kernels", action="store_true", help="skip the single-kernel configs")
    ap.add_argument("--no-m1", action="store_true", help="skip the one-token leg")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: fused sum + finish over peer memory (this library's kernel) or NCCL all-reduce + finishing pass")
    ap.add_argument("--profile-case", default=None,
                    choices=["q4_gemv", "q2_gemv", "q1_gemv", "q4_prefill", "q1_prefill", "mlp_gate_up", "mlp_down"],
                    help="run six plain launches of one kernel and exit (for profiler captures)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
