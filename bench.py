#!/usr/bin/env python
"""bench.py -- headline benchmark of the B200 quantized-inference hot path.

Metric: quant matvec HBM GB/s.  Workload at every N: benchmark configuration 1,
the GGUF Q4_K dequant-fused matvec K=2560 -> N=10240 at batch 1, run as a ring of R
distinct weight matrices (R * 14.7 MB >> the 126 MB L2), so that every launch streams its
weights from HBM as it does inside a real decode step.  One pass over the ring = R matvec
launches, captured in one CUDA graph; one "step" = `--passes` replays of it (default 100, so
that the timed region of 20 steps lasts about half a second).

  value    = algorithmic bytes of all ranks' launches / device time (inputs resident)
  e2e      = the same pass driven from HOST buffers through the C ABI: pinned-host
             activations copied H2D, R launches, outputs copied D2H, every pass of every step
             (the copies of neighbouring passes run on their own streams, double-buffered)
  roofline = the matvec kernel against the measured HBM copy peak (MEASURED_PEAKS.json)
  cpu_baseline = the CPU oracle (a C restatement of the reference's Lean spec; the
             reference itself cannot be built here) on the box's host cores
  extra    = the other benchmark configurations (ternary i2_s ring, Q8_0 ring, decode attention)

`--impl reference` times that CPU restatement alone, on the same workload and metric.
With N > 1 each rank streams its own ring (the path shards by weight tensor; no
data-path collective), "weak" scaling; timing is the max over ranks.
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

K1, N1 = 2560, 10240
Q4K_BYTES = 14_796_800      # weights 14 745 600 + x 10 240 + y 40 960
Q80_BYTES = 27_904_000
I2S_BYTES = 4_489_220       # K=2560, N=6912 ternary: W + scale + x + acc + y
FALLBACK_HBM_GBS = 6650.0


def measured_traffic():
    """DRAM bytes per launch of the headline kernel (read + written), from the committed
    profiler summary of that kernel; None when the summary is absent."""
    import re
    p = os.path.join(ROOT, "profiles", "kq_mv_q4k_K2560_N10240.md")
    try:
        txt = open(p).read()
        rd = re.search(r"dram__bytes_read\.sum\s*\|\s*([0-9.]+)\s*MB", txt)
        wr = re.search(r"dram__bytes_write\.sum\s*\|\s*([0-9.]+)\s*MB", txt)
        return (float(rd.group(1)) + float(wr.group(1))) * 1e6
    except Exception:
        return None


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ----------------------------------------------------------------------------- reference arm

def run_reference(args):
    """The reference's CPU definition of the path, restated in C (oracle/), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from hesper_b200 import formats
    from oracle import oracle as orc
    orc.lib()
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: ask for the cores again
    orc.set_num_threads(os.cpu_count() or 1)
    cores = orc.num_threads()
    ring, x = cpu_ring(0x1337C0DE)
    orc.q4k_matvec(ring[0], K1, N1, x)  # touch
    t1 = time.perf_counter()
    orc.q4k_matvec(ring[1], K1, N1, x)
    one = time.perf_counter() - t1
    reps = max(1, min(2000, int(1.0 / max(one, 1e-6))))  # ~1 s of CPU work per step
    for w in range(args.warmup):
        orc.q4k_matvec(ring[w % len(ring)], K1, N1, x)
    t0 = time.perf_counter()
    i = 0
    for _ in range(args.steps):
        for _ in range(reps):
            orc.q4k_matvec(ring[i % len(ring)], K1, N1, x)
            i += 1
    dt = time.perf_counter() - t0
    gbs = Q4K_BYTES * reps * args.steps / dt / 1e9
    sample = (f"{reps} Q4_K matvecs K={K1} N={N1} per step over a ring of {len(ring)} distinct "
              f"matrices ({len(ring) * Q4K_BYTES >> 20} MB), {cores} OpenMP threads")
    line = {
        "impl": "reference", "metric": "quant matvec HBM GB/s", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64 accumulate over f32 dequant", "data": "synthetic",
        "config": {"workload": f"cfg1 Q4_K matvec K={K1} N={N1} batch 1 on host cores"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)
    return 0


# ----------------------------------------------------------------------------- our arm

def build_ring(torch, ctx, fmt, K, N, R, seed):
    """R distinct weight tensors on the device: one random tensor rolled by whole rows."""
    from hesper_b200 import LinearLayer, formats
    rng = np.random.default_rng(seed)
    base = torch.from_numpy(formats.random_kquant(rng, fmt, N, K)).cuda()
    rb = formats.kquant_row_bytes(fmt, K)
    return [LinearLayer(ctx, base if r == 0 else torch.roll(base, r * rb * 7), fmt, K, N)
            for r in range(R)]


def time_graph(torch, st, fn, steps, warmup, passes=1):
    """Capture fn() on stream st; a step is `passes` replays.  Runs warmup + steps steps and
    returns (seconds per step, graph), timed with CUDA events on st."""
    # inputs were produced on the default stream: order the side stream after them
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        fn()
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            fn()
        for _ in range(warmup * passes):
            g.replay()
        st.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(steps * passes):
            g.replay()
        e1.record(st)
        st.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / steps, g


def cpu_ring(seed, R=8):
    """R distinct Q4_K matrices of the bench shape on the host (one random tensor rolled by
    whole rows: 118 MB, larger than the host's L2) and one activation vector."""
    from hesper_b200 import formats
    rng = np.random.default_rng(seed)
    base = formats.random_q4k(rng, N1, K1)
    rb = formats.kquant_row_bytes(12, K1)
    ring = [base if r == 0 else np.roll(base, r * rb * 7) for r in range(R)]
    return ring, rng.standard_normal((1, K1)).astype(np.float32)


def cpu_baseline(sample_seconds=12.0):
    from oracle import oracle as orc
    orc.lib()
    orc.set_num_threads(os.cpu_count() or 1)
    ring, x = cpu_ring(1)
    orc.q4k_matvec(ring[0], K1, N1, x)
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < sample_seconds:
        orc.q4k_matvec(ring[n % len(ring)], K1, N1, x)
        n += 1
    dt = time.perf_counter() - t0
    return {"value": Q4K_BYTES * n / dt / 1e9, "unit": "GB/s", "cores": orc.num_threads(),
            "kind": "port",
            "sample": f"{n} Q4_K matvecs K={K1} N={N1} over a ring of {len(ring)} distinct matrices "
                      f"(rows split over {orc.num_threads()} OpenMP threads), {dt:.1f} s"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import hesper_b200
    from hesper_b200 import BitLinear, LinearLayer, execute_flash_attention_v11, formats
    from hesper_b200 import flash_attention_workspace

    ctx = hesper_b200.Context(local)
    st = torch.cuda.Stream()
    R = args.ring
    layers = build_ring(torch, ctx, 12, K1, N1, R, 0x1337C0DE + rank)
    xs = torch.randn(R, K1, device="cuda")
    ys = torch.empty(R, N1, device="cuda")

    def ring_pass():
        for r, l in enumerate(layers):
            l.forward(xs[r:r + 1], out=ys[r:r + 1], stream=st)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput (the headline `value`) ----
    barrier()
    with ClockSampler(local) as clk:
        P = max(1, args.passes)
        sec, _ = time_graph(torch, st, ring_pass, args.steps, max(3, args.warmup), P)
    barrier()
    tsec = torch.tensor([sec], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tsec, op=dist.ReduceOp.MAX)
    sec_max = float(tsec.item())
    value = world * P * R * Q4K_BYTES / sec_max / 1e9
    per_launch = sec / (P * R)
    peak, peak_src = measured_peak()
    achieved = Q4K_BYTES / per_launch / 1e9

    # ---- end to end from host buffers ----
    # A host that drives the C ABI with its own streams pipelines the copies: two sets of
    # device buffers (and a graph of the same 40 launches on each), the activations of pass
    # i + 1 go up and the results of pass i - 1 come down on their own streams while pass i
    # computes.  Every pass's H2D and D2H lies inside the timed region.
    hx = [torch.randn(R, K1).pin_memory() for _ in range(2)]
    hy = [torch.empty(R, N1).pin_memory() for _ in range(2)]
    dx = [xs, torch.empty_like(xs)]
    dy = [ys, torch.empty_like(ys)]

    graphs = []
    torch.cuda.synchronize()
    for b_ in range(2):
        def one_pass(b_=b_):
            for r, l in enumerate(layers):
                l.forward(dx[b_][r:r + 1], out=dy[b_][r:r + 1], stream=st)

        with torch.cuda.stream(st):
            one_pass()
            st.synchronize()
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=st):
                one_pass()
            st.synchronize()
        graphs.append(g_)
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    ev_up = [torch.cuda.Event() for _ in range(2)]      # activations of the buffer are on the device
    ev_done = [torch.cuda.Event() for _ in range(2)]    # the buffer's launches have finished
    ev_down = [torch.cuda.Event() for _ in range(2)]    # its results are on the host

    def e2e_step():
        for i in range(P):
            b_ = i & 1
            with torch.cuda.stream(up):
                up.wait_event(ev_done[b_])      # the pass that last read this x has finished
                dx[b_].copy_(hx[b_], non_blocking=True)
                ev_up[b_].record(up)
            with torch.cuda.stream(st):
                st.wait_event(ev_up[b_])
                st.wait_event(ev_down[b_])      # the results this pass overwrites are on the host
                graphs[b_].replay()
                ev_done[b_].record(st)
            with torch.cuda.stream(down):
                down.wait_event(ev_done[b_])
                hy[b_].copy_(dy[b_], non_blocking=True)
                ev_down[b_].record(down)
        st.synchronize()
        down.synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_sec = (time.perf_counter() - t0) / args.steps
    te = torch.tensor([e2e_sec], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_val = world * P * R * Q4K_BYTES / float(te.item()) / 1e9

    extra = {}
    if rank == 0 and not args.no_extra:
        if world == 1:
            extra = run_extra(torch, ctx, st, hesper_b200, args)
        else:  # single-GPU sections: the other ranks would only wait for them
            extra = {"single_gpu_sections": "measured in the 1-GPU run only"}
    if not args.no_extra:
        # config 4 is tensor-parallel over all ranks of the job: every rank takes part
        tpd = run_tp_decode(torch, dist, ctx, hesper_b200, rank, world)
        if rank == 0:
            extra["cfg4_gemma_tp_decode"] = tpd
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline()
    ctx.check()

    if rank == 0:
        line = {
            "metric": "quant matvec HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": sec_max * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8 (4-bit quants) x s16 (two s8 planes) integer mma, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"cfg1 GGUF Q4_K matvec K={K1} N={N1} batch 1, ring of {R} "
                                   f"distinct matrices per GPU ({R * 14.7456:.0f} MB > L2: inputs "
                                   f"larger than L2, no flush needed), one CUDA graph per pass, "
                                   f"{P} passes per step, programmatic dependent launch between "
                                   "matvecs",
                       "pct_of_8TBs": value / world / 8000.0 * 100.0},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": measured_traffic(),
                         "peak_source": peak_src, "kernel": "kq_mv_kernel<12,false>",
                         "algorithmic_bytes_per_launch": Q4K_BYTES,
                         "us_per_launch": per_launch * 1e6},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": P * R * K1 * 4,
                    "d2h_bytes_per_step": P * R * N1 * 4},
            "gpu_launches": P * R * args.steps,
            "clocks": clk.summary(),
            "extra": extra,
        }
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_extra(torch, ctx, st, hb, args):
    """The other benchmark configurations, device-resident, each as GB/s of algorithmic bytes."""
    from hesper_b200 import BitLinear, formats
    out = {}
    steps, warm = max(5, args.steps // 2), 3
    # cfg0: ternary i2_s x int8, K=2560 N=6912, ring of 128
    rng = np.random.default_rng(7)
    K0, N0, R0 = 2560, 6912, 128
    base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N0, K0))).cuda()
    sc = torch.tensor([0.05], device="cuda")
    bl = [BitLinear(ctx, base if r == 0 else torch.roll(base, r * 640 * 3), sc, K0, N0)
          for r in range(R0)]
    x0 = torch.randn(1, K0, device="cuda")
    y0 = torch.empty(R0, N0, device="cuda")

    def p0():
        for r, l in enumerate(bl):
            l.forward(x0, out=y0[r:r + 1], stream=st)
    sec, _ = time_graph(torch, st, p0, steps, warm)
    out["cfg0_i2s_ring_GBs"] = R0 * I2S_BYTES / sec / 1e9
    out["cfg0_i2s_us_per_matvec"] = sec / R0 * 1e6
    del bl, base
    # cfg1 Q8_0 variant, ring of 24
    R8 = 24
    l8 = build_ring(torch, ctx, 8, K1, N1, R8, 11)
    x8 = torch.randn(1, K1, device="cuda")
    y8 = torch.empty(R8, N1, device="cuda")

    def p8():
        for r, l in enumerate(l8):
            l.forward(x8, out=y8[r:r + 1], stream=st)
    sec, _ = time_graph(torch, st, p8, steps, warm)
    out["cfg1_q8_0_ring_GBs"] = R8 * Q80_BYTES / sec / 1e9
    del l8
    # cfg2: decode attention 8q/2kv heads, D=256
    H, Hkv, D = 8, 2, 256
    att = {}
    for B, L in [(1, 4096), (1, 32768), (16, 4096), (64, 4096), (64, 32768)]:
        q = torch.randn(B, H, D, device="cuda").half()
        k = torch.randn(B, Hkv, L, D, device="cuda").half()
        v = torch.randn(B, Hkv, L, D, device="cuda").half()
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        ws = hb.flash_attention_workspace(ctx, B, H, Hkv, D, L)
        o = torch.empty(B, H, D, device="cuda")

        def pa():
            hb.execute_flash_attention_v11(ctx, q, k, v, lens, num_heads=H, num_kv_heads=Hkv,
                                           head_dim=D, max_seq_len=L, scale=1 / 16, workspace=ws,
                                           out=o, stream=st)
        sec, _ = time_graph(torch, st, pa, steps, warm)
        att[f"B{B}_L{L}"] = {"us": sec * 1e6, "GBs": B * (2048 * L + 12288) / sec / 1e9}
        del q, k, v
    out["cfg2_attention"] = att
    out["batched_64_tokens"] = run_batched(torch, ctx, st, steps, warm)
    out["cfg3_bitnet2b_decode"] = run_bitnet_decode(torch, ctx, hb)
    return out


def run_batched(torch, ctx, st, steps, warm):
    """The tensor-core paths at 64 tokens: ternary product (tcgen05 kind::i8, activation
    quantiser included) and the LM head (tcgen05 kind::f16), cold rings."""
    from hesper_b200 import BitLinear, formats, _lib
    out = {}
    rng = np.random.default_rng(3)
    M = 64
    sc = torch.tensor([0.05], device="cuda")
    for K, N in ((2560, 6912), (6912, 2560)):
        R = 64
        base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N, K))).cuda()
        bl = [BitLinear(ctx, base if r == 0 else torch.roll(base, r * 640 * 3), sc, K, N)
              for r in range(R)]
        x = torch.randn(M, K, device="cuda")
        y = torch.empty(M, N, device="cuda")

        def pb():
            for l in bl:
                l.forward(x, out=y, stream=st)
        sec, _ = time_graph(torch, st, pb, steps, warm)
        t = sec / R
        out[f"i2s_K{K}_N{N}"] = {"us": t * 1e6, "weight_GBs": N * K / 4 / t / 1e9,
                                 "int8_TOPs": 2.0 * M * K * N / t / 1e12}
        del bl, base
    lib = _lib.load()
    V, K = 128256, 2560
    tabs = [(torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(2)]
    x = torch.randn(M, K, device="cuda")
    arg = torch.zeros(M, dtype=torch.int32, device="cuda")
    scr = torch.zeros(M, dtype=torch.int64, device="cuda")

    def pl():
        for t_ in tabs:
            rc = lib.hb200_lmhead_argmax(ctx.handle, t_.data_ptr(), 0, V, K, x.data_ptr(), M, None,
                                         0.0, None, arg.data_ptr(), scr.data_ptr(), None, None, 0,
                                         st.cuda_stream)
            assert rc == 0
    sec, _ = time_graph(torch, st, pl, steps, warm)
    t = sec / len(tabs)
    peak = measured_peak()[0]
    out["lmhead_V128256_K2560"] = {"us": t * 1e6, "table_GBs": V * K * 2 / t / 1e9,
                                   "frac_of_hbm_peak": V * K * 2 / t / 1e9 / peak,
                                   "bf16_TFLOPs": 2.0 * 2 * M * V * K / t / 1e12}
    return out


def run_tp_decode(torch, dist, ctx, hb, rank, world):
    """Configuration 4: Gemma-4-E4B-shaped Q4_K model, tensor-parallel over `world` GPUs,
    random-init (every rank draws the same tensors and keeps its slice), decode at context
    ~8000 of 8192.  Beside the timing, the greedy tokens are checked: all ranks must hold the
    same tokens, and at world > 1 rank 0 also decodes the unsharded model from the same seed and
    reports how many of 8 greedy tokens after an 8-token prompt agree (random-init logits have
    near-ties, so a different summation order may legitimately flip a token: reported, not
    asserted)."""
    from hesper_b200 import tp
    S = tp.GemmaShape()
    out = {"tp": world}
    comm = None
    try:
        if world > 1:
            comm = tp.TensorParallel.from_torch_distributed(ctx)
        plan = tp.plan(S, rank, world)
        shard = tp.random_gemma_shard_device(S, plan, seed=7)
        # algorithmic bytes per token per the whole job: Q4_K layers + LM head + bf16 embedding
        # row + f16 KV (35 sliding-window layers x 512 positions, 7 global layers x ctx)
        wbytes = 42 * 51_609_600 + 377_487_360
        first8 = {}
        for B, steps in ((1, 64), (32, 16), (256, 8)):
            model = tp.GemmaModel(ctx, S, shard, plan, comm, batch=B, max_new_tokens=steps)
            model.set_position(8000)
            model.generate(None, 4, use_graph=True)       # warm-up (also captures once)
            model.set_position(8000)
            if world > 1:
                dist.barrier()
            toks, _, ms = model.generate(None, steps, use_graph=True)
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            kv = B * (35 * 512 + 7 * 8000) * 2048
            us = ms / steps * 1e3
            roof = (wbytes + kv) / world / measured_peak()[0] / 1e3
            rec = {"tok_s": B * steps / ms * 1e3, "us_per_step": us,
                   "roofline_us_at_measured_peak": roof, "frac_of_roofline": roof / us,
                   "allreduces_per_step": 84 if world > 1 else 0}
            n8 = min(8, steps)
            mine = torch.from_numpy(np.ascontiguousarray(toks[:, :n8])).cuda()
            if B == 1:  # a defined context for the comparison with the unsharded model
                pr = np.arange(11, 19, dtype=np.int32).reshape(1, 8)
                first8[B] = model.generate(pr, 8, use_graph=True)[0][0].tolist()
            if world > 1:
                allt = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(allt, mine)
                rec["ranks_agree"] = bool(all(torch.equal(allt[0], a) for a in allt))
                assert rec["ranks_agree"], "tensor-parallel ranks hold different greedy tokens"
            out[f"B{B}"] = rec
            model.close()
            del model
        if world > 1 and rank == 0:
            # the unsharded model from the same seed on this GPU, batch 1
            del shard
            torch.cuda.empty_cache()
            p1 = tp.plan(S, 0, 1)
            one = tp.GemmaModel(ctx, S, tp.random_gemma_shard_device(S, p1, seed=7), p1, None,
                                batch=1, max_new_tokens=8)
            t1, _, _ = one.generate(np.arange(11, 19, dtype=np.int32).reshape(1, 8), 8,
                                    use_graph=True)
            one.close()
            same = sum(int(a == b) for a, b in zip(t1[0].tolist(), first8[1]))
            out["B1"]["first8_equal_to_unsharded"] = same
    except AssertionError:
        raise
    except Exception as e:  # keep the headline line alive if a side measurement fails
        out["error"] = repr(e)[:300]
    finally:
        if comm is not None:
            comm.close()
    return out


def run_bitnet_decode(torch, ctx, hb):
    """Configuration 3: BitNet-b1.58-2B-shaped model, random-init, 2048-token random prompt
    then 128 greedy tokens at batch 1 and at batch 64 (decode by graph replay; the prompt is
    consumed in passes of 256 // batch positions through the batched kernels)."""
    from hesper_b200.models import BitNetShape, BitNetModel, random_bitnet_weights_device
    shape = BitNetShape.bitnet_2b(max_seq=2304)
    w = random_bitnet_weights_device(shape)
    out = {}
    peak = measured_peak()[0]
    for B, P, n_new in ((1, 2048, 128), (64, 2048, 128)):
        try:
            model = BitNetModel(ctx, shape, w, batch=B, max_new_tokens=n_new)
            prompt = np.random.default_rng(0).integers(0, shape.vocab, (B, P)).astype(np.int32)
            _, ms_p, ms_d = model.generate(prompt, n_new, use_graph=True)
            steps = n_new - 1
            us = ms_d / steps * 1e3
            # bytes per step: ternary layers + bf16 LM head + f16 KV at the mean decode position
            kv = B * 30 * 2 * 5 * 128 * 2 * (P + n_new // 2)
            byts = 521_011_200 + 656_670_720 + kv
            out[f"B{B}"] = {"tok_s": B * steps / ms_d * 1e3, "us_per_step": us,
                            "prompt_len": P, "new_tokens": n_new, "prefill_ms": ms_p,
                            "roofline_us_at_measured_peak": byts / peak / 1e3,
                            "frac_of_roofline": byts / peak / 1e3 / us}
            model.close()
            del model
        except Exception as e:
            out[f"B{B}"] = {"error": repr(e)[:300]}
    return out


# ----------------------------------------------------------------------------- profiler cases

CASES = """Small fixed workloads for profiler captures: `python bench.py --case <name>`.
Each runs a handful of launches of one kernel on inputs larger than the L2 but well under a
few GB, so that a full-metric capture of one to three launches ends in a minute.
  q4k      ring of 12 Q4_K matrices K=2560 N=10240 (177 MB), 3 passes
  q80      ring of 8 Q8_0 matrices (223 MB), 3 passes
  i2s      ring of 40 ternary matrices K=2560 N=6912 (177 MB), 3 passes
  attn     decode attention B=16 L=4096, 8q/2kv heads, D=256 (268 MB of KV), 6 calls
  attn_prefill  causal attention of a 256-token prompt chunk at context 8192, 8 sequences,
           8q/2kv heads, D=256 (134 MB of KV), 3 calls
  i2s_mma  64-token ternary product on the tensor cores, ring of 40 matrices (177 MB), 2 passes
  lmhead64 64-token LM head on the tensor cores, one bf16 table V=128256 K=2560 (657 MB), 3 calls
  q4k_b32  32-token Q4_K product on the tensor cores, ring of 12 matrices, 2 passes
  bitnet1 / bitnet64   BitNet-2B-shaped decode loop at batch 1 / 64: 2 prompt positions and
           3 new tokens, launched one by one (no graph) so that a launch list sees each kernel
  gemma1 / gemma32 / gemma256   Gemma-4-E4B-shaped Q4_K decode loop (one rank): 3 tokens at
           position 8000, launched one by one
"""


def run_case(name: str) -> int:
    import torch
    import hesper_b200 as hb
    from hesper_b200 import formats
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --case needs a CUDA device")
    ctx = hb.Context(0)
    rng = np.random.default_rng(0)
    if name in ("q4k", "q80"):
        fmt, R = (12, 12) if name == "q4k" else (8, 8)
        K, N = 2560, 10240
        base = torch.from_numpy(formats.random_kquant(rng, fmt, N, K)).cuda()
        rb = formats.kquant_row_bytes(fmt, K)
        layers = [hb.LinearLayer(ctx, torch.roll(base, r * rb), fmt, K, N) for r in range(R)]
        x = torch.randn(1, K, device="cuda")
        y = torch.empty(1, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            for l in layers:
                l.forward(x, out=y)
    elif name == "i2s":
        K, N, R = 2560, 6912, 40
        base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N, K))).cuda()
        sc = torch.tensor([0.05], device="cuda")
        layers = [hb.BitLinear(ctx, torch.roll(base, r * 640), sc, K, N) for r in range(R)]
        x = torch.randn(1, K, device="cuda")
        y = torch.empty(1, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            for l in layers:
                l.forward(x, out=y)
    elif name == "q4k_b32":
        K, N, R, M = 2560, 10240, 12, 32
        base = torch.from_numpy(formats.random_kquant(rng, 12, N, K)).cuda()
        rb = formats.kquant_row_bytes(12, K)
        layers = [hb.LinearLayer(ctx, torch.roll(base, r * rb), 12, K, N) for r in range(R)]
        x = torch.randn(M, K, device="cuda")
        y = torch.empty(M, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(2):
            for l in layers:
                l.forward(x, out=y)
    elif name == "i2s_mma":
        K, N, R, M = 2560, 6912, 40, 64
        base = torch.from_numpy(formats.i2s_pack(formats.random_ternary(rng, N, K))).cuda()
        sc = torch.tensor([0.05], device="cuda")
        layers = [hb.BitLinear(ctx, torch.roll(base, r * 640), sc, K, N) for r in range(R)]
        x = torch.randn(M, K, device="cuda")
        y = torch.empty(M, N, device="cuda")
        torch.cuda.synchronize()
        for _ in range(2):
            for l in layers:
                l.forward(x, out=y)
    elif name == "lmhead64":
        from hesper_b200 import _lib
        lib = _lib.load()
        V, K, M = 128256, 2560, 64
        table = (torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16)
        x = torch.randn(M, K, device="cuda")
        arg = torch.zeros(M, dtype=torch.int32, device="cuda")
        scr = torch.zeros(M, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            rc = lib.hb200_lmhead_argmax(ctx.handle, table.data_ptr(), 0, V, K, x.data_ptr(), M,
                                         None, 0.0, None, arg.data_ptr(), scr.data_ptr(), None,
                                         None, 0, None)
            assert rc == 0
    elif name in ("bitnet1", "bitnet64"):
        from hesper_b200.models import BitNetModel, BitNetShape, random_bitnet_weights_device
        B = 1 if name == "bitnet1" else 64
        shape = BitNetShape.bitnet_2b(max_seq=2304)
        w = random_bitnet_weights_device(shape)
        m = BitNetModel(ctx, shape, w, batch=B, max_new_tokens=8)
        prompt = rng.integers(0, shape.vocab, (B, 2)).astype(np.int32)
        m.generate(prompt, 3, use_graph=False)
        m.close()
    elif name in ("gemma1", "gemma32", "gemma256"):
        from hesper_b200 import tp
        B = int(name[5:])
        S = tp.GemmaShape()
        plan = tp.plan(S, 0, 1)
        shard = tp.random_gemma_shard_device(S, plan, seed=7)
        m = tp.GemmaModel(ctx, S, shard, plan, None, batch=B, max_new_tokens=8)
        m.set_position(8000)
        m.generate(None, 3, use_graph=False)
        m.close()
    elif name == "attn_prefill":
        B, T, H, Hkv, D, L = 8, 256, 8, 2, 256, 8192
        q = torch.randn(B, T, H, D, device="cuda")
        k = torch.randn(B, Hkv, L, D, device="cuda").half()
        v = torch.randn(B, Hkv, L, D, device="cuda").half()
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        for _ in range(3):
            hb.flash_attention_prefill(ctx, q, k, v, lens, num_heads=H, num_kv_heads=Hkv,
                                       head_dim=D, max_seq_len=L, scale=1 / 16)
    elif name == "attn":
        B, H, Hkv, D, L = 16, 8, 2, 256, 4096
        q = torch.randn(B, H, D, device="cuda").half()
        k = torch.randn(B, Hkv, L, D, device="cuda").half()
        v = torch.randn(B, Hkv, L, D, device="cuda").half()
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        ws = hb.flash_attention_workspace(ctx, B, H, Hkv, D, L)
        torch.cuda.synchronize()
        for _ in range(6):
            hb.execute_flash_attention_v11(ctx, q, k, v, lens, num_heads=H, num_kv_heads=Hkv,
                                           head_dim=D, max_seq_len=L, scale=1 / 16, workspace=ws)
    else:
        raise SystemExit(f"unknown case {name}")
    torch.cuda.synchronize()
    ctx.check()
    print("ok")
    return 0



_RESULT_FD = None


def emit(line: dict) -> None:
    """The one JSON line, on the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # stdout carries the one JSON line and nothing else: whatever a library prints there (NCCL's
    # version banner at NCCL_DEBUG=VERSION, for one) is sent to stderr by pointing file
    # descriptor 1 at it for the run; the result goes to a copy of the original descriptor
    global _RESULT_FD
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ring", type=int, default=40, help="distinct weight matrices per pass")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--passes", type=int, default=100, help="ring passes (graph replays) per step")
    ap.add_argument("--case", default=None, help="run one small profiler workload and exit:\n" + CASES)
    args = ap.parse_args()
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.case:
        return run_case(args.case)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
