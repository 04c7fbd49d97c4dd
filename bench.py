#!/usr/bin/env python
"""Benchmark of the decode GEMV hot path (the decode GEMV sweep) on N B200 GPUs of one node.

Workload: the decode GEMV sweep — M in {1,2,4,8} activation rows times the five Phi-1.5 layer
shapes (K->N: 2048->6144, 2048->2048, 2048->8192, 8192->2048, 2048->51200), f16 weights
~N(0,0.02) resident in HBM, activations ~N(0,1): 20 launches of the GEMV kernel, replayed as
one CUDA graph.  A "step" is SWEEPS_PER_STEP passes over the sweep (one pass is 0.2 ms on a
B200; the timed region of the default run lasts more than a second, so the clock samples are
taken under the measured load).  The metric is achieved HBM GB/s counted with the reference's
own byte formula 2*(M*K + K*N + M*N) (hgemm_trans.zig:580-593).  A pass touches 1.24 GB of
distinct weights, ten times the L2, so no flush is needed between iterations.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 is launched by torch.distributed.run; every rank runs the sweep on its own GPU
(independent requests are partitioned across GPUs, no collective on the data path), the
timed region is bracketed by barriers, the time is the max over ranks.

--impl reference times the CPU oracle (the C++ restatement of the reference's AVX2 path;
the Zig reference itself cannot be built on this box) on the host cores for the same sweep.
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

SHAPES = [(2048, 6144), (2048, 2048), (2048, 8192), (8192, 2048), (2048, 51200)]  # (K, N)
MS = [1, 2, 4, 8]
METRIC = "decode_gemv_hbm_gbs"
UNIT = "GB/s"


def algo_bytes(m, k, n):
    return 2 * (m * k + k * n + m * n)


SWEEP_BYTES = sum(algo_bytes(m, k, n) for m in MS for k, n in SHAPES)
SWEEPS_PER_STEP = 256
STEP_BYTES = SWEEPS_PER_STEP * SWEEP_BYTES
WORKLOAD = "decode GEMV sweep: M in {1,2,4,8} x the five Phi-1.5 layer shapes, 20 weight matrices of their own"


def workload_config():
    """The workload description both arms print (identical dicts)."""
    return {"workload": WORKLOAD, "bytes_per_sweep": SWEEP_BYTES, "sweeps_per_step": SWEEPS_PER_STEP,
            "bytes_per_step": STEP_BYTES,
            "l2": "inputs larger than L2: 1.24 GB of distinct weights per sweep, each byte read once per sweep"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t_begin = self.t_end = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # nvidia-smi needs most of a second to print its first line, so it is started before the warm-up; only the
        # lines that arrived between the start and the end of the timed region are used
        inside = [ln for (t, ln) in self.lines
                  if self.t_begin is None or (self.t_begin <= t <= (self.t_end or t) + 0.05)]
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": "timed region only"}


def make_inputs(seed=2000):
    """Seeded synthetic inputs of the sweep (weights ~N(0,0.02), activations ~N(0,1)).  Every one of the 20 problems
    owns its weight matrix, as in the reference's benchmark (a fresh B per case): the matrix of (M, shape) is the
    shape's base matrix rotated by M rows."""
    rng = np.random.default_rng(seed)
    base = [(rng.standard_normal((n, k), dtype=np.float32) * 0.02).astype(np.float16) for k, n in SHAPES]
    ws = {(m, i): (base[i] if m == MS[0] else np.roll(base[i], m, axis=0)) for m in MS for i in range(len(SHAPES))}
    xs = {(m, i): rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
          for m in MS for i, (k, n) in enumerate(SHAPES)}
    return ws, xs


def cpu_sweep(oracle, ws, xs):
    for m in MS:
        for i in range(len(SHAPES)):
            oracle.hgemm_nt(xs[(m, i)], ws[(m, i)])


def run_reference(args, rank):
    """The reference arm: the CPU oracle on the host cores, all threads.  A step of this arm is a bounded sample of
    the workload's step: one of its SWEEPS_PER_STEP sweeps (1.24 GB of weights, all 20 problems)."""
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    ws, xs = make_inputs()
    for _ in range(max(args.warmup, 1)):
        cpu_sweep(oracle, ws, xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_sweep(oracle, ws, xs)
    dt = (time.perf_counter() - t0) / args.steps
    val = SWEEP_BYTES / dt / 1e9
    cores = oracle.get_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * SWEEPS_PER_STEP, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "one sweep (all 20 problems, 1.24 GB) of the 256 sweeps of a step, per timed step; "
                                   "ms_per_step is the sample scaled to a full step (C++ restatement of "
                                   "hgemm_trans.zig; the Zig reference cannot be built here)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the per-shape and GEMM side measurements")
    ap.add_argument("--only", default=None, choices=sorted(ONLY_CASES),
                    help="run one small side workload alone (for profiling a kernel) and print its timing")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()

    pkg = entry.load_package()
    ctx = pkg.Context(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    # the weights are registered once and never written on this stream, so consecutive GEMVs may be
    # launched programmatically dependent (a kernel streams its first weights while its predecessor drains)
    ctx.set_option("pdl", 1)

    if args.only:
        print(json.dumps({"only": args.only, **run_only(ctx, torch, stream, args.only)}), flush=True)
        ctx.sync()
        if world > 1:
            dist.destroy_process_group()
        return

    ws_h, xs_h = make_inputs()
    # every one of the 20 problems owns its weight matrix, as in the reference's benchmark (a fresh B per case):
    # 1.24 GB of distinct weights per step, so no byte can be served twice from L2 inside a step either
    wsm = {key: torch.from_numpy(w).cuda() for key, w in ws_h.items()}
    xs = {key: torch.from_numpy(x).cuda() for key, x in xs_h.items()}
    ys = {(m, i): torch.empty((m, n), dtype=torch.float16, device="cuda") for m in MS for i, (k, n) in enumerate(SHAPES)}

    def sweep():
        for m in MS:
            for i, (k, n) in enumerate(SHAPES):
                ctx.hgemm_nt(xs[(m, i)].data_ptr(), wsm[(m, i)].data_ptr(), m, n, k, out=ys[(m, i)].data_ptr())

    # one eager pass (sets up everything), a parity spot check against torch f32, then capture
    sweep()
    ctx.sync()
    for key in [(1, 0), (8, 4)]:
        ref = xs[key].float() @ wsm[key].float().T
        err = (ys[key].float() - ref).abs().max().item()
        assert err <= 1e-2 * ref.abs().max().item(), f"parity check failed for {key}: {err}"
    # The 20 products of a sweep are independent problems with their own operands.  They are recorded as
    # SWEEP_BRANCHES parallel chains of one graph (fork / join with events inside the capture), so that the launch
    # gaps and drain phases of one chain are filled by the other chains' memory traffic; inside a chain
    # consecutive launches stay programmatically dependent.  Launches are dealt to the chains largest first.
    branches = max(1, int(os.environ.get("BENCH_SWEEP_BRANCHES", SWEEP_BRANCHES)))
    order = sorted(((m, i) for m in MS for i in range(len(SHAPES))), key=lambda mi: -SHAPES[mi[1]][0] * SHAPES[mi[1]][1])
    chains, load = [[] for _ in range(branches)], [0] * branches
    for m, i in order:
        b = load.index(min(load))
        chains[b].append((m, i))
        load[b] += SHAPES[i][0] * SHAPES[i][1]
    side = [torch.cuda.Stream() for _ in range(branches - 1)]

    def sweep_branched():
        fork = torch.cuda.Event()
        fork.record(stream)
        joins = []
        for b, chain in enumerate(chains):
            st = stream if b == 0 else side[b - 1]
            if b:
                st.wait_event(fork)
                ctx.set_stream(st.cuda_stream)
            for m, i in chain:
                k, n = SHAPES[i]
                ctx.hgemm_nt(xs[(m, i)].data_ptr(), wsm[(m, i)].data_ptr(), m, n, k, out=ys[(m, i)].data_ptr())
            if b:
                ev = torch.cuda.Event()
                ev.record(st)
                joins.append(ev)
                ctx.set_stream(stream.cuda_stream)
        for ev in joins:
            stream.wait_event(ev)

    def capture(fn):
        n0 = ctx.launch_count()
        ctx.graph_begin()
        fn()
        g = ctx.graph_end()
        return g, ctx.launch_count() - n0

    graph, launches_per_sweep = capture(sweep_branched if branches > 1 else sweep)

    def timed(g, steps, sampler=None):
        """`steps` steps of SWEEPS_PER_STEP graph replays each, CUDA events on the launching stream, barriers and
        synchronisation on both sides; returns the max over ranks of the mean ms per step."""
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        barrier()
        if sampler:
            sampler.mark_begin()
        ev0.record(stream)
        for _ in range(steps * SWEEPS_PER_STEP):
            ctx.graph_launch(g)
        ev1.record(stream)
        torch.cuda.synchronize()
        if sampler:
            sampler.mark_end()
        barrier()
        clk = sampler.stop() if sampler else None
        t = torch.tensor([ev0.elapsed_time(ev1)], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps, clk

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(warm * SWEEPS_PER_STEP):
        ctx.graph_launch(graph)
    ctx.sync()
    # the clock samples that count are those taken during the timed region (more than a second at 20 steps)
    ms_step, clocks = timed(graph, args.steps, sampler)
    value = world * STEP_BYTES / (ms_step * 1e-3) / 1e9
    launches_per_step = launches_per_sweep * SWEEPS_PER_STEP

    # the same 20 launches as ONE dependent chain (what a caller gets who cannot overlap independent products)
    single = None
    if branches > 1 and not args.no_extras:
        g1, _ = capture(sweep)
        for _ in range(3 * 16):
            ctx.graph_launch(g1)
        ms1, _ = timed(g1, max(2, args.steps // 4))
        single = {"value": world * STEP_BYTES / (ms1 * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms1,
                  "note": "the 20 GEMVs of a sweep as one programmatically dependent chain instead of four"}
        ctx.graph_destroy(g1)

    # ---- end to end through the C ABI with HOST buffers: H2D of the activations and D2H of the
    # result inside every call (weights registered once), as the Zig host would call it
    pin_x = {key: torch.from_numpy(x).pin_memory() for key, x in xs_h.items()}
    pin_y = {key: torch.empty(tuple(ys[key].shape), dtype=torch.float16).pin_memory() for key in ys}

    calls = [(pin_x[(m, i)].data_ptr(), wsm[(m, i)].data_ptr(), pin_y[(m, i)].data_ptr(), m, n, k)
             for m in MS for i, (k, n) in enumerate(SHAPES)]
    hgemm_nt, handle = ctx.lib.md_hgemm_nt, ctx.h

    def e2e_sweep():
        for x_ptr, w_ptr, y_ptr, m, n, k in calls:
            if hgemm_nt(handle, x_ptr, w_ptr, y_ptr, m, n, k) != 0:
                raise RuntimeError(ctx.lib.md_last_error(ctx.h).decode())

    import ctypes as C
    ctx.lib.md_hgemm_nt.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t]
    for _ in range(3):
        e2e_sweep()
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(SWEEPS_PER_STEP):     # one step
        e2e_sweep()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    barrier()
    t = torch.tensor([dt], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_val = world * STEP_BYTES / t.item() / 1e9
    h2d = SWEEPS_PER_STEP * sum(m * k * 2 for m in MS for k, n in SHAPES)
    d2h = SWEEPS_PER_STEP * sum(m * n * 2 for m in MS for k, n in SHAPES)
    err = (pin_y[(8, 4)].float() - (xs[(8, 4)].float() @ wsm[(8, 4)].float().T).cpu()).abs().max().item()
    assert err < 0.2, f"e2e parity check failed: {err}"

    colsplit = box = None
    if world > 1 and not args.no_extras:
        colsplit = colsplit_extras(ctx, torch, dist, stream, world, rank)
    if not args.no_extras:
        box = box_requests_extras(ctx, torch, dist if world > 1 else None, world, rank)

    if rank != 0:
        ctx.sync()
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    achieved = (STEP_BYTES / launches_per_step) / (ms_step * 1e-3 / launches_per_step) / 1e9
    config = workload_config()      # the same dict the reference arm prints
    launch = {"launches_per_step": launches_per_step, "sweep_chains": branches, "replay": "one CUDA graph per sweep",
              "parallelism": f"replicas x{world}"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": config, "launch": launch,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_kind": peak_kind, "kernel": "gemv_nt_mma_kernel",
                     "frac_of_nominal_8tbs": achieved / 8000.0,
                     "note": "four concurrent chains of independent GEMVs; as one dependent chain see single_chain"},
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "md_hgemm_nt with pinned HOST activations/outputs per call (activations fetched over the bus inside the call, results written by the kernel into the pinned host buffer), weights registered once; one step = 256 sweeps = 5120 synchronous calls"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if single is not None:
        single["frac"] = single["value"] / world / hbm_peak
        line["single_chain"] = single

    if not args.no_extras and world == 1:
        line["extras"] = extras(ctx, torch, stream, tensor_peak, hbm_peak)
        line["extras"].update(model_extras(ctx, torch))
    if colsplit is not None:
        line.setdefault("extras", {})["colsplit_gemm_8192"] = colsplit
    if box is not None:
        line.setdefault("extras", {})["box_requests"] = box

    # ---- CPU baseline: the oracle on this box's host cores, bounded sample
    from oracle import oracle
    oracle.build()
    cpu_sweep(oracle, ws_h, xs_h)
    best = None
    t_begin = time.perf_counter()
    for _ in range(5):
        t0 = time.perf_counter()
        cpu_sweep(oracle, ws_h, xs_h)
        d = time.perf_counter() - t0
        best = d if best is None else min(best, d)
        if time.perf_counter() - t_begin > 20:
            break
    line["cpu_baseline"] = {"value": SWEEP_BYTES / best / 1e9, "unit": UNIT, "cores": oracle.get_threads(), "kind": "port",
                            "sample": "best of up to 5 sweeps (1.24 GB each; a step is 256 of them) of the C++ "
                                      "restatement of hgemm_trans.zig on the host cores"}
    if not args.no_extras and world == 1:
        line["extras"]["cpu"] = cpu_extras(oracle)
        if box is not None and "cpu" in line["extras"]:
            c = line["extras"]["cpu"]["request_extrapolated"]
            box["cpu_requests_per_s_extrapolated"] = round(1.0 / c["seconds_per_request"], 4)
            box["cpu_decode_tok_s"] = c["decode_tok_s"]
    print(json.dumps(line), flush=True)
    ctx.graph_destroy(graph)
    ctx.sync()
    if world > 1:
        dist.destroy_process_group()


SWEEP_BRANCHES = 4  # parallel chains the sweep graph is recorded as
# dram__bytes_read.sum + dram__bytes_write.sum of gemv_nt_mma_kernel from an ncu capture of this workload (its
# summary sits under profiles/): 280.41 MB measured over the three captured launches (fc1, fc2, lm_head at
# M = 1) against 276.97 MB of algorithmic bytes, a factor of 1.0124; traffic grows in proportion to the weight
# bytes, so the average launch of the sweep is scaled by the same factor.
TRAFFIC_BYTES_PER_LAUNCH = int(round(1.0124 * SWEEP_BYTES / 20))


def colsplit_extras(ctx, torch, dist, stream, world, rank):
    """The 8192^3 f16 GEMM with N split over the ranks: all-gather baseline (ncclAllGather inside the library)
    against the fused push epilogue, both through the library's own communicator.  Device time per call, max over
    ranks.  Parity is asserted on every rank: the two forms agree bit for bit, and 64 sampled rows agree with an f32
    product of the same operands within 1e-2 * max|ref|."""
    import importlib
    import __graft_entry__ as entry
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    M = N = K = 8192
    g = torch.Generator(device="cuda").manual_seed(5000)          # same operands on every rank
    a = torch.randn(M, K, device="cuda", generator=g).half()
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.02).half()     # B^T, [N,K] layout
    bs = par.slice_b(b, 1, world, rank)
    rows = torch.arange(0, M, M // 64, device="cuda")
    ref = a[rows].float() @ b.float().T
    del b
    out = {"M": M, "N": N, "K": K, "world": world}
    peaks = measured_peaks()
    comm = par.Comm(ctx)
    results = {}
    # fused: the library's default way of pushing tiles; the other push form is measured beside it
    default_tma = ctx.get_option("push_tma")
    for mode in ("allgather", "fused", "fused_other_push"):
        ctx.set_option("push_tma", (1 - default_tma) if mode == "fused_other_push" else default_tma)
        gm = par.ColSplitGemm(comm, M, N, K, 1, mode="allgather" if mode == "allgather" else "fused")
        for _ in range(3):
            gm(a, bs)
        comm.barrier()
        ctx.sync()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(stream)
        for _ in range(reps):
            gm(a, bs)
        e1.record(stream)
        ctx.sync()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = t.item() * 1e3
        out[mode] = {"us": round(us, 1), "TFLOP/s_total": round(2.0 * M * N * K / us / 1e6, 1)}
        comm.barrier()
        results[mode] = torch.from_numpy(gm.result()).cuda()
        if mode != "allgather":
            out[mode]["tile"] = ctx.get_option("last_tc_tile")
            out[mode]["push"] = "tma stores from the staged chunks" if ctx.get_option("push_tma") else "push warps"
        dist.barrier()
        gm.close()
    ctx.set_option("push_tma", default_tma)
    same = bool(torch.equal(results["fused"], results["allgather"])) and \
        bool(torch.equal(results["fused_other_push"], results["allgather"]))
    err = (results["fused"][rows].float() - ref).abs().max().item()
    tol = 1e-2 * ref.abs().max().item()
    ok = torch.tensor([1 if (same and err <= tol) else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    assert ok.item() == 1, f"rank {rank}: column-split parity failed (forms equal: {same}, err {err} vs tol {tol})"
    out["parity_ok"] = True
    out["parity"] = "fused == allgather bit for bit on every rank; 64 sampled rows within 1e-2*max|ref| of an f32 product"
    # roofline of the fused kernel: the slower of the math and the bytes that must cross NVLink
    t_math = 2.0 * M * (N / world) * K / (peaks[1] * 1e12)
    t_link = M * (N / world) * 2 * (world - 1) / 770e9
    out["fused"]["target_us"] = round(max(t_math, t_link) * 1e6, 1)
    out["fused"]["frac_of_target"] = round(out["fused"]["target_us"] / out["fused"]["us"], 3)
    # the GEMM alone, for reference
    y = torch.empty(M, N // world, device="cuda", dtype=torch.float16)
    for _ in range(2):
        ctx.hgemm_nt(a.data_ptr(), bs.data_ptr(), M, N // world, K, out=y.data_ptr())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(10):
        ctx.hgemm_nt(a.data_ptr(), bs.data_ptr(), M, N // world, K, out=y.data_ptr())
    e1.record(stream)
    torch.cuda.synchronize()
    out["local_gemm_us"] = round(e0.elapsed_time(e1) / 10 * 1e3, 1)
    comm.close()
    del results, a, bs, y
    torch.cuda.empty_cache()
    return out


def extras(ctx, torch, stream, tensor_peak, hbm_peak):
    """Side measurements: per-shape GEMV GB/s (rotating weight copies so every
    launch streams from HBM), config 1 (64x2048 . 2048x8192) and large GEMMs on the tcgen05 kernel."""
    out = {"gemv": [], "gemm": []}

    def time_graph(fn, reps):
        fn()
        ctx.sync()
        ctx.graph_begin()
        fn()
        g = ctx.graph_end()
        for _ in range(3):
            ctx.graph_launch(g)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            ctx.graph_launch(g)
        e1.record(stream)
        torch.cuda.synchronize()
        ctx.graph_destroy(g)
        return e0.elapsed_time(e1) / reps

    for m in (1, 8):
        for k, n in SHAPES:
            copies = max(3, (300 << 20) // (n * k * 2) + 1)
            w = (torch.randn(copies, n, k, device="cuda") * 0.02).half()
            x = torch.randn(m, k, device="cuda").half()
            y = torch.empty(m, n, device="cuda", dtype=torch.float16)

            def fn():
                for c in range(copies):
                    ctx.hgemm_nt(x.data_ptr(), w[c].data_ptr(), m, n, k, out=y.data_ptr())
            us = time_graph(fn, 5) / copies * 1e3
            gbs = algo_bytes(m, k, n) / us / 1e3
            out["gemv"].append({"M": m, "K": k, "N": n, "us": round(us, 2), "GB/s": round(gbs, 1),
                                "frac_of_measured_hbm": round(gbs / hbm_peak, 3)})
            del w
    for (m, k, n, layout, copies) in [(64, 2048, 8192, "nn", 10), (64, 2048, 8192, "nt", 10),
                                      (761, 2048, 8192, "nt", 10), (9477, 1152, 4304, "nn", 4),
                                      (729, 1152, 3456, "nn", 16), (8192, 8192, 8192, "nt", 1)]:
        shape = (copies, n, k) if layout == "nt" else (copies, k, n)
        w = (torch.randn(*shape, device="cuda") * 0.02).half()
        x = torch.randn(m, k, device="cuda").half()
        y = torch.empty(m, n, device="cuda", dtype=torch.float16)
        call = ctx.hgemm_nt if layout == "nt" else ctx.hgemm_nn

        def fn():
            for c in range(copies):
                call(x.data_ptr(), w[c].data_ptr(), m, n, k, out=y.data_ptr())
        us = time_graph(fn, 5) / copies * 1e3
        tf = 2.0 * m * n * k / us / 1e6
        out["gemm"].append({"M": m, "K": k, "N": n, "layout": layout, "us": round(us, 2), "TFLOP/s": round(tf, 1),
                            "GB/s": round(algo_bytes(m, k, n) / us / 1e3, 1),
                            "frac_of_measured_tensor": round(tf / tensor_peak, 3)})
        del w
    return out


# name -> what `--only name` runs: a few launches of one kernel family on inputs larger than L2 where the bytes
# matter, so that a profiler capture of it stays small
ONLY_CASES = {
    "gemm_config1": "64x2048 . 2048x8192 (both layouts), ten weight matrices in turn",
    "gemm_8192": "8192^3 NT, three calls",
    "gemm_prefill": "761x2048 . 2048x8192 NT with bias + GELU, ten weight matrices in turn",
    "gemm_vit": "9477x1152 . 1152x4304 NN (13 crops, fc1) with bias + GELU, four weight matrices in turn",
    "prefill": "text prefill of 761 rows through all 24 layers, three passes",
    "decode": "text decode, one request, 761-row prefill then 40 steps",
    "decode8": "text decode, eight requests batched, 761-row prefill each then 40 steps",
    "vision1": "vision encode + projection, one crop, three passes",
    "vision13": "vision encode + projection, thirteen crops, three passes",
}


def run_only(ctx, torch, stream, case):
    g = torch.Generator(device="cuda").manual_seed(4000)

    def n(*shape, std=0.02):
        return (torch.randn(*shape, device="cuda", generator=g) * std).half()

    def timed(fn, reps):
        fn()
        ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        ctx.sync()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    if case.startswith("gemm_"):
        m, k, nn, layout, copies, glue = {"gemm_config1": (64, 2048, 8192, "both", 10, False),
                                          "gemm_8192": (8192, 8192, 8192, "nt", 1, False),
                                          "gemm_prefill": (761, 2048, 8192, "nt", 10, True),
                                          "gemm_vit": (9477, 1152, 4304, "nn", 4, True)}[case]
        x = torch.randn(m, k, device="cuda", generator=g).half()
        y = torch.empty(m, nn, device="cuda", dtype=torch.float16)
        bias = n(nn)
        out = {}
        for lay in (("nt", "nn") if layout == "both" else (layout,)):
            w = n(copies, nn, k) if lay == "nt" else n(copies, k, nn)

            def fn():
                for c in range(copies):
                    if glue:
                        ctx.hgemm_fused(x.data_ptr(), w[c].data_ptr(), y.data_ptr(), m, nn, k, 1 if lay == "nt" else 0,
                                        bias=bias.data_ptr(), gelu=True)
                    else:
                        (ctx.hgemm_nt if lay == "nt" else ctx.hgemm_nn)(x.data_ptr(), w[c].data_ptr(), m, nn, k,
                                                                        out=y.data_ptr())
            out[lay + "_us_per_call"] = round(timed(fn, 3) / copies, 2)
            out[lay + "_kernel"] = ctx.get_option("last_tc_tile")
            del w
        return out
    if case in ("prefill", "decode", "decode8"):
        _, _, w, tm, embeds = build_text_model(ctx, torch, g)
        batch = 8 if case == "decode8" else 1
        reqs = [tm.request() for _ in range(batch)]
        out = {}
        for rep in range(3 if case == "prefill" else 1):
            toks = []
            for r in reqs:
                r.reset()
                t0 = time.perf_counter()
                toks.append(tm.forward(r, embeds, want_hidden=False, want_logits=False)[2])
                out["prefill_ms"] = round((time.perf_counter() - t0) * 1e3, 3)
        if case != "prefill":
            t0 = time.perf_counter()
            if batch == 1:
                tm.generate(reqs[0], toks[0], 40)
            else:
                tm.generate_batch(reqs, toks, 40)
            out["us_per_step"] = round((time.perf_counter() - t0) / 40 * 1e6, 1)
        for r in reqs:
            r.close()
        tm.close()
        return out
    crops = 13 if case == "vision13" else 1
    vw, make_vm = build_vision_model(ctx, torch, g, n)
    vm = make_vm(crops)
    img = np.random.default_rng(crops).integers(0, 256, (crops, 378, 378, 3), dtype=np.uint8)
    for _ in range(3):
        t0 = time.perf_counter()
        vm.encode(img)
        ms = (time.perf_counter() - t0) * 1e3
    vm.close()
    return {"crops": crops, "encode_ms": round(ms, 3)}


def build_text_model(ctx, torch, g):
    """Random-init Moondream2 text decoder (24 layers, dim 2048, MLP 8192, vocab 51200) generated on the device."""
    import importlib
    import __graft_entry__ as entry
    models = importlib.import_module(entry.PKG_NAME + ".models")

    def n(*shape, std=0.02):
        return (torch.randn(*shape, device="cuda", generator=g) * std).half()

    L, D, F, V = 24, 2048, 8192, 51200
    ones, zeros = torch.ones(D, device="cuda").half(), torch.zeros(D, device="cuda").half()
    w = {"ln_w": [ones] * L, "ln_b": [zeros] * L,
         "wqkv": [n(3 * D, D) for _ in range(L)], "bqkv": [n(3 * D) for _ in range(L)],
         "wout": [n(D, D) for _ in range(L)], "bout": [n(D) for _ in range(L)],
         "wfc1": [n(F, D) for _ in range(L)], "bfc1": [n(F) for _ in range(L)],
         "wfc2": [n(D, F) for _ in range(L)], "bfc2": [n(D) for _ in range(L)],
         "ln_out_w": ones, "ln_out_b": zeros, "lm_w": n(V, D), "lm_b": n(V), "wte": n(V, D)}
    tm = models.TextModel(ctx, w)
    embeds = w["wte"][torch.randint(0, V, (761,), device="cuda", generator=g)].cpu().numpy()
    return models, n, w, tm, embeds


def decode_config4(tm, embeds, sync=None):
    """Config 4 on one request: prefill of 761 rows, 200 greedy steps. Returns (prefill seconds, decode seconds), each
    the best of the repetitions that replay the captured graphs (the first two record them); `sync` (a cross-rank
    barrier) runs before the timed decode when given."""
    req = tm.request()
    pre, dec = [], []
    for rep in range(5):
        req.reset()
        t0 = time.perf_counter()
        _, _, tok = tm.forward(req, embeds, want_hidden=False, want_logits=False)
        t1 = time.perf_counter()
        pre.append(t1 - t0)
        if sync:
            sync()
            t1 = time.perf_counter()
        tm.generate(req, tok, 200)
        t2 = time.perf_counter()
        dec.append(t2 - t1)
    req.close()
    return min(pre[2:]), min(dec[2:])


def build_vision_model(ctx, torch, g, n):
    """Random-init SigLIP-style ViT + projection weights of the real shapes on the device; returns the weight dict and
    a constructor taking the crop capacity."""
    import importlib
    import __graft_entry__ as entry
    models = importlib.import_module(entry.PKG_NAME + ".models")
    Lv, Dv, Fv = 27, 1152, 4304
    onev, zerov = torch.ones(Dv, device="cuda").half(), torch.zeros(Dv, device="cuda").half()
    vw = {"ln1_w": [onev] * Lv, "ln1_b": [zerov] * Lv, "ln2_w": [onev] * Lv, "ln2_b": [zerov] * Lv,
          "wqkv": [n(Dv, 3 * Dv) for _ in range(Lv)], "bqkv": [n(3 * Dv) for _ in range(Lv)],
          "wout": [n(Dv, Dv) for _ in range(Lv)], "bout": [n(Dv) for _ in range(Lv)],
          "wfc1": [n(Dv, Fv) for _ in range(Lv)], "bfc1": [n(Fv) for _ in range(Lv)],
          "wfc2": [n(Fv, Dv) for _ in range(Lv)], "bfc2": [n(Dv) for _ in range(Lv)],
          "patch_w": n(588, Dv), "patch_b": n(Dv), "pos_emb": n(729, Dv), "norm_w": onev, "norm_b": zerov,
          "proj_fc1_w": n(2 * Dv, 8192), "proj_fc1_b": n(8192), "proj_fc2_w": n(8192, 2048), "proj_fc2_b": n(2048)}
    return vw, (lambda crops: models.VisionModel(ctx, vw, max_crops=crops))


def box_requests_extras(ctx, torch, dist, world, rank):
    """The box-scale request workload: 64 independent requests (a random 378x378 image = one crop, 32 random prompt
    tokens, 200 greedy decode steps), request i on GPU i mod world, up to 8 requests of a GPU decoding together.
    Every rank holds a full replica (random-init weights of the real shapes); no collective on the data path, the
    token ids are gathered on the host at the end.  Host wall clock around the whole job, max over ranks."""
    import importlib
    import __graft_entry__ as entry
    par = importlib.import_module(entry.PKG_NAME + ".parallel")
    g = torch.Generator(device="cuda").manual_seed(4000)
    models, n, w, tm, _ = build_text_model(ctx, torch, g)
    vw, make_vm = build_vision_model(ctx, torch, g, n)
    vm = make_vm(8)      # the eight images of a decode group go through the encoder in one pass
    n_req, n_steps = 64, 200
    rng = np.random.default_rng(5100)
    requests = [par.Request(rng.integers(0, 256, (1, 378, 378, 3), dtype=np.uint8), rng.integers(0, 51200, 32))
                for _ in range(n_req)]
    state = {}
    par.serve_requests(ctx, vm, tm, requests[:2 * world * 8], world, rank, 8, state=state)      # warm-up: graphs, buffers
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    mine = par.serve_requests(ctx, vm, tm, requests, world, rank, n_steps, state=state)
    dt = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = t.item()
    everything = par.gather_tokens(mine, n_req)
    assert len(everything) == n_req and all(len(t) == n_steps + 1 for t in everything)
    for r in state.get("reqs", []):
        r.close()
    tm.close()
    vm.close()
    del w, vw, tm, vm, state
    torch.cuda.empty_cache()
    return {"requests": n_req, "decode_steps": n_steps, "prefill_rows": 761, "crops_per_image": 1, "gpus": world,
            "streams_per_gpu": 8, "seconds": round(dt, 3), "requests_per_s": round(n_req / dt, 2),
            "decode_tok_s_aggregate": round(n_req * n_steps / dt, 1),
            "note": "whole job: vision encode (the images of a group of 8 in one pass) + 761-row prefill + 200 decode "
                    "steps per request, images and prompts copied up from host memory, token ids gathered on the host; "
                    "time = slowest rank"}


def cpu_extras(oracle):
    """The oracle (C++ restatement of the reference's AVX2 path) on this box's host cores next to the two other
    headline quantities: the 64x2048 . 2048x8192 hgemm in TFLOP/s, and decode tokens/s.  Bounded samples."""
    out = {"cores": oracle.get_threads(), "kind": "port"}
    rng = np.random.default_rng(1000)
    a = rng.standard_normal((64, 2048), dtype=np.float32).astype(np.float16)
    wkn = (rng.standard_normal((2048, 8192), dtype=np.float32) * 0.02).astype(np.float16)
    oracle.hgemm_nn(a, wkn)
    best = min(_time(lambda: oracle.hgemm_nn(a, wkn)) for _ in range(5))
    out["hgemm_64x2048x8192"] = {"us": round(best * 1e6, 1), "TFLOP/s": round(2.0 * 64 * 2048 * 8192 / best / 1e12, 4),
                                 "sample": "best of 5 (the reference's own rule, hgemm.zig:446-542)"}

    # one layer of each stage, scaled by the layer count; the decode steps run against the cache the 761-row
    # prefill of that layer has just filled, i.e. at the request's own cache lengths 762, 763, ...
    def n(*shape, std=0.02):
        return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float16)
    D, F, V = 2048, 8192, 51200
    one, zero = np.ones(D, np.float16), np.zeros(D, np.float16)
    tw = {"ln_w": [one], "ln_b": [zero], "wqkv": [n(3 * D, D)], "bqkv": [n(3 * D)], "wout": [n(D, D)], "bout": [n(D)],
          "wfc1": [n(F, D)], "bfc1": [n(F)], "wfc2": [n(D, F)], "bfc2": [n(D)], "ln_out_w": one, "ln_out_b": zero,
          "lm_w": n(V, D), "lm_b": n(V), "wte": n(V, D)}
    tm = oracle.TextModel(tw)
    embeds = n(761, D, std=1.0)
    t_prefill_layer = _time(lambda: tm.decoder(embeds))
    steps = 3
    t0 = time.perf_counter()
    for _ in range(steps):
        h = tm.decoder(tm.embed([1]))
    t_layer_step = (time.perf_counter() - t0) / steps
    t_head = _time(lambda: tm.lm_head(h))
    t_step = 24 * t_layer_step + t_head
    Dv, Fv = 1152, 4304
    onev, zerov = np.ones(Dv, np.float16), np.zeros(Dv, np.float16)
    vw = {"ln1_w": [onev], "ln1_b": [zerov], "ln2_w": [onev], "ln2_b": [zerov], "wqkv": [n(Dv, 3 * Dv)],
          "bqkv": [n(3 * Dv)], "wout": [n(Dv, Dv)], "bout": [n(Dv)], "wfc1": [n(Dv, Fv)], "bfc1": [n(Fv)],
          "wfc2": [n(Fv, Dv)], "bfc2": [n(Dv)], "patch_w": n(588, Dv), "patch_b": n(Dv), "pos_emb": n(729, Dv),
          "norm_w": onev, "norm_b": zerov, "proj_fc1_w": n(2 * Dv, 8192), "proj_fc1_b": n(8192),
          "proj_fc2_w": n(8192, 2048), "proj_fc2_b": n(2048)}
    vm = oracle.VisionModel(vw)
    patches = n(1, 729, 588, std=1.0)
    t_vis_layer = _time(lambda: vm.encoder(patches))
    f = n(729, Dv, std=1.0)
    t_proj = _time(lambda: vm.projection(f, f))
    per_request = 27 * t_vis_layer + t_proj + 24 * t_prefill_layer + t_head + 200 * t_step
    out["decode"] = {"tok_s": round(1.0 / t_step, 3), "ms_per_token": round(t_step * 1e3, 1),
                     "sample": f"{steps} decode steps of one layer at cache length 762.. x 24 layers + one lm_head"}
    out["request_extrapolated"] = {
        "seconds_per_request": round(per_request, 1), "decode_tok_s": round(1.0 / t_step, 3),
        "vision_s": round(27 * t_vis_layer + t_proj, 2), "prefill_s": round(24 * t_prefill_layer + t_head, 2),
        "decode_s": round(200 * t_step, 1),
        "sample": "one ViT layer x 27 + projection, one decoder layer over 761 rows x 24, 200 x the decode step above; "
                  "64 requests = 64 x this on one host (extrapolated, not run)"}
    return out


def _time(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def model_extras(ctx, torch):
    """End-to-end numbers of the callers around the hot path, random-init Moondream2 shapes generated on the
    device: config 4 (prefill of 761 rows, 200 greedy decode steps, single stream and 8 batched streams)
    and config 3 (vision encoder + projection for 1 / 5 / 13 crops)."""
    g = torch.Generator(device="cuda").manual_seed(4000)
    models, n, w, tm, embeds = build_text_model(ctx, torch, g)
    out = {}
    pre, dec = decode_config4(tm, embeds)
    weights_bytes = 24 * 100663296 + 209715200
    kv_bytes = 196608 * 861   # mean kv_len over steps 762..961
    out["text_config4"] = {
        "prefill_761_ms": round(pre * 1e3, 2), "decode_tok_s": round(200 / dec, 1),
        "us_per_token": round(dec / 200 * 1e6, 1),
        "hbm_GB/s": round((weights_bytes + kv_bytes) / (dec / 200) / 1e9, 1),
        "note": "host wall clock around md_text_forward (H2D of the 761 embedding rows included) and md_text_generate "
                "(200 graph replays + D2H of the tokens); best of three replayed repetitions each"}
    reqs = [tm.request() for _ in range(8)]
    for _ in range(2):
        for r in reqs:
            r.reset()
            tm.forward(r, embeds, want_hidden=False, want_logits=False)
        t1 = time.perf_counter()
        tm.generate_batch(reqs, [1] * 8, 200)
        t2 = time.perf_counter()
    out["text_config4"]["decode_tok_s_8_streams"] = round(8 * 200 / (t2 - t1), 1)
    for r in reqs:
        r.close()
    tm.close()
    del w, tm
    torch.cuda.empty_cache()

    vw, make_vm = build_vision_model(ctx, torch, g, n)
    out["vision_config3"] = []
    for crops in (1, 5, 13):
        vm = make_vm(crops)
        img = np.random.default_rng(crops).integers(0, 256, (crops, 378, 378, 3), dtype=np.uint8)
        times = []
        for _ in range(6):
            t0 = time.perf_counter()
            vm.encode(img)
            times.append(time.perf_counter() - t0)
        best = min(times[2:])    # the first two calls size the buffers and record the graph
        flops = crops * 666.4e9 + 51.98e9
        out["vision_config3"].append({"crops": crops, "ms": round(best * 1e3, 2),
                                      "TFLOP/s": round(flops / best / 1e12, 1)})
        vm.close()
    return out


if __name__ == "__main__":
    main()
