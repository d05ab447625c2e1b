"""Benchmark of the low-latency GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1  workload "c2_fp8_decode": BASELINE config 2, W8A8 FP8 y[M,14336] = x[M,4096] @ w[14336,4096]^T with per-token
       activation scales, per-channel weight scales, bf16 output. One step = the five decode GEMMs M = 1, 2, 4, 8, 16,
       each on a different weight copy (copies rotate over > 512 MB, four times the L2, so every GEMM streams its weight
       from HBM). metric = achieved HBM GB/s = algorithmic bytes of the step / device time.
N > 1  workload "c5_tp_decode_step": BASELINE config 5, tensor-parallel decode layers (hidden 8192, QKV 10240,
       gate_up 57344, down 28672) in FP8 at M = 8, sharded over the N GPUs with an NCCL all-reduce after each
       row-parallel GEMM; strong scaling; the same metric (aggregate algorithmic bytes / max-over-ranks device time).
--impl reference: the reference semantics on the host cores (dequantise, torch fp32 matmul), the only CPU
       implementation this path has (the reference itself is CUDA-only).
Prints one JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT / "sm120-lowlat-gemm_b200", ROOT):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

N_OUT, K_IN = 14336, 4096
TOKENS = (1, 2, 4, 8, 16)
TP_M = 8
TP_KIND = "fp8"
# DRAM bytes one launch of the fp8 GEMM moved in the committed ncu capture (read 58.90 MB + write 0.09 MB, mean of three
# launches); bench.py cannot run ncu itself
NCU_DRAM_BYTES_PER_LAUNCH = 58.99e6


def peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.is_file():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.stop, self.index = [], threading.Event(), index
        self.t = threading.Thread(target=self._run, daemon=True)

    def _sample(self):
        try:
            out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                 capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
            if out:
                self.rows.append([c.strip() for c in out[0].split(",")])
        except Exception:
            pass

    def _run(self):
        while not self.stop.is_set():
            self._sample()
            self.stop.wait(0.1)

    def __enter__(self):
        self.t.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.t.join(timeout=15)
        if not self.rows:
            self._sample()

    def summary(self) -> dict:
        sm = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:]) if v.lower().startswith("active")})
        mx = max((int(r[1]) for r in self.rows if r[1].isdigit()), default=0)
        return {"sm_mhz": sm[len(sm) // 2] if sm else 0, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def step_bytes() -> int:
    from lowlat_gemm import timing
    return sum(timing.algorithmic_bytes("fp8", m, N_OUT, K_IN, 2, m, N_OUT) for m in TOKENS)


# ---------------------------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference semantics; the reference has no CPU implementation of its own)


def cpu_step_seconds(reps: int) -> tuple[float, int]:
    """Median seconds of one c2 step on the host: dequantise w and x to fp32, torch.matmul, scale, round to bf16."""
    import numpy as np
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    w8 = (torch.randn(N_OUT, K_IN, generator=g) * 4).to(torch.float8_e4m3fn)
    ws = (torch.rand(N_OUT, generator=g) * 1.5 + 0.5) * 1e-3
    table = torch.from_numpy(O.E4M3_VALUES.astype(np.float32))
    xs_all = {m: torch.randn(m, K_IN, generator=g) for m in TOKENS}
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        for m in TOKENS:
            xq, s = O.quantize_fp8(xs_all[m].numpy())
            xd = table[torch.from_numpy(xq.astype(np.int64))] * torch.from_numpy(s)[:, None]
            wd = table[w8.view(torch.uint8).long()] * ws[:, None]           # dequantised weight, fp32
            y = (xd @ wd.T).to(torch.bfloat16)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], threads


def cpu_tp_layer_seconds() -> tuple[float, int, int]:
    """Seconds of ONE config-5 decode layer (TP1 shapes, FP8 weights, M = 8) on the host, and its weight bytes."""
    import numpy as np
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    table = torch.from_numpy(O.E4M3_VALUES.astype(np.float32))
    shapes = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]
    x = torch.randn(TP_M, 8192, generator=g)
    total, nbytes = 0.0, 0
    for n, k in shapes:
        w8 = torch.randint(0, 0x7E, (n, k), generator=g, dtype=torch.uint8)
        ws = torch.rand(n, generator=g) * 1e-3
        xin = torch.randn(TP_M, k, generator=g)
        t0 = time.perf_counter()
        xq, s = O.quantize_fp8(xin.numpy())
        xd = table[torch.from_numpy(xq.astype(np.int64))] * torch.from_numpy(s)[:, None]
        y = torch.empty(TP_M, n)
        for r0 in range(0, n, 8192):  # dequantise in row blocks to bound host memory
            wd = table[w8[r0:r0 + 8192].long()] * ws[r0:r0 + 8192, None]
            y[:, r0:r0 + 8192] = xd @ wd.T
        total += time.perf_counter() - t0
        nbytes += n * k
        del w8
    return total, threads, nbytes


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.gpus > 1:
        sec, threads, nbytes = cpu_tp_layer_seconds()
        gbs = nbytes / sec / 1e9
        line = {"impl": "reference", "metric": "decode_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * args.layers, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
                "config": {"workload": "c5_tp_decode_step", "hidden": 8192, "qkv": 10240, "gate_up": 57344, "down": 28672,
                           "tokens": TP_M, "layers": args.layers, "parallelism": "host cpu"},
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                 "sample": "one decode layer (4 FP8 GEMMs, M=8, TP1 shapes): dequantise + fp32 torch.matmul on the host; "
                                           "ms_per_step extrapolates to the step's layers"},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    for _ in range(min(args.warmup, 1)):
        cpu_step_seconds(1)
    reps = max(1, min(args.steps, 5))
    sec, threads = cpu_step_seconds(reps)
    gbs = step_bytes() / sec / 1e9
    line = {"impl": "reference", "metric": "decode_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
            "config": {"workload": "c2_fp8_decode", "n": N_OUT, "k": K_IN, "tokens": list(TOKENS)},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                             "sample": f"median of {reps} c2 steps (5 GEMMs each, dequantise + fp32 torch.matmul) on the host"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# N = 1: config 2


def replay_timed(graphs_and_counts, total_steps: int) -> float:
    """Replays graphs so that exactly total_steps steps run; returns device milliseconds between CUDA events."""
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    left = total_steps
    for graph, n in graphs_and_counts:
        while left >= n and n > 0:
            graph.replay()
            left -= n
    b.record()
    torch.cuda.synchronize()
    assert left == 0
    return a.elapsed_time(b)


def capture(fn_step, nsteps: int):
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(nsteps):
            fn_step(i)
    return g


def run_single(args) -> None:
    import lowlat_gemm as L
    from lowlat_gemm import timing
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L.set_pdl(not args.no_pdl)
    cold = timing.ColdWeights("fp8", N_OUT, K_IN, dev)
    gen = torch.Generator().manual_seed(0)
    x_host = {m: torch.randn(m, K_IN, generator=gen).to(torch.bfloat16).pin_memory() for m in TOKENS}
    x_dev = {m: x_host[m].to(dev) for m in TOKENS}
    xq = {m: L.quantize_fp8(x_dev[m]) for m in TOKENS}            # resident, pre-quantised inputs for `value`
    y_dev = {m: torch.empty(m, N_OUT, dtype=torch.bfloat16, device=dev) for m in TOKENS}
    y_host = {m: torch.empty(m, N_OUT, dtype=torch.bfloat16).pin_memory() for m in TOKENS}
    elems = cnts = 0
    for m in TOKENS:
        e, c = L.workspace_need("fp8", N_OUT, K_IN, m, dev)
        elems, cnts = max(elems, e), max(cnts, c)
    L.reserve_workspace(dev, elems, cnts)
    ncopies = len(cold)
    pos = [0]

    def weights():
        w, kw = cold.items[pos[0] % ncopies]
        pos[0] += 1
        return w, kw

    def kernel_step(_i):  # inputs resident in HBM
        for m in TOKENS:
            w, kw = weights()
            L.gemm(xq[m][0], w, x_scale=xq[m][1], out=y_dev[m], **kw)

    copy_stream, in_stream = torch.cuda.Stream(), torch.cuda.Stream()
    x_in = [x_dev, {m: torch.empty_like(x_dev[m]) for m in TOKENS}]  # two sets: step i+1 arrives while step i computes
    read_done = [None, None]  # event after the quantizers that read a set

    def e2e_step(i):  # the call a user makes, from pinned host activations to pinned host results
        main = torch.cuda.current_stream()
        xs = x_in[i & 1]
        if i == 0:
            read_done[0] = read_done[1] = None  # a new capture (or the eager warm-up) starts: no events carried over
        if read_done[i & 1] is None:
            in_stream.wait_stream(main)
        else:
            in_stream.wait_event(read_done[i & 1])  # the set's previous contents have been consumed
        arrived = {}
        with torch.cuda.stream(in_stream):  # inputs come in on their own stream, ahead of the GEMMs that need them
            for m in TOKENS:
                xs[m].copy_(x_host[m], non_blocking=True)
                arrived[m] = in_stream.record_event()
        for m in TOKENS:
            w, kw = weights()
            main.wait_event(arrived[m])
            q, s = L.quantize_fp8(xs[m])
            if m == TOKENS[-1]:
                read_done[i & 1] = main.record_event()
            L.gemm(q, w, x_scale=s, out=y_dev[m], **kw)
            copy_stream.wait_stream(main)          # results leave on a second stream while the next GEMM runs
            with torch.cuda.stream(copy_stream):
                y_host[m].copy_(y_dev[m], non_blocking=True)
        main.wait_stream(copy_stream)
        main.wait_stream(in_stream)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kernel_step(0)
        e2e_step(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    chunk = min(args.steps, 64)
    rem = args.steps % chunk
    with torch.cuda.stream(side):
        graphs = [(capture(kernel_step, chunk), chunk)] + ([(capture(kernel_step, rem), rem)] if rem else [])
        egraphs = [(capture(e2e_step, chunk), chunk)] + ([(capture(e2e_step, rem), rem)] if rem else [])
    torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        graphs[0][0].replay()
        egraphs[0][0].replay()
    torch.cuda.synchronize()
    with ClockSampler(0) as clk:
        ms = replay_timed(graphs, args.steps)
        ms_e2e = replay_timed(egraphs, args.steps)
        if ms + ms_e2e < 400:  # keep the GPU busy long enough for the sampler to see loaded clocks
            t_end = time.time() + 0.5
            while time.time() < t_end:
                graphs[0][0].replay()
            torch.cuda.synchronize()
    sb = step_bytes()
    value = sb * args.steps / (ms * 1e-3) / 1e9
    e2e = sb * args.steps / (ms_e2e * 1e-3) / 1e9
    launches = args.steps * len(TOKENS)
    pk = peaks()
    per_launch_bytes = sb / len(TOKENS)
    per_launch_us = ms * 1e3 / launches
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
    cpu_sec, threads = cpu_step_seconds(3)
    from lowlat_gemm import _native
    status = _native.device_status()
    line = {
        "metric": "decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {"workload": "c2_fp8_decode", "n": N_OUT, "k": K_IN, "tokens": list(TOKENS), "out": "bf16",
                   "cold_weights": f"{ncopies} weight copies rotate ({ncopies * cold.nbytes >> 20} MB > 4x L2)",
                   "pdl": L.pdl_enabled(), "launch": "cuda_graph", "us_per_gemm": per_launch_us,
                   "pct_of_8tbs": 100 * value / 8000.0},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": sum(m * K_IN * 2 for m in TOKENS),
                "d2h_bytes_per_step": sum(m * N_OUT * 2 for m in TOKENS), "ms_per_step": ms_e2e / args.steps,
                "path": "pinned host x -> H2D (own stream, one step ahead) -> quantize_fp8 -> gemm -> D2H pinned y (copy-out on a second stream), captured in a CUDA graph"},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "peak_source": pk["source"],
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, profiles/umma_gemm_fp8_c2_decode.md",
                     "kernel": "umma_gemm_kernel<FAM_F8,16,2>", "algorithmic_bytes_per_launch": per_launch_bytes},
        "cpu_baseline": {"value": sb / cpu_sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "median of 3 c2 steps (5 GEMMs each, dequantise + fp32 torch.matmul) on the host"},
        "clocks": clk.summary(), "device_status": status,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# N > 1: config 5, tensor-parallel decode step


def _progress(msg: str) -> None:
    """Progress marker for multi-rank runs (rank 0 only), flushed at once so a stalled run shows where it stopped."""
    if os.environ.get("RANK", "0") == "0":
        print(f"[bench {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def run_tp(args) -> None:
    import torch.distributed as dist
    import lowlat_gemm as L
    from lowlat_gemm import tp as TP
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=dev)
    _progress("process group up")
    L.set_pdl(not args.no_pdl)
    layers = args.layers
    comm, comm_note = None, ("nccl all_reduce" if multi else "none (one rank)")
    if args.allreduce in ("auto", "oneshot") and multi:
        # the library's own one-shot all-reduce over peer memory; "auto" falls back to NCCL on every rank together
        # when the peer mappings cannot be set up on any of them
        from lowlat_gemm import comm as CM
        try:
            comm = CM.OneShotAllReduce(None, dev, max_bytes=TP_M * 8192 * 2, ctas=16)
            failed = ""
        except Exception as exc:  # noqa: BLE001 - any setup failure means "use NCCL"
            if args.allreduce == "oneshot":
                raise
            failed = type(exc).__name__
        flag = torch.tensor([0 if failed else 1], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 1:
            comm_note = "one-shot peer-memory all-reduce"
        else:
            comm = None
            comm_note = "nccl all_reduce (peer-memory setup failed" + (f": {failed})" if failed else " on another rank)")
    step = TP.DecodeStep(TP_KIND, layers, world, rank, dev, prefetch_bytes=0, comm=comm)
    _progress("weights built")
    x = torch.randn(TP_M, step.shape.hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).to(torch.bfloat16) * 0.05
    elems = cnts = 0
    for n, k in step.shape.shards(world).values():
        e, c = L.workspace_need(TP_KIND, n, k, TP_M, dev)
        elems, cnts = max(elems, e), max(cnts, c)
    L.reserve_workspace(dev, elems, cnts)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step.run(x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    if comm is not None:
        # a bounded wait that expired in the library's all-reduce shows in the device status word: then every rank
        # goes back to NCCL together instead of timing waits
        from lowlat_gemm import _native as NV
        bad = torch.tensor([NV.device_status()], device=dev, dtype=torch.int32)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) != 0:
            comm, comm_note = None, f"nccl all_reduce (the library's all-reduce reported status {int(bad.item())} in the warm-up)"
            step = TP.DecodeStep(TP_KIND, layers, world, rank, dev, prefetch_bytes=0, comm=None)
            with torch.cuda.stream(side):
                step.run(x)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
    _progress("eager warm-up done")
    step.gemms = step.collectives = step.quants = 0
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step.run(x)
    gemms_per_step = step.gemms
    # the library's own launches per step: GEMMs, quantizer / gated-activation kernels, and its all-reduces
    own_per_step = step.gemms + step.quants + (step.collectives if comm is not None else 0)
    _progress("step captured")
    # end to end: the step's activations come from pinned host memory and its result goes back there, every step
    x_host = x.cpu().pin_memory()
    y_host = torch.empty(TP_M, step.shape.hidden, dtype=torch.bfloat16).pin_memory()
    with torch.cuda.stream(side):
        egraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(egraph):
            x.copy_(x_host, non_blocking=True)
            y_host.copy_(step.run(x), non_blocking=True)
    _progress("e2e step captured")
    for _ in range(max(args.warmup, 3)):
        graph.replay()
        egraph.replay()
    torch.cuda.synchronize()
    _progress("graph warm-up done")

    def timed(gr) -> float:
        if multi:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device=dev)
        if multi:
            dist.barrier()
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with ClockSampler(local) as clk:
        ms = timed(graph)
        ms_e2e = timed(egraph)
    total_bytes = step.weight_bytes() * world  # every rank streams its shard; activations are negligible
    if rank == 0:
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        pk = peaks()
        line = {"metric": "decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
                "config": {"workload": "c5_tp_decode_step", "hidden": 8192, "qkv": 10240, "gate_up": 57344, "down": 28672,
                           "tokens": TP_M, "layers": layers, "parallelism": f"tp{world}",
                           "collective": comm_note + (" x2 per layer" if multi else ""),
                           "us_per_layer": ms * 1e3 / args.steps / layers, "pdl": L.pdl_enabled(), "launch": "cuda_graph",
                           "cold_weights": f"{layers} layers of distinct weights ({step.weight_bytes() >> 20} MB per rank)"},
                "e2e": {"value": total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": TP_M * 8192 * 2, "d2h_bytes_per_step": TP_M * 8192 * 2,
                        "ms_per_step": ms_e2e / args.steps,
                        "path": "pinned host x -> H2D -> decode layers (quantize_fp8 + gemm + all_reduce) -> D2H pinned y, in a CUDA graph"},
                "gpu_launches": args.steps * own_per_step,
                "roofline": {"bound": "hbm", "achieved": value / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": value / world / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                             "note": "per-GPU weight bytes of the step / step time, collectives included"},
                "cpu_baseline": None, "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    # CUDA graphs that hold NCCL kernels must go before the communicator does, or teardown can block; a watchdog ends
    # the process in any case once the result is out
    if not multi:
        return
    threading.Timer(30.0, lambda: os._exit(0)).start()
    del graph, egraph
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--allreduce", choices=("auto", "nccl", "oneshot"), default="auto")
    ap.add_argument("--workload", choices=("auto", "c2", "c5"), default="auto",
                    help="auto: config 2 on one GPU, config 5 (tensor-parallel decode step) on several")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.workload == "c5":
        run_tp(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
