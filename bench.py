"""Benchmark of the low-latency GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload auto|c2|c5] [--kind fp8|bf16|nvfp4] [--tokens M] [--layers L] [--allreduce ...]

N = 1  workload "c2_fp8_decode": W8A8 FP8 y[M,14336] = x[M,4096] @ w[14336,4096]^T with per-token activation scales,
       per-channel weight scales, bf16 output. One step = the five decode GEMMs M = 1, 2, 4, 8, 16, each on a different
       weight copy (copies rotate over > 512 MB, four times the L2, so every GEMM streams its weight from HBM).
       metric = achieved HBM GB/s = algorithmic bytes of the step / device time. The line also carries one row per
       other precision (bf16, int8, nvfp4, W4A16, W8A16 at M = 1 and 16) and the tensor-parallel decode step at TP1.
N > 1  workload "c5_tp_decode_step": tensor-parallel decode layers (hidden 8192, QKV 10240, gate_up 57344, down 28672),
       FP8 at M = 8 unless --kind / --tokens say otherwise, sharded over the N GPUs, one sum over ranks after each
       row-parallel GEMM; strong scaling; the same metric (aggregate weight bytes / max-over-ranks device time). Rank 0
       also times the same step on one GPU afterwards, so every line carries its own TP1 figure and speed-up.
--impl reference: the reference semantics on the host cores (dequantise, torch fp32 matmul), the only CPU
       implementation this path has (the reference itself is CUDA-only).
Timing: the step is captured in CUDA graphs; rounds of exactly --steps steps are replayed between CUDA events until at
least 0.25 s have been timed; the median round gives the reported numbers, the fastest is reported beside it.
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
MIN_TIMED_SECONDS = 0.25
# DRAM bytes one launch of the fp8 GEMM moved in the committed profiler capture (read 58.90 MB + write 0.09 MB, mean of
# three launches); bench.py cannot run the profiler itself
NCU_DRAM_BYTES_PER_LAUNCH = 58.99e6
# one row per precision beside the headline: (kind, N, K)
KIND_ROWS = (("bf16", 11008, 4096), ("int8", 4096, 4096), ("w8a16_bf16", 14336, 4096), ("nvfp4", 28672, 8192),
             ("w4a16_bf16", 28672, 8192))
TP_SHAPES = ((10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672))  # qkv, o, gate_up, down at TP1


def peaks() -> dict:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.is_file():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


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


def c2_step_bytes() -> int:
    """Algorithmic bytes of one c2 step; the formula of the oracle, so the CPU arm needs nothing of the CUDA package."""
    from oracle import oracle as O
    return sum(O.gemm_bytes("fp8", m, N_OUT, K_IN, 2, m, N_OUT) for m in TOKENS)


def timed_rounds(replay_round, steps: int, barrier=None, reduce_max=None) -> dict:
    """Replays rounds of exactly `steps` steps between CUDA events until MIN_TIMED_SECONDS have been timed (at least
    three rounds). With several ranks every round starts at a barrier and counts as its slowest rank."""
    times, total = [], 0.0
    while len(times) < 3 or (total < MIN_TIMED_SECONDS * 1e3 and len(times) < 2000):
        if barrier is not None:
            barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        replay_round()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if reduce_max is not None:
            ms = reduce_max(ms)
        times.append(ms)
        total += ms
    times.sort()
    return {"ms_median": times[len(times) // 2], "ms_min": times[0], "rounds": len(times), "timed_ms": total, "steps": steps}


# ---------------------------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference semantics; the reference has no CPU implementation of its own)


def cpu_c2_step(reps: int) -> dict:
    """One c2 step on the host, median of `reps`: quantize x, dequantise x and w to fp32, torch.matmul, round to bf16.
    Reported twice: with the weight's dequantisation inside the timed region, and with the weight dequantised before."""
    import numpy as np
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    w8 = (torch.randn(N_OUT, K_IN, generator=g) * 4).to(torch.float8_e4m3fn)
    ws = (torch.rand(N_OUT, generator=g) * 1.5 + 0.5) * 1e-3
    table = torch.from_numpy(O.E4M3_VALUES.astype(np.float32))
    xs_all = {m: torch.randn(m, K_IN, generator=g) for m in TOKENS}

    def act(m):
        xq, s = O.quantize_fp8(xs_all[m].numpy())
        return table[torch.from_numpy(xq.astype(np.int64))] * torch.from_numpy(s)[:, None]

    def dequant_w():
        return table[w8.view(torch.uint8).long()] * ws[:, None]

    incl, excl = [], []
    for _ in range(reps):
        t0 = time.perf_counter()
        for m in TOKENS:
            (act(m) @ dequant_w().T).to(torch.bfloat16)
        incl.append(time.perf_counter() - t0)
    wd = dequant_w()
    for _ in range(reps):
        t0 = time.perf_counter()
        for m in TOKENS:
            (act(m) @ wd.T).to(torch.bfloat16)
        excl.append(time.perf_counter() - t0)
    incl.sort()
    excl.sort()
    return {"seconds": incl[len(incl) // 2], "seconds_dequant_excluded": excl[len(excl) // 2], "threads": threads, "reps": reps}


def cpu_tp_layer(tokens: int) -> dict:
    """ONE decode layer (TP1 shapes, FP8 weights) on the host: seconds, and the weight bytes it streams."""
    import numpy as np
    from oracle import oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    table = torch.from_numpy(O.E4M3_VALUES.astype(np.float32))
    total, nbytes = 0.0, 0
    for n, k in TP_SHAPES:
        w8 = torch.randint(0, 0x7E, (n, k), generator=g, dtype=torch.uint8)
        ws = torch.rand(n, generator=g) * 1e-3
        xin = torch.randn(tokens, k, generator=g)
        t0 = time.perf_counter()
        xq, s = O.quantize_fp8(xin.numpy())
        xd = table[torch.from_numpy(xq.astype(np.int64))] * torch.from_numpy(s)[:, None]
        y = torch.empty(tokens, n)
        for r0 in range(0, n, 8192):  # dequantise in row blocks to bound host memory
            wd = table[w8[r0:r0 + 8192].long()] * ws[r0:r0 + 8192, None]
            y[:, r0:r0 + 8192] = xd @ wd.T
        total += time.perf_counter() - t0
        nbytes += n * k
        del w8
    return {"seconds": total, "threads": threads, "bytes": nbytes}


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if args.gpus > 1 or args.workload == "c5":
        # one "step" of this arm is one decode layer; the number of steps actually run is what the line reports
        steps = max(1, min(args.steps, 3))
        runs = sorted((cpu_tp_layer(args.tokens) for _ in range(steps)), key=lambda r: r["seconds"])
        meta = runs[len(runs) // 2]
        sec = meta["seconds"]
        gbs = meta["bytes"] / sec / 1e9
        line = {"impl": "reference", "metric": "decode_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": 0, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
                "config": {"workload": "c5_tp_decode_step", "hidden": 8192, "qkv": 10240, "gate_up": 57344, "down": 28672,
                           "tokens": args.tokens, "layers": 1, "parallelism": "host cpu",
                           "note": "a step of this arm is ONE decode layer (4 FP8 GEMMs, TP1 shapes); steps = layers actually run"},
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": meta["threads"], "kind": "port",
                                 "sample": f"median of {steps} decode layers: dequantise + fp32 torch.matmul on the host"},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return
    for _ in range(min(args.warmup, 1)):
        cpu_c2_step(1)
    reps = max(1, min(args.steps, 5))
    r = cpu_c2_step(reps)
    sb = c2_step_bytes()
    gbs = sb / r["seconds"] / 1e9
    line = {"impl": "reference", "metric": "decode_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": reps, "warmup": min(args.warmup, 1), "ms_per_step": r["seconds"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
            "config": {"workload": "c2_fp8_decode", "n": N_OUT, "k": K_IN, "tokens": list(TOKENS)},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": r["threads"], "kind": "port",
                             "value_dequant_excluded": sb / r["seconds_dequant_excluded"] / 1e9,
                             "sample": f"median of {reps} c2 steps (5 GEMMs each) on the host; value: weight dequantisation + fp32 "
                                       "torch.matmul timed together, value_dequant_excluded: matmul on a weight dequantised beforehand"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# shared pieces of the GPU arms


def capture(fn_step, nsteps: int, finish=None):
    """nsteps calls of fn_step in one CUDA graph; `finish` joins whatever side streams the steps forked."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(nsteps):
            fn_step(i)
        if finish is not None:
            finish()
    return g


def replayer(graphs_and_counts, total_steps: int):
    """A callable that replays the captured graphs so that exactly total_steps steps run."""
    plan, left = [], total_steps
    for graph, n in graphs_and_counts:
        while n > 0 and left >= n:
            plan.append(graph)
            left -= n
    assert left == 0

    def run():
        for g in plan:
            g.replay()
    return run


def kind_rows(dev, pk: dict) -> list:
    """One row per other precision at M = 1 and 16: microseconds per GEMM over cold weights (a CUDA graph of calls on
    rotating weight copies, median of five replays), achieved GB/s from the algorithmic bytes, fraction of the measured
    copy bandwidth."""
    import lowlat_gemm as L
    from lowlat_gemm import api, timing
    rows = []
    for kind, n, k in KIND_ROWS:
        cold = timing.ColdWeights(kind, n, k, dev)
        e, c = L.workspace_need(kind, n, k, 16, dev)
        L.reserve_workspace(dev, e, c)
        for m in (1, 16):
            x, x_kw = timing.make_input(kind, m, k, dev)
            out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            us = timing.time_per_call(lambda w, kw, nxt: L.gemm(x, w, out=out, **kw, **x_kw), cold, replays=5)
            xs, ws = (m, n) if kind in ("fp8", "int8") else (0, n) if kind.startswith("w8a16") else (0, 0)
            nbytes = timing.algorithmic_bytes(kind, m, n, k, 2, xs, ws, 0)
            gbs = nbytes / us / 1e3
            plan = L.get_plan(kind, n, k, dev)
            engine = "skinny" if plan.skinny is not None and m <= min(plan.skinny_max_m, 16) else "tcgen05"
            rows.append({"kind": kind, "n": n, "k": k, "m": m, "us": us, "gbs": gbs, "frac": gbs / pk["hbm_gbs"],
                         "pct_of_8tbs": gbs / 80.0, "engine": engine})
        del cold
        torch.cuda.empty_cache()
    # the tensor-bound end of the same entry point: hundreds to thousands of token rows (256-row tiles on CTA pairs);
    # bf16 against the measured cuBLAS bf16 rate, fp8 against the nominal dense rate (no measured figure exists)
    for kind, n, k, peak, peak_name in (("bf16", 11008, 4096, pk["bf16_tflops"], "measured cuBLAS bf16 burst"),
                                        ("fp8", 14336, 4096, 4500.0, "nominal dense fp8")):
        cold = timing.ColdWeights(kind, n, k, dev)
        for m in (256, 2048):
            x, x_kw = timing.make_input(kind, m, k, dev)
            out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            us = timing.time_per_call(lambda w, kw, nxt: L.gemm(x, w, out=out, **kw, **x_kw), cold, calls=16, replays=5)
            tf = 2.0 * m * n * k / us / 1e6
            choice = api.tc_choice_for(kind, m, n, k, L.get_plan(kind, n, k, dev), dev)
            rows.append({"kind": kind, "n": n, "k": k, "m": m, "us": us, "tflops": tf, "bound": "tensor", "peak_tflops": peak,
                         "peak": peak_name, "frac": tf / peak, "engine": "tcgen05 cta_group::2" if choice.cfg in L.PAIR_CFGS else "tcgen05"})
        del cold
        torch.cuda.empty_cache()
    return rows


class TpRun:
    """The tensor-parallel decode step of one rank, captured in a CUDA graph: weights, the library's all-reduce in its
    push form (also on one rank, where the same kernels run over local memory), residual stream."""

    def __init__(self, kind: str, tokens: int, layers: int, world: int, rank: int, dev, allreduce: str, group=None):
        import lowlat_gemm as L
        from lowlat_gemm import comm as CM, tp as TP
        self.kind, self.tokens, self.layers, self.world, self.dev = kind, tokens, layers, world, dev
        self.note = "none (one rank)" if world == 1 else "nccl all_reduce"
        comm = None
        if allreduce in ("auto", "push", "pull"):
            comm = CM.OneShotAllReduce(group, dev, max_bytes=tokens * 8192 * 2, ctas=16, local=world == 1)
            form = "pull" if allreduce == "pull" else "push"
            self.note = {"push": "pushed from the row-parallel GEMM's epilogue, local sum + residual + quantizer in one kernel",
                         "pull": "one-shot peer-memory all-reduce kernel"}[form] + (" (one rank: local memory)" if world == 1 else "")
        self.form = "nccl" if comm is None else form
        self.step = TP.DecodeStep(kind, layers, world, rank, dev, prefetch_bytes=0, comm=comm, residual=True,
                                  push=comm is not None and form == "push")
        self.x = (torch.randn(tokens, self.step.shape.hidden, device=dev,
                              generator=torch.Generator(device=dev).manual_seed(1)) * 0.05).to(torch.bfloat16)
        elems = cnts = 0
        for n, k in self.step.shape.shards(world).values():
            e, c = L.workspace_need(kind, n, k, tokens, dev)
            elems, cnts = max(elems, e), max(cnts, c)
        L.reserve_workspace(dev, elems, cnts)
        self.side = torch.cuda.Stream()

    def eager(self, times: int = 2) -> torch.Tensor:
        self.side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.side):
            for _ in range(times):
                y = self.step.run(self.x)
        torch.cuda.current_stream().wait_stream(self.side)
        torch.cuda.synchronize()
        return y

    def capture(self):
        st = self.step
        st.gemms = st.collectives = st.quants = st.reduces = 0
        with torch.cuda.stream(self.side):
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.y = st.run(self.x)
        # launches of the library's own kernels per step: GEMMs, quantizer / gated-activation kernels, sum kernels
        self.own_launches = st.gemms + st.quants + st.reduces
        self.x_host = self.x.cpu().pin_memory()
        self.y_host = torch.empty(self.tokens, st.shape.hidden, dtype=torch.bfloat16).pin_memory()
        with torch.cuda.stream(self.side):
            self.egraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.egraph):
                self.x.copy_(self.x_host, non_blocking=True)
                self.y_host.copy_(st.run(self.x), non_blocking=True)
        torch.cuda.synchronize()

    def weight_bytes(self) -> int:
        return self.step.weight_bytes()


def tp1_record(dev, kind: str, tokens: int, layers: int, steps: int) -> dict:
    """The decode step on ONE GPU with the same kernels the multi-GPU step uses: the like-for-like base of the scaling."""
    run = TpRun(kind, tokens, layers, 1, 0, dev, "push")
    run.eager()
    run.capture()
    for _ in range(3):
        run.graph.replay()
    torch.cuda.synchronize()
    t = timed_rounds(lambda: [run.graph.replay() for _ in range(steps)], steps)
    ms_step = t["ms_median"] / steps
    rec = {"kind": kind, "tokens": tokens, "layers": layers, "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3 / layers,
           "gbs": run.weight_bytes() / (ms_step * 1e-3) / 1e9, "launches_per_step": run.own_launches, "rounds": t["rounds"]}
    del run
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------------------------------------------
# N = 1: the FP8 decode GEMMs


def run_single(args) -> None:
    import lowlat_gemm as L
    from lowlat_gemm import _native, timing
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L.set_pdl(not args.no_pdl)
    cold = timing.ColdWeights("fp8", N_OUT, K_IN, dev)
    gen = torch.Generator().manual_seed(0)
    # the step's activations: one pinned host matrix holding the five token groups one after the other
    rows_of, at = {}, 0
    for m in TOKENS:
        rows_of[m] = slice(at, at + m)
        at += m
    x_host_all = torch.randn(at, K_IN, generator=gen).to(torch.bfloat16).pin_memory()
    x_host = {m: x_host_all[rows_of[m]] for m in TOKENS}
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
    x_in = [torch.empty(at, K_IN, dtype=torch.bfloat16, device=dev) for _ in range(2)]  # two sets: step i+1 arrives while step i computes
    read_done = [None, None]  # event after the GEMMs of the step that used a set

    keep = []  # quantized inputs stay referenced while the graphs that use them live
    y_sets = [y_dev, {m: torch.empty_like(y_dev[m]) for m in TOKENS}]  # results of step i leave while step i + 1 computes
    copied = [None, None]  # event after the copy-out of the step that used a result set

    def e2e_step(i):  # the calls a user makes, from pinned host activations to pinned host results
        # Input side (its own stream, at most two steps ahead of the GEMMs): H2D copy of the step's activations and
        # their quantize_fp8. Compute side: the step's five gemm() calls as one chain of dependent launches. Output
        # side (a third stream): D2H of each result, behind the GEMMs by at most two steps.
        main = torch.cuda.current_stream()
        xs, ys = x_in[i & 1], y_sets[i & 1]
        if i == 0:  # a new capture (or the eager warm-up) starts: no events carried over
            read_done[0] = read_done[1] = copied[0] = copied[1] = None
        if read_done[i & 1] is None:
            in_stream.wait_stream(main)
        else:
            in_stream.wait_event(read_done[i & 1])  # the GEMMs of step i - 2 are done: bounded look-ahead
        with torch.cuda.stream(in_stream):
            # one copy and one quantize_fp8 call for the step's 31 token rows (the quantizer works row by row, so the
            # groups' results are what five separate calls would give); a copy and a launch per group made this
            # stream, not the GEMMs, the step's critical path (87 against 55 us)
            xs.copy_(x_host_all, non_blocking=True)
            q_all, s_all = L.quantize_fp8(xs)
            qs = {m: (q_all[rows_of[m]], s_all[rows_of[m]]) for m in TOKENS}
            arrived = in_stream.record_event()
        keep.append((q_all, s_all))
        main.wait_event(arrived)  # one join per step: the GEMM chain below stays a chain of programmatic launches
        if copied[i & 1] is not None:
            main.wait_event(copied[i & 1])  # the results of step i - 2 have left this set
        for m in TOKENS:
            w, kw = weights()
            q, sc = qs[m]
            L.gemm(q, w, x_scale=sc, out=ys[m], **kw)
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                y_host[m].copy_(ys[m], non_blocking=True)
        read_done[i & 1] = main.record_event()
        copied[i & 1] = copy_stream.record_event()

    def e2e_finish():  # every forked stream rejoins the capturing stream
        main = torch.cuda.current_stream()
        main.wait_stream(copy_stream)
        main.wait_stream(in_stream)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kernel_step(0)
        e2e_step(0)
        e2e_finish()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    chunk = min(args.steps, 64)
    rem = args.steps % chunk
    with torch.cuda.stream(side):
        graphs = [(capture(kernel_step, chunk), chunk)] + ([(capture(kernel_step, rem), rem)] if rem else [])
        egraphs = [(capture(e2e_step, chunk, e2e_finish), chunk)] + ([(capture(e2e_step, rem, e2e_finish), rem)] if rem else [])
    torch.cuda.synchronize()
    warm = max(args.warmup, 3)
    for _ in range(warm):
        graphs[0][0].replay()
        egraphs[0][0].replay()
    torch.cuda.synchronize()
    with ClockSampler(0) as clk:
        t_dev = timed_rounds(replayer(graphs, args.steps), args.steps)
        t_e2e = timed_rounds(replayer(egraphs, args.steps), args.steps)
    status = _native.device_status()
    sb = c2_step_bytes()
    ms, ms_e2e = t_dev["ms_median"], t_e2e["ms_median"]
    value = sb * args.steps / (ms * 1e-3) / 1e9
    e2e = sb * args.steps / (ms_e2e * 1e-3) / 1e9
    launches_per_round = args.steps * len(TOKENS)
    pk = peaks()
    per_launch_bytes = sb / len(TOKENS)
    per_launch_us = ms * 1e3 / launches_per_round
    achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
    del graphs, egraphs, cold
    torch.cuda.empty_cache()
    # the other precisions and the one-GPU decode step, each timed on its own after the headline
    rows = [] if args.no_extras else kind_rows(dev, pk)
    tp1 = None if args.no_extras else tp1_record(dev, args.kind, args.tokens, args.layers, 10)
    status = max(status, _native.device_status())
    cpu = cpu_c2_step(3)
    line = {
        "metric": "decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8", "data": "synthetic",
        "config": {"workload": "c2_fp8_decode", "n": N_OUT, "k": K_IN, "tokens": list(TOKENS), "out": "bf16",
                   "cold_weights": f"{ncopies} weight copies rotate ({ncopies * timing.weight_bytes('fp8', N_OUT, K_IN) >> 20} MB > 4x L2)",
                   "pdl": L.pdl_enabled(), "launch": "cuda_graph", "us_per_gemm": per_launch_us,
                   "us_per_gemm_fastest_round": t_dev["ms_min"] * 1e3 / launches_per_round,
                   "pct_of_8tbs": 100 * value / 8000.0,
                   "timing": {"rounds": t_dev["rounds"], "steps_per_round": args.steps, "timed_ms": t_dev["timed_ms"],
                              "statistic": "median round"},
                   "kinds": rows, "tp1_step": tp1},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": sum(m * K_IN * 2 for m in TOKENS),
                "d2h_bytes_per_step": sum(m * N_OUT * 2 for m in TOKENS), "ms_per_step": ms_e2e / args.steps,
                "rounds": t_e2e["rounds"],
                "path": "pinned host x (the step's 31 token rows) -> one H2D copy + one quantize_fp8 call on an input stream, at most two steps ahead -> the step's five gemm() calls as one dependent chain -> D2H of each result to pinned y on a third stream; every step's copies and quantizer are inside the timed CUDA graph"},
        "gpu_launches": launches_per_round * t_dev["rounds"], "gpu_launches_per_round": launches_per_round,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "peak_source": pk["source"],
                     "traffic_source": "constant: dram__bytes_read.sum + dram__bytes_write.sum per launch of the committed profiler "
                                       "capture of this kernel and shape, not measured by this run",
                     "kernel": "umma_gemm_kernel<FAM_F8,16,2>", "algorithmic_bytes_per_launch": per_launch_bytes},
        "cpu_baseline": {"value": sb / cpu["seconds"] / 1e9, "unit": "GB/s", "cores": cpu["threads"], "kind": "port",
                         "value_dequant_excluded": sb / cpu["seconds_dequant_excluded"] / 1e9,
                         "sample": "median of 3 c2 steps (5 GEMMs each, dequantise + fp32 torch.matmul) on the host"},
        "clocks": clk.summary(), "device_status": status,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
# N > 1 (or --workload c5): tensor-parallel decode step


def _progress(msg: str) -> None:
    """Progress marker for multi-rank runs (rank 0 only), flushed at once so a stalled run shows where it stopped."""
    if os.environ.get("RANK", "0") == "0":
        print(f"[bench {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def run_tp(args) -> None:
    import torch.distributed as dist
    import lowlat_gemm as L
    from lowlat_gemm import _native as NV
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=dev)
    _progress("process group up")
    L.set_pdl(not args.no_pdl)
    kind, tokens, layers = args.kind, args.tokens, args.layers

    def all_max(v: float) -> float:
        if not multi:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # the library's own all-reduce; "auto" falls back to NCCL on every rank together when the peer mappings cannot be
    # set up on any of them, or when a bounded wait expired in the warm-up
    want = args.allreduce
    run, fallback = None, ""
    if want != "nccl":
        try:
            run = TpRun(kind, tokens, layers, world, rank, dev, want)
            failed = 0.0
        except Exception as exc:  # noqa: BLE001 - any setup failure means "use NCCL"
            if want != "auto":
                raise
            failed, fallback = 1.0, f"peer-memory setup failed: {type(exc).__name__}"
        if all_max(failed) > 0:
            run, fallback = None, fallback or "peer-memory setup failed on another rank"
    if run is not None:
        run.eager()
        bad = all_max(float(NV.device_status()))
        if bad > 0 and want == "auto":
            run, fallback = None, f"the library's all-reduce reported status {int(bad)} in the warm-up"
    if run is None:
        run = TpRun(kind, tokens, layers, world, rank, dev, "nccl")
        run.eager()
    _progress("weights built, eager warm-up done")

    # one step checked before anything is timed: the step with the library's all-reduce against the same step (same
    # weights, same input) with NCCL's, on every rank
    check = {"against": "same step over torch.distributed.all_reduce", "max_rel_diff": None, "ok": None}
    if multi and run.form != "nccl":
        from lowlat_gemm import tp as TP
        y_lib = run.eager(1).float()
        ref_step = TP.DecodeStep(kind, layers, world, rank, dev, prefetch_bytes=0, comm=None, residual=True)
        ref_step.layers = run.step.layers  # the very same weight shards
        y_ref = ref_step.run(run.x).float()
        torch.cuda.synchronize()
        rel = float(((y_lib - y_ref).abs().max() / y_ref.abs().max().clamp_min(1e-6)).item())
        finite = bool(torch.isfinite(y_lib).all().item())
        rel = all_max(rel if finite else float("inf"))
        # bf16 partials are rounded before NCCL adds them and the library adds them in fp32: a few bf16 ulps per layer.
        # With NVFP4 activations such an ulp can move a value across a 4-bit quantization boundary in the next
        # projection, so two equally valid orders of summation differ by a 4-bit step here and there: wider bound.
        bound = 1e-1 if kind == "nvfp4" else 3e-2
        check.update(max_rel_diff=rel, bound=bound, ok=bool(rel < bound))
        del ref_step
    run.capture()
    _progress("step captured")
    for _ in range(max(args.warmup, 3)):
        run.graph.replay()
        run.egraph.replay()
    torch.cuda.synchronize()
    barrier = dist.barrier if multi else None
    with ClockSampler(local) as clk:
        t_dev = timed_rounds(lambda: [run.graph.replay() for _ in range(args.steps)], args.steps, barrier, all_max)
        t_e2e = timed_rounds(lambda: [run.egraph.replay() for _ in range(args.steps)], args.steps, barrier, all_max)
    status = int(all_max(float(NV.device_status())))
    _progress("timed")
    total_bytes = run.weight_bytes() * world  # every rank streams its shard; activations are negligible
    own, form, note, wb = run.own_launches, run.form, run.note + (f"; fell back: {fallback}" if fallback else ""), run.weight_bytes()
    tp1 = None
    if rank == 0 and multi and not args.no_extras:
        # the same step on ONE GPU (rank 0 alone, the others wait): the base the speed-up of this line refers to
        del run
        torch.cuda.empty_cache()
        tp1 = tp1_record(dev, kind, tokens, layers, args.steps)
        _progress("TP1 timed")
    if rank == 0:
        ms = t_dev["ms_median"]
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        us_layer = ms * 1e3 / args.steps / layers
        pk = peaks()
        line = {"metric": "decode_gemm_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": kind, "data": "synthetic",
                "config": {"workload": "c5_tp_decode_step", "hidden": 8192, "qkv": 10240, "gate_up": 57344, "down": 28672,
                           "kind": kind, "tokens": tokens, "layers": layers, "parallelism": f"tp{world}", "residual": True,
                           "collective": note + (" x2 per layer" if multi else ""), "allreduce_form": form,
                           "us_per_layer": us_layer, "us_per_layer_fastest_round": t_dev["ms_min"] * 1e3 / args.steps / layers,
                           "pdl": L.pdl_enabled(), "launch": "cuda_graph",
                           "cold_weights": f"{layers} layers of distinct weights ({wb >> 20} MB per rank)",
                           "timing": {"rounds": t_dev["rounds"], "steps_per_round": args.steps, "timed_ms": t_dev["timed_ms"],
                                      "statistic": "median round, each round the max over ranks"},
                           "tp1_step": tp1,
                           "speedup_vs_tp1": (tp1["us_per_layer"] / us_layer) if tp1 else None},
                "e2e": {"value": total_bytes * args.steps / (t_e2e["ms_median"] * 1e-3) / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": tokens * 8192 * 2, "d2h_bytes_per_step": tokens * 8192 * 2,
                        "ms_per_step": t_e2e["ms_median"] / args.steps,
                        "path": "pinned host x -> H2D -> decode layers (quantizer, gemm, sum over ranks, residual) -> D2H pinned y, in a CUDA graph"},
                "gpu_launches": args.steps * own * t_dev["rounds"], "gpu_launches_per_step": own,
                "roofline": {"bound": "hbm", "achieved": value / world, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": value / world / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                             "note": "per-GPU weight bytes of the step / step time, collectives included"},
                "cpu_baseline": None, "clocks": clk.summary(), "device_status": status, "check": check}
        print(json.dumps(line), flush=True)
    if not multi:
        return
    # CUDA graphs that hold NCCL kernels must go before the communicator does, or teardown can block; a watchdog ends
    # the process in any case once the result is out
    threading.Timer(60.0, lambda: os._exit(0)).start()
    run = None
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-precision rows and the TP1 record")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--kind", choices=("fp8", "bf16", "nvfp4"), default="fp8", help="precision of the decode step (c5)")
    ap.add_argument("--tokens", type=int, default=8, help="token batch of the decode step (c5): 1, 4, 8, 32")
    ap.add_argument("--allreduce", choices=("auto", "push", "pull", "nccl"), default="auto",
                    help="sum over ranks: the library's push form (auto, push), its one-shot kernel (pull) or NCCL")
    ap.add_argument("--workload", choices=("auto", "c2", "c5"), default="auto",
                    help="auto: the FP8 decode GEMMs on one GPU, the tensor-parallel decode step on several")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.workload == "c5":
        run_tp(args)
    else:
        run_single(args)


if __name__ == "__main__":
    main()
