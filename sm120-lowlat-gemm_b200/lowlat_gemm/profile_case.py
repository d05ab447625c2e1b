"""A small, self-contained case of one kernel for a profiler capture.

    python -m lowlat_gemm.profile_case gemm  --kind fp8 --n 14336 --k 4096 --m 16 [--engine tc|skinny|plan] [--calls 8]
    python -m lowlat_gemm.profile_case quant --mode fp8|int8|nvfp4|gated_fp8 --m 8 --k 8192
    python -m lowlat_gemm.profile_case step  --kind fp8 --tokens 8 --layers 2        (one-GPU decode step, push form)
    python -m lowlat_gemm.profile_case allreduce --rows 8 --cols 8192                (pull-form kernels, one rank on local memory)
    python -m lowlat_gemm.profile_case relayout --rows 28672 --cols 512              (block-scale layout converter)

Every call of `gemm` reads a different copy of the weight and the copies together exceed the L2 cache, so DRAM counters
mean what they mean in a decode step, while the whole case holds well under 2 GB on the device and launches only a
few kernels: a capture of one to three launches ends by itself in about a minute. Run it once without the profiler
first; give the profiler --clock-control none.
"""

from __future__ import annotations

import argparse

import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, timing


def run_gemm(a) -> None:
    dev = torch.device("cuda", 0)
    cold = timing.ColdWeights(a.kind, a.n, a.k, dev, min_bytes=a.rotate_mb << 20, max_copies=16)
    x, x_kw = timing.make_input(a.kind, a.m, a.k, dev)
    out_dt = torch.float16 if a.kind.endswith("_f16") or a.kind == "f16" else torch.bfloat16
    y = torch.empty(a.m, a.n, device=dev, dtype=out_dt)
    plan = L.get_plan(a.kind, a.n, a.k, dev)
    if a.engine == "tc":
        plan = Plan(tc=plan.tc)
    elif a.engine == "skinny":
        plan = Plan(skinny=plan.skinny or L.default_skinny_order(a.n, a.k, 148), skinny_max_m=16)
    e, c = L.workspace_need(a.kind, a.n, a.k, a.m, dev)
    L.reserve_workspace(dev, max(e, 16 * a.m * a.n), max(c, 4096))
    L.set_pdl(a.pdl)
    for i in range(a.calls):
        w, kw = cold.items[i % len(cold)]
        L.gemm(x, w, out=y, plan=plan, **kw, **x_kw)
    torch.cuda.synchronize()
    print(f"gemm {a.kind} {a.n}x{a.k} M={a.m}: {a.calls} calls over {len(cold)} weight copies, |y| sum {float(y.float().abs().sum()):.4g}")


def run_quant(a) -> None:
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    width = 2 * a.k if a.mode.startswith("gated") else a.k
    xs = [torch.randn(a.m, width, device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
    gs = torch.tensor([64.0], device=dev)
    for i in range(a.calls):
        x = xs[i % 4]
        if a.mode == "fp8":
            L.quantize_fp8(x)
        elif a.mode == "int8":
            L.quantize_int8(x)
        elif a.mode == "nvfp4":
            L.quantize_nvfp4(x, gs)
        else:
            L.silu_mul_quantize_fp8(x)
    torch.cuda.synchronize()
    print(f"quant {a.mode} [{a.m}, {a.k}]: {a.calls} calls")


def run_step(a) -> None:
    from lowlat_gemm import comm as CM, tp as TP
    dev = torch.device("cuda", 0)
    L.set_pdl(a.pdl)
    ar = CM.OneShotAllReduce(None, dev, max_bytes=a.tokens * 8192 * 2, local=True)
    step = TP.DecodeStep(a.kind, a.layers, 1, 0, dev, comm=ar, residual=True, push=True)
    x = (torch.randn(a.tokens, 8192, device=dev, generator=torch.Generator(device=dev).manual_seed(1)) * 0.05).to(torch.bfloat16)
    for _ in range(2):
        y = step.run(x)
    torch.cuda.synchronize()
    print(f"decode step {a.kind} tokens={a.tokens} layers={a.layers}: finite={bool(torch.isfinite(y.float()).all())}")


def run_allreduce(a) -> None:
    """The pull-form kernels with a single rank on ordinary device memory: same code path as with peers (flag
    handshake with itself, rank-order sum of one partial), so a one-GPU capture shows their fixed costs."""
    from lowlat_gemm import comm as CM
    dev = torch.device("cuda", 0)
    ar = CM.OneShotAllReduce(None, dev, max_bytes=a.rows * a.cols * 2, local=True)
    g = torch.Generator(device=dev).manual_seed(2)
    out = torch.empty(a.rows, a.cols, device=dev, dtype=torch.bfloat16)
    for i in range(a.calls):
        ar.view(i, (a.rows, a.cols), torch.bfloat16).copy_(torch.randn(a.rows, a.cols, device=dev, generator=g).to(torch.bfloat16))
        if i % 2:
            ar.reduce_quantize_fp8(i, a.rows, a.cols, torch.bfloat16, out=out)
        else:
            ar.reduce(i, out)
    torch.cuda.synchronize()
    print(f"all-reduce (pull form, one rank) [{a.rows}, {a.cols}]: {a.calls} calls, |out| sum {float(out.float().abs().sum()):.4g}")


def run_relayout(a) -> None:
    from lowlat_gemm import convert as CV
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    sfs = [torch.randint(0, 256, (a.rows, a.cols), device=dev, generator=g, dtype=torch.uint8) for _ in range(4)]
    ok = True
    for i in range(a.calls):
        tiled = CV.scales_to_tiled(sfs[i % 4])
        back = CV.scales_to_rowmajor(tiled, a.rows, a.cols)
        ok = ok and bool(torch.equal(back.view(torch.uint8), sfs[i % 4]))
    torch.cuda.synchronize()
    print(f"scale relayout [{a.rows}, {a.cols}]: {a.calls} round trips, restored={ok}")


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--kind", default="fp8")
    g.add_argument("--n", type=int, default=14336)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--m", type=int, default=16)
    g.add_argument("--engine", choices=("plan", "tc", "skinny"), default="plan")
    g.add_argument("--calls", type=int, default=8)
    g.add_argument("--rotate-mb", type=int, default=256, help="weight copies rotate over at least this much (twice the L2)")
    g.add_argument("--pdl", action="store_true")
    q = sub.add_parser("quant")
    q.add_argument("--mode", choices=("fp8", "int8", "nvfp4", "gated_fp8"), default="fp8")
    q.add_argument("--m", type=int, default=8)
    q.add_argument("--k", type=int, default=8192)
    q.add_argument("--calls", type=int, default=8)
    s = sub.add_parser("step")
    s.add_argument("--kind", default="fp8")
    s.add_argument("--tokens", type=int, default=8)
    s.add_argument("--layers", type=int, default=2)
    s.add_argument("--pdl", action="store_true")
    r = sub.add_parser("allreduce")
    r.add_argument("--rows", type=int, default=8)
    r.add_argument("--cols", type=int, default=8192)
    r.add_argument("--calls", type=int, default=8)
    t = sub.add_parser("relayout")
    t.add_argument("--rows", type=int, default=28672)
    t.add_argument("--cols", type=int, default=512)
    t.add_argument("--calls", type=int, default=6)
    a = ap.parse_args()
    {"gemm": run_gemm, "quant": run_quant, "step": run_step, "allreduce": run_allreduce, "relayout": run_relayout}[a.what](a)


if __name__ == "__main__":
    main()
