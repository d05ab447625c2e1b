"""Time gemm() on the benchmark configurations and print microseconds per GEMM with achieved HBM bandwidth.

    python -m lowlat_gemm.perf_table [--configs c1,c2,c3,c4] [--plans plans.json] [--pdl] [--json out.json]

Cold-weight CUDA-graph timing (lowlat_gemm/timing.py). Bandwidth = algorithmic bytes of the GEMM (every operand touched
once) / time, reported against the nominal 8 TB/s and against a measured copy bandwidth when --measured-gbs gives one. The
counterpart of the reference's tools/bench.py:44-85.
"""

from __future__ import annotations

import argparse
import json

import torch

import lowlat_gemm as L
from lowlat_gemm import timing

CONFIGS = {
    "c1": [("bf16", 11008, 4096, (1, 2, 4, 8, 16))],
    "c2": [("fp8", 14336, 4096, (1, 2, 4, 8, 16, 64, 256)), ("w8a16_bf16", 14336, 4096, (1, 2, 4, 8, 16))],
    "c3": [("int8", 4096, 4096, (1, 8, 32, 128))],
    "c4": [("nvfp4", 28672, 8192, (1, 2, 4, 8, 16, 128)), ("w4a16_bf16", 28672, 8192, (1, 2, 4, 8, 16, 128))],
}


def scale_lens(kind: str, m: int, n: int) -> tuple[int, int, int]:
    """(x_scale len, w_scale len, bias bytes) the synthetic operands of timing.make_* carry."""
    if kind in ("fp8", "int8"):
        return m, n, 0
    if kind.startswith("w8a16"):
        return 0, n, 0
    return 0, 0, 0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="c1,c2,c3,c4")
    ap.add_argument("--plans")
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--prefetch-next", action="store_true")
    ap.add_argument("--prefetch-mb", type=float, default=16)
    ap.add_argument("--measured-gbs", type=float, default=0.0, help="measured copy bandwidth of this GPU in GB/s; 0 leaves that column out")
    ap.add_argument("--json")
    ap.add_argument("--replays", type=int, default=20)
    args = ap.parse_args()
    if args.plans:
        L.load_plans(args.plans)
    dev = torch.device("cuda", torch.cuda.current_device())
    L.set_pdl(args.pdl)
    rows = []
    print(f"{torch.cuda.get_device_name(dev)}; us per GEMM, cold weights, CUDA-graph replay; pdl={args.pdl} prefetch_next={args.prefetch_next}")
    print(f"{'kind':11s} {'N':>6s} {'K':>5s} {'M':>4s} {'us':>8s} {'GB/s':>8s} {'%8TB/s':>7s} {'%meas':>6s}  plan")
    for cname in args.configs.split(","):
        for kind, n, k, tokens in CONFIGS[cname]:
            cold = timing.ColdWeights(kind, n, k, dev)
            e, c = L.workspace_need(kind, n, k, max(tokens), dev)
            L.reserve_workspace(dev, e, c)
            for m in tokens:
                x, x_kw = timing.make_input(kind, m, k, dev)
                out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)

                def call(w, kw, nxt):
                    if args.prefetch_next:
                        return L.gemm(x, w, out=out, prefetch=nxt, prefetch_bytes=int(args.prefetch_mb * (1 << 20)), **kw, **x_kw)
                    return L.gemm(x, w, out=out, **kw, **x_kw)

                us = timing.time_per_call(call, cold, replays=args.replays)
                xs, ws, bb = scale_lens(kind, m, n)
                nbytes = timing.algorithmic_bytes(kind, m, n, k, 2, xs, ws, bb)
                gbs = nbytes / us / 1e3
                plan = L.get_plan(kind, n, k, dev)
                if plan.skinny is not None and m <= min(plan.skinny_max_m, 16):
                    desc = f"skinny lanes={plan.skinny.lanes_per_row} ks={plan.skinny.ksplit} {plan.skinny.tile(m)}"
                else:
                    ch = L._tc_lookup(plan.tc, m) or L.default_tc_choice(kind, m, n, k, torch.cuda.get_device_properties(dev).multi_processor_count)
                    desc = f"cfg{ch.cfg} swap={int(ch.swap)} st={ch.stages} ks={ch.ksplit}{' cl' if ch.cluster else ''}"
                print(f"{kind:11s} {n:6d} {k:5d} {m:4d} {us:8.2f} {gbs:8.0f} {gbs / 80:7.1f} {(100 * gbs / args.measured_gbs) if args.measured_gbs else float('nan'):6.1f}  {desc}", flush=True)
                rows.append({"config": cname, "kind": kind, "n": n, "k": k, "m": m, "us": us, "bytes": nbytes, "gbs": gbs,
                             "pct_8tbs": gbs / 80, "pct_measured": (100 * gbs / args.measured_gbs) if args.measured_gbs else None, "plan": desc})
            del cold
            torch.cuda.empty_cache()
    if args.json:
        json.dump({"device": torch.cuda.get_device_name(dev), "pdl": args.pdl, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
