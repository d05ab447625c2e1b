"""Measure plans for a shape list and write a plan file (load it with LLG_PLAN_FILE or lowlat_gemm.load_plans, or
install it as lowlat_gemm/plans/<device>.json).

    python -m lowlat_gemm.tune --shapes shapes.json --kinds bf16,fp8 --out plans.json [--tokens 1,2,4,8,16,64]

Same procedure as the reference's tuner (tools/tune.py:32-134): every tensor-core candidate (config, orientation,
stages, K split, cluster) is timed per token count over cold weights and the fastest kept; for W16A16 the skinny
summation order (lanes per row, K split) is chosen once per (N, K) - results stay bit-identical across token counts -
with a tile per token count, and skinny serves the token counts where it beats the tensor-core choice, up to the first
one where it does not. The plan file is rewritten after every shape, so an interrupted run resumes from its --out.
The candidate grid is the B200 one: 128-row tiles, up to 16 stages of 227 KB shared memory, two CTAs per SM.
"""

from __future__ import annotations

import argparse
import itertools
import json
import os

import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, SkinnyOrder, SkinnyTile, TcChoice, timing

SKINNY_TILES = [SkinnyTile(r, u, w) for (r, u), w in itertools.product([(1, 4), (1, 8), (2, 2), (2, 4), (4, 2)], (4, 8))]
KSPLITS = (1, 2, 3, 4, 5, 6, 8, 10, 12, 16)


def tc_candidates(kind: str, m: int, n: int, k: int, sm_count: int, quick: bool = False):
    for cfg in range(L.NUM_CFGS):
        top = L.max_stages(kind, cfg)
        if top < 2:
            continue
        bp, bq, _, stage = L.tc_info(kind, cfg)
        nk = -(-k // (L.KINDS[kind][1] * L.cfg_atoms(cfg)))
        for swap in ((True,) if kind in L._MIXED else (True, False)):
            p, q = (n, m) if swap else (m, n)
            if (bq > 2 * q and bq > 16) or (not swap and p < 64):  # tile far wider than the problem
                continue
            tiles = -(-p // bp) * -(-q // bq)
            two_per_sm = max(2, min(top, ((L.smem_budget() - 4096) // 2) // stage))
            for stages in sorted({min(4, top), two_per_sm, top} if quick else {min(3, top), min(4, top), two_per_sm, min(8, top), top}):
                for ks in KSPLITS:
                    if ks > 1 and (nk // ks < 2 or tiles * ks > 6 * sm_count):
                        continue
                    if ks == 1 and tiles * 8 < sm_count and nk >= 8:  # a handful of CTAs cannot stream at HBM rate
                        continue
                    yield TcChoice(cfg=cfg, swap=swap, stages=stages, ksplit=ks)
                    if 1 < ks <= 8 and not quick:
                        yield TcChoice(cfg=cfg, swap=swap, stages=stages, ksplit=ks, cluster=True)


def tune_shape(kind: str, n: int, k: int, tokens, dev, replays: int = 7, max_calls: int = 0, quick: bool = False,
               log=print, prefetch_bytes: int = 0) -> Plan:
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    cold = timing.ColdWeights(kind, n, k, dev)
    calls = min(max(len(cold), 32), max_calls) if max_calls else max(len(cold), 32)
    plan = Plan()
    tc_us = {}
    out_dt = torch.float16 if kind == "f16" or kind.endswith("_f16") else torch.bfloat16
    for m in tokens:
        x, x_kw = timing.make_input(kind, m, k, dev)
        out = torch.empty(m, n, device=dev, dtype=out_dt)
        best = None
        for c in tc_candidates(kind, m, n, k, sm_count, quick):
            try:
                pf = (lambda nxt: {"prefetch": nxt, "prefetch_bytes": prefetch_bytes}) if prefetch_bytes else (lambda nxt: {})
                t = timing.time_per_call(lambda w, kw, nxt: L.gemm(x, w, out=out, plan=Plan(tc={m: c}), **kw, **x_kw, **pf(nxt)),
                                         cold, calls=calls, replays=replays)
            except RuntimeError:
                continue
            if best is None or t < best[0]:
                best = (t, c)
        tc_us[m], plan.tc[m] = best
        log(f"  {kind} {n}x{k} M={m}: {best[0]:.2f} us  {best[1]}")
    if kind in ("bf16", "f16"):
        skinny_ms = [m for m in tokens if m <= L.SKINNY_MAX_TOKENS]
        kv = k // 8
        best_order = None
        for lanes, ks, clu in itertools.product((32, 16, 8), (1, 2, 4, 8), (False, True)):
            if (ks > 1 and kv // ks < lanes) or (clu and not 1 < ks <= 8) or (quick and clu):
                continue
            tiles, total = {}, 0.0
            for m in skinny_ms:
                x, _ = timing.make_input(kind, m, k, dev)
                out = torch.empty(m, n, device=dev, dtype=x.dtype)
                bt = None
                for tile in SKINNY_TILES:
                    pl = Plan(skinny=SkinnyOrder(lanes_per_row=lanes, ksplit=ks, default_tile=tile, cluster=clu),
                              skinny_max_m=L.SKINNY_MAX_TOKENS)
                    pf = (lambda nxt: {"prefetch": nxt, "prefetch_bytes": prefetch_bytes}) if prefetch_bytes else (lambda nxt: {})
                    t = timing.time_per_call(lambda w, kw, nxt: L.gemm(x, w, out=out, plan=pl, **pf(nxt)), cold, calls=calls, replays=replays)
                    if bt is None or t < bt[0]:
                        bt = (t, tile)
                tiles[m] = bt
                total += bt[0]
            if best_order is None or total < best_order[0]:
                best_order = (total, lanes, ks, clu, tiles)
        if best_order is not None and skinny_ms:
            _, lanes, ks, clu, tiles = best_order
            plan.skinny = SkinnyOrder(lanes_per_row=lanes, ksplit=ks, cluster=clu, tiles={m: t for m, (_, t) in tiles.items()})
            plan.skinny_max_m = 0
            for m in skinny_ms:
                if tiles[m][0] < tc_us[m]:
                    plan.skinny_max_m = m
                else:
                    break
            log(f"  {kind} {n}x{k} skinny lanes={lanes} ksplit={ks} cluster={clu} max_m={plan.skinny_max_m} "
                + " ".join(f"M{m}:{tiles[m][0]:.2f}" for m in skinny_ms))
    del cold
    torch.cuda.empty_cache()
    return plan


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", required=True, help='JSON {"shapes": [{"name", "n", "k"}, ...]}')
    ap.add_argument("--kinds", default="bf16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128,256")
    ap.add_argument("--replays", type=int, default=7)
    ap.add_argument("--max-calls", type=int, default=0, help="cap the calls per timed graph (faster; weights may stay in L2)")
    ap.add_argument("--quick", action="store_true", help="smaller candidate grid")
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--prefetch-next-mb", type=float, default=0, help="every call prefetches this much of the next weight into L2")
    args = ap.parse_args()

    dev = torch.device("cuda", torch.cuda.current_device())
    name = torch.cuda.get_device_name(dev)
    L.set_pdl(args.pdl)
    tokens = [int(t) for t in args.tokens.split(",")]
    shapes = json.load(open(args.shapes))["shapes"]
    max_n = max(s["n"] for s in shapes)
    L.reserve_workspace(dev, max(KSPLITS) * max(tokens) * max_n, 4 * max_n)
    plans: dict[tuple[str, int, int], Plan] = {}
    if os.path.isfile(args.out):  # resume
        for key, d in json.load(open(args.out)).get("plans", {}).items():
            kind, shape = key.split(":")
            n, k = (int(v) for v in shape.split("x"))
            plans[(kind, n, k)] = Plan.from_json(d)
    for kind in args.kinds.split(","):
        for s in shapes:
            n, k = s["n"], s["k"]
            if (kind, n, k) in plans or k % L.KINDS[kind][2]:
                continue
            only = s.get("kinds")
            if only and kind not in only:
                continue
            toks = [t for t in tokens if t <= s.get("max_m", 1 << 30)]
            print(f"{kind} {s.get('name', '')} {n}x{k}", flush=True)
            plans[(kind, n, k)] = tune_shape(kind, n, k, toks, dev, args.replays, args.max_calls, args.quick,
                                             prefetch_bytes=int(args.prefetch_next_mb * (1 << 20)))
            L.save_plans(args.out, plans, name)


if __name__ == "__main__":
    main()
