"""Measure plans for a shape list and write a plan file (load it with LLG_PLAN_FILE or lowlat_gemm.load_plans, or
install it as lowlat_gemm/plans/<device>.json).

    python -m lowlat_gemm.tune --shapes shapes.json --kinds bf16,fp8 --out plans.json [--tokens 1,2,4,8,16,64] [--pdl]

What it does is what the reference's tuner does (tools/tune.py:32-134): per (precision, N, K) and token count, time every
candidate over cold weights and keep the fastest; for W16A16 also pick one skinny summation order per (N, K) - results
must stay bit-identical across token counts - with a tile per token count, and let the skinny engine serve the token
counts, from one upwards, for which it beats the tensor-core choice. The plan file is rewritten after every shape, so
an interrupted run resumes from its --out.

How it is organised here: a `Workbench` owns the cold weights of one (kind, N, K) and times one plan at one token
count; `tc_space()` and `skinny_space()` enumerate the B200 search spaces (128-row tcgen05 tiles with one or two K
atoms per stage and 256-row tiles on CTA pairs, rings up to 227 KB, cluster or workspace split-K; persistent skinny
CTAs of 8 or 16 warps);
`search()` walks them. On B200 the skinny engine only competes at one or two tokens, so its space is searched up to
--skinny-tokens (default 2).
"""

from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass

import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, SkinnyOrder, SkinnyTile, TcChoice, timing

KSPLITS = (1, 2, 3, 4, 5, 6, 8, 10, 12, 16)


@dataclass
class Workbench:
    """Cold weights of one (kind, N, K) and a stopwatch for plans on them."""

    kind: str
    n: int
    k: int
    dev: torch.device
    replays: int = 7
    max_calls: int = 0
    prefetch_bytes: int = 0

    def __post_init__(self):
        self.cold = timing.ColdWeights(self.kind, self.n, self.k, self.dev)
        self.calls = max(len(self.cold), 32)
        if self.max_calls:
            self.calls = min(self.calls, self.max_calls)
        self.out_dtype = torch.float16 if self.kind == "f16" or self.kind.endswith("_f16") else torch.bfloat16
        self._inputs: dict[int, tuple] = {}

    def inputs(self, m: int):
        if m not in self._inputs:
            x, x_kw = timing.make_input(self.kind, m, self.k, self.dev)
            self._inputs[m] = (x, x_kw, torch.empty(m, self.n, device=self.dev, dtype=self.out_dtype))
        return self._inputs[m]

    def microseconds(self, m: int, plan: Plan, with_scales: bool = True) -> float | None:
        """Per-call time of gemm() under `plan`, or None when the library refuses the configuration."""
        x, x_kw, out = self.inputs(m)

        def call(w, kw, nxt):
            extra = {"prefetch": nxt, "prefetch_bytes": self.prefetch_bytes} if self.prefetch_bytes else {}
            scales = {**kw, **x_kw} if with_scales else {}
            return L.gemm(x, w, out=out, plan=plan, **scales, **extra)

        try:
            return timing.time_per_call(call, self.cold, calls=self.calls, replays=self.replays)
        except RuntimeError:
            return None

    def close(self):
        del self.cold
        self._inputs.clear()
        torch.cuda.empty_cache()


def tc_space(kind: str, m: int, n: int, k: int, sm_count: int, quick: bool = False):
    """Tensor-core candidates worth timing for this problem on a GPU with sm_count SMs."""
    mixed = kind in L._MIXED
    for cfg in range(L.NUM_CFGS):
        deepest = L.max_stages(kind, cfg)
        if deepest < 2:
            continue
        bp, bq, _, stage_bytes = L.tc_info(kind, cfg)
        k_tiles = -(-k // (L.KINDS[kind][1] * L.cfg_atoms(cfg)))
        for swap in ((True,) if mixed else (True, False)):
            p, q = (n, m) if swap else (m, n)
            if (bq > 2 * q and bq > 16) or (not swap and p < 64):
                continue  # a tile far wider than the problem, or a handful of token rows on the 128-row side
            tiles = -(-p // bp) * -(-q // bq)
            co_resident = max(2, min(deepest, ((L.smem_budget() - 4096) // 2) // stage_bytes))  # two CTAs per SM
            depths = {min(4, deepest), co_resident, deepest}
            if not quick:
                depths |= {min(3, deepest), min(8, deepest)}
            for stages in sorted(depths):
                for ks in ((1,) if cfg in L.PAIR_CFGS else KSPLITS):  # 256-row pair tiles have no split-K
                    if ks > 1 and (k_tiles // ks < 2 or tiles * ks > 6 * sm_count):
                        continue
                    if ks == 1 and tiles * 8 < sm_count and k_tiles >= 8:
                        continue  # a few CTAs cannot stream a long K at the HBM rate
                    yield TcChoice(cfg=cfg, swap=swap, stages=stages, ksplit=ks)
                    if 1 < ks <= 8 and not quick:
                        yield TcChoice(cfg=cfg, swap=swap, stages=stages, ksplit=ks, cluster=True)


def skinny_space(k: int, quick: bool = False):
    """(lanes per row, K split, cluster) orders and the tiles to try under each."""
    kv = k // 8
    tiles = [SkinnyTile(2, 4, 4), SkinnyTile(2, 4, 8), SkinnyTile(4, 2, 4), SkinnyTile(1, 4, 4)]
    if not quick:
        tiles += [SkinnyTile(4, 2, 8), SkinnyTile(1, 8, 4), SkinnyTile(2, 2, 4)]
    for lanes in (32, 16, 8):
        for ks in (1, 2, 4, 8):
            if ks > 1 and kv // ks < 2 * lanes:
                continue
            for cluster in ((False,) if ks == 1 else (True,) if quick else (True, False)):
                yield lanes, ks, cluster, tiles


def search(kind: str, n: int, k: int, tokens, dev, replays: int = 7, max_calls: int = 0, quick: bool = False, log=print,
           prefetch_bytes: int = 0, skinny_tokens: int = 2) -> Plan:
    sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
    bench = Workbench(kind, n, k, dev, replays, max_calls, prefetch_bytes)
    plan, tc_time = Plan(), {}
    for m in tokens:
        winner = None
        for choice in tc_space(kind, m, n, k, sm_count, quick):
            t = bench.microseconds(m, Plan(tc={m: choice}))
            if t is not None and (winner is None or t < winner[0]):
                winner = (t, choice)
        tc_time[m], plan.tc[m] = winner
        log(f"  {kind} {n}x{k} M={m}: {winner[0]:.2f} us  {winner[1]}")
    small = [m for m in tokens if m <= min(skinny_tokens, L.SKINNY_MAX_TOKENS)]
    if kind in ("bf16", "f16") and small:
        best = None  # (summed time, order fields, {m: (time, tile)})
        for lanes, ks, cluster, tiles in skinny_space(k, quick):
            per_m, total = {}, 0.0
            for m in small:
                timed = [(bench.microseconds(m, Plan(skinny=SkinnyOrder(lanes, ks, default_tile=t, cluster=cluster),
                                                     skinny_max_m=L.SKINNY_MAX_TOKENS), with_scales=False), t) for t in tiles]
                timed = [(us, t) for us, t in timed if us is not None]
                if not timed:
                    break
                per_m[m] = min(timed, key=lambda e: e[0])
                total += per_m[m][0]
            if len(per_m) == len(small) and (best is None or total < best[0]):
                best = (total, (lanes, ks, cluster), per_m)
        if best is not None:
            _, (lanes, ks, cluster), per_m = best
            plan.skinny = SkinnyOrder(lanes_per_row=lanes, ksplit=ks, cluster=cluster, tiles={m: t for m, (_, t) in per_m.items()},
                                      default_tile=per_m[small[0]][1])
            plan.skinny_max_m = 0
            for m in small:  # skinny serves 1..m while it keeps beating the tensor cores
                if per_m[m][0] >= tc_time[m]:
                    break
                plan.skinny_max_m = m
            log(f"  {kind} {n}x{k} skinny lanes={lanes} ksplit={ks} cluster={cluster} max_m={plan.skinny_max_m} "
                + " ".join(f"M{m}:{per_m[m][0]:.2f}" for m in small))
    bench.close()
    return plan


def _read_plans(path: str) -> dict:
    if not os.path.isfile(path):
        return {}
    out = {}
    for key, d in json.load(open(path)).get("plans", {}).items():
        kind, shape = key.split(":")
        n, k = (int(v) for v in shape.split("x"))
        out[(kind, n, k)] = Plan.from_json(d)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", required=True, help='JSON {"shapes": [{"name", "n", "k", optional "kinds", "max_m"}, ...]}')
    ap.add_argument("--kinds", default="bf16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokens", default="1,2,4,8,16,32,64,128,256")
    ap.add_argument("--replays", type=int, default=7)
    ap.add_argument("--max-calls", type=int, default=0, help="cap the calls per timed graph (faster; weights may stay in L2)")
    ap.add_argument("--quick", action="store_true", help="smaller candidate grid")
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--prefetch-next-mb", type=float, default=0, help="every call prefetches this much of the next weight into L2")
    ap.add_argument("--skinny-tokens", type=int, default=2, help="largest token count the skinny engine is tried at")
    args = ap.parse_args()

    dev = torch.device("cuda", torch.cuda.current_device())
    name = torch.cuda.get_device_name(dev)
    L.set_pdl(args.pdl)
    tokens = [int(t) for t in args.tokens.split(",")]
    shapes = json.load(open(args.shapes))["shapes"]
    widest = max(s["n"] for s in shapes)
    L.reserve_workspace(dev, max(KSPLITS) * max(tokens) * widest, 4 * widest)
    plans = _read_plans(args.out)  # resume
    for kind in args.kinds.split(","):
        for s in shapes:
            n, k = s["n"], s["k"]
            if (kind, n, k) in plans or k % L.KINDS[kind][2] or (s.get("kinds") and kind not in s["kinds"]):
                continue
            print(f"{kind} {s.get('name', '')} {n}x{k}", flush=True)
            plans[(kind, n, k)] = search(kind, n, k, [t for t in tokens if t <= s.get("max_m", 1 << 30)], dev, args.replays,
                                         args.max_calls, args.quick, prefetch_bytes=int(args.prefetch_next_mb * (1 << 20)),
                                         skinny_tokens=args.skinny_tokens)
            L.save_plans(args.out, plans, name)


if __name__ == "__main__":
    main()
