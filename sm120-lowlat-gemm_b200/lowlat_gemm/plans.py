"""Plans: which engine and tiling serves each token count of a (precision, N, K) problem.

Surface and semantics follow the reference's planner (lowlat_gemm/__init__.py:83-349): the dataclasses with their
validation and JSON form, the "largest tuned M <= m, valid up to twice the largest tuned M" lookup, a per-device-name
registry filled from set_plan(), LLG_PLAN_FILE, the packaged plans/<device>.json and finally heuristics. The tile
table and the heuristics themselves are B200's: every config is a 128-row tcgen05 tile (128 x {16,32,64,128,256},
one or two 128-byte K atoms per pipeline stage) and the shared-memory budget is the 227 KB of sm_100.
"""

from __future__ import annotations

import json
import os
import threading
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from . import _native as N

SKINNY_MAX_TOKENS = 16
NUM_CFGS = 10
MAX_STAGES = 16

# kind -> (id, K elements per 128-byte atom of the streamed operand, K multiple required)
KINDS = {
    "bf16": (0, 64, 8),
    "f16": (1, 64, 8),
    "fp8": (2, 128, 16),
    "int8": (3, 128, 16),
    "nvfp4": (4, 256, 64),
    "w8a16_bf16": (5, 128, 16),
    "w8a16_f16": (6, 128, 16),
    "w4a16_bf16": (7, 256, 64),
    "w4a16_f16": (8, 256, 64),
}
_MIXED = {"w8a16_bf16", "w8a16_f16", "w4a16_bf16", "w4a16_f16"}
_SKINNY_TILES = {(1, 2), (1, 4), (1, 8), (2, 2), (2, 4), (4, 2)}


@dataclass(frozen=True)
class SkinnyTile:
    """Per-M tiling of the skinny kernel; never changes a result bit."""

    rows: int = 1
    unroll: int = 4
    warps: int = 4

    def __post_init__(self):
        if (self.rows, self.unroll) not in _SKINNY_TILES:
            raise ValueError(f"unsupported skinny (rows, unroll) {(self.rows, self.unroll)}")
        if not 1 <= self.warps <= 8:
            raise ValueError(f"warps must be in [1, 8], got {self.warps}")


@dataclass
class SkinnyOrder:
    """Summation order of the skinny kernel (fixed per N, K so results are M-invariant) plus per-M tiles."""

    lanes_per_row: int = 32
    ksplit: int = 1
    tiles: dict[int, SkinnyTile] = field(default_factory=dict)
    default_tile: SkinnyTile = field(default_factory=SkinnyTile)
    cluster: bool = False

    def __post_init__(self):
        if self.lanes_per_row not in (8, 16, 32):
            raise ValueError(f"lanes_per_row must be 8, 16 or 32, got {self.lanes_per_row}")
        if not 1 <= self.ksplit <= 64:
            raise ValueError(f"ksplit must be in [1, 64], got {self.ksplit}")
        if self.cluster and self.ksplit > 8:
            raise ValueError(f"cluster split-K needs ksplit <= 8, got {self.ksplit}")

    def tile(self, m: int) -> SkinnyTile:
        return _nearest(self.tiles, m, self.default_tile)


@dataclass(frozen=True)
class TcChoice:
    cfg: int
    swap: bool              # the weight is the MMA's 128-row operand (few tokens)
    stages: int = 4
    ksplit: int = 1
    cluster: bool = False   # split-K reduced through cluster shared memory (ksplit <= 8, no workspace)

    def __post_init__(self):
        if not 0 <= self.cfg < NUM_CFGS:
            raise ValueError(f"cfg must be in [0, {NUM_CFGS}), got {self.cfg}")
        if not 1 <= self.ksplit <= 64 or not 2 <= self.stages <= MAX_STAGES:
            raise ValueError(f"bad ksplit/stages {self.ksplit}/{self.stages}")
        if self.cluster and self.ksplit > 8:
            raise ValueError(f"cluster split-K needs ksplit <= 8, got {self.ksplit}")


@dataclass
class Plan:
    """Per (kind, N, K): engine and tiling for each M; the nearest lower listed M wins."""

    skinny: SkinnyOrder | None = None
    skinny_max_m: int = 0
    tc: dict[int, TcChoice] = field(default_factory=dict)
    prefer_vendor: list[int] = field(default_factory=list)

    def to_json(self) -> dict:
        out: dict = {"skinny_max_m": self.skinny_max_m,
                     "tc": {str(m): asdict(self.tc[m]) for m in sorted(self.tc)}}
        if self.prefer_vendor:
            out["prefer_vendor"] = sorted(self.prefer_vendor)
        if self.skinny is not None:
            s = self.skinny
            out["skinny"] = {"lanes_per_row": s.lanes_per_row, "ksplit": s.ksplit, "cluster": s.cluster,
                             "default_tile": asdict(s.default_tile),
                             "tiles": {str(m): asdict(s.tiles[m]) for m in sorted(s.tiles)}}
        return out

    @classmethod
    def from_json(cls, d: dict) -> "Plan":
        skinny = None
        if d.get("skinny") is not None:
            s = d["skinny"]
            skinny = SkinnyOrder(lanes_per_row=int(s["lanes_per_row"]), ksplit=int(s["ksplit"]),
                                 cluster=bool(s.get("cluster", False)),
                                 default_tile=SkinnyTile(**s.get("default_tile", {})),
                                 tiles={int(m): SkinnyTile(**t) for m, t in s.get("tiles", {}).items()})
        return cls(skinny=skinny, skinny_max_m=int(d.get("skinny_max_m", 0)),
                   tc={int(m): TcChoice(**c) for m, c in d.get("tc", {}).items()},
                   prefer_vendor=[int(m) for m in d.get("prefer_vendor", [])])


def _tc_lookup(table: dict, m: int):
    """Tuned entry for m: that of the largest tuned M <= m; no answer beyond twice the largest tuned M."""
    if m in table:
        return table[m]
    if not table or m > 2 * max(table):
        return None
    below = [t for t in table if t <= m]
    return table[max(below)] if below else table[min(table)]


def _nearest(table: dict, m: int, default):
    if m in table:
        return table[m]
    below = [t for t in table if t <= m]
    if below:
        return table[max(below)]
    return table[min(table)] if table else default


# ---------------------------------------------------------------------------------------------------------------
# tile facts and heuristics

_info: dict[tuple[int, int], tuple[int, int, int, int]] = {}


def tc_info(kind: str, cfg: int) -> tuple[int, int, int, int]:
    """(BP, BQ, threads, shared-memory bytes per pipeline stage); stage bytes 0 = config unavailable for the kind."""
    key = (KINDS[kind][0], cfg)
    if key not in _info:
        _info[key] = tuple(N.tc_info(*key))
    return _info[key]


def smem_budget() -> int:
    return int(N.lib.llg_smem_budget())


def max_stages(kind: str, cfg: int) -> int:
    stage = tc_info(kind, cfg)[3]
    return min(MAX_STAGES, smem_budget() // stage) if stage else 0


def cfg_atoms(cfg: int) -> int:
    return 1 + cfg // 5


def skinny_ranges(n: int, ksplit: int, sm_count: int) -> int:
    """Upper bound of the row ranges (CTAs along N, and split-K counters) of a skinny launch: one wave of CTAs, two to
    an SM for small CTAs, never more than rows."""
    return max(1, min(n, max(1, 2 * sm_count // ksplit)))


def default_skinny_order(n: int, k: int, sm_count: int) -> SkinnyOrder:
    """Summation order and tile for the persistent skinny kernel when nothing was tuned: 32 virtual lanes per row where
    K gives each at least two vectors (the widest K chunk per row and pipeline stage), CTAs of 8 warps that run two to
    an SM, and a K split only while a CTA would otherwise own fewer than 8 rows and the splits stay long enough to
    amortise a pipeline stage. Measured on B200 (11008 x 4096, one token): 15.8 us against 15.9 us on the tensor
    cores; from two tokens on the tensor-core engine is faster, so default_plan() hands it those."""
    kv = k // 8
    lanes = 32 if kv >= 64 else 16 if kv >= 32 else 8
    ksplit = 1
    while n * ksplit < 8 * 2 * sm_count and kv // (2 * ksplit) >= 4 * lanes and ksplit < 8:
        ksplit *= 2
    return SkinnyOrder(lanes_per_row=lanes, ksplit=ksplit, cluster=ksplit > 1,
                       default_tile=SkinnyTile(rows=2, unroll=4, warps=4))


def _fit_cfg(kind: str, cfg: int) -> int:
    while max_stages(kind, cfg) < 2:
        cfg = cfg - 5 if cfg >= 5 else cfg - 1
        if cfg < 0:
            raise ValueError(f"no tensor-core config fits shared memory for {kind}")
    return cfg


_WBITS = {"bf16": 16, "f16": 16, "fp8": 8, "int8": 8, "nvfp4": 4, "w8a16_bf16": 8, "w8a16_f16": 8, "w4a16_bf16": 4,
          "w4a16_f16": 4}


def default_tc_choice(kind: str, m: int, n: int, k: int, sm_count: int) -> TcChoice:
    """Weight on the 128-row side ("swap") while the token count fits one narrow tile, activations there otherwise;
    two K atoms per stage where they fit (fewer barrier round trips per byte). The K split is picked with a small cost
    model: weight bytes over the fraction of SMs kept busy by the last round, plus the split-K partial traffic, plus a
    fixed cost per round and per stage of the chain one CTA walks; splits up to 8 reduce over the cluster. Without a split, kinds that stream (everything but
    the mixed ones) take three stages when three fit 110 KB: two CTAs then fit an SM, so the next kernel of a dependent
    chain is resident early (what the tuner finds on B200 for every baseline shape)."""
    swap = kind in _MIXED or m <= 64
    if swap:
        cfg = 5 if m <= 16 else 6 if m <= 32 else 7 if m <= 64 else 3 if m <= 128 else 4
    else:
        cfg = 4 if n >= 2048 and m >= 256 else 3
    cfg = _fit_cfg(kind, cfg)
    bp, bq, _, stage = tc_info(kind, cfg)
    p, q = (n, m) if swap else (m, n)
    tiles = -(-p // bp) * -(-q // bq)
    nk = -(-k // (KINDS[kind][1] * cfg_atoms(cfg)))
    weight = n * k * _WBITS[kind] / 8
    best, best_t = 1, None
    for ks in range(1, 9):  # up to what a cluster can reduce
        if ks > 1 and nk // ks < 2:
            break
        items = tiles * ks
        rounds = -(-items // sm_count)
        busy = items / (rounds * sm_count)
        if ks == 1 and swap:
            # without a split the launcher shortens the row pitch (down to 32 rows) so that the tiles fill whole rounds
            tq = -(-q // bq)
            want = -(-tiles // sm_count) * sm_count // tq
            pitch = min(bp, max(32, -(-p // max(want, 1))))
            items = -(-p // pitch) * tq
            rounds = -(-items // sm_count)
            busy = items / (rounds * sm_count)
        partials = 2.0 * ks * p * q * 4 if ks > 1 else 0.0
        # microseconds: streaming, a fixed cost per round, and the serial chain of stages one CTA walks per item
        t = (weight / busy + 0.5 * partials) / 6.5e6 + rounds * 0.4 + (nk / ks) * 0.12
        if best_t is None or t < best_t - 1e-9:
            best, best_t = ks, t
    top = max_stages(kind, cfg)
    if best == 1 and kind not in _MIXED and 3 * stage <= 110 * 1024:
        stages = 3
    elif kind in _MIXED:
        stages = min(top, 4)
    else:
        stages = top
    stages = max(2, min(stages, top, nk + 1))
    return TcChoice(cfg=cfg, swap=swap, stages=stages, ksplit=best, cluster=best > 1)


def default_plan(kind: str, n: int, k: int, sm_count: int) -> Plan:
    plan = Plan()
    if kind in ("bf16", "f16"):
        plan.skinny = default_skinny_order(n, k, sm_count)
        plan.skinny_max_m = 1
    for m in (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024, 4096):
        plan.tc[m] = default_tc_choice(kind, m, n, k, sm_count)
    return plan


# ---------------------------------------------------------------------------------------------------------------
# registry

_lock = threading.Lock()
_plans: dict[tuple[str, str, int, int], Plan] = {}
_loaded: set[str] = set()
_sm_counts: dict[int, int] = {}


def _dev(device: torch.device | None) -> torch.device:
    if device is None or device.index is None:
        return torch.device("cuda", torch.cuda.current_device())
    return device


def _sm_count(device: torch.device) -> int:
    if device.index not in _sm_counts:
        _sm_counts[device.index] = torch.cuda.get_device_properties(device.index).multi_processor_count
    return _sm_counts[device.index]


def _file_key(name: str) -> str:
    return "".join(ch if ch.isalnum() else "_" for ch in name).strip("_").lower()


def _packaged_path(name: str) -> Path:
    return Path(__file__).with_name("plans") / f"{_file_key(name)}.json"


def _ingest(data: dict, name: str) -> int:
    entries = data.get("plans", {})
    with _lock:
        for key, d in entries.items():
            kind, shape = key.split(":")
            n, k = (int(v) for v in shape.lower().split("x"))
            _plans[(name, kind, n, k)] = Plan.from_json(d)
    return len(entries)


def _ensure_loaded(name: str) -> None:
    if name in _loaded:
        return
    with _lock:
        if name in _loaded:
            return
        _loaded.add(name)
    packaged = _packaged_path(name)
    if packaged.is_file():
        _ingest(json.loads(packaged.read_text()), name)
    env = os.environ.get("LLG_PLAN_FILE")
    if env:
        data = json.loads(Path(env).read_text())
        _ingest(data, data.get("device") or name)


def load_plans(path: str | os.PathLike, device_name: str | None = None) -> int:
    """Load {"device": ..., "plans": {"<kind>:<N>x<K>": plan}}; these win over the packaged plans. Returns the count."""
    data = json.loads(Path(path).read_text())
    name = device_name or data.get("device")
    if not name:
        raise ValueError(f"{path}: no device name in the file and none given")
    _ensure_loaded(name)
    return _ingest(data, name)


def save_plans(path: str | os.PathLike, plans: dict[tuple[str, int, int], Plan], device_name: str) -> None:
    body = {f"{kind}:{n}x{k}": p.to_json() for (kind, n, k), p in plans.items()}
    Path(path).write_text(json.dumps({"device": device_name, "plans": body}, indent=1))


def set_plan(kind: str, n: int, k: int, plan: Plan, device: torch.device | None = None) -> None:
    name = torch.cuda.get_device_name(_dev(device))
    _ensure_loaded(name)
    with _lock:
        _plans[(name, kind, n, k)] = plan


def get_plan(kind: str, n: int, k: int, device: torch.device | None = None) -> Plan:
    device = _dev(device)
    name = torch.cuda.get_device_name(device)
    _ensure_loaded(name)
    plan = _plans.get((name, kind, n, k))
    if plan is None:
        fresh = default_plan(kind, n, k, _sm_count(device))
        with _lock:
            plan = _plans.setdefault((name, kind, n, k), fresh)
    return plan


def prefer_lowlat(kind: str, n: int, k: int, m: int, device: torch.device | None = None) -> bool:
    """False when the plan recorded the vendor library as faster at the nearest tuned M (<= m, within 2x)."""
    plan = get_plan(kind, n, k, device)
    if not plan.prefer_vendor or not plan.tc:
        return True
    tuned = [t for t in plan.tc if t <= m]
    if not tuned or m > 2 * max(plan.tc):
        return True
    return max(tuned) not in plan.prefer_vendor
