"""Plans: which engine and tiling serves each token count of a (precision, N, K) problem.

Surface and semantics follow the reference's planner (lowlat_gemm/__init__.py:83-349): the dataclasses with their
validation and JSON form, the "largest tuned M <= m, valid up to twice the largest tuned M" lookup, a per-device-name
registry filled from set_plan(), LLG_PLAN_FILE, the packaged plans/<device>.json and finally heuristics. The tile
table and the heuristics themselves are B200's: configs 0-9 are 128-row tcgen05 tiles (128 x {16,32,64,128,256}, one
or two 128-byte K atoms per pipeline stage), configs 10 and 11 are 256 x {128,256} tiles computed by a pair of CTAs
(bf16, f16, fp8, int8; no split-K), and the shared-memory budget is the 227 KB of sm_100.
"""

from __future__ import annotations

import bisect
import json
import os
import threading
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from . import _native as N

SKINNY_MAX_TOKENS = 16
NUM_CFGS = 12
PAIR_CFGS = (10, 11)  # 256-row tiles on CTA pairs
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
        if self.cfg in PAIR_CFGS and self.ksplit > 1:
            raise ValueError(f"cfg {self.cfg} (256-row tiles on CTA pairs) runs without split-K, got ksplit {self.ksplit}")


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


def _floor_entry(table: dict, m: int):
    """(largest key <= m, its value), falling back to the smallest key when every key is larger; None for an empty
    table. The rule both lookups share: an entry tuned for M tokens also serves the token counts above it."""
    if not table:
        return None
    keys = sorted(table)
    at = bisect.bisect_right(keys, m)
    key = keys[at - 1] if at else keys[0]
    return key, table[key]


def _tc_lookup(table: dict, m: int):
    """Tuned tensor-core entry for m tokens: that of the largest tuned M <= m, but no answer at all beyond twice the
    largest tuned M - there the heuristics decide (reference lowlat_gemm/__init__.py:177-184)."""
    hit = _floor_entry(table, m)
    if hit is None or m > 2 * max(table):
        return None
    return hit[1]


def _nearest(table: dict, m: int, default):
    hit = _floor_entry(table, m)
    return default if hit is None else hit[1]


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
    _, bq, _, stage = tc_info(kind, cfg)
    # the pair kernel keeps its epilogue scratch (16 KB of line buffers and 16 bytes per tile column) behind the ring
    budget = smem_budget() - (16384 + 16 * bq if cfg in PAIR_CFGS else 0)
    return min(MAX_STAGES, budget // stage) if stage else 0


def cfg_atoms(cfg: int) -> int:
    return 1 if cfg in PAIR_CFGS else 1 + cfg // 5


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
    if cfg in PAIR_CFGS and max_stages(kind, cfg) < 2:
        cfg = 4 if cfg == 11 else 3  # the kind has no pair kernel: the single-CTA tile of the same width
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
    elif m >= 192 and n >= 256:
        cfg = 11  # 256 x 256 on CTA pairs (measured on B200: fp8 14336x4096 at M = 256 / 1024 / 4096 25.5 / 60 / 175 us
        #           against 27.8 / 75.8 / 266 us for the best single-CTA tile); kinds without a pair kernel fall back
    else:
        cfg = 4 if n >= 2048 and m >= 256 else 3
    cfg = _fit_cfg(kind, cfg)
    bp, bq, _, stage = tc_info(kind, cfg)
    if cfg in PAIR_CFGS:
        return TcChoice(cfg=cfg, swap=False, stages=max_stages(kind, cfg), ksplit=1)
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


_HEURISTIC_TOKENS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024, 4096)


def default_plan(kind: str, n: int, k: int, sm_count: int) -> Plan:
    """Plan from heuristics alone: a tensor-core choice per power-of-two token count and, for W16A16, the skinny engine
    for the single-token call (the only one where it matches the tensor cores on B200)."""
    w16 = kind in ("bf16", "f16")
    return Plan(skinny=default_skinny_order(n, k, sm_count) if w16 else None, skinny_max_m=1 if w16 else 0,
                tc={m: default_tc_choice(kind, m, n, k, sm_count) for m in _HEURISTIC_TOKENS})


# ---------------------------------------------------------------------------------------------------------------
# registry: plans per device name. Sources in rising priority: heuristics, the packaged plans/<device>.json, the file
# named by LLG_PLAN_FILE, load_plans(), set_plan() (reference lowlat_gemm/__init__.py:265-349).


def _dev(device: torch.device | None) -> torch.device:
    if device is not None and device.index is not None:
        return device
    return torch.device("cuda", torch.cuda.current_device())


def _file_key(name: str) -> str:
    """Device name -> file stem: lower case, every run of other characters an underscore ("NVIDIA B200" -> nvidia_b200)."""
    return "".join(ch if ch.isalnum() else "_" for ch in name).strip("_").lower()


def _packaged_path(name: str) -> Path:
    return Path(__file__).with_name("plans") / f"{_file_key(name)}.json"


def _parse_key(key: str) -> tuple[str, int, int]:
    kind, shape = key.split(":")
    n, k = shape.lower().split("x")
    return kind, int(n), int(k)


class _PlanStore:
    """All plans of the process, keyed by (device name, kind, N, K), behind one lock."""

    def __init__(self):
        self._lock = threading.Lock()
        self._plans: dict[tuple[str, str, int, int], Plan] = {}
        self._seeded: set[str] = set()      # device names whose packaged / environment plans have been read
        self._sms: dict[int, int] = {}

    def sm_count(self, device: torch.device) -> int:
        if device.index not in self._sms:
            self._sms[device.index] = torch.cuda.get_device_properties(device.index).multi_processor_count
        return self._sms[device.index]

    def ingest(self, data: dict, name: str) -> int:
        parsed = {_parse_key(key): Plan.from_json(body) for key, body in data.get("plans", {}).items()}
        with self._lock:
            for (kind, n, k), plan in parsed.items():
                self._plans[(name, kind, n, k)] = plan
        return len(parsed)

    def seed(self, name: str) -> None:
        """First use of a device name: read its packaged plans, then the file LLG_PLAN_FILE names (which wins)."""
        with self._lock:
            if name in self._seeded:
                return
            self._seeded.add(name)
        packaged = _packaged_path(name)
        if packaged.is_file():
            self.ingest(json.loads(packaged.read_text()), name)
        extra = os.environ.get("LLG_PLAN_FILE")
        if extra:
            data = json.loads(Path(extra).read_text())
            self.ingest(data, data.get("device") or name)

    def put(self, name: str, kind: str, n: int, k: int, plan: Plan) -> None:
        self.seed(name)
        with self._lock:
            self._plans[(name, kind, n, k)] = plan

    def get(self, name: str, kind: str, n: int, k: int, sm_count: int) -> Plan:
        self.seed(name)
        key = (name, kind, n, k)
        plan = self._plans.get(key)
        if plan is None:
            fresh = default_plan(kind, n, k, sm_count)  # computed outside the lock: it queries the library
            with self._lock:
                plan = self._plans.setdefault(key, fresh)
        return plan


_store = _PlanStore()


def _sm_count(device: torch.device) -> int:
    return _store.sm_count(device)


def load_plans(path: str | os.PathLike, device_name: str | None = None) -> int:
    """Load {"device": ..., "plans": {"<kind>:<N>x<K>": plan}}; these win over the packaged plans. Returns the count."""
    data = json.loads(Path(path).read_text())
    name = device_name or data.get("device")
    if not name:
        raise ValueError(f"{path}: no device name in the file and none given")
    _store.seed(name)
    return _store.ingest(data, name)


def save_plans(path: str | os.PathLike, plans: dict[tuple[str, int, int], Plan], device_name: str) -> None:
    body = {f"{kind}:{n}x{k}": p.to_json() for (kind, n, k), p in plans.items()}
    Path(path).write_text(json.dumps({"device": device_name, "plans": body}, indent=1))


def set_plan(kind: str, n: int, k: int, plan: Plan, device: torch.device | None = None) -> None:
    _store.put(torch.cuda.get_device_name(_dev(device)), kind, n, k, plan)


def get_plan(kind: str, n: int, k: int, device: torch.device | None = None) -> Plan:
    device = _dev(device)
    return _store.get(torch.cuda.get_device_name(device), kind, n, k, _store.sm_count(device))


def prefer_lowlat(kind: str, n: int, k: int, m: int, device: torch.device | None = None) -> bool:
    """False when the plan recorded the vendor library as faster at the tuned token count that serves m (the largest
    tuned M <= m, within twice the largest tuned M); True whenever nothing was recorded for m."""
    plan = get_plan(kind, n, k, device)
    if not plan.prefer_vendor or _tc_lookup(plan.tc, m) is None:
        return True
    served_by = _floor_entry(plan.tc, m)[0]
    return served_by > m or served_by not in plan.prefer_vendor
