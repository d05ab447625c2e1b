"""Cold-weight timing of gemm() calls and synthetic operands per precision.

Method (the one the reference's tools use, tools/common.py:57-125): every timed call reads a different copy of the
weight and the copies together exceed the L2 cache several times, so each call streams its weight from HBM as in a
decode step; the calls are captured once into a CUDA graph, the graph is replayed and timed with CUDA events on the
replaying stream, and the median replay is reported per call. B200's L2 is 126 MB, so at least 512 MB rotate.

Operands are described by one table (`_SPECS`): storage bits of weight and activation, whether a side carries e4m3
block scales, and how values and scale vectors are drawn; `make_weight` / `make_input` / `weight_bytes` /
`algorithmic_bytes` all read it.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FP8 = torch.float8_e4m3fn
FP4 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)
MIN_ROTATION_BYTES = 512 << 20


@dataclass(frozen=True)
class _Spec:
    w_bits: int
    x_bits: int
    w_blocks: bool = False    # one e4m3 scale per 16 weights
    x_blocks: bool = False
    w_scale: float | None = None  # magnitude of the per-channel weight scale vector (None: no vector)
    x_scale: bool = False         # per-token activation scale vector


_SPECS = {
    "bf16": _Spec(16, 16), "f16": _Spec(16, 16),
    "fp8": _Spec(8, 8, w_scale=1e-3, x_scale=True), "int8": _Spec(8, 8, w_scale=1e-2, x_scale=True),
    "nvfp4": _Spec(4, 4, w_blocks=True, x_blocks=True),
    "w8a16_bf16": _Spec(8, 16, w_scale=1e-3), "w8a16_f16": _Spec(8, 16, w_scale=1e-3),
    "w4a16_bf16": _Spec(4, 16, w_blocks=True), "w4a16_f16": _Spec(4, 16, w_blocks=True),
}


def _act_dtype(kind: str) -> torch.dtype:
    return torch.float16 if kind == "f16" or kind.endswith("_f16") else torch.bfloat16


def weight_bytes(kind: str, n: int, k: int) -> int:
    s = _SPECS[kind]
    return n * k * s.w_bits // 8 + (n * (k // 16) if s.w_blocks else 0)


def algorithmic_bytes(kind: str, m: int, n: int, k: int, out_bytes: int = 2, x_scale_len: int = 0, w_scale_len: int = 0,
                      bias_bytes: int = 0) -> int:
    """Bytes one GEMM must move when every operand is touched exactly once (split-K workspace traffic not counted):
    weight + weight block scales + activations + activation block scales + output + scale vectors + bias."""
    s = _SPECS[kind]
    acts = m * k * s.x_bits // 8 + (m * (k // 16) if s.x_blocks else 0)
    return weight_bytes(kind, n, k) + acts + m * n * out_bytes + 4 * (x_scale_len + w_scale_len) + bias_bytes


def _values(rows: int, k: int, bits: int, dtype16: torch.dtype, spread: float, g: torch.Generator, device) -> torch.Tensor:
    """Synthetic values of one operand: normal for 16-bit and fp8, uniform integers for int8 (handled by the caller),
    uniform random bytes for packed fp4 (every code occurs)."""
    if bits == 16:
        return (torch.randn(rows, k, device=device, generator=g) * spread).to(dtype16)
    if bits == 8:
        return (torch.randn(rows, k, device=device, generator=g) * 4).to(FP8)
    return torch.randint(0, 256, (rows, k // 2), device=device, generator=g, dtype=torch.uint8).view(FP4)


def _block_scales(rows: int, k: int, g: torch.Generator, device) -> torch.Tensor:
    # moderate positive e4m3 codes, as the reference's tests draw them (tests/test_gemm.py:33-83)
    return torch.randint(0x18, 0x48, (rows, k // 16), device=device, generator=g, dtype=torch.uint8).view(FP8)


def make_weight(kind: str, n: int, k: int, g: torch.Generator, device) -> tuple[torch.Tensor, dict]:
    """A synthetic weight of this precision and the gemm() keyword arguments that go with it."""
    s = _SPECS.get(kind)
    if s is None:
        raise ValueError(kind)
    if kind == "int8":
        w = torch.randint(-127, 128, (n, k), device=device, generator=g, dtype=torch.int8)
    else:
        w = _values(n, k, s.w_bits, _act_dtype(kind), 0.02, g, device)
    kw: dict = {}
    if s.w_scale is not None:
        lo, width = (0.5, 1.5) if s.w_scale == 1e-3 else (0.5, 1.0)
        kw["w_scale"] = (torch.rand(n, device=device, generator=g) * width + lo) * s.w_scale
    if s.w_blocks:
        kw.update(w_block_scale=_block_scales(n, k, g, device), w_scale=1e-3)
    return w, kw


def make_input(kind: str, m: int, k: int, device, seed: int = 1234) -> tuple[torch.Tensor, dict]:
    s = _SPECS.get(kind)
    if s is None:
        raise ValueError(kind)
    g = torch.Generator(device=device).manual_seed(seed)
    if kind == "int8":
        x = torch.randint(-127, 128, (m, k), device=device, generator=g, dtype=torch.int8)
    else:
        x = _values(m, k, s.x_bits, _act_dtype(kind), 1.0, g, device)
    kw: dict = {}
    if s.x_scale:
        kw["x_scale"] = torch.rand(m, device=device, generator=g) + 0.5
    if s.x_blocks:
        kw["x_block_scale"] = _block_scales(m, k, g, device)
    return x, kw


class ColdWeights:
    """Enough distinct copies of one (kind, N, K) weight that consecutive calls never find theirs in L2. `items` is a
    list of (weight, gemm keyword arguments); the copies share values (content does not matter for timing) but not
    addresses."""

    def __init__(self, kind: str, n: int, k: int, device, min_bytes: int = MIN_ROTATION_BYTES, max_copies: int = 4096):
        self.kind, self.n, self.k = kind, n, k
        self.nbytes = weight_bytes(kind, n, k)
        copies = max(2, min(max_copies, -(-min_bytes // self.nbytes)))
        w, kw = make_weight(kind, n, k, torch.Generator(device=device).manual_seed(0), device)
        self.items = [(w, kw)] + [(w.clone(), {a: (b.clone() if torch.is_tensor(b) else b) for a, b in kw.items()})
                                  for _ in range(copies - 1)]

    def __len__(self) -> int:
        return len(self.items)


def time_graph(build, replays: int = 20, warm_replays: int = 2) -> float:
    """Captures build() (which issues work on the current stream) into a CUDA graph; returns the median replay time
    in microseconds, timed with CUDA events on the replaying stream."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        build()  # once outside capture: lazy plan loading, workspace growth, module loading
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        build()
    for _ in range(warm_replays):
        graph.replay()
    torch.cuda.synchronize()
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(replays)]
    for start, stop in marks:
        start.record()
        graph.replay()
        stop.record()
    torch.cuda.synchronize()
    del graph
    times = sorted(start.elapsed_time(stop) * 1000.0 for start, stop in marks)
    return times[len(times) // 2]


def time_per_call(fn, weights: ColdWeights, calls: int | None = None, replays: int = 20, before=None) -> float:
    """Median microseconds per fn(w, w_kwargs, next_w) over a graph of `calls` calls on rotating weights. With `before`
    (a small producer kernel launched ahead of every call) the time of a producer-only graph is subtracted."""
    calls = calls or max(len(weights), 64)
    ring = weights.items
    schedule = [(ring[i % len(ring)], ring[(i + 1) % len(ring)][0]) for i in range(calls)]

    def chain(include_fn: bool):
        def run():
            for (w, kw), nxt in schedule:
                if before is not None:
                    before()
                if include_fn:
                    fn(w, kw, nxt)
        return run

    per_call = time_graph(chain(True), replays) / calls
    if before is not None:
        per_call -= time_graph(chain(False), replays) / calls
    return per_call
