"""Cold-weight timing of gemm() calls and synthetic operands per precision.

Method (the one the reference's tools use, tools/common.py:57-125): every timed call reads a different copy of the
weight and the copies together exceed the L2 cache several times, so each call streams its weight from HBM as in a
decode step; the calls are captured once into a CUDA graph, the graph is replayed and timed with CUDA events on the
replaying stream, and the median replay is reported per call. B200's L2 is 126 MB, so at least 512 MB rotate.
"""

from __future__ import annotations

import torch

FP8 = torch.float8_e4m3fn
FP4 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)
MIN_ROTATION_BYTES = 512 << 20


def weight_bytes(kind: str, n: int, k: int) -> int:
    bits = {"bf16": 16, "f16": 16, "fp8": 8, "int8": 8, "nvfp4": 4}.get(kind, 8 if kind.startswith("w8") else 4)
    return n * k * bits // 8 + (n * (k // 16) if (kind == "nvfp4" or kind.startswith("w4a16")) else 0)


def algorithmic_bytes(kind: str, m: int, n: int, k: int, out_bytes: int = 2, x_scale_len: int = 0, w_scale_len: int = 0,
                      bias_bytes: int = 0) -> int:
    """Bytes one GEMM must move when every operand is touched exactly once (split-K workspace traffic not counted):
    weight + weight block scales + activations + activation block scales + output + scale vectors + bias."""
    xbits = {"fp8": 8, "int8": 8, "nvfp4": 4}.get(kind, 16)
    sf_x = m * (k // 16) if kind == "nvfp4" else 0
    return weight_bytes(kind, n, k) + m * k * xbits // 8 + sf_x + m * n * out_bytes + 4 * (x_scale_len + w_scale_len) + bias_bytes


def make_weight(kind: str, n: int, k: int, g: torch.Generator, device) -> tuple[torch.Tensor, dict]:
    """A synthetic weight of this precision and the gemm() keyword arguments that go with it."""
    if kind in ("bf16", "f16"):
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        return (torch.randn(n, k, device=device, generator=g) * 0.02).to(dt), {}
    if kind == "fp8" or kind.startswith("w8a16"):
        return (torch.randn(n, k, device=device, generator=g) * 4).to(FP8), {
            "w_scale": (torch.rand(n, device=device, generator=g) * 1.5 + 0.5) * 1e-3}
    if kind == "int8":
        return torch.randint(-127, 128, (n, k), device=device, generator=g, dtype=torch.int8), {
            "w_scale": (torch.rand(n, device=device, generator=g) + 0.5) * 1e-2}
    if kind == "nvfp4" or kind.startswith("w4a16"):
        w = torch.randint(0, 256, (n, k // 2), device=device, generator=g, dtype=torch.uint8).view(FP4)
        sf = torch.randint(0x18, 0x48, (n, k // 16), device=device, generator=g, dtype=torch.uint8).view(FP8)
        return w, {"w_block_scale": sf, "w_scale": 1e-3}
    raise ValueError(kind)


def make_input(kind: str, m: int, k: int, device, seed: int = 1234) -> tuple[torch.Tensor, dict]:
    g = torch.Generator(device=device).manual_seed(seed)
    if kind == "bf16" or kind.endswith("_bf16"):
        return torch.randn(m, k, device=device, generator=g).to(torch.bfloat16), {}
    if kind == "f16" or kind.endswith("_f16"):
        return torch.randn(m, k, device=device, generator=g).to(torch.float16), {}
    if kind == "fp8":
        return (torch.randn(m, k, device=device, generator=g) * 4).to(FP8), {
            "x_scale": torch.rand(m, device=device, generator=g) + 0.5}
    if kind == "int8":
        return torch.randint(-127, 128, (m, k), device=device, generator=g, dtype=torch.int8), {
            "x_scale": torch.rand(m, device=device, generator=g) + 0.5}
    if kind == "nvfp4":
        x = torch.randint(0, 256, (m, k // 2), device=device, generator=g, dtype=torch.uint8).view(FP4)
        sf = torch.randint(0x18, 0x48, (m, k // 16), device=device, generator=g, dtype=torch.uint8).view(FP8)
        return x, {"x_block_scale": sf}
    raise ValueError(kind)


class ColdWeights:
    """Enough distinct copies of one (kind, N, K) weight that consecutive calls never find theirs in L2."""

    def __init__(self, kind: str, n: int, k: int, device, min_bytes: int = MIN_ROTATION_BYTES, max_copies: int = 4096):
        self.kind, self.n, self.k = kind, n, k
        self.nbytes = weight_bytes(kind, n, k)
        copies = max(2, min(max_copies, -(-min_bytes // self.nbytes)))
        g = torch.Generator(device=device).manual_seed(0)
        first = make_weight(kind, n, k, g, device)
        self.items = [first]
        for _ in range(copies - 1):  # same values, different addresses: content does not matter for timing
            w, kw = first
            self.items.append((w.clone(), {a: (b.clone() if torch.is_tensor(b) else b) for a, b in kw.items()}))

    def __len__(self) -> int:
        return len(self.items)


def time_graph(build, replays: int = 20, warm_replays: int = 2) -> float:
    """Captures build() (which issues work on the current stream) into a CUDA graph; returns the median replay time
    in microseconds, timed with CUDA events on the replaying stream."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        build()  # warm-up outside capture: lazy plan loading, workspace growth, module loading
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        build()
    for _ in range(warm_replays):
        graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) * 1000.0)
    del graph
    times.sort()
    return times[len(times) // 2]


def time_per_call(fn, weights: ColdWeights, calls: int | None = None, replays: int = 20, before=None) -> float:
    """Median microseconds per fn(w, w_kwargs, next_w) over a graph of `calls` calls on rotating weights. With `before`
    (a small producer kernel launched ahead of every call) the time of a producer-only graph is subtracted."""
    calls = calls or max(len(weights), 64)
    seq = [weights.items[i % len(weights)] for i in range(calls)]
    nxt = [weights.items[(i + 1) % len(weights)][0] for i in range(calls)]

    def build(with_fn: bool):
        def run():
            for i, (w, kw) in enumerate(seq):
                if before is not None:
                    before()
                if with_fn:
                    fn(w, kw, nxt[i])
        return run

    t = time_graph(build(True), replays) / calls
    if before is not None:
        t -= time_graph(build(False), replays) / calls
    return t
