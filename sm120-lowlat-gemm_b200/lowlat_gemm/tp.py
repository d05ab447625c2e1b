"""Tensor-parallel decode step over the GEMM library: one process per GPU, weights sharded Megatron-style.

Per layer (hidden H, intermediate I; the attention itself is outside the GEMM path and is stood in for by a slice):
    qkv      [QKV/tp, H]   column-parallel (no communication)
    o        [H, H/tp]     row-parallel    -> all-reduce(sum) of y[M, H]
    gate_up  [2*I/tp, H]   column-parallel, gate and up halves sharded separately so SiLU(gate)*up stays local
    down     [H, I/tp]     row-parallel    -> all-reduce(sum) of y[M, H]
The reference has no multi-GPU code; its nearest analogue is the single-GPU step replay tools/decode_step.py:27-172,
whose structure (per-layer weights so every GEMM streams from HBM, one CUDA graph per variant, PDL and next-weight
prefetch as options) this module keeps.

The GEMM and quantizer callables are parameters so the sharding and collective logic can run on CPU ranks (gloo) in
tests with a host matmul; the defaults are the library's own CUDA entry points.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import timing

FP8 = torch.float8_e4m3fn


@dataclass(frozen=True)
class LayerShape:
    hidden: int = 8192
    qkv: int = 10240
    inter: int = 28672

    def shards(self, tp: int) -> dict[str, tuple[int, int]]:
        """Per-rank (N, K) of the four projections."""
        for v in (self.qkv, self.hidden, self.inter):
            if v % tp:
                raise ValueError(f"{v} is not divisible by tp={tp}")
        return {"qkv": (self.qkv // tp, self.hidden), "o": (self.hidden, self.hidden // tp),
                "gate_up": (2 * self.inter // tp, self.hidden), "down": (self.hidden, self.inter // tp)}


def shard_rows(w: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Column-parallel shard: a contiguous block of output rows."""
    n = w.shape[0] // tp
    return w[rank * n:(rank + 1) * n]


def shard_cols(w: torch.Tensor, tp: int, rank: int, per_elem: int = 1) -> torch.Tensor:
    """Row-parallel shard: a contiguous block of K columns (per_elem = stored columns per K element, e.g. 1/2 for fp4
    is expressed by the caller passing the packed width)."""
    k = w.shape[1] // tp
    return w[:, rank * k:(rank + 1) * k].contiguous()


def shard_gate_up(w: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """gate_up [2I, H] = [gate; up]: each half is sharded by rows and the two shards are stacked again."""
    half = w.shape[0] // 2
    n = half // tp
    return torch.cat([w[rank * n:(rank + 1) * n], w[half + rank * n: half + (rank + 1) * n]], dim=0)


class DecodeLayer:
    """One rank's shard of one layer, with synthetic weights of the requested precision."""

    def __init__(self, kind: str, shape: LayerShape, tp: int, rank: int, device, seed: int = 0):
        self.kind, self.shape, self.tp, self.rank = kind, shape, tp, rank
        g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
        self.w = {name: timing.make_weight(kind, n, k, g, device) for name, (n, k) in shape.shards(tp).items()}
        if kind in ("bf16", "f16"):
            # 16-bit weights of N(0, 0.02) grow the hidden state by 0.02 * sqrt(K) per projection and overflow within a
            # few layers of the residual stream: rescale to 0.5 / sqrt(full K) so that values stay finite (timing is
            # value-independent, the check against NCCL is not)
            full_k = {"qkv": shape.hidden, "o": shape.hidden, "gate_up": shape.hidden, "down": shape.inter}
            self.w = {name: (w * (0.5 / (0.02 * full_k[name] ** 0.5)), kw) for name, (w, kw) in self.w.items()}

    def weight_bytes(self) -> int:
        return sum(timing.weight_bytes(self.kind, *nk) for nk in self.shape.shards(self.tp).values())


def _default_fns():
    from . import api
    return api.gemm, api.quantize_fp8, api.quantize_nvfp4, api


class DecodeStep:
    """`layers` decode layers on this rank; run() executes them in order on the current stream.

    residual=True keeps the hidden state of a decoder: h = h + all_reduce(o(...)), h = h + all_reduce(down(...)).
    comm: None (NCCL all_reduce, or no collective on one rank), or a comm.OneShotAllReduce. With a comm, `push=True`
    sends the row-parallel projections through the push form - the GEMM's epilogue stores into every rank's buffer, one
    consumer kernel sums, adds the residual and quantizes for the next projection - and `push=False` through the pull
    form (separate all-reduce kernel, fused with the FP8 quantizer where `fuse_quant` allows, residual added by an
    elementwise kernel). A single-rank comm (local=True) gives a one-GPU step the very same kernels."""

    def __init__(self, kind: str, layers: int, tp: int, rank: int, device, shape: LayerShape = LayerShape(), group=None,
                 gemm_fn=None, prefetch_bytes: int = 0, nvfp4_global: float = 64.0, comm=None, fuse_quant: bool = True,
                 residual: bool = False, push: bool = False):
        self.kind, self.tp, self.rank, self.group, self.device = kind, tp, rank, group, device
        self.shape = shape
        self.layers = [DecodeLayer(kind, shape, tp, rank, device, seed=i) for i in range(layers)]
        g, q8, q4, api = _default_fns() if gemm_fn is None else (gemm_fn, None, None, None)
        self._gemm, self._q8, self._q4, self._api = g, q8, q4, api
        self.prefetch_bytes = prefetch_bytes
        self.act_dtype = torch.float16 if kind.endswith("f16") and not kind.endswith("bf16") else torch.bfloat16
        self._g4 = torch.tensor([nvfp4_global], device=device) if kind == "nvfp4" else None
        self._g4_host = float(nvfp4_global)  # host copy: nothing on the launch path may read the device
        self.collectives = 0
        self.gemms = 0
        self.quants = 0
        self.reduces = 0  # the library's own all-reduce / local-sum kernels
        self.comm = comm if (tp > 1 or push) else None  # a comm.OneShotAllReduce, or None for NCCL all_reduce
        self.push = bool(push and self.comm is not None)
        self.residual = residual
        self._ar_index = 0
        self.fuse_quant = fuse_quant  # FP8 with `comm`: all-reduce and the next activation quantizer as one kernel

    def weight_bytes(self) -> int:
        return sum(l.weight_bytes() for l in self.layers)

    def _order(self):
        return [(li, name) for li in range(len(self.layers)) for name in ("qkv", "o", "gate_up", "down")]

    def _project(self, h, w, kw: dict, nxt, out=None, gated: bool = False, gemm=None) -> torch.Tensor:
        """One projection: activation quantization where the precision needs it, then the GEMM (`gemm`, default the
        library's gemm()). With `gated`, h is [gate | up] and the projection's input is silu(gate) * up, fused into the
        quantizer's kernel. h may be a (q, scale) pair that an earlier fused kernel already produced."""
        gemm = gemm or self._gemm
        extra = {} if out is None else {"out": out}
        if nxt is not None and self.prefetch_bytes:
            extra.update(prefetch=nxt, prefetch_bytes=min(self.prefetch_bytes, nxt.numel() * nxt.element_size()))
        self.gemms += 1
        if isinstance(h, tuple):
            q, s = h
            return gemm(q, w, x_scale=s, out_dtype=self.act_dtype, **kw, **extra)
        if gated and self._api is None:  # host stand-in used by the CPU tests
            half = h.shape[1] // 2
            h, gated = torch.nn.functional.silu(h[:, :half]) * h[:, half:], False
        if self.kind in ("fp8", "nvfp4") or gated:
            self.quants += 1  # one quantizer / activation kernel of the library
        if self.kind == "fp8":
            q, s = self._api.silu_mul_quantize_fp8(h) if gated else self._q8(h)
            return gemm(q, w, x_scale=s, out_dtype=self.act_dtype, **kw, **extra)
        if self.kind == "nvfp4":
            q, sf = self._api.silu_mul_quantize_nvfp4(h, self._g4) if gated else self._q4(h, self._g4)
            return gemm(q, w, x_block_scale=sf, x_scale=1.0 / self._g4_host, out_dtype=self.act_dtype, **kw, **extra)
        if gated:
            h = self._api.silu_mul(h)
        return gemm(h, w, out_dtype=self.act_dtype, **kw, **extra)

    def _row_parallel(self, h, w, kw: dict, nxt, resid, gated: bool = False, feeds_gemm: bool = False):
        """Row-parallel projection, sum over ranks, residual add. Returns (input of the next projection, hidden state);
        the former is a (q, scale) pair when a fused kernel already quantized it for an FP8 projection."""
        rows = h[0].shape[0] if isinstance(h, tuple) else h.shape[0]
        cols = w.shape[0]
        add = resid if self.residual else None
        if self.push:
            idx = self._ar_index
            self._ar_index += 1
            self.collectives += 1 if self.tp > 1 else 0
            self.reduces += 1

            def pushed(x, wt, *, out_dtype, **kwargs):
                self.comm.gemm_push(idx, x, wt, out_dtype=out_dtype, **kwargs)

            self._project(h, w, kw, nxt, gated=gated, gemm=pushed)
            quant = feeds_gemm and self.kind == "fp8"
            out, q, s = self.comm.reduce_local(idx, rows, cols, self.act_dtype, residual=add,
                                               want_out=self.residual or not quant, quantize=quant)
            return ((q, s) if quant else out), out
        if self.tp == 1:
            y = self._project(h, w, kw, nxt, gated=gated)
        else:
            self.collectives += 1
            if self.comm is None:
                y = self._project(h, w, kw, nxt, gated=gated)
                dist.all_reduce(y, group=self.group)
            else:
                idx = self._ar_index
                self._ar_index += 1
                self.reduces += 1
                part = self._project(h, w, kw, nxt, out=self.comm.view(idx, (rows, cols), self.act_dtype), gated=gated)
                fused = (feeds_gemm and self.fuse_quant and self.kind == "fp8" and add is None and rows <= 64
                         and cols % 8 == 0 and cols <= 16384)
                if fused:
                    return self.comm.reduce_quantize_fp8(idx, rows, cols, self.act_dtype), None
                y = self.comm.reduce(idx, torch.empty_like(part))
        if add is not None:
            y = y + add
        return y, y

    def run(self, x: torch.Tensor) -> torch.Tensor:
        """x [M, hidden] replicated on every rank -> [M, hidden] replicated (after the last all-reduce)."""
        self._ar_index = 0
        order = self._order()
        nxt_w = {order[i]: self.layers[order[(i + 1) % len(order)][0]].w[order[(i + 1) % len(order)][1]][0]
                 for i in range(len(order))}
        a_width = self.shape.hidden // self.tp
        h_in, hidden = x, x
        for li, layer in enumerate(self.layers):
            qkv = self._project(h_in, *layer.w["qkv"], nxt_w[(li, "qkv")])
            attn = qkv[:, :a_width]  # stand-in for this rank's attention heads' output
            if attn.data_ptr() % 16 or (attn.stride(0) * attn.element_size()) % 16:
                attn = attn.contiguous()  # the GEMM takes strided rows as long as they stay 16-byte aligned
            o_in, hidden = self._row_parallel(attn, *layer.w["o"], nxt_w[(li, "o")], hidden, feeds_gemm=True)
            gu = self._project(o_in, *layer.w["gate_up"], nxt_w[(li, "gate_up")])
            # the last layer's sum is the step's result; every other one also feeds the next layer's QKV projection
            last = li + 1 == len(self.layers)
            h_in, hidden = self._row_parallel(gu, *layer.w["down"], nxt_w[(li, "down")], hidden, gated=True,
                                              feeds_gemm=not last)
        return hidden if hidden is not None else h_in
