"""gemm() and the activation quantizers: the call surface of the reference (lowlat_gemm/__init__.py:355-620) on top
of the sm_100a core.

    y = alpha * (x * x_scale) @ (w * w_scale)^T + bias

Precision comes from the dtypes of x and w (bf16/f16 x same, x fp8, x fp4 weights; fp8 x fp8; int8 x int8;
fp4 x fp4). fp4 tensors are torch.float4_e2m1fn_x2 (or uint8 together with a block scale): two values per byte, the
even element in the low nibble, one e4m3 block scale per 16 values.

How a call is put together here: `_Problem` pins down kind, shapes and the output; `_route` picks the engine from the
plan; the skinny route goes straight to its op, the tensor-core route builds a `TcLaunch` (operand orientation, scale
folding, split-K buffers) whose `op_args()` are the positional arguments of torch.ops.lowlat_gemm.tc_gemm. The
tensor-parallel code reuses `TcLaunch` to send the same launch through the push entry point of the C ABI.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _ops  # noqa: F401  (registers torch.ops.lowlat_gemm)
from .plans import (KINDS, SKINNY_MAX_TOKENS, _MIXED, Plan, TcChoice, _dev, _sm_count, _tc_lookup, default_tc_choice,
                    get_plan, skinny_ranges, tc_info)

_FP4 = getattr(torch, "float4_e2m1fn_x2", None)
_FP8 = torch.float8_e4m3fn
_FP4_KINDS = ("nvfp4", "w4a16_bf16", "w4a16_f16")
_ACT16 = {torch.bfloat16: "bf16", torch.float16: "f16"}
_MIN_PARTIALS, _MIN_COUNTERS = 1 << 20, 1 << 12

# one (4-byte partials, int32 counters) pair per device; every launch on a stream reuses it and leaves the counters
# at zero (reference lowlat_gemm/__init__.py:353-394)
_ws: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


# ---------------------------------------------------------------------------------------------------------------
# process-wide switches and the split-K buffers


def set_pdl(on: bool = True) -> None:
    """Programmatic dependent launch for all later gemm() calls (process-wide). A GEMM may then begin while the
    previous kernel of the stream still runs: it streams its weight first and touches activations, outputs and
    split-K buffers only after that kernel has finished. Enable it only when nothing in flight writes the weights.
    CUDA graphs keep the setting they were captured with."""
    torch.ops.lowlat_gemm.set_pdl(bool(on))


def pdl_enabled() -> bool:
    return bool(torch.ops.lowlat_gemm.pdl_enabled())


def reserve_workspace(device: torch.device, elems: int, counters: int) -> None:
    """Grow the split-K buffers of `device` to at least `elems` partials and `counters` counters. Call before CUDA
    graph capture: growing during capture raises."""
    device = _dev(device)
    have = _ws.get(device.index)
    if have is not None and have[0].numel() >= elems and have[1].numel() >= counters:
        return
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError(f"lowlat_gemm: split-K workspace too small during CUDA graph capture (need {elems} partials, "
                           f"{counters} counters); call reserve_workspace() before capture")
    old_p, old_c = (have[0].numel(), have[1].numel()) if have is not None else (0, 0)
    _ws[device.index] = (torch.empty(max(elems, _MIN_PARTIALS, old_p), dtype=torch.float32, device=device),
                         torch.zeros(max(counters, _MIN_COUNTERS, old_c), dtype=torch.int32, device=device))


def _workspace(device: torch.device, elems: int, counters: int):
    device = _dev(device)
    reserve_workspace(device, elems, counters)
    return _ws[device.index]


# ---------------------------------------------------------------------------------------------------------------
# what a call is: precision, shapes, output


def _is_fp4(t: torch.Tensor, block_scale) -> bool:
    return (_FP4 is not None and t.dtype == _FP4) or (t.dtype == torch.uint8 and block_scale is not None)


def kind_of(x: torch.Tensor, w: torch.Tensor, x_block_scale=None, w_block_scale=None) -> str:
    act = _ACT16.get(x.dtype)
    if act is not None:
        if w.dtype == x.dtype:
            return act
        if w.dtype == _FP8:
            return "w8a16_" + act
        if _is_fp4(w, w_block_scale):
            return "w4a16_" + act
    else:
        pair = (x.dtype, w.dtype)
        if pair == (_FP8, _FP8):
            return "fp8"
        if pair == (torch.int8, torch.int8):
            return "int8"
        if _is_fp4(x, x_block_scale) and _is_fp4(w, w_block_scale):
            return "nvfp4"
    raise TypeError(f"lowlat_gemm: unsupported dtype pair x={x.dtype}, w={w.dtype}")


def _k_of(kind: str, w: torch.Tensor) -> int:
    return w.shape[1] * 2 if kind in _FP4_KINDS else w.shape[1]


def _rows_ok(t: torch.Tensor) -> bool:
    """2-D, unit inner stride, rows 16-byte aligned and a 16-byte multiple apart: what a TMA map (and the reference) needs."""
    return t.dim() == 2 and t.stride(1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0


def supports(x: torch.Tensor, w: torch.Tensor, x_block_scale=None, w_block_scale=None) -> bool:
    """True when gemm(x, w, ...) can run on these operands (dtype pair, K alignment, 16-byte rows)."""
    if not (x.is_cuda and w.is_cuda and w.dim() == 2 and x.dim() >= 1):
        return False
    try:
        kind = kind_of(x, w, x_block_scale, w_block_scale)
    except TypeError:
        return False
    k = _k_of(kind, w)
    x_k = x.shape[-1] * (2 if kind == "nvfp4" else 1)
    if k == 0 or k % KINDS[kind][2] or x_k != k:
        return False
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 and x.is_contiguous() else x
    return _rows_ok(x2) and _rows_ok(w)


@dataclass
class _Problem:
    kind: str
    m: int
    n: int
    k: int
    x2: torch.Tensor      # activations as [M, K]
    w: torch.Tensor
    y2: torch.Tensor      # output as [M, N]
    result: torch.Tensor  # what gemm() returns (y2 in the caller's shape, or `out` itself)
    device: torch.device


def _problem(x, w, x_block_scale, w_block_scale, out_dtype, out) -> _Problem:
    kind = kind_of(x, w, x_block_scale, w_block_scale)
    x2 = x.reshape(-1, x.shape[-1])
    m, n, k = x2.shape[0], w.shape[0], _k_of(kind, w)
    x_k = x2.shape[1] * (2 if kind == "nvfp4" else 1)
    if x_k != k:
        raise ValueError(f"lowlat_gemm: x has K={x2.shape[1]} but w {tuple(w.shape)} implies K={k}")
    device = _dev(x2.device)
    if out is not None:  # out wins over out_dtype
        y2, result = out.view(-1, n), out
    else:
        dt = out_dtype or (x.dtype if x.dtype in _ACT16 else torch.bfloat16)
        y2 = torch.empty(m, n, dtype=dt, device=device)
        result = y2.view(*x.shape[:-1], n)
    return _Problem(kind, m, n, k, x2, w, y2, result, device)


# ---------------------------------------------------------------------------------------------------------------
# engine choice and the two launch paths


def _skinny_serves(pr: _Problem, plan: Plan, plain: bool) -> bool:
    """The CUDA-core GEMV takes W16A16 calls without any epilogue term, up to the plan's token limit."""
    return (plan.skinny is not None and pr.m <= min(plan.skinny_max_m, SKINNY_MAX_TOKENS) and plain
            and pr.y2.dtype in (pr.x2.dtype, torch.float32))


def _launch_skinny(pr: _Problem, plan: Plan, prefetch, prefetch_bytes) -> None:
    order = plan.skinny
    tile = order.tile(pr.m)
    split = order.ksplit > 1 and not order.cluster
    ws, cnt = _workspace(pr.device, order.ksplit * pr.m * pr.n if split else 0,
                         skinny_ranges(pr.n, order.ksplit, _sm_count(pr.device)) if split else 0)
    torch.ops.lowlat_gemm.skinny_out(pr.y2, pr.x2, pr.w, ws, cnt, tile.rows, tile.unroll, order.lanes_per_row, tile.warps,
                                     order.ksplit, order.cluster, prefetch, prefetch_bytes)


def _bytes(t):
    if t is None:
        return None
    return t.view(torch.uint8) if t.dtype != torch.uint8 and t.element_size() == 1 else t


def _scale_split(v):
    """A scale given as a python number folds into the host alpha; a tensor becomes a contiguous fp32 vector."""
    if v is None:
        return 1.0, None
    if torch.is_tensor(v):
        vec = v.reshape(-1)
        return 1.0, vec if vec.dtype == torch.float32 and vec.is_contiguous() else vec.float().contiguous()
    return float(v), None


@dataclass
class TcLaunch:
    """One tensor-core launch, ready for the op: operands already in (A, B) orientation."""

    y2: torch.Tensor
    a: torch.Tensor
    b: torch.Tensor
    a_sf: torch.Tensor | None
    b_sf: torch.Tensor | None
    row_scale: torch.Tensor | None
    col_scale: torch.Tensor | None
    bias: torch.Tensor | None
    alpha_t: torch.Tensor | None
    alpha: float
    kind_id: int
    swap: bool
    choice: TcChoice
    ws: torch.Tensor = field(repr=False, default=None)
    counters: torch.Tensor = field(repr=False, default=None)
    prefetch: torch.Tensor | None = None
    prefetch_bytes: int = 0

    def op_args(self) -> tuple:
        c = self.choice
        return (self.y2, self.a, self.b, self.a_sf, self.b_sf, self.row_scale, self.col_scale, self.bias, self.alpha_t,
                self.alpha, self.kind_id, self.swap, self.swap, c.cfg, c.stages, c.ksplit, self.ws, self.counters, c.cluster,
                self.prefetch, self.prefetch_bytes)


def tc_launch_for(pr: _Problem, choice: TcChoice, *, x_scale=None, w_scale=None, x_block_scale=None, w_block_scale=None,
                  alpha=None, bias=None, prefetch=None, prefetch_bytes: int = 0) -> TcLaunch:
    """Orientation, scale folding and split-K buffers of a tensor-core call. With few tokens the weight is operand A
    (its rows fill the 128-row MMA tile, the result is stored transposed): the scales and block scales swap sides
    with the operands. Python numbers never become tensors here, so capture into a CUDA graph stays legal."""
    fx, xs = _scale_split(x_scale)
    fw, wsc = _scale_split(w_scale)
    host_alpha = fx * fw
    alpha_t = None
    if torch.is_tensor(alpha):
        alpha_t = alpha.reshape(1)
        alpha_t = alpha_t if alpha_t.dtype == torch.float32 else alpha_t.float()
    elif alpha is not None:
        host_alpha *= float(alpha)
    narrow_x = pr.kind == "nvfp4" or pr.x2.element_size() == 1
    act = (_bytes(pr.x2) if narrow_x else pr.x2, _bytes(x_block_scale), xs, pr.m)
    wgt = (_bytes(pr.w) if pr.w.element_size() == 1 else pr.w, _bytes(w_block_scale), wsc, pr.n)
    swap = choice.swap or pr.kind in _MIXED
    (a, a_sf, row_s, p), (b, b_sf, col_s, q) = (wgt, act) if swap else (act, wgt)
    if pr.kind.startswith("w4a16"):
        a_sf, b_sf = wgt[1], None  # only the weight carries block scales, and it is always operand A
    bp, bq, _, _ = tc_info(pr.kind, choice.cfg)
    via_ws = choice.ksplit > 1 and not choice.cluster
    ws, cnt = _workspace(pr.device, choice.ksplit * p * q if via_ws else 0, -(-p // bp) * -(-q // bq) if via_ws else 0)
    return TcLaunch(pr.y2, a, b, a_sf, b_sf, row_s, col_s, bias, alpha_t, host_alpha, KINDS[pr.kind][0], swap, choice, ws, cnt,
                    prefetch, prefetch_bytes)


def tc_choice_for(kind: str, m: int, n: int, k: int, plan: Plan, device: torch.device) -> TcChoice:
    return _tc_lookup(plan.tc, m) or default_tc_choice(kind, m, n, k, _sm_count(device))


def gemm(x: torch.Tensor, w: torch.Tensor, *, x_scale=None, w_scale=None, x_block_scale: torch.Tensor | None = None,
         w_block_scale: torch.Tensor | None = None, alpha=None, bias: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None, plan: Plan | None = None,
         prefetch: torch.Tensor | None = None, prefetch_bytes: int = 0) -> torch.Tensor:
    """y[..., N] = alpha * (x * x_scale) @ (w * w_scale)^T + bias.

    x_scale / w_scale: None, a float, or a float32 tensor with 1 element or one per row (M for x, N for w).
    alpha: None, a float or a 1-element float32 tensor (a device scalar stays valid inside CUDA graphs).
    out wins over out_dtype. prefetch: a contiguous tensor (usually the weight of the GEMM that runs next) whose first
    prefetch_bytes (0 = all) the kernel pulls into L2 once its own weight is streaming.
    """
    pr = _problem(x, w, x_block_scale, w_block_scale, out_dtype, out)
    if pr.m == 0:
        return pr.result
    plan = plan or get_plan(pr.kind, pr.n, pr.k, pr.device)
    plain = x_scale is None and w_scale is None and alpha is None and bias is None
    if _skinny_serves(pr, plan, plain):
        _launch_skinny(pr, plan, prefetch, prefetch_bytes)
    else:
        launch = tc_launch_for(pr, tc_choice_for(pr.kind, pr.m, pr.n, pr.k, plan, pr.device), x_scale=x_scale, w_scale=w_scale,
                               x_block_scale=x_block_scale, w_block_scale=w_block_scale, alpha=alpha, bias=bias,
                               prefetch=prefetch, prefetch_bytes=prefetch_bytes)
        torch.ops.lowlat_gemm.tc_gemm(*launch.op_args())
    return pr.result


def workspace_need(kind: str, n: int, k: int, max_m: int, device: torch.device | None = None) -> tuple[int, int]:
    """(partials, counters) the split-K buffers need for every M <= max_m of this (kind, N, K)."""
    device = _dev(device)
    plan = get_plan(kind, n, k, device)
    sms = _sm_count(device)
    need_p = need_c = 0
    for m in range(1, max_m + 1):
        if plan.skinny is not None and m <= min(plan.skinny_max_m, SKINNY_MAX_TOKENS):
            o = plan.skinny  # note: whether a call is plain enough for the skinny engine is not known here; both are counted
            if o.ksplit > 1 and not o.cluster:
                need_p, need_c = max(need_p, o.ksplit * m * n), max(need_c, skinny_ranges(n, o.ksplit, sms))
        c = tc_choice_for(kind, m, n, k, plan, device)
        if c.ksplit > 1 and not c.cluster:
            bp, bq, _, _ = tc_info(kind, c.cfg)
            p, q = (n, m) if (c.swap or kind in _MIXED) else (m, n)
            need_p, need_c = max(need_p, c.ksplit * p * q), max(need_c, -(-p // bp) * -(-q // bq))
    return need_p, need_c


# ---------------------------------------------------------------------------------------------------------------
# activation quantizers (reference lowlat_gemm/__init__.py:586-620)

_Q_FP8_STATIC, _Q_FP8_TOKEN, _Q_INT8_TOKEN, _Q_NVFP4, _Q_NONE = 0, 1, 2, 3, 4


def _rows(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


def quantize_fp8(x: torch.Tensor, scale: torch.Tensor | None = None, min_scale: float = 1e-12):
    """x [M, K] bf16/f16/f32 -> (q float8_e4m3fn [M, K], scale). Static when `scale` (a 1-element float32 tensor) is
    given, else dynamic per token: scale[m] = amax(x[m]) / 448."""
    x2 = _rows(x)
    q = torch.empty(x2.shape, dtype=_FP8, device=x.device)
    static = scale is not None
    s = scale.reshape(1).float() if static else torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    torch.ops.lowlat_gemm.quant(x2, q.view(torch.uint8), None, s if static else None, None if static else s,
                                _Q_FP8_STATIC if static else _Q_FP8_TOKEN, min_scale)
    return q.view(*x.shape), s


def quantize_int8(x: torch.Tensor, min_scale: float = 1e-12):
    """x [M, K] -> (q int8 [M, K], scale float32 [M]); scale[m] = amax(x[m]) / 127, round to nearest even."""
    x2 = _rows(x)
    q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    torch.ops.lowlat_gemm.quant(x2, q, None, None, s, _Q_INT8_TOKEN, min_scale)
    return q.view(*x.shape), s


def _fp4_pair(q: torch.Tensor, sf: torch.Tensor):
    return (q.view(_FP4) if _FP4 is not None else q), sf.view(_FP8)


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor):
    """x [M, K] -> (q fp4 [M, K/2], block_scale float8_e4m3fn [M, K/16]). Per 16 elements sf = e4m3(amax / 6 * g) and
    q = e2m1(x * g / sf), so x ~= q * sf / g: pass x_scale = 1 / g to gemm()."""
    x2 = _rows(x)
    rows, k = x2.shape
    q = torch.empty(rows, k // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(rows, k // 16, dtype=torch.uint8, device=x.device)
    torch.ops.lowlat_gemm.quant(x2, q, sf, global_scale.reshape(1).float(), None, _Q_NVFP4, 0.0)
    return _fp4_pair(q, sf)


# ---------------------------------------------------------------------------------------------------------------
# gated activation fused with the quantizer (input side of the down projection; no counterpart in the reference)

_DT_CODE = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}


def _gated(gate_up: torch.Tensor, mode: int, global_scale: torch.Tensor | None, want_act: bool):
    import ctypes as C

    from . import _native as N

    gu = _rows(gate_up)
    rows, two_k = gu.shape
    k = two_k // 2
    if two_k % 2 or gu.stride(1) != 1 or gu.dtype not in _DT_CODE or not gu.is_cuda:
        raise RuntimeError("lowlat_gemm: gate_up must be a CUDA [M, 2K] bf16/f16/f32 tensor with unit last stride")
    a = N.GatedQuantArgs()
    a.q.mode, a.q.in_dtype, a.q.M, a.q.K = mode, _DT_CODE[gu.dtype], rows, k
    a.q.x, a.q.ldx = gu.data_ptr(), gu.stride(0)
    a.up, a.ldup = gu.data_ptr() + k * gu.element_size(), gu.stride(0)
    act = q = s = sf = None
    if want_act or mode == _Q_NONE:
        act = torch.empty(rows, k, dtype=gu.dtype, device=gu.device)
        a.act, a.ldact = act.data_ptr(), act.stride(0)
    if mode == _Q_FP8_TOKEN:
        q = torch.empty(rows, k, dtype=_FP8, device=gu.device)
        s = torch.empty(rows, dtype=torch.float32, device=gu.device)
        a.q.q, a.q.ldq, a.q.scale_out, a.q.min_scale = q.data_ptr(), q.stride(0), s.data_ptr(), 1e-12
    elif mode == _Q_NVFP4:
        q = torch.empty(rows, k // 2, dtype=torch.uint8, device=gu.device)
        sf = torch.empty(rows, k // 16, dtype=torch.uint8, device=gu.device)
        g = global_scale.reshape(1).float()
        a.q.q, a.q.ldq, a.q.sf_out, a.q.ldsf, a.q.scale_in = q.data_ptr(), q.stride(0), sf.data_ptr(), sf.stride(0), g.data_ptr()
    with torch.cuda.device(gu.device):
        N.check(N.lib.llg_gated_quant(C.byref(a), C.c_void_p(torch.cuda.current_stream(gu.device).cuda_stream)))
    return act, q, s, sf


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[M, 2K] = [gate | up] -> silu(gate) * up as [M, K] in the input type (fp32 arithmetic, one rounding)."""
    return _gated(gate_up, _Q_NONE, None, True)[0]


def silu_mul_quantize_fp8(gate_up: torch.Tensor):
    """quantize_fp8(silu_mul(gate_up)) in one kernel: (q float8_e4m3fn [M, K], scale float32 [M])."""
    _, q, s, _ = _gated(gate_up, _Q_FP8_TOKEN, None, False)
    return q, s


def silu_mul_quantize_nvfp4(gate_up: torch.Tensor, global_scale: torch.Tensor):
    """quantize_nvfp4(silu_mul(gate_up), global_scale) in one kernel: (q fp4 [M, K/2], block scales e4m3 [M, K/16])."""
    _, q, _, sf = _gated(gate_up, _Q_NVFP4, global_scale, False)
    return _fp4_pair(q, sf)
