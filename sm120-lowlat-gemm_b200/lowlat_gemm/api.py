"""gemm() and the activation quantizers: the call surface of the reference (lowlat_gemm/__init__.py:355-620) on top
of the sm_100a core.

    y = alpha * (x * x_scale) @ (w * w_scale)^T + bias

Precision comes from the dtypes of x and w (bf16/f16 x same, x fp8, x fp4 weights; fp8 x fp8; int8 x int8;
fp4 x fp4). fp4 tensors are torch.float4_e2m1fn_x2 (or uint8 together with a block scale): two values per byte, the
even element in the low nibble, one e4m3 block scale per 16 values.
"""

from __future__ import annotations

import torch

from . import _ops  # noqa: F401  (registers torch.ops.lowlat_gemm)
from .plans import (KINDS, SKINNY_MAX_TOKENS, _MIXED, Plan, _dev, _sm_count, _tc_lookup, default_tc_choice, get_plan,
                    skinny_ranges, tc_info)

_FP4 = getattr(torch, "float4_e2m1fn_x2", None)
_FP8 = torch.float8_e4m3fn
_FP4_KINDS = ("nvfp4", "w4a16_bf16", "w4a16_f16")

# one (4-byte partials, int32 counters) pair per device; every launch on a stream reuses it and leaves the counters
# at zero (reference lowlat_gemm/__init__.py:353-394)
_ws: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


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
    ws, cnt = _ws.get(device.index, (None, None))
    if ws is not None and ws.numel() >= elems and cnt.numel() >= counters:
        return
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError(f"lowlat_gemm: split-K workspace too small during CUDA graph capture (need {elems} partials, "
                           f"{counters} counters); call reserve_workspace() before capture")
    elems = max(elems, 1 << 20, ws.numel() if ws is not None else 0)
    counters = max(counters, 1 << 12, cnt.numel() if cnt is not None else 0)
    _ws[device.index] = (torch.empty(elems, dtype=torch.float32, device=device),
                         torch.zeros(counters, dtype=torch.int32, device=device))


def _workspace(device: torch.device, elems: int, counters: int):
    device = _dev(device)
    reserve_workspace(device, elems, counters)
    return _ws[device.index]


def _is_fp4(t: torch.Tensor, block_scale) -> bool:
    return (_FP4 is not None and t.dtype == _FP4) or (t.dtype == torch.uint8 and block_scale is not None)


def kind_of(x: torch.Tensor, w: torch.Tensor, x_block_scale=None, w_block_scale=None) -> str:
    xt, wt = x.dtype, w.dtype
    if xt in (torch.bfloat16, torch.float16):
        tag = "bf16" if xt == torch.bfloat16 else "f16"
        if wt == xt:
            return tag
        if wt == _FP8:
            return "w8a16_" + tag
        if _is_fp4(w, w_block_scale):
            return "w4a16_" + tag
    elif xt == _FP8 and wt == _FP8:
        return "fp8"
    elif xt == torch.int8 and wt == torch.int8:
        return "int8"
    elif _is_fp4(x, x_block_scale) and _is_fp4(w, w_block_scale):
        return "nvfp4"
    raise TypeError(f"lowlat_gemm: unsupported dtype pair x={xt}, w={wt}")


def supports(x: torch.Tensor, w: torch.Tensor, x_block_scale=None, w_block_scale=None) -> bool:
    """True when gemm(x, w, ...) can run on these operands (dtype pair, K alignment, 16-byte rows)."""
    if not (x.is_cuda and w.is_cuda and w.dim() == 2 and x.dim() >= 1):
        return False
    try:
        kind = kind_of(x, w, x_block_scale, w_block_scale)
    except TypeError:
        return False
    k = w.shape[1] * (2 if kind in _FP4_KINDS else 1)
    if k == 0 or k % KINDS[kind][2] or x.shape[-1] * (2 if kind == "nvfp4" else 1) != k:
        return False
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() != 2 and x.is_contiguous() else x
    for t in (x2, w):
        if t.dim() != 2 or t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
            return False
    return True


def workspace_need(kind: str, n: int, k: int, max_m: int, device: torch.device | None = None) -> tuple[int, int]:
    """(partials, counters) the split-K buffers need for every M <= max_m of this (kind, N, K)."""
    device = _dev(device)
    plan = get_plan(kind, n, k, device)
    elems = counters = 0
    for m in range(1, max_m + 1):
        if plan.skinny is not None and m <= min(plan.skinny_max_m, SKINNY_MAX_TOKENS):
            o = plan.skinny
            if o.ksplit > 1 and not o.cluster:
                elems = max(elems, o.ksplit * m * n)
                counters = max(counters, skinny_ranges(n, o.ksplit, _sm_count(device)))
            continue
        c = _tc_lookup(plan.tc, m) or default_tc_choice(kind, m, n, k, _sm_count(device))
        if c.ksplit > 1 and not c.cluster:
            bp, bq, _, _ = tc_info(kind, c.cfg)
            p, q = (n, m) if (c.swap or kind in _MIXED) else (m, n)
            elems = max(elems, c.ksplit * p * q)
            counters = max(counters, -(-p // bp) * -(-q // bq))
    return elems, counters


def _bytes_view(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype != torch.uint8 and t.element_size() == 1 else t


def _f32_vec(v: torch.Tensor) -> torch.Tensor:
    v = v.reshape(-1)
    return v if v.dtype == torch.float32 and v.is_contiguous() else v.float().contiguous()


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
    kind = kind_of(x, w, x_block_scale, w_block_scale)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    m, n = x2.shape[0], w.shape[0]
    k = w.shape[1] * (2 if kind in _FP4_KINDS else 1)
    if x2.shape[1] * (2 if kind == "nvfp4" else 1) != k:
        raise ValueError(f"lowlat_gemm: x has K={x2.shape[1]} but w {tuple(w.shape)} implies K={k}")
    device = _dev(x2.device)
    if out is not None:
        out_dtype = out.dtype
    elif out_dtype is None:
        out_dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
    y2 = out.view(-1, n) if out is not None else torch.empty(m, n, dtype=out_dtype, device=device)
    result = out if out is not None else y2.view(*lead, n)
    if m == 0:
        return result
    plan = plan or get_plan(kind, n, k, device)

    plain = x_scale is None and w_scale is None and alpha is None and bias is None
    if (plan.skinny is not None and m <= min(plan.skinny_max_m, SKINNY_MAX_TOKENS) and plain
            and y2.dtype in (x.dtype, torch.float32)):
        order = plan.skinny
        tile = order.tile(m)
        if order.ksplit > 1 and not order.cluster:
            ws, cnt = _workspace(device, order.ksplit * m * n, skinny_ranges(n, order.ksplit, _sm_count(device)))
        else:
            ws, cnt = _workspace(device, 0, 0)
        torch.ops.lowlat_gemm.skinny_out(y2, x2, w, ws, cnt, tile.rows, tile.unroll, order.lanes_per_row, tile.warps,
                                         order.ksplit, order.cluster, prefetch, prefetch_bytes)
        return result

    c = _tc_lookup(plan.tc, m) or default_tc_choice(kind, m, n, k, _sm_count(device))
    swap = c.swap or kind in _MIXED
    # python numbers fold into one host float: no tensor is created, so capture into a CUDA graph stays legal
    host_alpha = 1.0
    for v in (x_scale, w_scale):
        if v is not None and not torch.is_tensor(v):
            host_alpha *= float(v)
    xs = _f32_vec(x_scale) if torch.is_tensor(x_scale) else None
    wsc = _f32_vec(w_scale) if torch.is_tensor(w_scale) else None
    alpha_t = None
    if torch.is_tensor(alpha):
        alpha_t = alpha.reshape(1)
        alpha_t = alpha_t if alpha_t.dtype == torch.float32 else alpha_t.float()
    elif alpha is not None:
        host_alpha *= float(alpha)
    xa = _bytes_view(x2) if (kind == "nvfp4" or x2.element_size() == 1) else x2
    wa = _bytes_view(w) if w.element_size() == 1 else w
    xsf = _bytes_view(x_block_scale) if x_block_scale is not None else None
    wsf = _bytes_view(w_block_scale) if w_block_scale is not None else None
    if swap:
        a, b, a_sf, b_sf, row_s, col_s, p, q = wa, xa, wsf, xsf, wsc, xs, n, m
    else:
        a, b, a_sf, b_sf, row_s, col_s, p, q = xa, wa, xsf, wsf, xs, wsc, m, n
    if kind in ("w4a16_bf16", "w4a16_f16"):
        a_sf, b_sf = wsf, None
    bp, bq, _, _ = tc_info(kind, c.cfg)
    tiles = -(-p // bp) * -(-q // bq)
    use_ws = c.ksplit > 1 and not c.cluster
    wsp, cnt = _workspace(device, c.ksplit * p * q if use_ws else 0, tiles if use_ws else 0)
    torch.ops.lowlat_gemm.tc_gemm(y2, a, b, a_sf, b_sf, row_s, col_s, bias, alpha_t, host_alpha, KINDS[kind][0], swap,
                                  swap, c.cfg, c.stages, c.ksplit, wsp, cnt, c.cluster, prefetch, prefetch_bytes)
    return result


# ---------------------------------------------------------------------------------------------------------------
# activation quantizers (reference lowlat_gemm/__init__.py:586-620)


def quantize_fp8(x: torch.Tensor, scale: torch.Tensor | None = None, min_scale: float = 1e-12):
    """x [M, K] bf16/f16/f32 -> (q float8_e4m3fn [M, K], scale). Static when `scale` (a 1-element float32 tensor) is
    given, else dynamic per token: scale[m] = amax(x[m]) / 448."""
    x2 = x.reshape(-1, x.shape[-1])
    q = torch.empty(x2.shape, dtype=_FP8, device=x.device)
    if scale is not None:
        s = scale.reshape(1).float()
        torch.ops.lowlat_gemm.quant(x2, q.view(torch.uint8), None, s, None, 0, min_scale)
    else:
        s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        torch.ops.lowlat_gemm.quant(x2, q.view(torch.uint8), None, None, s, 1, min_scale)
    return q.view(*x.shape), s


def quantize_int8(x: torch.Tensor, min_scale: float = 1e-12):
    """x [M, K] -> (q int8 [M, K], scale float32 [M]); scale[m] = amax(x[m]) / 127, round to nearest even."""
    x2 = x.reshape(-1, x.shape[-1])
    q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    torch.ops.lowlat_gemm.quant(x2, q, None, None, s, 2, min_scale)
    return q.view(*x.shape), s


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor):
    """x [M, K] -> (q fp4 [M, K/2], block_scale float8_e4m3fn [M, K/16]). Per 16 elements sf = e4m3(amax / 6 * g) and
    q = e2m1(x * g / sf), so x ~= q * sf / g: pass x_scale = 1 / g to gemm()."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, k = x2.shape
    q = torch.empty(rows, k // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(rows, k // 16, dtype=torch.uint8, device=x.device)
    torch.ops.lowlat_gemm.quant(x2, q, sf, global_scale.reshape(1).float(), None, 3, 0.0)
    return (q.view(_FP4) if _FP4 is not None else q), sf.view(_FP8)


# ---------------------------------------------------------------------------------------------------------------
# gated activation fused with the quantizer (input side of the down projection; no counterpart in the reference)

_DT_CODE = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}


def _gated(gate_up: torch.Tensor, mode: int, global_scale: torch.Tensor | None, want_act: bool):
    import ctypes as C

    from . import _native as N

    gu = gate_up.reshape(-1, gate_up.shape[-1])
    rows, two_k = gu.shape
    k = two_k // 2
    if two_k % 2 or gu.stride(1) != 1 or gu.dtype not in _DT_CODE or not gu.is_cuda:
        raise RuntimeError("lowlat_gemm: gate_up must be a CUDA [M, 2K] bf16/f16/f32 tensor with unit last stride")
    a = N.GatedQuantArgs()
    a.q.mode, a.q.in_dtype, a.q.M, a.q.K = mode, _DT_CODE[gu.dtype], rows, k
    a.q.x, a.q.ldx = gu.data_ptr(), gu.stride(0)
    a.up, a.ldup = gu.data_ptr() + k * gu.element_size(), gu.stride(0)
    act = q = s = sf = None
    if want_act or mode == 4:
        act = torch.empty(rows, k, dtype=gu.dtype, device=gu.device)
        a.act, a.ldact = act.data_ptr(), act.stride(0)
    if mode == 1:
        q = torch.empty(rows, k, dtype=_FP8, device=gu.device)
        s = torch.empty(rows, dtype=torch.float32, device=gu.device)
        a.q.q, a.q.ldq, a.q.scale_out, a.q.min_scale = q.data_ptr(), q.stride(0), s.data_ptr(), 1e-12
    elif mode == 3:
        q = torch.empty(rows, k // 2, dtype=torch.uint8, device=gu.device)
        sf = torch.empty(rows, k // 16, dtype=torch.uint8, device=gu.device)
        g = global_scale.reshape(1).float()
        a.q.q, a.q.ldq, a.q.sf_out, a.q.ldsf, a.q.scale_in = q.data_ptr(), q.stride(0), sf.data_ptr(), sf.stride(0), g.data_ptr()
    with torch.cuda.device(gu.device):
        N.check(N.lib.llg_gated_quant(C.byref(a), C.c_void_p(torch.cuda.current_stream(gu.device).cuda_stream)))
    return act, q, s, sf


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[M, 2K] = [gate | up] -> silu(gate) * up as [M, K] in the input type (fp32 arithmetic, one rounding)."""
    return _gated(gate_up, 4, None, True)[0]


def silu_mul_quantize_fp8(gate_up: torch.Tensor):
    """quantize_fp8(silu_mul(gate_up)) in one kernel: (q float8_e4m3fn [M, K], scale float32 [M])."""
    _, q, s, _ = _gated(gate_up, 1, None, False)
    return q, s


def silu_mul_quantize_nvfp4(gate_up: torch.Tensor, global_scale: torch.Tensor):
    """quantize_nvfp4(silu_mul(gate_up), global_scale) in one kernel: (q fp4 [M, K/2], block scales e4m3 [M, K/16])."""
    _, q, _, sf = _gated(gate_up, 3, global_scale, False)
    return (q.view(_FP4) if _FP4 is not None else q), sf.view(_FP8)
