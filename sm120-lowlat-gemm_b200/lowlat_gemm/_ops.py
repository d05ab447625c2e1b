"""torch.ops.lowlat_gemm.*: the custom-op boundary, with the schema strings of the reference's TORCH_LIBRARY block
(csrc/ops.cpp:420-440) so callers written against it (tests, tools, serving hooks) work unchanged.

Two registrations of the same seven ops exist, both thin layers over the C ABI of libllg_core:
  * the C++ torch extension lowlat_gemm._C (csrc/ops.cpp, the counterpart of the reference's extension module): used
    whenever it has been built;
  * this module's torch.library registration over ctypes: the torch-free binding's sibling, used when _C is absent or
    when LLG_OPS=ctypes asks for it.
BACKEND says which one is active. Each op checks what only a tensor knows (device, dtype, contiguity; reference
csrc/ops.cpp:26-28, 63-83, 170-199, 308-360), then hands raw pointers, sizes and strides to libllg_core, which
validates the rest and launches on the current CUDA stream of the operand's device. Errors surface as
RuntimeError("lowlat_gemm: ...").
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _native as N

_DT = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}

def _try_cpp() -> bool:
    import os

    if os.environ.get("LLG_OPS", "").lower() == "ctypes":
        return False
    try:
        from . import _C  # noqa: F401  (its import registers the ops)
    except ImportError:
        return False
    return True


BACKEND = "cpp" if _try_cpp() else "ctypes"
_lib = torch.library.Library("lowlat_gemm", "DEF" if BACKEND == "ctypes" else "FRAGMENT")
if BACKEND == "ctypes":
    _lib.define("skinny(Tensor x, Tensor w, Tensor ws, Tensor counters, int rows, int unroll, int lanes_per_row, "
                "int warps, int ksplit, bool out_fp32=False, bool cluster=False, Tensor? prefetch=None, "
                "int prefetch_bytes=0) -> Tensor")
    _lib.define("skinny_out(Tensor(a!) y, Tensor x, Tensor w, Tensor ws, Tensor counters, int rows, int unroll, "
                "int lanes_per_row, int warps, int ksplit, bool cluster=False, Tensor? prefetch=None, "
                "int prefetch_bytes=0) -> ()")
    _lib.define("tc_gemm(Tensor(a!) y, Tensor a, Tensor b, Tensor? a_sf, Tensor? b_sf, Tensor? row_scale, "
                "Tensor? col_scale, Tensor? bias, Tensor? alpha_t, float alpha, int kind, bool swap, bool bias_on_p, "
                "int cfg, int stages, int ksplit, Tensor ws, Tensor counters, bool cluster=False, Tensor? prefetch=None, "
                "int prefetch_bytes=0) -> ()")
    _lib.define("quant(Tensor x, Tensor(a!) q, Tensor(b!)? sf, Tensor? scale_in, Tensor(c!)? scale_out, int mode, "
                "float min_scale) -> ()")
    _lib.define("tc_info(int kind, int cfg) -> int[]")
    _lib.define("set_pdl(bool on) -> ()")
    _lib.define("pdl_enabled() -> bool")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError("lowlat_gemm: " + msg)


def _same_device(ref: torch.Tensor, t: torch.Tensor, name: str) -> None:
    _need(t.is_cuda and t.device == ref.device, f"{name} must be on {ref.device}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _prefetch(args, ref: torch.Tensor, t: torch.Tensor | None, nbytes: int) -> None:
    if t is None:
        return
    _same_device(ref, t, "prefetch")
    _need(t.is_contiguous(), "prefetch tensor must be contiguous and 16-byte aligned")
    total = t.numel() * t.element_size()
    args.prefetch = t.data_ptr()
    args.prefetch_bytes = nbytes if 0 < nbytes < total else total


def _skinny_run(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster, prefetch, prefetch_bytes):
    _need(x.is_cuda, "x must be on CUDA")
    _same_device(x, w, "w")
    _same_device(x, y, "y")
    _need(x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype,
          f"skinny: x and w must both be bfloat16 or both float16, got {x.dtype} and {w.dtype}")
    _need(y.dtype in (x.dtype, torch.float32), f"skinny: output must be {x.dtype} or float32, got {y.dtype}")
    _need(x.dim() == 2 and w.dim() == 2 and y.dim() == 2, "x, w, y must be 2-D")
    m, k = x.shape
    n = w.shape[0]
    _need(w.shape[1] == k, f"x is [{m}, {k}] but w is [{n}, {w.shape[1]}]")
    _need(tuple(y.shape) == (m, n), f"output must be [{m}, {n}]")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and y.stride(1) == 1, "x, w, y need unit stride in the last dimension")
    a = N.SkinnyArgs()
    a.x, a.ldx, a.w, a.ldw, a.y, a.ldy = x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), y.data_ptr(), y.stride(0)
    a.M, a.N, a.K = m, n, k
    a.f16 = int(x.dtype == torch.float16)
    a.out_fp32 = int(y.dtype == torch.float32)
    a.rows, a.unroll, a.lanes_per_row, a.warps, a.ksplit, a.cluster = rows, unroll, lanes_per_row, warps, ksplit, int(cluster)
    if ksplit > 1 and not (cluster and ksplit > 1):
        _same_device(x, ws, "workspace")
        _same_device(x, counters, "counters")
        _need(ws.dtype == torch.float32 and ws.is_contiguous() and counters.dtype == torch.int32 and counters.is_contiguous(),
              "workspace must be contiguous float32, counters contiguous int32")
        a.ws, a.ws_elems, a.counters, a.counters_elems = ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel()
    _prefetch(a, x, prefetch, prefetch_bytes)
    with torch.cuda.device(x.device):
        N.check(N.lib.llg_skinny(C.byref(a), _stream(x)))


def _skinny(x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, out_fp32=False, cluster=False,
            prefetch=None, prefetch_bytes=0):
    y = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32 if out_fp32 else x.dtype, device=x.device)
    _skinny_run(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster, prefetch, prefetch_bytes)
    return y


def _skinny_meta(x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, out_fp32=False, cluster=False,
                 prefetch=None, prefetch_bytes=0):
    return torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32 if out_fp32 else x.dtype, device=x.device)


def _skinny_out(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster=False, prefetch=None,
                prefetch_bytes=0):
    _skinny_run(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster, prefetch, prefetch_bytes)


_A_BITS = {0: 16, 1: 16, 2: 8, 3: 8, 4: 4, 5: 8, 6: 8, 7: 4, 8: 4}
_HAS_SF = {4: (True, True), 7: (True, False), 8: (True, False)}


def _operand(t: torch.Tensor, name: str) -> None:
    _need(t.dim() == 2, f"{name} must be 2-D")
    _need(t.stride(1) == 1, f"{name} needs unit stride in the last dimension")


def _scales(t: torch.Tensor, rows: int, kblocks: int, name: str) -> None:
    _need(t.dim() == 2 and t.element_size() == 1, f"{name} must be a 2-D 1-byte (e4m3) tensor")
    _need(tuple(t.shape) == (rows, kblocks), f"{name} must be [{rows}, {kblocks}], got {list(t.shape)}")
    _need(t.stride(1) == 1, f"{name} needs unit column stride, a row stride that is a multiple of 4 and 4-byte alignment")


def _vec(ref, t, full: int, name: str):
    if t is None:
        return None, 0
    _same_device(ref, t, name)
    _need(t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be a contiguous float32 tensor")
    _need(t.numel() in (1, full), f"{name} must have 1 or {full} elements, got {t.numel()}")
    return t.data_ptr(), (1 if t.numel() == 1 else full)


def fill_tc_args(y, a, b, a_sf, b_sf, row_scale, col_scale, bias, alpha_t, alpha, kind, swap, bias_on_p, cfg, stages,
                 ksplit, ws, counters, cluster=False, prefetch=None, prefetch_bytes=0) -> N.TcArgs:
    """Tensor-level validation of a tc_gemm call and translation into the C-ABI descriptor."""
    _need(kind in _A_BITS, f"unknown kind {kind}")
    _need(a.is_cuda, "operands must be on CUDA")
    _same_device(a, b, "b")
    _same_device(a, y, "y")
    _operand(a, "a")
    _operand(b, "b")
    p, q = a.shape[0], b.shape[0]
    _need(y.dim() == 2 and y.stride(1) == 1, "y must be 2-D with unit last stride")
    want = (q, p) if swap else (p, q)
    _need(tuple(y.shape) == want, f"y must be [{want[0]}, {want[1]}], got {list(y.shape)}")
    _need(y.dtype in _DT, "y must be bfloat16, float16 or float32")
    t = N.TcArgs()
    t.kind, t.cfg, t.stages, t.ksplit, t.cluster, t.swap = kind, cfg, stages, ksplit, int(cluster), int(swap)
    t.a, t.a_rows, t.a_row_bytes, t.lda_bytes = a.data_ptr(), p, a.shape[1] * a.element_size(), a.stride(0) * a.element_size()
    t.b, t.b_rows, t.b_row_bytes, t.ldb_bytes = b.data_ptr(), q, b.shape[1] * b.element_size(), b.stride(0) * b.element_size()
    k = t.a_row_bytes * 8 // _A_BITS[kind]
    need_a, need_b = _HAS_SF.get(kind, (False, False))
    if need_a:
        _need(a_sf is not None, "this kind needs block scales for a")
        _same_device(a, a_sf, "a_sf")
        _scales(a_sf, p, k // 16, "a_sf")
        t.a_sf, t.lda_sf = a_sf.data_ptr(), a_sf.stride(0)
    if need_b:
        _need(b_sf is not None, "this kind needs block scales for b")
        _same_device(a, b_sf, "b_sf")
        _scales(b_sf, q, k // 16, "b_sf")
        t.b_sf, t.ldb_sf = b_sf.data_ptr(), b_sf.stride(0)
    t.row_scale, t.row_scale_len = _vec(a, row_scale, p, "row_scale")
    t.col_scale, t.col_scale_len = _vec(a, col_scale, q, "col_scale")
    if bias is not None:
        _same_device(a, bias, "bias")
        n_bias = p if bias_on_p else q
        _need(bias.dtype in _DT and bias.is_contiguous() and bias.numel() == n_bias,
              f"bias must be a contiguous bf16/f16/f32 vector of {n_bias} elements")
        t.bias, t.bias_dtype = bias.data_ptr(), _DT[bias.dtype]
    t.bias_on_p = int(bias_on_p)
    if alpha_t is not None:
        _same_device(a, alpha_t, "alpha")
        _need(alpha_t.dtype == torch.float32 and alpha_t.numel() == 1, "alpha tensor must be one float32")
        t.alpha_ptr = alpha_t.data_ptr()
    t.alpha = float(alpha)
    t.y, t.ldy, t.out_dtype = y.data_ptr(), y.stride(0), _DT[y.dtype]
    if ksplit > 1 and not cluster:
        _same_device(a, ws, "workspace")
        _same_device(a, counters, "counters")
        _need(ws.element_size() == 4 and ws.is_contiguous() and counters.dtype == torch.int32 and counters.is_contiguous(),
              "workspace must be a contiguous 4-byte tensor, counters contiguous int32")
        t.ws, t.ws_elems, t.counters, t.counters_elems = ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel()
    _prefetch(t, a, prefetch, prefetch_bytes)
    return t


def _tc_gemm(y, a, b, a_sf, b_sf, row_scale, col_scale, bias, alpha_t, alpha, kind, swap, bias_on_p, cfg, stages,
             ksplit, ws, counters, cluster=False, prefetch=None, prefetch_bytes=0):
    t = fill_tc_args(y, a, b, a_sf, b_sf, row_scale, col_scale, bias, alpha_t, alpha, kind, swap, bias_on_p, cfg,
                     stages, ksplit, ws, counters, cluster, prefetch, prefetch_bytes)
    with torch.cuda.device(a.device):
        N.check(N.lib.llg_tc_gemm(C.byref(t), _stream(a)))


def _quant(x, q, sf, scale_in, scale_out, mode, min_scale):
    _need(x.is_cuda and x.dim() == 2 and x.stride(1) == 1, "quant: x must be a 2-D CUDA tensor with unit last stride")
    _same_device(x, q, "q")
    _need(x.dtype in _DT, "quant: x must be bf16, f16 or f32")
    m, k = x.shape
    _need(q.dim() == 2 and q.shape[0] == m and q.stride(1) == 1 and q.element_size() == 1,
          "quant: q must be a 2-D 1-byte tensor with M rows")
    a = N.QuantArgs()
    a.mode, a.in_dtype, a.x, a.ldx, a.q, a.ldq = mode, _DT[x.dtype], x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0)
    a.min_scale, a.M, a.K = float(min_scale), m, k
    if mode in (1, 2):
        _need(q.shape[1] == k, "quant: q must be [M, K]")
        _need(scale_out is not None and scale_out.dtype == torch.float32 and scale_out.is_contiguous()
              and scale_out.numel() == m, "quant: per-token modes need scale_out float32[M]")
        _same_device(x, scale_out, "scale_out")
        a.scale_out = scale_out.data_ptr()
    if mode in (0, 3):
        _need(scale_in is not None and scale_in.dtype == torch.float32 and scale_in.numel() == 1,
              "quant: this mode needs scale_in float32[1]")
        _same_device(x, scale_in, "scale_in")
        a.scale_in = scale_in.data_ptr()
    if mode == 0:
        _need(q.shape[1] == k, "quant: q must be [M, K]")
    if mode == 3:
        _need(k % 16 == 0, "quant: nvfp4 needs K % 16 == 0")
        _need(q.shape[1] == k // 2, "quant: q must be [M, K/2] bytes with 8-byte aligned rows")
        _need(sf is not None and sf.dim() == 2 and tuple(sf.shape) == (m, k // 16) and sf.element_size() == 1
              and sf.stride(1) == 1, "quant: nvfp4 needs sf [M, K/16] bytes")
        _same_device(x, sf, "sf")
        a.sf_out, a.ldsf = sf.data_ptr(), sf.stride(0)
    with torch.cuda.device(x.device):
        N.check(N.lib.llg_quant(C.byref(a), _stream(x)))


def _tc_info(kind, cfg):
    return list(N.tc_info(kind, cfg))


def _set_pdl(on):
    N.lib.llg_set_pdl(int(bool(on)))


def _pdl_enabled():
    return bool(N.lib.llg_pdl_enabled())


if BACKEND == "ctypes":
    _lib.impl("skinny", _skinny, "CUDA")
    _lib.impl("skinny", _skinny_meta, "Meta")
    _lib.impl("skinny_out", _skinny_out, "CUDA")
    _lib.impl("tc_gemm", _tc_gemm, "CUDA")
    _lib.impl("quant", _quant, "CUDA")
    _lib.impl("tc_info", _tc_info, "CompositeExplicitAutograd")
    _lib.impl("set_pdl", _set_pdl, "CompositeExplicitAutograd")
    _lib.impl("pdl_enabled", _pdl_enabled, "CompositeExplicitAutograd")
