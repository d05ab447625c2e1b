"""ctypes binding of libllg_core.so (C ABI declared in include/llg_core.h).

The shared library is the only compute backend: if it is missing or does not match the header, importing this module
raises. There is no CPU fallback anywhere in the package.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_NAME = "libllg_core.so"

c_i32, c_i64, c_f32, c_ptr = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class SkinnyArgs(C.Structure):
    _fields_ = [
        ("x", c_ptr), ("ldx", c_i64), ("w", c_ptr), ("ldw", c_i64), ("y", c_ptr), ("ldy", c_i64),
        ("M", c_i32), ("N", c_i32), ("K", c_i32), ("f16", c_i32), ("out_fp32", c_i32),
        ("rows", c_i32), ("unroll", c_i32), ("lanes_per_row", c_i32), ("warps", c_i32), ("ksplit", c_i32),
        ("cluster", c_i32),
        ("ws", c_ptr), ("ws_elems", c_i64), ("counters", c_ptr), ("counters_elems", c_i64),
        ("prefetch", c_ptr), ("prefetch_bytes", c_i64),
    ]


class TcArgs(C.Structure):
    _fields_ = [
        ("kind", c_i32), ("cfg", c_i32), ("stages", c_i32), ("ksplit", c_i32), ("cluster", c_i32), ("swap", c_i32),
        ("a", c_ptr), ("a_rows", c_i64), ("a_row_bytes", c_i64), ("lda_bytes", c_i64),
        ("b", c_ptr), ("b_rows", c_i64), ("b_row_bytes", c_i64), ("ldb_bytes", c_i64),
        ("a_sf", c_ptr), ("lda_sf", c_i64), ("b_sf", c_ptr), ("ldb_sf", c_i64),
        ("row_scale", c_ptr), ("row_scale_len", c_i32), ("col_scale", c_ptr), ("col_scale_len", c_i32),
        ("bias", c_ptr), ("bias_dtype", c_i32), ("bias_on_p", c_i32),
        ("alpha_ptr", c_ptr), ("alpha", c_f32),
        ("y", c_ptr), ("ldy", c_i64), ("out_dtype", c_i32),
        ("ws", c_ptr), ("ws_elems", c_i64), ("counters", c_ptr), ("counters_elems", c_i64),
        ("prefetch", c_ptr), ("prefetch_bytes", c_i64),
    ]


class QuantArgs(C.Structure):
    _fields_ = [
        ("mode", c_i32), ("in_dtype", c_i32), ("x", c_ptr), ("ldx", c_i64), ("q", c_ptr), ("ldq", c_i64),
        ("sf_out", c_ptr), ("ldsf", c_i64), ("scale_in", c_ptr), ("scale_out", c_ptr), ("min_scale", c_f32),
        ("M", c_i32), ("K", c_i32),
    ]


class GatedQuantArgs(C.Structure):
    _fields_ = [("q", QuantArgs), ("up", c_ptr), ("ldup", c_i64), ("act", c_ptr), ("ldact", c_i64)]


class PushArgs(C.Structure):
    _fields_ = [("world", c_i32), ("rank", c_i32), ("rows", c_i32), ("reserved", c_i32), ("dst", c_ptr * 8),
                ("flags", c_ptr * 8), ("done", c_ptr)]


# every symbol include/llg_core.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "llg_skinny": (c_i32, [C.POINTER(SkinnyArgs), c_ptr]),
    "llg_skinny_ranges": (c_i32, [c_i32, c_i32]),
    "llg_tc_gemm": (c_i32, [C.POINTER(TcArgs), c_ptr]),
    "llg_tc_info": (c_i32, [c_i32, c_i32, C.POINTER(c_i32 * 4)]),
    "llg_smem_budget": (c_i32, []),
    "llg_quant": (c_i32, [C.POINTER(QuantArgs), c_ptr]),
    "llg_gated_quant": (c_i32, [C.POINTER(GatedQuantArgs), c_ptr]),
    "llg_set_pdl": (None, [c_i32]),
    "llg_pdl_enabled": (c_i32, []),
    "llg_allreduce_oneshot": (c_i32, [c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_i32, c_i32, c_i32, c_ptr]),
    "llg_allreduce_quant_fp8": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_i32, c_i32, c_i32, C.c_float, c_i32,
                                        c_i32, c_ptr]),
    "llg_tc_gemm_static_ws": (c_i32, [C.POINTER(TcArgs), c_ptr]),
    "llg_tc_gemm_push": (c_i32, [C.POINTER(TcArgs), C.POINTER(PushArgs), c_ptr]),
    "llg_reduce_local": (c_i32, [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_i32, c_i32, c_i32, C.c_float, c_i32,
                                 c_ptr]),
    "llg_set_wait_limit": (None, [c_i64]),
    "llg_sf_relayout": (c_i32, [c_ptr, c_ptr, c_i32, c_i32, c_i64, c_i32, c_ptr]),
    "llg_tc_gemm_host": (c_i32, [C.POINTER(TcArgs), c_ptr, c_ptr, c_i64, c_ptr, c_i64, c_ptr]),
    "llg_device_status": (c_i32, [C.POINTER(C.c_uint32)]),
    "llg_struct_sizes": (None, [C.POINTER(c_i32 * 5)]),
    "llg_last_error": (C.c_char_p, []),
    "llg_abi_version": (c_i32, []),
}
ABI_VERSION = 2
AR_MAX_CTAS = 64      # LLG_AR_MAX_CTAS: flag sets (CTAs, or rows of the fused all-reduce + quantizer) per all-reduce


def library_path() -> Path:
    env = os.environ.get("LLG_CORE_LIB")
    return Path(env) if env else Path(__file__).with_name(_LIB_NAME)


def _load() -> C.CDLL:
    path = library_path()
    if not path.is_file():
        raise ImportError(
            f"lowlat_gemm: {path} not found. Build it with `make -C {Path(__file__).resolve().parent.parent / 'csrc'} -j` "
            "(needs nvcc with sm_100a support); there is no fallback implementation.")
    lib = C.CDLL(str(path))
    for name, (res, args) in SYMBOLS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"lowlat_gemm: {path} does not export {name}") from e
        fn.restype, fn.argtypes = res, args
    if lib.llg_abi_version() != ABI_VERSION:
        raise ImportError(f"lowlat_gemm: {path} has ABI {lib.llg_abi_version()}, this package needs {ABI_VERSION}")
    sizes = (c_i32 * 5)()
    lib.llg_struct_sizes(C.byref(sizes))
    want = (C.sizeof(SkinnyArgs), C.sizeof(TcArgs), C.sizeof(QuantArgs), C.sizeof(GatedQuantArgs), C.sizeof(PushArgs))
    if tuple(sizes) != want:
        raise ImportError(f"lowlat_gemm: struct layout mismatch, library {tuple(sizes)} vs binding {want}")
    return lib


lib = _load()


def check(rc: int) -> None:
    """Raise the library's error as RuntimeError("lowlat_gemm: ...") like the reference's TORCH_CHECK does."""
    if rc != 0:
        raise RuntimeError(lib.llg_last_error().decode())


def tc_info(kind: int, cfg: int) -> tuple[int, int, int, int]:
    out = (c_i32 * 4)()
    check(lib.llg_tc_info(kind, cfg, C.byref(out)))
    return tuple(out)


def device_status() -> int:
    v = C.c_uint32(0)
    check(lib.llg_device_status(C.byref(v)))
    return int(v.value)
