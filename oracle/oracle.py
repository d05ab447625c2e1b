"""CPU oracle for the low-latency GEMM path: a numpy restatement of the reference's arithmetic.

TEST INFRASTRUCTURE ONLY. Nothing in the product imports this module; only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs may use it, and only as the checker or as the timed CPU baseline.

Pinning: the format decoders and the dequantised GEMM are checked against golden vectors produced by the reference's
own CPU emulator of its tensor-core kernel (tests/emulate_tc.py) and the quantizers against the reference's test
expressions (tests/test_gemm.py:200-218); see tests/golden/make_golden.py. The NVFP4 activation quantizer has no
bit-level pin in the reference's CPU tests (its test only bounds the round-trip error, tests/test_gemm.py:221-228); it
and the skinny summation order are pinned on the GPU instead, byte for byte against the reference's own kernels
(csrc/quant.cu, csrc/gemv_lpr*.cu) compiled for sm_100a by oracle/Makefile (tests/test_gpu_ref_pin.py).

Each function cites the reference lines it follows (paths relative to the reference repository).
"""

from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------------------------------------------
# number formats

# e2m1 code -> value (tests/test_gemm.py:15, tests/emulate_tc.py:37)
E2M1_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float64)


def _e4m3_value(b: int) -> float:
    """float8_e4m3fn: bias 7, subnormals m/8 * 2^-6, 0x7f / 0xff are NaN (tests/emulate_tc.py:40-48)."""
    if (b & 0x7F) == 0x7F:
        return float("nan")
    sign = -1.0 if b & 0x80 else 1.0
    e, m = (b >> 3) & 0xF, b & 7
    return sign * (m / 8.0) * 2.0**-6 if e == 0 else sign * (1 + m / 8.0) * 2.0 ** (e - 7)


E4M3_VALUES = np.array([_e4m3_value(b) for b in range(256)], dtype=np.float64)
_E4M3_POS = E4M3_VALUES[:0x7F].astype(np.float64)  # codes 0x00..0x7e, increasing, finite
_E2M1_POS = E2M1_VALUES[:8]


def _round_to_table(mag: np.ndarray, table: np.ndarray) -> np.ndarray:
    """Index of the table entry nearest to mag (>= 0), ties to the even index, saturating at the last entry.
    The tables are the non-negative values of a small float format in code order, so "even index" is "even
    mantissa": round-to-nearest-even as cvt.rn.satfinite does (csrc/ptx.cuh:199-213)."""
    mag = np.asarray(mag, dtype=np.float64)
    hi = np.searchsorted(table, mag, side="left")  # first entry >= mag
    hi = np.clip(hi, 0, len(table) - 1)
    lo = np.clip(hi - 1, 0, len(table) - 1)
    d_lo, d_hi = mag - table[lo], table[hi] - mag
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    idx = np.where(pick_hi, hi, lo)
    return np.where(mag >= table[-1], len(table) - 1, idx)


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e4m3x2.f32 per element (csrc/ptx.cuh:199-203): RNE, +-448 saturation, sign of zero kept,
    NaN -> 0x7f."""
    x = np.asarray(x, dtype=np.float32)
    code = _round_to_table(np.abs(x.astype(np.float64)), _E4M3_POS).astype(np.uint8)
    code = np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)
    return np.where(np.isnan(x), np.uint8(0x7F), code).astype(np.uint8)


def f32_to_e2m1(x: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e2m1x2.f32 per element (csrc/ptx.cuh:205-213): 4-bit code, RNE, +-6 saturation."""
    x = np.asarray(x, dtype=np.float32)
    code = _round_to_table(np.abs(x.astype(np.float64)), _E2M1_POS).astype(np.uint8)
    return np.where(np.signbit(x), code | 0x8, code).astype(np.uint8)


def unpack_fp4(q: np.ndarray) -> np.ndarray:
    """[rows, K/2] packed bytes -> [rows, K] float64, element 2i in the low nibble (tests/test_gemm.py:22-26)."""
    q = np.asarray(q).view(np.uint8)
    out = np.empty(q.shape[:-1] + (q.shape[-1] * 2,), dtype=np.float64)
    out[..., 0::2] = E2M1_VALUES[q & 0xF]
    out[..., 1::2] = E2M1_VALUES[q >> 4]
    return out


def expand_block_scales(sf: np.ndarray) -> np.ndarray:
    """[rows, K/16] e4m3 bytes -> [rows, K] float64 (tests/test_gemm.py:29-30)."""
    return np.repeat(E4M3_VALUES[np.asarray(sf).view(np.uint8)], 16, axis=-1)


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (np.asarray(u16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (what __float2bfloat16_rn does for finite values)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


# ---------------------------------------------------------------------------------------------------------------
# quantizers (csrc/quant.cu)


def quantize_fp8(x: np.ndarray, scale: float | None = None, min_scale: float = 1e-12):
    """csrc/quant.cu:43-65. x [M,K] (any float dtype, widened exactly to fp32). Per token when scale is None:
    s = max(amax/448, min_scale) with IEEE fp32 division, q = e4m3(x * (1/s)). Returns (q uint8 [M,K], s fp32)."""
    xf = np.asarray(x, dtype=np.float32)
    if scale is None:
        s = np.maximum(np.abs(xf).max(axis=1) / np.float32(448.0), np.float32(min_scale)).astype(np.float32)
    else:
        s = np.full((1,), scale, dtype=np.float32)
    inv = (np.float32(1.0) / s).astype(np.float32)
    q = f32_to_e4m3(xf * (inv[:, None] if scale is None else inv[0]))
    return q, s


def quantize_int8(x: np.ndarray, min_scale: float = 1e-12):
    """csrc/quant.cu:67-82: s = max(amax/127, min_scale), q = clamp(rint(x * (1/s)), -127, 127)."""
    xf = np.asarray(x, dtype=np.float32)
    s = np.maximum(np.abs(xf).max(axis=1) / np.float32(127.0), np.float32(min_scale)).astype(np.float32)
    inv = (np.float32(1.0) / s).astype(np.float32)
    q = np.clip(np.rint(xf * inv[:, None]), -127, 127).astype(np.int8)
    return q, s


def quantize_nvfp4(x: np.ndarray, g: float):
    """csrc/quant.cu:85-114: per 16 elements sf = e4m3(amax / 6 * g); inv = g / decode(sf) (0 when sf decodes to 0);
    nibble = e2m1(x * inv), even element in the low nibble. Returns (q uint8 [M,K/2], sf uint8 [M,K/16])."""
    xf = np.asarray(x, dtype=np.float32)
    m, k = xf.shape
    g = np.float32(g)
    blk = xf.reshape(m, k // 16, 16)
    amax = np.abs(blk).max(axis=2).astype(np.float32)
    sf = f32_to_e4m3(((amax / np.float32(6.0)).astype(np.float32) * g).astype(np.float32))
    sfv = E4M3_VALUES[sf].astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(sfv > 0, (g / sfv).astype(np.float32), np.float32(0)).astype(np.float32)
    codes = f32_to_e2m1((blk * inv[:, :, None]).astype(np.float32)).reshape(m, k)
    q = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return q, sf


# ---------------------------------------------------------------------------------------------------------------
# GEMM semantics: y = alpha * (x * x_scale) @ (w * w_scale)^T + bias  (lowlat_gemm/__init__.py:15-17, 506)


def dequant(kind_side: str, t: np.ndarray, block_scale: np.ndarray | None = None) -> np.ndarray:
    """Operand bytes -> float64 values. kind_side in {bf16, f16, fp8, int8, fp4}."""
    if kind_side == "bf16":
        return bf16_bits_to_f32(np.asarray(t).view(np.uint16)).astype(np.float64)
    if kind_side == "f16":
        return np.asarray(t).view(np.float16).astype(np.float64)
    if kind_side == "fp8":
        return E4M3_VALUES[np.asarray(t).view(np.uint8)]
    if kind_side == "int8":
        return np.asarray(t).view(np.int8).astype(np.float64)
    if kind_side == "fp4":
        v = unpack_fp4(t)
        return v * expand_block_scales(block_scale) if block_scale is not None else v
    raise ValueError(kind_side)


def gemm_f64(x_deq: np.ndarray, w_deq: np.ndarray, alpha: float = 1.0, bias: np.ndarray | None = None) -> np.ndarray:
    """float64 reference used for the reference's own 2e-5 tolerance (tests/test_gemm.py:86-102)."""
    y = alpha * (x_deq @ w_deq.T)
    return y if bias is None else y + np.asarray(bias, dtype=np.float64)


def gemm_f32(x_deq: np.ndarray, w_deq: np.ndarray, alpha: float = 1.0, bias: np.ndarray | None = None) -> np.ndarray:
    """fp32 host matmul of the dequantised operands: the baseline the 1e-2 x RMS tolerance is stated against."""
    y = np.float32(alpha) * (x_deq.astype(np.float32) @ w_deq.astype(np.float32).T)
    return y if bias is None else y + np.asarray(bias, dtype=np.float32)


def epilogue_f32(acc: np.ndarray, alpha: float, row_scale, col_scale, bias, bias_on_rows: bool) -> np.ndarray:
    """Epilogue on an accumulator acc[p,q] in the reference's operand order, every operation rounded to fp32:
    v = ((acc * alpha) * row_scale[p]) * col_scale[q]; v += bias (csrc/tc_gemm.cuh:159-161). int32 accumulators are
    converted with one rounding first (:422)."""
    v = np.asarray(acc).astype(np.float32)
    v = (v * np.float32(alpha)).astype(np.float32)
    rs = np.float32(1) if row_scale is None else np.asarray(row_scale, dtype=np.float32).reshape(-1, 1)
    cs = np.float32(1) if col_scale is None else np.asarray(col_scale, dtype=np.float32).reshape(1, -1)
    v = (v * rs).astype(np.float32)
    v = (v * cs).astype(np.float32)
    if bias is not None:
        b = np.asarray(bias, dtype=np.float32)
        v = (v + (b.reshape(-1, 1) if bias_on_rows else b.reshape(1, -1))).astype(np.float32)
    return v


def gemm_int8_exact(x: np.ndarray, w: np.ndarray, x_scale, w_scale, alpha: float = 1.0, bias=None) -> np.ndarray:
    """INT8 W8A8 as the swapped tensor-core path computes it: exact int32 accumulation, then the fp32 epilogue with
    the weight scale as row scale and the activation scale as column scale, bias per weight row
    (lowlat_gemm/__init__.py:565-566; csrc/tc_gemm.cuh:159-161). Returns fp32 y[M,N]."""
    acc = np.asarray(w).view(np.int8).astype(np.int64) @ np.asarray(x).view(np.int8).astype(np.int64).T  # [N, M]
    assert np.abs(acc).max() < 2**31
    return epilogue_f32(acc.astype(np.int32), alpha, w_scale, x_scale, bias, bias_on_rows=True).T


# ---------------------------------------------------------------------------------------------------------------
# skinny GEMV: bit-exact emulation of the summation order (csrc/gemv.cuh:6-12, 85-88, 108-154, 214-231)


def skinny_gemv_exact(x: np.ndarray, w: np.ndarray, lanes_per_row: int, ksplit: int = 1) -> np.ndarray:
    """x [M,K], w [N,K] as float32 arrays holding bf16/f16-representable values. Returns fp32 y[M,N] with exactly the
    bits the GPU kernel produces: lane sl of a row's lane group adds vectors vbeg+sl, vbeg+sl+LPR, ... elementwise in
    order (each product of two 16-bit floats is exact in fp32, so fma == multiply then add), lanes are combined by an
    xor butterfly (offsets LPR/2 ... 1), split partials are added in split order."""
    x = np.asarray(x, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    m, k = x.shape
    n = w.shape[0]
    kv = k // 8
    lpr = lanes_per_row
    total = None
    for s in range(ksplit):
        vbeg, vend = kv * s // ksplit, kv * (s + 1) // ksplit
        acc = np.zeros((lpr, m, n), dtype=np.float32)
        steps = -(-(vend - vbeg) // lpr) if vend > vbeg else 0
        for j in range(steps):
            v = vbeg + np.arange(lpr) + lpr * j          # vector index per lane
            live = v < vend
            vv = np.where(live, v, vbeg)
            for e in range(8):
                col = vv * 8 + e
                prod = w[:, col].T[:, None, :] * x[:, col].T[:, :, None]   # [lpr, m, n], exact in fp32
                acc = np.where(live[:, None, None], (acc + prod).astype(np.float32), acc)
        off = lpr // 2
        while off >= 1:
            acc = (acc + acc[np.arange(lpr) ^ off]).astype(np.float32)
            off //= 2
        part = acc[0]
        total = part if total is None else (total + part).astype(np.float32)
    return total


def splitk_sum_order(parts: np.ndarray) -> np.ndarray:
    """Sum of split-K partials [ksplit, ...] in split order starting from partial 0 (csrc/tc_gemm.cuh:484-498)."""
    total = parts[0]
    for kk in range(1, parts.shape[0]):
        total = (total + parts[kk]).astype(parts.dtype)
    return total


# ---------------------------------------------------------------------------------------------------------------
# block-scale layouts. The reference takes block scales row-major, [rows, K/16] (lowlat_gemm/__init__.py:10-16);
# checkpoints prepared for block-scaled tensor-core GEMMs hold them in tiles of 128 rows x 4 columns (the published
# layout of the vendor GEMM libraries' scale-factor operand): 512 contiguous bytes per tile, byte (r, c) of a tile at
# (r % 32) * 16 + (r // 32) * 4 + c, tiles row-tile major, rows and columns padded to whole tiles with zeros.


def sf_to_tiled(sf: np.ndarray) -> np.ndarray:
    rows, cols = sf.shape
    rt, ct = -(-rows // 128), -(-cols // 4)
    out = np.zeros(rt * ct * 512, dtype=np.uint8)
    for r in range(rows):
        for c in range(cols):
            out[((r // 128) * ct + c // 4) * 512 + ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + c % 4] = sf[r, c]
    return out


def sf_from_tiled(tiled: np.ndarray, rows: int, cols: int) -> np.ndarray:
    ct = -(-cols // 4)
    out = np.zeros((rows, cols), dtype=np.uint8)
    for r in range(rows):
        for c in range(cols):
            out[r, c] = tiled[((r // 128) * ct + c // 4) * 512 + ((r % 128) % 32) * 16 + ((r % 128) // 32) * 4 + c % 4]
    return out


# ---------------------------------------------------------------------------------------------------------------
# algorithmic bytes of one GEMM (every operand touched once; split-K workspace traffic not counted)


def gemm_bytes(kind: str, m: int, n: int, k: int, out_bytes: int = 2, x_scale_len: int = 0, w_scale_len: int = 0,
               bias_bytes: int = 0) -> int:
    wbits = {"bf16": 16, "f16": 16, "fp8": 8, "int8": 8, "nvfp4": 4}.get(kind, 8 if kind.startswith("w8") else 4)
    xbits = {"fp8": 8, "int8": 8, "nvfp4": 4}.get(kind, 16)
    sf_w = n * (k // 16) if (kind == "nvfp4" or kind.startswith("w4a16")) else 0
    sf_x = m * (k // 16) if kind == "nvfp4" else 0
    return n * k * wbits // 8 + sf_w + m * k * xbits // 8 + sf_x + m * n * out_bytes + 4 * x_scale_len + 4 * w_scale_len + bias_bytes
