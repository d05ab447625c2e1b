"""Load-time converters: checkpoint tensors -> the operand layouts gemm() takes.

gemm() wants what the reference's gemm() wants (lowlat_gemm/__init__.py:10-16): e4m3 weights [N, K] with one float32
scale per output channel (or one for the tensor); packed e2m1 weights [N, K/2] (even element in the low nibble) with
row-major e4m3 block scales [N, K/16] and one global float32 scale. Checkpoints differ in three ways this module
covers, each once at load time and never on the hot path:

* block scales stored in the 128 x 4 tiled form that block-scaled tensor-core GEMM libraries read: `scales_to_rowmajor`
  (and `scales_to_tiled` for the way back), one HBM-bound kernel of the core library (`llg_sf_relayout`);
* scale tensors of other shapes or reciprocal meaning: `fp8_weight`, `nvfp4_weight` normalise them;
* 16-bit weights that should be served quantized: `quantize_weight_fp8` / `quantize_weight_nvfp4` run the library's own
  quantizers over the weight rows (per-channel FP8; NVFP4 with the global scale amax / (6 * 448)) - weights then carry
  exactly the rounding the activation quantizers are pinned to.

The reference has no such helpers: its callers are expected to hold weights in these layouts already.
"""

from __future__ import annotations

import torch

from . import _native as N
from .api import quantize_fp8, quantize_nvfp4

FP8 = torch.float8_e4m3fn
FP4 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def tiled_scale_bytes(rows: int, cols: int) -> int:
    return -(-rows // 128) * -(-cols // 4) * 512


def scales_to_rowmajor(tiled: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Tiled block scales (any shape, `tiled_scale_bytes(rows, cols)` one-byte elements) -> [rows, cols] e4m3, row-major."""
    flat = tiled.contiguous().view(torch.uint8).reshape(-1)
    if flat.numel() != tiled_scale_bytes(rows, cols):
        raise ValueError(f"lowlat_gemm: tiled scales of a [{rows}, {cols}] matrix hold {tiled_scale_bytes(rows, cols)} bytes, "
                         f"got {flat.numel()}")
    if not flat.is_cuda:
        raise ValueError("lowlat_gemm: scales must be CUDA tensors")
    out = torch.empty(rows, cols, dtype=torch.uint8, device=flat.device)
    with torch.cuda.device(flat.device):
        N.check(N.lib.llg_sf_relayout(flat.data_ptr(), out.data_ptr(), rows, cols, cols, 0, _stream(flat)))
    return out.view(FP8)


def scales_to_tiled(sf: torch.Tensor) -> torch.Tensor:
    """[rows, cols] block scales (unit column stride) -> the tiled form, a flat uint8 tensor (padding zero)."""
    if sf.dim() != 2 or sf.element_size() != 1 or sf.stride(1) != 1 or not sf.is_cuda:
        raise ValueError("lowlat_gemm: scales must be a 2-D one-byte CUDA tensor with unit column stride")
    rows, cols = sf.shape
    out = torch.empty(tiled_scale_bytes(rows, cols), dtype=torch.uint8, device=sf.device)
    with torch.cuda.device(sf.device):
        N.check(N.lib.llg_sf_relayout(sf.data_ptr(), out.data_ptr(), rows, cols, sf.stride(0), 1, _stream(sf)))
    return out


def fp8_weight(weight: torch.Tensor, scale: torch.Tensor | float, reciprocal: bool = False) -> dict:
    """An e4m3 checkpoint weight [N, K] (float8 or raw bytes) with a per-tensor or per-channel scale of shape (), [1],
    [N] or [N, 1] -> gemm() keyword arguments {w, w_scale}. reciprocal=True: the checkpoint stores 1 / scale."""
    w = weight.view(FP8) if weight.dtype == torch.uint8 else weight
    if w.dtype != FP8 or w.dim() != 2:
        raise ValueError("lowlat_gemm: an FP8 weight is a 2-D float8_e4m3fn (or uint8) tensor")
    s = torch.as_tensor(scale, dtype=torch.float32, device=w.device).reshape(-1)
    if s.numel() not in (1, w.shape[0]):
        raise ValueError(f"lowlat_gemm: weight scale must have 1 or {w.shape[0]} elements, got {s.numel()}")
    if reciprocal:
        s = torch.reciprocal(s)
    return {"w": w.contiguous(), "w_scale": s.contiguous()}


def nvfp4_weight(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor | float,
                 tiled_scales: bool = False, reciprocal: bool = False) -> dict:
    """A packed e2m1 checkpoint weight [N, K/2] with e4m3 block scales (row-major [N, K/16], or the tiled form when
    tiled_scales) and the tensor-wide second-level scale -> gemm() keyword arguments {w, w_block_scale, w_scale}."""
    if packed.dim() != 2 or packed.element_size() != 1:
        raise ValueError("lowlat_gemm: a packed FP4 weight is a 2-D one-byte tensor [N, K/2]")
    n, k = packed.shape[0], packed.shape[1] * 2
    if k % 16:
        raise ValueError(f"lowlat_gemm: K must be a multiple of 16, got {k}")
    sf = scales_to_rowmajor(block_scale, n, k // 16) if tiled_scales else block_scale.view(FP8)
    if tuple(sf.shape) != (n, k // 16):
        raise ValueError(f"lowlat_gemm: block scales must be [{n}, {k // 16}], got {tuple(sf.shape)}")
    g = torch.as_tensor(global_scale, dtype=torch.float32, device=packed.device).reshape(-1)
    if g.numel() != 1:
        raise ValueError("lowlat_gemm: the global scale of an NVFP4 weight has one element")
    if reciprocal:
        g = torch.reciprocal(g)
    return {"w": packed.contiguous().view(FP4), "w_block_scale": sf.contiguous(), "w_scale": g}


def quantize_weight_fp8(weight: torch.Tensor) -> dict:
    """bf16 / f16 / f32 weight [N, K] -> per-channel FP8: {w, w_scale [N]} (the quantizer of quantize_fp8 over rows)."""
    q, s = quantize_fp8(weight)
    return {"w": q, "w_scale": s}


def quantize_weight_nvfp4(weight: torch.Tensor) -> dict:
    """bf16 / f16 / f32 weight [N, K] -> NVFP4 {w, w_block_scale, w_scale}. The quantizer multiplies by a tensor-wide
    factor g before it forms the block scales (sf = e4m3(block amax / 6 * g)); g = 6 * 448 / amax puts the largest
    block scale at the top of the e4m3 range, and the weight's global scale is its reciprocal."""
    amax = weight.float().abs().max().clamp_min(1e-12)
    g = (6.0 * 448.0 / amax).reshape(1)
    q, sf = quantize_nvfp4(weight, g)
    return {"w": q, "w_block_scale": sf, "w_scale": torch.reciprocal(g)}
