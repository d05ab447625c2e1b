"""Low-latency GEMM for NVIDIA B200 (sm_100a): drop-in for the Python surface of Cerynitius/sm120-lowlat-gemm.

    y = lowlat_gemm.gemm(x, w, ...)      # y[..., N] = alpha * (x * x_scale) @ (w[N, K] * w_scale)^T + bias

    x bf16/f16, w same            W16A16
    x bf16/f16, w float8_e4m3fn   W8A16   (w_scale: per tensor or per channel)
    x bf16/f16, w fp4             W4A16   (w_block_scale [N, K/16] e4m3; w_scale: global)
    x float8_e4m3fn, w same       W8A8 FP8
    x int8, w int8                W8A8 INT8 (int32 accumulation)
    x fp4, w fp4                  W4A4 NVFP4 (block scales on both sides)

Two engines behind one call: a CUDA-core streaming GEMV for W16A16 with at most 16 rows (bit-identical for every M)
and a TMA-fed tcgen05 tensor-core kernel with tensor-memory accumulators for every precision and any M. A plan per
(precision, N, K) picks engine and tiling per M. All compute runs in libllg_core.so (hand-written CUDA, C ABI in
include/llg_core.h); nothing falls back to the CPU or to a vendor GEMM.
"""

from .api import (_FP4_KINDS, _workspace, _ws, gemm, kind_of, pdl_enabled, quantize_fp8, quantize_int8,  # noqa: F401
                  quantize_nvfp4, reserve_workspace, set_pdl, silu_mul, silu_mul_quantize_fp8, silu_mul_quantize_nvfp4, supports,
                  workspace_need)
from .plans import (KINDS, MAX_STAGES, NUM_CFGS, PAIR_CFGS, SKINNY_MAX_TOKENS, _MIXED, Plan, SkinnyOrder, SkinnyTile,  # noqa: F401
                    TcChoice, _file_key, _nearest, _packaged_path, _tc_lookup, cfg_atoms, default_plan,
                    default_skinny_order, default_tc_choice, get_plan, load_plans, max_stages, prefer_lowlat,
                    save_plans, set_plan, skinny_ranges, smem_budget, tc_info)

__all__ = [
    "KINDS", "Plan", "SkinnyOrder", "SkinnyTile", "TcChoice", "default_plan", "gemm", "get_plan", "kind_of",
    "prefer_lowlat", "load_plans", "quantize_fp8", "quantize_int8", "quantize_nvfp4", "reserve_workspace",
    "save_plans", "set_pdl", "set_plan", "supports", "workspace_need",
]
