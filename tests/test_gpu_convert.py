"""Load-time converters on the GPU: the block-scale relayout kernel against the oracle's index arithmetic (bit-exact,
both directions, ragged sizes, padded row pitch), and checkpoint-style weights through gemm() against the same
weights handed over in the native layout."""
import numpy as np
import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import convert as CV
from oracle import oracle as O

from _cases import FP4, FP8, operands, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows,cols", [(1, 1), (128, 4), (130, 7), (300, 512), (1000, 130), (4096, 256)])
def test_scale_relayout_is_the_oracles_permutation(rows, cols):
    g = torch.Generator().manual_seed(rows * 31 + cols)
    sf = torch.randint(0, 256, (rows, cols), generator=g, dtype=torch.uint8)
    want = O.sf_to_tiled(sf.numpy())
    tiled = CV.scales_to_tiled(sf.to(DEV))
    assert tiled.numel() == CV.tiled_scale_bytes(rows, cols) == want.size
    assert np.array_equal(tiled.cpu().numpy(), want)  # padding bytes included: written as zero
    back = CV.scales_to_rowmajor(tiled, rows, cols)
    assert torch.equal(back.view(torch.uint8).cpu(), sf)
    assert np.array_equal(O.sf_from_tiled(want, rows, cols), sf.numpy())
    # a source whose rows are padded (and not 4-byte aligned) goes through the byte path
    wide = torch.zeros(rows, cols + 3, dtype=torch.uint8, device=DEV)
    wide[:, :cols] = sf.to(DEV)
    assert torch.equal(CV.scales_to_tiled(wide[:, :cols]), tiled)


def test_relayout_refuses_bad_arguments():
    with pytest.raises(ValueError, match="hold"):
        CV.scales_to_rowmajor(torch.zeros(512, dtype=torch.uint8, device=DEV), 129, 4)
    with pytest.raises(ValueError, match="unit column stride"):
        CV.scales_to_tiled(torch.zeros(8, 8, dtype=torch.uint8, device=DEV).t())


def test_checkpoint_weights_through_gemm():
    m, n, k = 5, 300, 1024
    # NVFP4 weight whose block scales arrive tiled and whose global scale arrives as a reciprocal
    x, w, kw, xd, wd = operands("w4a16_bf16", m, n, k, seed=4)
    native = L.gemm(x, w, out_dtype=torch.float32, **kw)
    ck = CV.nvfp4_weight(w.view(torch.uint8), CV.scales_to_tiled(kw["w_block_scale"]), 1.0 / kw["w_scale"].double(),
                         tiled_scales=True, reciprocal=True)
    y = L.gemm(x, ck["w"], out_dtype=torch.float32, w_block_scale=ck["w_block_scale"], w_scale=ck["w_scale"])
    assert torch.equal(ck["w_block_scale"].view(torch.uint8), kw["w_block_scale"].view(torch.uint8))
    assert rel_err(y, xd @ wd.T) < 2e-5 and rel_err(y, native.double().cpu().numpy()) < 1e-6
    # FP8 weight with an [N, 1] scale
    x, w, kw, xd, wd = operands("w8a16_bf16", m, n, k, seed=5)
    ck = CV.fp8_weight(w.view(torch.uint8), kw["w_scale"].reshape(n, 1))
    y = L.gemm(x, ck["w"], out_dtype=torch.float32, w_scale=ck["w_scale"])
    assert torch.equal(y, L.gemm(x, w, out_dtype=torch.float32, **kw))


def test_weight_quantizers_round_trip():
    g = torch.Generator().manual_seed(9)
    w16 = (torch.randn(257, 512, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    x = torch.randn(3, 512, generator=g).to(torch.bfloat16).to(DEV)
    ref = x.double() @ w16.double().T
    q8 = CV.quantize_weight_fp8(w16)
    y8 = L.gemm(x, q8["w"], w_scale=q8["w_scale"], out_dtype=torch.float32)
    assert float((y8.double() - ref).abs().max() / ref.abs().max()) < 0.05  # e4m3: 3 mantissa bits per weight
    q4 = CV.quantize_weight_nvfp4(w16)
    assert q4["w_block_scale"].view(torch.uint8).max() <= 0x7E and float(q4["w_block_scale"].float().max()) > 224.0
    y4 = L.gemm(x, q4["w"], w_block_scale=q4["w_block_scale"], w_scale=q4["w_scale"], out_dtype=torch.float32)
    assert float((y4.double() - ref).abs().max() / ref.abs().max()) < 0.25  # e2m1: 1 mantissa bit per weight
    # bit-exact against the oracle's quantizer on the same rows
    gs = 6.0 * 448.0 / w16.float().abs().max().clamp_min(1e-12)  # the factor the converter computes, same fp32 operations
    assert torch.equal(torch.reciprocal(gs.reshape(1)), q4["w_scale"])
    oq, osf = O.quantize_nvfp4(w16.float().cpu().numpy(), float(gs.item()))
    assert np.array_equal(q4["w"].view(torch.uint8).cpu().numpy(), oq) and np.array_equal(q4["w_block_scale"].view(torch.uint8).cpu().numpy(), osf)
