"""The CPU oracle against the golden fixtures made from the reference (tests/golden/make_golden.py) and against
torch's own float8 / float4 casts. No GPU."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O

G = Path(__file__).parent / "golden"
KINDS = ["bf16", "f16", "fp8", "int8", "nvfp4", "w8a16_bf16", "w8a16_f16", "w4a16_bf16", "w4a16_f16"]
SIDE = {"bf16": ("bf16", "bf16"), "f16": ("f16", "f16"), "fp8": ("fp8", "fp8"), "int8": ("int8", "int8"),
        "nvfp4": ("fp4", "fp4"), "w8a16_bf16": ("fp8", "bf16"), "w8a16_f16": ("fp8", "f16"),
        "w4a16_bf16": ("fp4", "bf16"), "w4a16_f16": ("fp4", "f16")}


def test_decode_tables_match_reference_emulator():
    f = np.load(G / "formats.npz")
    finite = ~np.isnan(O.E4M3_VALUES)
    assert np.array_equal(O.E4M3_VALUES[finite], f["e4m3"][finite])
    assert np.array_equal(O.E2M1_VALUES, f["e2m1"]) and np.array_equal(np.signbit(O.E2M1_VALUES), np.signbit(f["e2m1"]))


@pytest.mark.parametrize("kind", KINDS)
def test_dequantised_gemm_matches_reference_emulator(kind):
    """y = alpha * rs[p] * cs[q] * sum_k A[p,k] B[q,k] on the emulator's operands, within float64 round-off."""
    f = np.load(G / f"tc_{kind}.npz")
    sa, sb = SIDE[kind]
    k = int(f["k"])
    a = O.dequant(sa, f["a"], f["asf"] if f["asf"].size else None)[:, :k]
    b = O.dequant(sb, f["b"], f["bsf"] if f["bsf"].size else None)[:, :k]
    y = (a @ b.T) * float(f["alpha"]) * f["rs"][:, None] * f["cs"][None, :]
    ref = f["y"].T  # stored swapped: y[q, p]
    assert np.abs(y - ref).max() <= 1e-12 * np.abs(ref).max()


def test_fp8_and_int8_quantizers_match_reference_test_expressions():
    f = np.load(G / "quant.npz")
    x = O.bf16_bits_to_f32(f["x_bf16_bits"])
    q, s = O.quantize_fp8(x)
    assert np.array_equal(s, f["fp8_scale"]) and np.array_equal(q, f["fp8_q"])
    q2, _ = O.quantize_fp8(x, scale=float(f["fp8_static_scale"][0]))
    assert np.array_equal(q2, f["fp8_static_q"])
    qi, si = O.quantize_int8(f["x_f32"])
    assert np.array_equal(si, f["int8_scale"]) and np.array_equal(qi, f["int8_q"])


def test_nvfp4_quantizer_roundtrip_bound():
    """The only property the reference's tests pin for this quantizer (tests/test_gemm.py:221-228)."""
    f = np.load(G / "quant.npz")
    x = O.bf16_bits_to_f32(f["x4_bf16_bits"]).astype(np.float64)
    g = 448 * 6 / np.abs(x).max()
    q, sf = O.quantize_nvfp4(x, g)
    deq = O.unpack_fp4(q) * O.expand_block_scales(sf) / np.float64(np.float32(g))
    blk = np.repeat(np.abs(x).reshape(6, -1, 16).max(-1), 16, axis=-1)
    assert (np.abs(deq - x) <= blk * 0.26 + 1e-6).all()


def test_e4m3_encoder_matches_torch_cast_on_all_interesting_values():
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(20000) * s for s in (1e-3, 0.02, 1, 30, 400)]).astype(np.float32)
    mids = (O.E4M3_VALUES[:0x7E] + O.E4M3_VALUES[1:0x7F]) / 2          # every rounding tie
    vals = np.concatenate([vals, mids.astype(np.float32), -mids.astype(np.float32), O.E4M3_VALUES[:0x7F].astype(np.float32),
                           np.float32([0.0, -0.0, 448, -448, 464, 1e9, -1e9])])
    ours = O.f32_to_e4m3(vals)
    theirs = torch.from_numpy(vals).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)


def test_e2m1_encoder_ties_and_saturation():
    x = np.float32([0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6, 7, 100, -0.25, -0.75, -2.5, -9, -0.0, 0.24])
    want = np.uint8([0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 7, 7, 8, 10, 12, 15, 8, 0])  # ties go to the even code
    assert np.array_equal(O.f32_to_e2m1(x), want)


def test_int8_exact_and_epilogue_order():
    rng = np.random.default_rng(1)
    x = rng.integers(-127, 128, (3, 64)).astype(np.int8)
    w = rng.integers(-127, 128, (7, 64)).astype(np.int8)
    xs, ws = rng.uniform(0.5, 1.5, 3).astype(np.float32), rng.uniform(0.5, 1.5, 7).astype(np.float32)
    bias = rng.standard_normal(7).astype(np.float32)
    y = O.gemm_int8_exact(x, w, xs, ws, 0.5, bias)
    acc = (w.astype(np.int64) @ x.astype(np.int64).T).astype(np.float32)
    manual = ((acc * np.float32(0.5)) * ws[:, None]) * xs[None, :] + bias[:, None]
    assert y.dtype == np.float32 and np.array_equal(y, manual.T.astype(np.float32))


def test_skinny_order_emulation_is_m_invariant_and_close():
    rng = np.random.default_rng(2)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((5, 256)).astype(np.float32)))
    w = O.bf16_bits_to_f32(O.f32_to_bf16_bits((rng.standard_normal((9, 256)) / 16).astype(np.float32)))
    for lpr, ks in [(8, 1), (16, 2), (32, 1), (8, 4)]:
        y = O.skinny_gemv_exact(x, w, lpr, ks)
        for i in range(5):
            assert np.array_equal(O.skinny_gemv_exact(x[i:i + 1], w, lpr, ks)[0], y[i])
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        assert np.abs(y - ref).max() < 2e-5 * np.abs(ref).max()


def test_block_scale_tiling_is_a_permutation_with_zero_padding():
    """The tiled block-scale layout of the oracle: every source byte lands exactly once, padding stays zero, the inverse
    restores the matrix, and the first tile has the published order (row r, column c at (r % 32) * 16 + (r // 32) * 4 + c)."""
    rng = np.random.default_rng(3)
    for rows, cols in [(1, 1), (128, 4), (129, 5), (300, 18)]:
        sf = rng.integers(1, 256, size=(rows, cols), dtype=np.uint8)  # no zeros: padding is recognisable
        tiled = O.sf_to_tiled(sf)
        assert tiled.size == -(-rows // 128) * -(-cols // 4) * 512
        assert np.count_nonzero(tiled) == rows * cols
        assert np.array_equal(O.sf_from_tiled(tiled, rows, cols), sf)
    sf = np.arange(128 * 4, dtype=np.uint16).reshape(128, 4).astype(np.uint8)
    tiled = O.sf_to_tiled(sf)
    for r, c in [(0, 0), (1, 0), (31, 3), (32, 0), (33, 2), (127, 3)]:
        assert tiled[(r % 32) * 16 + (r // 32) * 4 + c] == sf[r, c]
