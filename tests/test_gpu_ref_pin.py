"""Pins to the reference's own GPU code: its quantizer kernels (csrc/quant.cu) and its GEMV (csrc/gemv.cuh), compiled
unmodified for sm_100a by oracle/Makefile into oracle/_ref/libref_sm100.so, are run on the same seeded inputs as this
repository's kernels, and the output BYTES must be equal - to the kernels and to the numpy oracle. This is what pins
the NVFP4 activation quantizer (the reference's tests only bound its error) and the GEMV's summation order.
Skipped when the library was not built (it needs the reference checkout at build time, not at run time)."""
import ctypes as C
import itertools
from pathlib import Path

import numpy as np
import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, SkinnyOrder, SkinnyTile
from oracle import oracle as O

pytestmark = pytest.mark.gpu
REF_SO = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libref_sm100.so"
DEV = "cuda"
_DT = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}


@pytest.fixture(scope="module")
def ref():
    if not REF_SO.is_file():
        pytest.skip("oracle/_ref/libref_sm100.so not built (make -C oracle REF=<reference checkout>)")
    lib = C.CDLL(str(REF_SO))
    lib.ref_quant.restype = C.c_int
    lib.ref_quant.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                              C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]
    lib.ref_gemv.restype = C.c_int
    lib.ref_gemv.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong] + [C.c_int] * 11 + \
                            [C.c_void_p, C.c_void_p]
    return lib


def _inputs(dt, m, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g) * torch.logspace(-3, 2, m)[:, None]  # rows of very different magnitude
    x[0, : k // 2] = 0
    if m > 2:
        x[2] = 0  # an all-zero row takes the min_scale branch
    return x.to(dt)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_quantizers_match_the_reference_kernels_byte_for_byte(ref, dt):
    torch.cuda.synchronize()
    for m, k in [(1, 4096), (5, 8192), (16, 1024), (3, 48), (2, 20000)]:
        x = _inputs(dt, m, k, seed=m * 7 + k).to(DEV)
        xf = x.float().cpu().numpy()
        # FP8 per token and static, INT8 per token
        for mode, ours in ((1, lambda: L.quantize_fp8(x)), (2, lambda: L.quantize_int8(x))):
            q_ref = torch.empty(m, k, dtype=torch.uint8, device=DEV)
            s_ref = torch.empty(m, dtype=torch.float32, device=DEV)
            assert ref.ref_quant(mode, _DT[dt], x.data_ptr(), x.stride(0), q_ref.data_ptr(), k, None, 0, None, s_ref.data_ptr(),
                                 1e-12, m, k) == 0
            q, s = ours()
            assert torch.equal(q.view(torch.uint8), q_ref) and torch.equal(s, s_ref), (mode, m, k, dt)
            oq, os_ = (O.quantize_fp8 if mode == 1 else O.quantize_int8)(xf)
            assert np.array_equal(q_ref.cpu().numpy(), oq.view(np.uint8)) and np.array_equal(s_ref.cpu().numpy(), os_)
        st = torch.tensor([0.37], device=DEV)
        q_ref = torch.empty(m, k, dtype=torch.uint8, device=DEV)
        assert ref.ref_quant(0, _DT[dt], x.data_ptr(), x.stride(0), q_ref.data_ptr(), k, None, 0, st.data_ptr(), None, 0.0, m, k) == 0
        assert torch.equal(L.quantize_fp8(x, scale=st)[0].view(torch.uint8), q_ref)
        # NVFP4: packed nibbles and block scales, for several global scales (tiny, usual, one that saturates the scales)
        if k % 16 == 0:
            for g in (1.0, 64.0, 448.0 * 6.0 / max(float(x.float().abs().max()), 1e-6), 1e6):
                gt = torch.tensor([g], device=DEV, dtype=torch.float32)
                q_ref = torch.empty(m, k // 2, dtype=torch.uint8, device=DEV)
                sf_ref = torch.empty(m, k // 16, dtype=torch.uint8, device=DEV)
                assert ref.ref_quant(3, _DT[dt], x.data_ptr(), x.stride(0), q_ref.data_ptr(), k // 2, sf_ref.data_ptr(), k // 16,
                                     gt.data_ptr(), None, 0.0, m, k) == 0
                q, sf = L.quantize_nvfp4(x, gt)
                assert torch.equal(q.view(torch.uint8), q_ref), (m, k, dt, g)
                assert torch.equal(sf.view(torch.uint8), sf_ref), (m, k, dt, g)
                oq, osf = O.quantize_nvfp4(xf, float(np.float32(g)))
                assert np.array_equal(q_ref.cpu().numpy(), oq) and np.array_equal(sf_ref.cpu().numpy(), osf), (m, k, dt, g)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_skinny_gemv_matches_the_reference_kernel_bit_for_bit(ref, dt):
    for n, k in [(33, 136), (513, 1024), (96, 2560), (1000, 4104)]:
        g = torch.Generator().manual_seed(n + k)
        x = torch.randn(16, k, generator=g).to(dt).to(DEV)
        w = (torch.randn(n, k, generator=g) / k**0.5).to(dt).to(DEV)
        for (lanes, ks, cl), m in itertools.product([(32, 1, False), (16, 4, False), (8, 2, False), (16, 4, True), (8, 8, True)],
                                                    (1, 3, 8, 16)):
            y_ref = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
            ws = torch.empty(ks * m * n, dtype=torch.float32, device=DEV)
            cnt = torch.zeros(n, dtype=torch.int32, device=DEV)
            rc = ref.ref_gemv(x.data_ptr(), w.data_ptr(), y_ref.data_ptr(), x.stride(0), w.stride(0), n, m, n, k,
                              int(dt == torch.float16), 1, 1, 4, lanes, 4, ks, int(cl), ws.data_ptr(), cnt.data_ptr())
            assert rc == 0
            order = SkinnyOrder(lanes_per_row=lanes, ksplit=ks, cluster=cl, default_tile=SkinnyTile(2, 4, 4))
            y = L.gemm(x[:m], w, out_dtype=torch.float32, plan=Plan(skinny=order, skinny_max_m=16))
            assert torch.equal(y, y_ref), (n, k, lanes, ks, cl, m, dt)
            assert int(cnt.abs().sum()) == 0
        want = O.skinny_gemv_exact(x[:3].float().cpu().numpy(), w.float().cpu().numpy(), 16, 4)
        y = L.gemm(x[:3], w, out_dtype=torch.float32,
                   plan=Plan(skinny=SkinnyOrder(lanes_per_row=16, ksplit=4, default_tile=SkinnyTile(1, 4, 8)), skinny_max_m=16))
        assert np.array_equal(y.cpu().numpy(), want)
