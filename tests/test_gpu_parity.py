"""GPU parity tests: the CUDA path (through lowlat_gemm -> torch.ops.lowlat_gemm -> the C ABI of libllg_core.so)
against the CPU oracle on identical seeded inputs. Modelled on the reference's tests/test_gemm.py.

Bars: quantizers, INT8 accumulation and the skinny GEMV bit-exact; floating-point tensor-core results within 2e-5 of
max|ref| for fp32 outputs (the reference's own gate) and within 1e-2 x RMS(ref) at the benchmark configurations.
"""
import itertools
from pathlib import Path

import numpy as np
import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, SkinnyOrder, SkinnyTile, TcChoice, _native as N
from oracle import oracle as O

from _cases import ALL_KINDS, FP4, FP8, KIND_K, operands, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = Path(__file__).parent / "golden"
TOL = 2e-5


def sms():
    return torch.cuda.get_device_properties(0).multi_processor_count


def no_expired_wait():
    assert N.device_status() == 0, "a kernel gave up a bounded wait"


# ---------------------------------------------------------------------------------------------------------------
# quantizers: bit-exact


@pytest.mark.parametrize("shape,dt", [((5, 384), torch.bfloat16), ((3, 4096), torch.bfloat16), ((2, 100), torch.float32),
                                      ((16, 8192), torch.float16), ((1, 8), torch.bfloat16), ((4, 20000), torch.bfloat16), ((3, 28672), torch.bfloat16), ((2, 40000), torch.float16),
                                      ((7, 1000), torch.float32)])
def test_quantizers_bit_exact(shape, dt):
    g = torch.Generator().manual_seed(shape[0] * 7919 + shape[1])
    x = torch.randn(*shape, generator=g).to(dt)
    x[0, : min(16, shape[1])] = 0  # an all-zero block: nvfp4 scale 0
    xn, xc = x.float().numpy(), x.to(DEV)
    q, s = L.quantize_fp8(xc)
    oq, osc = O.quantize_fp8(xn)
    assert q.dtype == FP8 and np.array_equal(s.cpu().numpy(), osc) and np.array_equal(q.view(torch.uint8).cpu().numpy(), oq)
    q, _ = L.quantize_fp8(xc, torch.tensor([0.02], device=DEV))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), O.quantize_fp8(xn, scale=float(np.float32(0.02)))[0])
    q, s = L.quantize_int8(xc)
    oq, osc = O.quantize_int8(xn)
    assert np.array_equal(s.cpu().numpy(), osc) and np.array_equal(q.cpu().numpy(), oq)
    if shape[1] % 16 == 0:
        gs = torch.tensor([448 * 6 / float(np.abs(xn).max())], device=DEV)
        q, sf = L.quantize_nvfp4(xc, gs)
        oq, osf = O.quantize_nvfp4(xn, float(gs.item()))
        assert sf.dtype == FP8 and np.array_equal(sf.view(torch.uint8).cpu().numpy(), osf)
        assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq)


def test_quantizers_on_reference_golden_inputs():
    f = np.load(G / "quant.npz")
    x = torch.from_numpy(f["x_bf16_bits"].view(np.int16)).view(torch.bfloat16).to(DEV)
    q, s = L.quantize_fp8(x)
    assert np.array_equal(s.cpu().numpy(), f["fp8_scale"]) and np.array_equal(q.view(torch.uint8).cpu().numpy(), f["fp8_q"])
    q, _ = L.quantize_fp8(x, torch.from_numpy(f["fp8_static_scale"]).to(DEV))
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), f["fp8_static_q"])
    q, s = L.quantize_int8(torch.from_numpy(f["x_f32"]).to(DEV))
    assert np.array_equal(s.cpu().numpy(), f["int8_scale"]) and np.array_equal(q.cpu().numpy(), f["int8_q"])


def test_quantizer_strided_rows_and_empty():
    x = torch.randn(6, 512, device=DEV).to(torch.bfloat16)[:, :256]  # row stride 512, K 256
    q, s = L.quantize_fp8(x)
    oq, osc = O.quantize_fp8(x.float().cpu().numpy())
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), osc)
    q, s = L.quantize_int8(torch.empty(0, 64, device=DEV))
    assert q.shape == (0, 64) and s.shape == (0,)


def test_gated_activation_fused_with_quantizers():
    """silu(gate) * up fused into the quantizer kernel: the activation matches an fp32 torch evaluation to one rounding
    and the quantized outputs are exactly what the stand-alone quantizers give on that activation."""
    g = torch.Generator().manual_seed(3)
    for dt, rows, k in [(torch.bfloat16, 5, 512), (torch.float16, 3, 4096), (torch.bfloat16, 2, 28672 // 2)]:
        gu = torch.randn(rows, 2 * k, generator=g).to(dt).to(DEV)
        act = L.silu_mul(gu)
        ref = (torch.nn.functional.silu(gu[:, :k].float()) * gu[:, k:].float())
        ulp = ref.abs() * (2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10) + 6.0e-8  # f16 subnormal spacing
        assert act.dtype == dt and bool(((act.float() - ref).abs() <= ulp).all())
        q, s = L.silu_mul_quantize_fp8(gu)
        q0, s0 = L.quantize_fp8(act)
        assert torch.equal(q.view(torch.uint8), q0.view(torch.uint8)) and torch.equal(s, s0)
        gs = torch.tensor([448 * 6 / act.float().abs().max().item()], device=DEV)
        q4, sf = L.silu_mul_quantize_nvfp4(gu, gs)
        q40, sf0 = L.quantize_nvfp4(act, gs)
        assert torch.equal(q4.view(torch.uint8), q40.view(torch.uint8)) and torch.equal(sf.view(torch.uint8), sf0.view(torch.uint8))
    view = torch.randn(4, 3 * 256, generator=g).to(torch.bfloat16).to(DEV)[:, :512]  # strided rows
    assert torch.equal(L.silu_mul(view), L.silu_mul(view.contiguous()))


# ---------------------------------------------------------------------------------------------------------------
# skinny GEMV: bit-exact against the order emulation, M- and tile-invariant


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_skinny_bit_exact_against_oracle(dt):
    for n, k in [(33, 136), (96, 2560), (1, 8), (513, 1024)]:
        g = torch.Generator().manual_seed(n * 31 + k)
        x = torch.randn(16, k, generator=g).to(dt)
        w = (torch.randn(n, k, generator=g) / k**0.5).to(dt)
        for lanes, ks, cl in [(32, 1, False), (8, 2, False), (16, 4, False), (16, 4, True), (8, 8, True)]:
            want = O.skinny_gemv_exact(x.float().numpy(), w.float().numpy(), lanes, ks)
            for tile, m in itertools.product([SkinnyTile(1, 4, 4), SkinnyTile(2, 2, 8), SkinnyTile(4, 2, 1), SkinnyTile(1, 8, 2)],
                                             (1, 3, 5, 16)):
                order = SkinnyOrder(lanes_per_row=lanes, ksplit=ks, default_tile=tile, cluster=cl)
                y = L.gemm(x[:m].to(DEV), w.to(DEV), out_dtype=torch.float32, plan=Plan(skinny=order, skinny_max_m=16))
                assert np.array_equal(y.cpu().numpy(), want[:m]), (n, k, lanes, ks, cl, tile, m)
    _, cnt = L._ws[torch.cuda.current_device()]
    assert int(cnt.abs().sum()) == 0


def test_skinny_batch_invariance_large_shapes():
    """Row i of an M-row call equals the 1-row call on x[i] for every M and tile (reference tests/test_gemm.py:147-157)."""
    for n, k in [(336, 10240), (2560, 6144), (10240, 320)]:
        x, w, _, _, _ = operands("bf16", 16, n, k, seed=1)
        base = L.default_skinny_order(n, k, sms())
        single = torch.cat([L.gemm(x[i:i + 1], w, plan=Plan(skinny=base, skinny_max_m=16)) for i in range(16)])
        for (r, u), wp in itertools.product([(1, 2), (1, 4), (1, 8), (2, 2), (2, 4), (4, 2)], (1, 4, 8)):
            order = SkinnyOrder(lanes_per_row=base.lanes_per_row, ksplit=base.ksplit, default_tile=SkinnyTile(r, u, wp))
            for m in (1, 2, 3, 5, 9, 16):
                y = L.gemm(x[:m], w, plan=Plan(skinny=order, skinny_max_m=16))
                assert torch.equal(y, single[:m]), (n, k, r, u, wp, m)


def test_skinny_16bit_output_rounding():
    x, w, _, xd, wd = operands("bf16", 4, 96, 2560)
    order = L.default_skinny_order(96, 2560, sms())
    y32 = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(skinny=order, skinny_max_m=16))
    y16 = L.gemm(x, w, plan=Plan(skinny=order, skinny_max_m=16))
    assert y16.dtype == torch.bfloat16 and torch.equal(y16, y32.to(torch.bfloat16))


# ---------------------------------------------------------------------------------------------------------------
# tensor-core engine


@pytest.mark.parametrize("kind", ALL_KINDS)
@pytest.mark.parametrize("m", [1, 3, 8, 17, 64, 200])
def test_default_plan_matches_reference(kind, m):
    n, k = 333, 4 * 256 + KIND_K[kind]  # odd N, partial last K tile
    x, w, kw, xd, wd = operands(kind, m, n, k)
    plan = Plan(tc=L.default_plan(kind, n, k, sms()).tc)  # tensor-core engine also where skinny would serve
    y = L.gemm(x, w, out_dtype=torch.float32, plan=plan, **kw)
    assert y.shape == (m, n) and y.dtype == torch.float32
    assert rel_err(y, xd @ wd.T) < TOL, kind
    no_expired_wait()


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_reference_emulator_golden_problem(kind):
    """The operands the reference's CPU emulator was run on (tests/golden/tc_<kind>.npz): same answer."""
    f = np.load(G / f"tc_{kind}.npz")
    k = int(f["k"])
    a_bits = {"nvfp4": 4, "w4a16_bf16": 4, "w4a16_f16": 4, "bf16": 16, "f16": 16}.get(kind, 8)
    b_bits = 4 if kind == "nvfp4" else 8 if kind in ("fp8", "int8") else 16
    wt = torch.from_numpy(f["a"][:, : k * a_bits // 8].copy())
    xt = torch.from_numpy(f["b"][:, : k * b_bits // 8].copy())
    views = {16: None, 8: FP8, 4: FP4}
    def as_operand(t, bits, int8):
        if bits == 16:
            return t.view(torch.bfloat16 if kind in ("bf16", "w8a16_bf16", "w4a16_bf16") else torch.float16)
        return t.view(torch.int8) if int8 else t.view(views[bits])
    w = as_operand(wt, a_bits, kind == "int8").to(DEV)
    x = as_operand(xt, b_bits, kind == "int8").to(DEV)
    kw = {}
    if f["asf"].size:
        kw["w_block_scale"] = torch.from_numpy(f["asf"]).view(FP8).to(DEV)
    if f["bsf"].size:
        kw["x_block_scale"] = torch.from_numpy(f["bsf"]).view(FP8).to(DEV)
    rs, cs = torch.from_numpy(f["rs"]).float().to(DEV), torch.from_numpy(f["cs"]).float().to(DEV)
    y = L.gemm(x, w, w_scale=rs, x_scale=cs, alpha=float(f["alpha"]), out_dtype=torch.float32,
               plan=Plan(tc={5: TcChoice(cfg=0, swap=True, stages=3, ksplit=1)}), **kw)
    # the emulator used float64 scales; ours are their fp32 roundings: 3 roundings of 2^-24 each
    assert rel_err(y, f["y"]) < 1e-6 + (TOL if kind != "int8" else 0)


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_every_config_orientation_and_split(kind):
    n, k = 200, 2 * 256 + KIND_K[kind]
    for m in (5, 70):
        x, w, kw, xd, wd = operands(kind, m, n, k, seed=m)
        ref = xd @ wd.T
        for cfg, swap, ksplit in itertools.product(range(L.NUM_CFGS), (False, True), (1, 3)):
            if L.max_stages(kind, cfg) < 2 or (kind in L._MIXED and not swap) or (cfg in L.PAIR_CFGS and ksplit > 1):
                continue
            c = TcChoice(cfg=cfg, swap=swap, stages=min(3, L.max_stages(kind, cfg)), ksplit=ksplit)
            y = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: c}), **kw)
            e = rel_err(y, ref)
            assert e < TOL, f"{kind} m={m} {c}: rel err {e}"
    no_expired_wait()


@pytest.mark.parametrize("kind", ["bf16", "f16", "fp8", "int8"])
def test_tiles_on_cta_pairs(kind):
    """The 256-row tiles that a pair of CTAs computes together: both orientations, ragged edges on every side (rows that
    leave the second CTA of a pair without data, columns that leave it without its half of B, a K tail), rings of 2 and
    5 stages, 16-bit outputs (vector stores) equal to the rounded fp32 result, bias on either side; INT8 bit-identical to
    the single-CTA tile. The last shape gives every pair several tiles, so both accumulator buffers are reused."""
    out16 = torch.float16 if kind == "f16" else torch.bfloat16
    for m, n, k in [(300, 712, 2 * 256 + KIND_K[kind]), (129, 130, 256), (520, 1100, 3 * 256), (2048, 2560, 512)]:
        x, w, kw, xd, wd = operands(kind, m, n, k, seed=m)
        bias = torch.randn(n, generator=torch.Generator().manual_seed(m)).to(DEV)
        ref = xd @ wd.T + bias.double().cpu().numpy()
        # the epilogue multiplies by the scale of the MMA's row side first, so bits are compared within an orientation
        single = {sw: L.gemm(x, w, bias=bias, out_dtype=torch.float32, plan=Plan(tc={m: TcChoice(cfg=3, swap=sw, stages=3)}), **kw)
                  for sw in (False, True)}
        for cfg, swap, stages in itertools.product(L.PAIR_CFGS, (False, True), (2, 5)):
            plan = Plan(tc={m: TcChoice(cfg=cfg, swap=swap, stages=stages)})
            y = L.gemm(x, w, bias=bias, out_dtype=torch.float32, plan=plan, **kw)
            e = rel_err(y, ref)
            assert e < TOL, f"{kind} {m}x{n}x{k} cfg={cfg} swap={swap} stages={stages}: rel err {e}"
            if kind == "int8":
                assert torch.equal(y, single[swap])
            y16 = L.gemm(x, w, bias=bias, out_dtype=out16, plan=plan, **kw)
            assert torch.equal(y16, y.to(out16)), f"{kind} cfg={cfg} swap={swap}: 16-bit output is not the rounded fp32 result"
    no_expired_wait()


def test_pair_tiles_in_a_pdl_chain_and_graph():
    """Three dependent GEMMs on pair tiles (the middle one between two single-CTA launches' worth of rows), eagerly
    with and without programmatic dependent launch and from a replayed CUDA graph with poisoned outputs: same bits."""
    g = torch.Generator().manual_seed(11)
    m, dims = 384, [1024, 2048, 768, 1536]
    ws = [(torch.randn(dims[i + 1], dims[i], generator=g) / dims[i] ** 0.5).to(torch.bfloat16).to(DEV) for i in range(3)]
    plans = [Plan(tc={m: TcChoice(cfg=11, swap=False, stages=6)}), Plan(tc={m: TcChoice(cfg=10, swap=True, stages=3)}),
             Plan(tc={m: TcChoice(cfg=11, swap=False, stages=2)})]
    x = torch.randn(m, dims[0], generator=g).to(torch.bfloat16).to(DEV)
    outs = [torch.empty(m, d, device=DEV, dtype=torch.bfloat16) for d in dims[1:]]

    def chain():
        h = x
        for w, p, o in zip(ws, plans, outs):
            L.gemm(h, w, out=o, plan=p)
            h = o

    L.set_pdl(False)
    chain()
    ref = [o.clone() for o in outs]
    want = x.double() @ ws[0].double().T
    assert rel_err(ref[0].double(), want.cpu().numpy()) < 1e-2  # bf16 output of a correct product
    try:
        L.set_pdl(True)
        chain()
        assert all(torch.equal(o, r) for o, r in zip(outs, ref))
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            chain()
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(3):
                chain()
        for _ in range(10):
            for o in outs:
                o.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert all(torch.equal(o, r) for o, r in zip(outs, ref))
    finally:
        L.set_pdl(False)
    no_expired_wait()


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_deep_pipelines(kind):
    m, n, k = 5, 72, 24 * 256
    x, w, kw, xd, wd = operands(kind, m, n, k, seed=3)
    ref = xd @ wd.T
    for cfg, ksplit in itertools.product(range(L.NUM_CFGS), (1, 2)):
        if cfg in L.PAIR_CFGS and ksplit > 1:
            continue
        top = L.max_stages(kind, cfg)
        for stages in sorted({s for s in (2, 8, 12, top) if 2 <= s <= top}):
            c = TcChoice(cfg=cfg, swap=True, stages=stages, ksplit=ksplit)
            y = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: c}), **kw)
            e = rel_err(y, ref)
            assert e < TOL, f"{kind} {c}: rel err {e}"
    no_expired_wait()


@pytest.mark.parametrize("kind", ["nvfp4", "w4a16_bf16", "w4a16_f16"])
def test_block_scales_by_tma_equal_per_thread_copies(kind):
    """Block scales whose rows are 16-byte aligned travel by TMA, others by per-thread 4-byte copies: the same numbers
    through both routes (the second time from a buffer shifted by 4 bytes) must give the same bits."""
    n, k = 300, 5 * 256  # K / 16 = 80 scale bytes per row: a multiple of 16
    for m, cfg, ksplit in [(3, 0, 1), (16, 5 if kind == "nvfp4" else 0, 1), (40, 2, 2)]:
        x, w, kw, xd, wd = operands(kind, m, n, k, seed=11 + m)
        c = TcChoice(cfg=cfg, swap=True, stages=3, ksplit=ksplit)
        y_tma = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: c}), **kw)
        shifted = dict(kw)
        for name in ("w_block_scale", "x_block_scale"):
            if name in kw:
                t = kw[name]
                buf = torch.empty(t.numel() + 16, dtype=torch.uint8, device=t.device)
                view = buf[4:4 + t.numel()].view(t.shape)
                view.copy_(t.view(torch.uint8))
                assert view.data_ptr() % 16 == 4
                shifted[name] = view.view(t.dtype)
        y_cp = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: c}), **shifted)
        assert torch.equal(y_tma, y_cp), (kind, m, c)
        assert rel_err(y_tma, xd @ wd.T) < TOL
    no_expired_wait()


@pytest.mark.parametrize("kind", ["bf16", "fp8", "nvfp4", "w4a16_bf16"])
def test_epilogue_bias_alpha_and_16bit_out(kind):
    m, n, k = 7, 130, 512
    x, w, kw, xd, wd = operands(kind, m, n, k)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    base_alpha = kw.pop("alpha", None)  # nvfp4: already folded into wd
    alpha = 0.5 * (base_alpha.item() if base_alpha is not None else 1.0)
    ref = 0.5 * (xd @ wd.T) + bias.double().numpy()
    y = L.gemm(x, w, alpha=alpha, bias=bias.to(DEV), out_dtype=torch.bfloat16, plan=Plan(tc=L.default_plan(kind, n, k, sms()).tc), **kw)
    assert y.dtype == torch.bfloat16 and rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("m,ksplit,cluster", [(1, 1, False), (8, 4, False), (32, 8, False), (8, 4, True), (128, 2, False)])
def test_int8_bit_exact(m, ksplit, cluster):
    """INT8: int32 accumulation exact, epilogue in the pinned order -> every output bit equals the oracle's."""
    n, k = 512, 4096
    g = torch.Generator().manual_seed(m)
    xf = torch.randn(m, k, generator=g).to(torch.bfloat16)
    x, xs = L.quantize_int8(xf.to(DEV))
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    ws = (torch.rand(n, generator=g) + 0.5) * 1e-2
    bias = (torch.randn(n, generator=g) * 0.1).to(torch.bfloat16)
    want = O.gemm_int8_exact(x.cpu().numpy(), w.numpy(), xs.cpu().numpy(), ws.numpy(), 1.0, bias.float().numpy())
    for swap, cfg in [(True, 0 if m <= 16 else 2), (False, 3)]:
        c = TcChoice(cfg=cfg if m <= 64 or not swap else 3, swap=swap, stages=4, ksplit=ksplit, cluster=cluster)
        y32 = L.gemm(x, w.to(DEV), x_scale=xs, w_scale=ws.to(DEV), bias=bias.to(DEV), out_dtype=torch.float32, plan=Plan(tc={m: c}))
        if swap:  # oracle epilogue order is the swapped orientation's: (acc*alpha)*w_scale*x_scale
            assert np.array_equal(y32.cpu().numpy(), want), (m, c)
        else:
            assert rel_err(y32, want.astype(np.float64)) < 1e-6
        y16 = L.gemm(x, w.to(DEV), x_scale=xs, w_scale=ws.to(DEV), bias=bias.to(DEV), plan=Plan(tc={m: c}))
        assert y16.dtype == torch.bfloat16 and torch.equal(y16, y32.to(torch.bfloat16))
    # raw accumulators: unit scales, fp32 out, |acc| < 2^24 holds for these magnitudes only statistically -> compare in int
    acc = L.gemm(x, w.to(DEV), out_dtype=torch.float32, plan=Plan(tc={m: TcChoice(cfg=0, swap=True, stages=4, ksplit=ksplit, cluster=cluster)}))
    exact = x.cpu().numpy().astype(np.int64) @ w.numpy().astype(np.int64).T
    assert np.array_equal(acc.cpu().numpy(), exact.astype(np.float32))


def test_split_k_deterministic_and_counters_reset():
    x, w, kw, _, _ = operands("fp8", 4, 336, 4096)
    plan = Plan(tc={4: TcChoice(cfg=0, swap=True, stages=4, ksplit=8)})
    first = L.gemm(x, w, plan=plan, **kw)
    for _ in range(20):
        assert torch.equal(L.gemm(x, w, plan=plan, **kw), first)
    _, cnt = L._ws[torch.cuda.current_device()]
    assert int(cnt.abs().sum()) == 0


@pytest.mark.parametrize("kind", ALL_KINDS)
def test_cluster_split_k_matches_workspace_bitwise(kind):
    n, k = 200, 4 * 256 + KIND_K[kind]
    for m in (3, 70):
        x, w, kw, xd, wd = operands(kind, m, n, k, seed=m + 1)
        ref = xd @ wd.T
        for cfg, swap, ksplit in itertools.product(range(L.NUM_CFGS), (False, True), (2, 5, 8)):
            st = L.max_stages(kind, cfg)
            if st < 2 or (kind in L._MIXED and not swap) or cfg in L.PAIR_CFGS:
                continue
            c = TcChoice(cfg=cfg, swap=swap, stages=min(3, st), ksplit=ksplit)
            y_ws = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: c}), **kw)
            cc = TcChoice(cfg=cfg, swap=swap, stages=min(3, st), ksplit=ksplit, cluster=True)
            y_cl = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={m: cc}), **kw)
            assert torch.equal(y_cl, y_ws), f"{kind} m={m} {cc}"
            assert rel_err(y_cl, ref) < TOL
    no_expired_wait()


def test_cuda_graph_replay():
    x, w, kw, _, _ = operands("nvfp4", 4, 512, 2048)
    plan = Plan(tc={4: TcChoice(cfg=0, swap=True, stages=4, ksplit=4)})
    eager = L.gemm(x, w, plan=plan, **kw)
    out = torch.empty_like(eager)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        L.gemm(x, w, out=out, plan=plan, **kw)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        L.gemm(x, w, out=out, plan=plan, **kw)
    for _ in range(5):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)


def test_workspace_growth_during_capture_raises():
    x, w, kw, _, _ = operands("fp8", 4, 256, 1024)
    L.reserve_workspace(torch.device(DEV), 0, 0)
    big = L._ws[torch.cuda.current_device()][0].numel() + 1
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with pytest.raises(RuntimeError, match="reserve_workspace"):
            with torch.cuda.graph(g):
                L.reserve_workspace(torch.device(DEV), big, 1)


@pytest.mark.parametrize("m", [1, 4, 40])
def test_pdl_chain_matches_serial(m):
    """Five chained GEMMs sharing one workspace; with PDL each may start early, so any read of activations or
    workspace before the dependency wait changes a bit here (reference tests/test_gemm.py:298-349)."""
    g = torch.Generator().manual_seed(7)
    dims = [2048, 1536, 4096, 512, 2048, 1024]
    ws = [(torch.randn(dims[i + 1], dims[i], generator=g) / dims[i] ** 0.5).to(torch.bfloat16).to(DEV) for i in range(len(dims) - 1)]
    skinny = Plan(skinny=SkinnyOrder(lanes_per_row=16, ksplit=4, default_tile=SkinnyTile(1, 4, 4)), skinny_max_m=16)
    plans = [Plan(tc={m: TcChoice(cfg=0 if m <= 16 else 2, swap=True, stages=4, ksplit=8, cluster=True)}),
             skinny if m <= 16 else Plan(tc={m: TcChoice(cfg=2, swap=True, stages=3, ksplit=2)}),
             Plan(tc={m: TcChoice(cfg=1 if m <= 32 else 2, swap=True, stages=3, ksplit=4)}),
             Plan(tc={m: TcChoice(cfg=3, swap=False, stages=2, ksplit=2)}),
             Plan(tc={m: TcChoice(cfg=5 if m <= 16 else 7, swap=False if m > 16 else True, stages=6, ksplit=1)})]
    x = torch.randn(m, dims[0], generator=g).to(torch.bfloat16).to(DEV)
    outs = [torch.empty(m, d, device=DEV, dtype=torch.bfloat16) for d in dims[1:]]

    def chain(prefetch=False):
        h = x
        for i, (w, p, o) in enumerate(zip(ws, plans, outs)):
            nxt = ws[(i + 1) % len(ws)] if prefetch else None
            L.gemm(h, w, out=o, plan=p, prefetch=nxt, prefetch_bytes=(1 << 20) if i % 2 else 0)
            h = o

    L.reserve_workspace(torch.device(DEV), 8 * 4096 * 64, 4096)
    L.set_pdl(False)
    chain()
    ref = [o.clone() for o in outs]
    try:
        L.set_pdl(True)
        chain()
        assert all(torch.equal(o, r) for o, r in zip(outs, ref))
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            chain()
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for r in range(4):
                chain(prefetch=r % 2 == 1)
        for _ in range(20):
            for o in outs:
                o.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            for i, (o, r) in enumerate(zip(outs, ref)):
                assert torch.equal(o, r), f"stage {i} differs under PDL"
    finally:
        L.set_pdl(False)
    _, cnt = L._ws[torch.cuda.current_device()]
    assert int(cnt.abs().sum()) == 0
    no_expired_wait()


def test_supports_and_shapes():
    x, w, _, _, _ = operands("bf16", 4, 64, 64)
    assert L.supports(x, w) and not L.supports(x.float(), w)
    x12 = torch.randn(2, 12, device=DEV).to(torch.bfloat16)
    assert not L.supports(x12, torch.randn(3, 12, device=DEV).to(torch.bfloat16))
    y = L.gemm(x.view(2, 2, 64), w)
    assert y.shape == (2, 2, 64) and y.dtype == torch.bfloat16
    assert L.gemm(x[:0], w).shape == (0, 64)
    out = torch.empty(4, 64, device=DEV, dtype=torch.float32)
    assert L.gemm(x, w, out=out, out_dtype=torch.bfloat16) is out  # out wins over out_dtype
    with pytest.raises(ValueError):
        L.gemm(x[:, :32], w)
    with pytest.raises(RuntimeError, match="lowlat_gemm:"):
        torch.ops.lowlat_gemm.tc_gemm(out, x, w, None, None, None, None, None, None, 1.0, 0, False, False, L.NUM_CFGS, 2, 1,
                                      *L._workspace(torch.device(DEV), 0, 0))


# ---------------------------------------------------------------------------------------------------------------
# the benchmark configurations at full size: max-abs error <= 1e-2 x RMS(ref) against the fp32 host matmul.
# The bound is applied to the fp32-output result. A 16-bit output is then required to be exactly that result rounded
# to the output type: rounding a correct value to bf16 alone moves it by up to 2^-9 of its magnitude, which at the
# largest of 44k N(0, s) outputs (4.3 s) is already 1.2e-2 x RMS, so the bound cannot be asked of a bf16 tensor.


def _check(call, ref32):
    y32 = call(torch.float32)
    err = np.abs(y32.double().cpu().numpy() - ref32.astype(np.float64)).max()
    assert err <= 1e-2 * np.sqrt(np.mean(ref32.astype(np.float64) ** 2)), err
    y16 = call(torch.bfloat16)
    assert y16.dtype == torch.bfloat16 and torch.equal(y16, y32.to(torch.bfloat16))


def test_config1_bf16():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 4096, generator=g).to(torch.bfloat16)
    w = (torch.randn(11008, 4096, generator=g) * 0.02).to(torch.bfloat16)
    ref = O.gemm_f32(x.float().numpy(), w.float().numpy())
    xc, wc = x.to(DEV), w.to(DEV)
    for plan in (None, Plan(tc=L.default_plan("bf16", 11008, 4096, sms()).tc)):  # skinny engine, tensor-core engine
        _check(lambda dt: L.gemm(xc, wc, plan=plan, out_dtype=dt), ref)


def test_config2_fp8_and_w8a16():
    """W8A8 FP8 and W8A16 at 14336 x 4096 for every token count of the configuration."""
    g = torch.Generator().manual_seed(0)
    w_scale = (torch.rand(14336, generator=g) * 1.5 + 0.5) * 1e-3
    w = ((torch.randn(14336, 4096, generator=g) * 0.02) / w_scale[:, None]).clamp(-448, 448).to(FP8)
    wc, wsc = w.to(DEV), w_scale.to(DEV)
    wd = (O.dequant("fp8", w.view(torch.uint8).numpy()) * w_scale.double().numpy()[:, None]).astype(np.float32)
    for m in (1, 2, 4, 8, 16, 64, 256):
        x = torch.randn(m, 4096, generator=g).to(torch.bfloat16)
        xc = x.to(DEV)
        xq, xs = L.quantize_fp8(xc)
        xd = O.dequant("fp8", xq.view(torch.uint8).cpu().numpy()) * xs.double().cpu().numpy()[:, None]
        _check(lambda dt: L.gemm(xq, wc, x_scale=xs, w_scale=wsc, out_dtype=dt), O.gemm_f32(xd, wd))
        _check(lambda dt: L.gemm(xc, wc, w_scale=wsc, out_dtype=dt), O.gemm_f32(x.double().numpy(), wd))


@pytest.mark.parametrize("m", [1, 8, 32, 128])
@pytest.mark.parametrize("ksplit", [1, 4, 8])
def test_config3_int8(m, ksplit):
    g = torch.Generator().manual_seed(0)
    xf = torch.randn(m, 4096, generator=g).to(torch.bfloat16)
    w = torch.randint(-127, 128, (4096, 4096), generator=g, dtype=torch.int8)
    ws = (torch.rand(4096, generator=g) + 0.5) * 1e-2
    bias = (torch.randn(4096, generator=g) * 0.1).to(torch.bfloat16)
    x, xs = L.quantize_int8(xf.to(DEV))
    want = O.gemm_int8_exact(x.cpu().numpy(), w.numpy(), xs.cpu().numpy(), ws.numpy(), 1.0, bias.float().numpy())
    c = TcChoice(cfg=0 if m <= 16 else 1 if m <= 32 else 3, swap=True, stages=6, ksplit=ksplit)
    y = L.gemm(x, w.to(DEV), x_scale=xs, w_scale=ws.to(DEV), bias=bias.to(DEV), out_dtype=torch.float32, plan=Plan(tc={m: c}))
    assert np.array_equal(y.cpu().numpy(), want)
    y = L.gemm(x, w.to(DEV), x_scale=xs, w_scale=ws.to(DEV), bias=bias.to(DEV))  # the default plan, bf16 out
    assert _close_bf16(y, want)


def _close_bf16(y, want32):
    """Default plans may pick the unswapped orientation, whose scale order differs by one fp32 rounding: allow one bf16 ulp."""
    a = y.float().cpu().numpy()
    b = torch.from_numpy(want32).to(torch.bfloat16).float().numpy()
    return bool((np.abs(a - b) <= np.abs(b) * 2.0**-7 + 1e-30).all())


def test_config4_nvfp4():
    """W4A16 and W4A4 at 28672 x 8192 for every token count of the configuration."""
    n, k = 28672, 8192
    g = torch.Generator().manual_seed(0)
    wf = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    gw = torch.tensor([448 * 6 / wf.float().abs().max().item()], device=DEV)
    wq, wsf = L.quantize_nvfp4(wf, gw)           # weights quantised with the library's own (reference-pinned) quantizer
    del wf
    wd = (O.dequant("fp4", wq.view(torch.uint8).cpu().numpy(), wsf.view(torch.uint8).cpu().numpy()) / float(gw.item())).astype(np.float32)
    for m in (1, 2, 4, 8, 16, 128):
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
        _check(lambda dt: L.gemm(x, wq, w_block_scale=wsf, w_scale=1.0 / gw.item(), out_dtype=dt),
               O.gemm_f32(x.double().cpu().numpy(), wd))
        gx = torch.tensor([448 * 6 / x.float().abs().max().item()], device=DEV)
        xq, xsf = L.quantize_nvfp4(x, gx)
        xd = O.dequant("fp4", xq.view(torch.uint8).cpu().numpy(), xsf.view(torch.uint8).cpu().numpy()) / float(gx.item())
        _check(lambda dt: L.gemm(xq, wq, x_block_scale=xsf, w_block_scale=wsf, x_scale=1.0 / gx.item(), w_scale=1.0 / gw.item(),
                                 out_dtype=dt), O.gemm_f32(xd, wd))
