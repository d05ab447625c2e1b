"""Host-side logic and the C ABI surface; no GPU (the library loads and validates arguments without one)."""
import ctypes as C
import json
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, SkinnyOrder, SkinnyTile, TcChoice, _native as N

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "llg_core.h").read_text()
    declared = set(re.findall(r"LLG_API[^;(]*?\b(llg_\w+)\s*\(", header))
    assert declared == set(N.SYMBOLS), declared ^ set(N.SYMBOLS)
    for name in declared:
        assert hasattr(N.lib, name)
    assert N.lib.llg_abi_version() == N.ABI_VERSION == int(re.search(r"#define LLG_ABI_VERSION (\d+)", header).group(1))


def test_struct_layout_matches_library():
    sizes = (C.c_int32 * 5)()
    N.lib.llg_struct_sizes(C.byref(sizes))
    assert tuple(sizes) == (C.sizeof(N.SkinnyArgs), C.sizeof(N.TcArgs), C.sizeof(N.QuantArgs), C.sizeof(N.GatedQuantArgs),
                            C.sizeof(N.PushArgs))


def test_tc_info_table():
    assert L.NUM_CFGS == 12 and L.PAIR_CFGS == (10, 11)
    for kind in L.KINDS:
        for cfg in range(10):
            bp, bq, threads, stage = L.tc_info(kind, cfg)
            want = 448 if kind.startswith(("w4a16", "w8a16")) else 320 if kind == "nvfp4" else 192
            assert bp == 128 and bq == 16 << (cfg % 5) and threads == want
            assert stage % 1024 == 0 and (stage == 0) == (L.max_stages(kind, cfg) == 0)
        for cfg, width in zip(L.PAIR_CFGS, (128, 256)):  # 256-row tiles on CTA pairs: unconverted operands only
            bp, bq, threads, stage = L.tc_info(kind, cfg)
            assert (bp, bq, threads) == (256, width, 192) and L.cfg_atoms(cfg) == 1
            assert stage == ((128 + width // 2) * 128 if kind in ("bf16", "f16", "fp8", "int8") else 0)
    with pytest.raises(ValueError, match="runs without split-K"):
        L.TcChoice(cfg=10, swap=False, ksplit=2)
    assert L.tc_info("bf16", 0)[3] == 128 * 128 + 16 * 128
    assert L.tc_info("nvfp4", 4)[3] == 0 and L.tc_info("w4a16_bf16", 5)[3] == 0
    with pytest.raises(RuntimeError, match="lowlat_gemm: unknown kind"):
        N.tc_info(99, 0)


def test_validation_errors_come_from_the_library_with_prefix():
    a = N.TcArgs()
    a.kind, a.cfg, a.ksplit = 0, 12, 1
    assert N.lib.llg_tc_gemm(C.byref(a), None) == -1
    assert N.lib.llg_last_error().decode().startswith("lowlat_gemm: cfg must be in [0, 12)")
    a.cfg, a.ksplit = 0, 65
    assert N.lib.llg_tc_gemm(C.byref(a), None) == -1 and b"ksplit must be in [1, 64]" in N.lib.llg_last_error()
    a.ksplit, a.a, a.lda_bytes = 1, 4096, 24
    assert N.lib.llg_tc_gemm(C.byref(a), None) == -1 and b"row stride must be a multiple of 16 bytes" in N.lib.llg_last_error()
    s = N.SkinnyArgs()
    s.rows, s.unroll, s.lanes_per_row, s.warps, s.ksplit = 3, 3, 32, 4, 1
    assert N.lib.llg_skinny(C.byref(s), None) == -1 and b"unsupported (rows, unroll)" in N.lib.llg_last_error()
    s.rows, s.unroll, s.lanes_per_row = 1, 4, 12
    assert N.lib.llg_skinny(C.byref(s), None) == -1 and b"lanes_per_row must be 8, 16 or 32" in N.lib.llg_last_error()
    q = N.QuantArgs()
    q.mode, q.in_dtype = 9, 1
    assert N.lib.llg_quant(C.byref(q), None) == -1 and b"unknown mode" in N.lib.llg_last_error()
    q.mode, q.K = 3, 24
    assert N.lib.llg_quant(C.byref(q), None) == -1 and b"nvfp4 needs K % 16 == 0" in N.lib.llg_last_error()


def test_pdl_switch_and_custom_op_schema():
    assert not L.pdl_enabled()
    L.set_pdl(True)
    assert L.pdl_enabled() and torch.ops.lowlat_gemm.pdl_enabled()
    L.set_pdl(False)
    assert not L.pdl_enabled()
    sch = str(torch.ops.lowlat_gemm.tc_gemm.default._schema)
    assert "Tensor(a!) y, Tensor a, Tensor b, Tensor? a_sf" in sch and "bool cluster=False" in sch
    assert list(torch.ops.lowlat_gemm.tc_info(2, 1)) == list(L.tc_info("fp8", 1))
    meta = torch.ops.lowlat_gemm.skinny(torch.empty(3, 64, dtype=torch.bfloat16, device="meta"),
                                        torch.empty(9, 64, dtype=torch.bfloat16, device="meta"),
                                        torch.empty(0, device="meta"), torch.empty(0, device="meta"), 1, 4, 32, 4, 1, True)
    assert meta.shape == (3, 9) and meta.dtype == torch.float32


def test_dataclass_validation():
    for bad in [dict(rows=3, unroll=2), dict(warps=9), dict(rows=2, unroll=8)]:
        with pytest.raises(ValueError):
            SkinnyTile(**bad)
    for bad in [dict(lanes_per_row=4), dict(ksplit=65), dict(ksplit=16, cluster=True)]:
        with pytest.raises(ValueError):
            SkinnyOrder(**bad)
    for bad in [dict(cfg=12, swap=True), dict(cfg=11, swap=True, ksplit=2), dict(cfg=0, swap=True, stages=1), dict(cfg=0, swap=True, stages=17),
                dict(cfg=0, swap=True, ksplit=0), dict(cfg=0, swap=True, ksplit=9, cluster=True)]:
        with pytest.raises(ValueError):
            TcChoice(**bad)


def test_plan_lookup_range_and_json_roundtrip(tmp_path):
    a, b = TcChoice(cfg=0, swap=True, stages=4, ksplit=2), TcChoice(cfg=1, swap=True, stages=4, ksplit=1)
    table = {1: a, 16: b}
    assert L._tc_lookup(table, 1) is a and L._tc_lookup(table, 15) is a
    assert L._tc_lookup(table, 16) is b and L._tc_lookup(table, 32) is b
    assert L._tc_lookup(table, 33) is None and L._tc_lookup({}, 1) is None
    order = SkinnyOrder(lanes_per_row=16, ksplit=4, cluster=True, tiles={2: SkinnyTile(2, 2, 8)})
    assert order.tile(1) == SkinnyTile(2, 2, 8) and order.tile(9) == SkinnyTile(2, 2, 8)
    plan = Plan(skinny=order, skinny_max_m=4, tc=dict(table), prefer_vendor=[16])
    back = Plan.from_json(json.loads(json.dumps(plan.to_json())))
    assert back == plan
    f = tmp_path / "p.json"
    L.save_plans(f, {("bf16", 4160, 1024): plan}, "Test Device 9000")
    assert L.load_plans(f) == 1
    data = json.loads(f.read_text())
    assert data["device"] == "Test Device 9000" and "bf16:4160x1024" in data["plans"]
    assert L._file_key("NVIDIA B200") == "nvidia_b200"
    with pytest.raises(ValueError):
        (tmp_path / "q.json").write_text('{"plans": {}}')
        L.load_plans(tmp_path / "q.json")


def test_heuristics_fill_the_gpu():
    sms = 148
    for kind, m, n, k in [("bf16", 4, 11008, 4096), ("fp8", 16, 14336, 4096), ("int8", 128, 4096, 4096),
                          ("nvfp4", 1, 28672, 8192), ("w4a16_bf16", 16, 28672, 8192), ("fp8", 256, 14336, 4096)]:
        c = L.default_tc_choice(kind, m, n, k, sms)
        bp, bq, _, stage = L.tc_info(kind, c.cfg)
        assert stage > 0 and 2 <= c.stages <= L.max_stages(kind, c.cfg)
        assert c.swap == (kind in L._MIXED or m <= 64)
        p, q = (n, m) if c.swap else (m, n)
        ctas = -(-p // bp) * -(-q // bq) * c.ksplit * (2 if c.cfg in L.PAIR_CFGS else 1)  # a pair tile occupies two SMs
        assert ctas >= sms // 2 or kind == "int8"
    # what the tuner finds on B200 for the baseline shapes: two K atoms per stage for decode batches; the streaming
    # kinds unsplit with three stages where the row pitch can spread the tiles; small weights split over a cluster
    c = L.default_tc_choice("fp8", 16, 14336, 4096, sms)
    assert (c.cfg, c.stages, c.ksplit, c.cluster) == (5, 3, 1, False)
    c = L.default_tc_choice("nvfp4", 8, 28672, 8192, sms)
    assert c.cfg == 5 and c.ksplit == 1 and c.stages == L.max_stages("nvfp4", 5)
    c = L.default_tc_choice("int8", 8, 4096, 4096, sms)
    assert c.cfg == 5 and 2 <= c.ksplit <= 8 and c.cluster
    assert L.default_tc_choice("w4a16_bf16", 4, 28672, 8192, sms).cfg == 0  # two atoms do not fit for W4A16
    for m in (1, 16, 64, 256):
        assert L.default_tc_choice("fp8", m, 1280, 8192, sms).ksplit <= 8
    # skinny engine: one wave of small CTAs, two to an SM, each with a contiguous row range
    o = L.default_skinny_order(11008, 4096, sms)
    assert o.lanes_per_row == 32 and o.ksplit == 1 and L.skinny_ranges(11008, o.ksplit, sms) == 2 * sms
    small = L.default_skinny_order(96, 2560, sms)
    assert small.ksplit > 1 and small.cluster and L.skinny_ranges(96, small.ksplit, sms) * small.ksplit <= 2 * sms
    assert L.default_skinny_order(1, 8, sms).lanes_per_row == 8 and L.skinny_ranges(1, 1, sms) == 1
    plan = L.default_plan("bf16", 11008, 4096, sms)
    assert plan.skinny is not None and plan.skinny_max_m >= 1 and set(plan.tc) >= {1, 16, 256}
    assert L.default_plan("fp8", 4096, 4096, sms).skinny is None


def test_kind_detection_on_cpu_tensors():
    bf, f8 = torch.zeros(2, 64, dtype=torch.bfloat16), torch.zeros(3, 64, dtype=torch.float8_e4m3fn)
    u8, sf = torch.zeros(3, 32, dtype=torch.uint8), torch.zeros(3, 4, dtype=torch.float8_e4m3fn)
    assert L.kind_of(bf, bf) == "bf16" and L.kind_of(bf.half(), f8) == "w8a16_f16"
    assert L.kind_of(bf, u8, None, sf) == "w4a16_bf16" and L.kind_of(u8, u8, sf, sf) == "nvfp4"
    assert L.kind_of(f8, f8) == "fp8" and L.kind_of(u8.view(torch.int8), u8.view(torch.int8)) == "int8"
    with pytest.raises(TypeError):
        L.kind_of(bf.float(), bf)
    assert not L.supports(bf, bf)  # not on a GPU


def test_missing_library_fails_loudly(tmp_path):
    code = "import sys; sys.path.insert(0, %r); import lowlat_gemm" % str(ROOT / "sm120-lowlat-gemm_b200")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                       env={"LLG_CORE_LIB": str(tmp_path / "nope.so"), "PATH": "/usr/bin"})
    assert r.returncode != 0 and "there is no fallback implementation" in r.stderr


def test_cpp_extension_registers_the_reference_schemas():
    """With lowlat_gemm._C built, the ops come from the C++ extension; either way the seven schemas are the reference's
    (csrc/ops.cpp:420-440), and the ctypes registration can still be asked for in a fresh interpreter."""
    from lowlat_gemm import _ops
    built = any((ROOT / "sm120-lowlat-gemm_b200" / "lowlat_gemm").glob("_C*.so"))
    assert _ops.BACKEND == ("cpp" if built else "ctypes")
    ns = torch.ops.lowlat_gemm
    assert str(ns.tc_info.default._schema) == "lowlat_gemm::tc_info(int kind, int cfg) -> int[]"
    assert "bool out_fp32=False, bool cluster=False, Tensor? prefetch=None, int prefetch_bytes=0) -> Tensor" in str(ns.skinny.default._schema)
    assert "Tensor(a!) y, Tensor a, Tensor b, Tensor? a_sf, Tensor? b_sf, Tensor? row_scale" in str(ns.tc_gemm.default._schema)
    assert "Tensor(a!) q, Tensor(b!)? sf, Tensor? scale_in, Tensor(c!)? scale_out, int mode, float min_scale" in str(ns.quant.default._schema)
    assert list(ns.tc_info(0, 0)) == list(N.tc_info(0, 0)) and ns.pdl_enabled() in (True, False)
    y = ns.skinny(torch.empty(3, 64, dtype=torch.bfloat16, device="meta"), torch.empty(7, 64, dtype=torch.bfloat16, device="meta"),
                  torch.empty(0, device="meta"), torch.empty(0, device="meta"), 1, 4, 32, 4, 1, True)
    assert tuple(y.shape) == (3, 7) and y.dtype == torch.float32
    code = "import sys; sys.path.insert(0, %r); from lowlat_gemm import _ops; print(_ops.BACKEND)" % str(ROOT / "sm120-lowlat-gemm_b200")
    import os
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=dict(os.environ, LLG_OPS="ctypes"), check=True)
    assert r.stdout.strip().splitlines()[-1] == "ctypes"
