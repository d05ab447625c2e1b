"""Plans on the GPU: every tuned entry of the plan file packaged for this device runs and matches a float64 reference
(the reference's tests/test_gemm.py:277-295, including the per-rank shapes of the tensor-parallel decode layer that
the multi-GPU benchmark depends on); plans loaded through LLG_PLAN_FILE win over the packaged ones in a fresh
interpreter (tests/test_gemm.py:257-274); and one full-size decode layer on one GPU against the oracle chain."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, TcChoice, _native as N, timing, tp as TP
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
ROOT = Path(__file__).resolve().parent.parent
E2M1 = [0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6]


def _fp4_f64(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """[rows, K/2] packed nibbles (even element low) x [rows, K/16] e4m3 block scales -> float64 [rows, K]."""
    b = q.view(torch.uint8)
    table = torch.tensor(E2M1, dtype=torch.float64, device=b.device)
    vals = torch.stack([table[(b & 15).long()], table[(b >> 4).long()]], dim=-1).reshape(b.shape[0], -1)
    return vals * sf.view(torch.float8_e4m3fn).double().repeat_interleave(16, dim=1)


def _deq(kind: str, t: torch.Tensor, kw: dict, side: str) -> torch.Tensor:
    """Operand -> float64 including its scales, on the GPU (the reference's tests build their expectation the same way)."""
    bs, sc = kw.get(f"{side}_block_scale"), kw.get(f"{side}_scale")
    fp4 = kind == "nvfp4" or (kind.startswith("w4a16") and side == "w")
    v = _fp4_f64(t, bs) if fp4 else t.double() if t.dtype != torch.float8_e4m3fn else t.float().double()
    if torch.is_tensor(sc):
        v = v * sc.double().reshape(-1, 1) if sc.numel() > 1 else v * sc.double()
    elif sc is not None:
        v = v * float(np.float32(sc))
    return v


def test_packaged_plans_match_float64_reference():
    path = L._packaged_path(torch.cuda.get_device_name(DEV))
    if not path.is_file():
        pytest.skip(f"no packaged plans for {torch.cuda.get_device_name(DEV)}")
    entries = json.loads(path.read_text())["plans"]
    checked = 0
    for key in sorted(entries):
        kind, shape = key.split(":")
        n, k = (int(v) for v in shape.split("x"))
        plan = Plan.from_json(entries[key])
        g = torch.Generator(device=DEV).manual_seed(n + k)
        w, w_kw = timing.make_weight(kind, n, k, g, DEV)
        wd = _deq(kind, w, w_kw, "w")
        tokens = sorted(set(plan.tc) | ({m for m in (1, 2, 4, 8, 16) if m <= plan.skinny_max_m} if plan.skinny else set()))
        e, c = L.workspace_need(kind, n, k, max(tokens), DEV)
        L.reserve_workspace(DEV, e, c)
        for m in tokens:
            x, x_kw = timing.make_input(kind, m, k, DEV, seed=m)
            ref = _deq(kind, x, x_kw, "x") @ wd.T
            y = L.gemm(x, w, out_dtype=torch.float32, plan=plan, **w_kw, **x_kw)
            err = float((y.double() - ref).abs().max() / ref.abs().max())
            assert err < 2e-5, (key, m, err)
            if m in plan.tc and plan.skinny is not None and m <= plan.skinny_max_m:  # both engines are tuned for this M
                y_tc = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc=plan.tc), **w_kw, **x_kw)
                assert float((y_tc.double() - ref).abs().max() / ref.abs().max()) < 2e-5, (key, m, "tc")
            checked += 1
        del w, wd
        torch.cuda.empty_cache()
    assert checked >= len(entries) and N.device_status() == 0


def test_plan_file_from_environment_overrides_packaged(tmp_path):
    name = torch.cuda.get_device_name(DEV)
    mark = Plan(tc={4: TcChoice(cfg=2, swap=True, stages=5, ksplit=3)})
    L.save_plans(tmp_path / "mine.json", {("fp8", 14336, 4096): mark}, name)
    code = ("import sys, json, torch; sys.path.insert(0, %r); import lowlat_gemm as L; "
            "p = L.get_plan('fp8', 14336, 4096); q = L.get_plan('int8', 4096, 4096); "
            "print(json.dumps([p.to_json(), sorted(q.tc)]))" % str(ROOT / "sm120-lowlat-gemm_b200"))
    env = dict(os.environ, LLG_PLAN_FILE=str(tmp_path / "mine.json"))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, check=True).stdout
    got, other = json.loads(out.strip().splitlines()[-1])
    assert got == mark.to_json()                       # the file named by the environment wins for its shape ...
    if L._packaged_path(name).is_file():
        assert len(other) > 0                          # ... and the packaged plans still serve the others
    env.pop("LLG_PLAN_FILE")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, check=True).stdout
    assert json.loads(out.strip().splitlines()[-1])[0] != mark.to_json()


@pytest.mark.parametrize("kind", ["fp8", "bf16", "nvfp4"])
def test_full_size_decode_layer_on_one_gpu(kind):
    """One decode layer at hidden 8192 (QKV 10240, gate_up 57344, down 28672), 8 tokens, with the residual stream, against
    the same chain evaluated with float64 matmuls on dequantised operands. Activation quantizers are applied by the
    library (they are pinned bit for bit elsewhere), so the reference re-uses their outputs and what is checked is every
    GEMM of the layer at its real size, in the order and with the inputs the step produces."""
    m, shape = 8, TP.LayerShape()
    step = TP.DecodeStep(kind, 1, 1, 0, DEV, shape=shape, residual=True)
    x = (torch.randn(m, shape.hidden, generator=torch.Generator().manual_seed(3)) * 0.05).to(torch.bfloat16).to(DEV)
    seen = []
    real = step._gemm

    def spy(xa, w, **kw):
        y = real(xa, w, **kw)
        seen.append((xa, w, {a: b for a, b in kw.items() if "scale" in a}, y))
        return y

    step._gemm = spy
    out = step.run(x)
    assert len(seen) == 4 and torch.isfinite(out.float()).all()
    for xa, w, kw, y in seen:
        ref = _deq(kind, xa, kw, "x") @ _deq(kind, w, kw, "w").T
        err = float((y.double() - ref).abs().max())
        rms = float(ref.pow(2).mean().sqrt())
        assert err <= 1e-2 * rms + float(ref.abs().max()) * 2.0**-8, (kind, tuple(w.shape), err, rms)  # + one bf16 rounding of y
    assert N.device_status() == 0
