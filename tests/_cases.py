"""Seeded operands per precision, generated on the CPU so the oracle and the GPU see identical bytes. Distributions
follow the reference's test generator (tests/test_gemm.py:33-83): activations N(0,1), 16-bit weights N(0,1)/sqrt(K),
fp8 = 4*N(0,1) cast, fp4 = uniform random bytes, block scales = uniform e4m3 bytes in [0x18, 0x48), per-row scales
U(0.5, 1.5)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O

FP8 = torch.float8_e4m3fn
FP4 = getattr(torch, "float4_e2m1fn_x2", torch.uint8)
KIND_K = {"bf16": 8, "f16": 8, "fp8": 16, "int8": 16, "nvfp4": 64, "w8a16_bf16": 16, "w8a16_f16": 16,
          "w4a16_bf16": 64, "w4a16_f16": 64}
ALL_KINDS = list(KIND_K)


def _fp8(g, rows, k):
    return (torch.randn(rows, k, generator=g) * 4).to(FP8)


def _fp4(g, rows, k):
    return torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8)


def _sf(g, rows, k):
    return torch.randint(0x18, 0x48, (rows, k // 16), generator=g, dtype=torch.uint8)


def operands(kind: str, m: int, n: int, k: int, seed: int = 0, dev: str = "cuda"):
    """(x, w, kwargs) on `dev` plus float64 numpy dequantised (x_deq, w_deq) including scales."""
    g = torch.Generator().manual_seed(seed)
    kw = {}
    if kind in ("bf16", "f16"):
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        x = torch.randn(m, k, generator=g).to(dt)
        w = (torch.randn(n, k, generator=g) / k**0.5).to(dt)
        xd, wd = x.double().numpy(), w.double().numpy()
    elif kind.startswith("w8a16"):
        dt = torch.bfloat16 if kind.endswith("bf16") else torch.float16
        x = torch.randn(m, k, generator=g).to(dt)
        w = _fp8(g, n, k)
        ws = torch.rand(n, generator=g) + 0.5
        kw["w_scale"] = ws
        xd, wd = x.double().numpy(), O.dequant("fp8", w.view(torch.uint8).numpy()) * ws.double().numpy()[:, None]
    elif kind.startswith("w4a16"):
        dt = torch.bfloat16 if kind.endswith("bf16") else torch.float16
        x = torch.randn(m, k, generator=g).to(dt)
        w, wsf = _fp4(g, n, k), _sf(g, n, k)
        kw.update(w_block_scale=wsf.view(FP8), w_scale=torch.tensor([0.01]))
        xd, wd = x.double().numpy(), O.dequant("fp4", w.numpy(), wsf.numpy()) * float(np.float32(0.01))
        w = w.view(FP4)
    elif kind == "fp8":
        x, w = _fp8(g, m, k), _fp8(g, n, k)
        xs, ws = torch.rand(m, generator=g) + 0.5, torch.rand(n, generator=g) + 0.5
        kw.update(x_scale=xs, w_scale=ws)
        xd = O.dequant("fp8", x.view(torch.uint8).numpy()) * xs.double().numpy()[:, None]
        wd = O.dequant("fp8", w.view(torch.uint8).numpy()) * ws.double().numpy()[:, None]
    elif kind == "int8":
        x = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8)
        w = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8)
        xs, ws = torch.rand(m, generator=g) + 0.5, torch.rand(n, generator=g) + 0.5
        kw.update(x_scale=xs, w_scale=ws)
        xd, wd = x.double().numpy() * xs.double().numpy()[:, None], w.double().numpy() * ws.double().numpy()[:, None]
    elif kind == "nvfp4":
        x, w = _fp4(g, m, k), _fp4(g, n, k)
        xsf, wsf = _sf(g, m, k), _sf(g, n, k)
        kw.update(x_block_scale=xsf.view(FP8), w_block_scale=wsf.view(FP8), alpha=torch.tensor([1e-3]))
        xd = O.dequant("fp4", x.numpy(), xsf.numpy())
        wd = O.dequant("fp4", w.numpy(), wsf.numpy()) * float(np.float32(1e-3))
        x, w = x.view(FP4), w.view(FP4)
    else:
        raise ValueError(kind)
    to = lambda t: t.to(dev) if torch.is_tensor(t) else t
    return to(x), to(w), {a: to(b) for a, b in kw.items()}, xd, wd


def rel_err(y: torch.Tensor, ref: np.ndarray) -> float:
    return float(np.abs(y.double().cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30))
