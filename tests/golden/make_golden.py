"""Regenerates the golden fixtures in this directory from the reference checkout (run where it is mounted):

    python tests/golden/make_golden.py /path/to/sm120-lowlat-gemm

What is stored (small .npz files, inputs and expected outputs only - no reference source):
  * formats.npz   - the reference emulator's e4m3 / e2m1 decode tables (tests/emulate_tc.py:37-48).
  * tc_<kind>.npz - one small problem per precision: packed operand bytes, block scales, epilogue vectors and the
                    output Y of the reference's CPU emulation of its tensor-core kernel
                    (tests/emulate_tc.py:run_kernel, float64 arithmetic over the kernel's exact index logic).
  * quant.npz     - seeded activations with the outputs of the reference's *test expressions* for the FP8 and INT8
                    quantizers evaluated with torch on the CPU (tests/test_gemm.py:200-218), i.e. the values the
                    reference's own GPU tests require bit for bit.
The NVFP4 quantizer has no bit-level expectation in the reference; its fixture holds only the round-trip bound
inputs (tests/test_gemm.py:221-228).
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "tests"))
    import emulate_tc as E  # the reference's own CPU emulator

    np.savez(HERE / "formats.npz", e4m3=E.E4M3, e2m1=E.E2M1)

    fmt_a = {"bf16": "bf16", "f16": "f16", "fp8": "e4m3", "int8": "s8", "nvfp4": "e2m1", "w8a16_bf16": "e4m3",
             "w8a16_f16": "e4m3", "w4a16_bf16": "e2m1", "w4a16_f16": "e2m1"}
    for kind, (a_bits, b_bits, bk, mixed, bscaled, wbscaled, int_acc, t16) in E.KINDS.items():
        rng = np.random.default_rng(11)
        kal = 64 if a_bits == 4 else 16
        p, q, k = 70, 5, 2 * bk + kal  # weight rows, tokens, a partial last K tile
        a, _ = E.make_operand(rng, p, k, fmt_a[kind])
        b, _ = E.make_operand(rng, q, k, t16 if mixed else fmt_a[kind])
        asf = bsf = None
        if bscaled or wbscaled:
            asf, _ = E.make_scales(rng, p, k)
        if bscaled:
            bsf, _ = E.make_scales(rng, q, k)
        rs, cs, alpha = rng.uniform(0.5, 2, p), rng.uniform(0.5, 2, q), 0.75
        y = E.run_kernel(kind, 0, p, q, k, a, b, asf, bsf, 1, 3, True, rs, cs, alpha)  # swap: y[q, p]
        np.savez(HERE / f"tc_{kind}.npz", a=a, b=b, asf=asf if asf is not None else np.zeros(0, np.uint8),
                 bsf=bsf if bsf is not None else np.zeros(0, np.uint8), rs=rs, cs=cs, alpha=alpha, y=y,
                 k=k)

    g = torch.Generator().manual_seed(5)
    x = torch.randn(5, 384, generator=g).to(torch.bfloat16)
    s_ref = x.float().abs().amax(dim=1) / torch.full((5,), 448.0)
    q_ref = (x.float() * (1 / s_ref)[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    st = torch.tensor([0.02])
    q_static = (x.float() * (1 / st)).clamp(-448, 448).to(torch.float8_e4m3fn)
    xi = torch.randn(5, 384, generator=g)
    si_ref = xi.abs().amax(dim=1) / torch.full((5,), 127.0)
    qi_ref = torch.round(xi * (1 / si_ref)[:, None]).clamp(-127, 127).to(torch.int8)
    x4 = torch.randn(6, 512, generator=g).to(torch.bfloat16)
    np.savez(HERE / "quant.npz",
             x_bf16_bits=x.view(torch.int16).numpy().view(np.uint16), fp8_scale=s_ref.numpy(),
             fp8_q=q_ref.view(torch.uint8).numpy(), fp8_static_scale=st.numpy(), fp8_static_q=q_static.view(torch.uint8).numpy(),
             x_f32=xi.numpy(), int8_scale=si_ref.numpy(), int8_q=qi_ref.numpy(),
             x4_bf16_bits=x4.view(torch.int16).numpy().view(np.uint16))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
