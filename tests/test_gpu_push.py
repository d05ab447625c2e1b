"""The push form of the row-parallel boundary on ONE GPU: a single-rank OneShotAllReduce (ordinary device memory, no
process group) drives exactly the kernels a multi-GPU step uses - llg_tc_gemm_push storing from the GEMM's epilogue and
signalling, llg_reduce_local waiting for the signals, summing, adding the residual and quantizing - so their
arithmetic is pinned where only one GPU is available. Also the failure path: a wait for a signal that never comes
runs out after a short limit, the kernel returns, the status word reports it, and the device stays usable."""
import ctypes as C

import numpy as np
import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import Plan, TcChoice, _native as N, comm as CM, tp as TP

from _cases import operands

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev():
    return torch.device("cuda", torch.cuda.current_device())


@pytest.mark.parametrize("kind", ["fp8", "bf16", "nvfp4", "w8a16_bf16"])
@pytest.mark.parametrize("choice", [TcChoice(cfg=0, swap=True, stages=4, ksplit=1), TcChoice(cfg=5, swap=True, stages=3, ksplit=3),
                                    TcChoice(cfg=1, swap=True, stages=4, ksplit=4, cluster=True),
                                    TcChoice(cfg=3, swap=False, stages=3, ksplit=1)])
def test_pushed_gemm_plus_local_reduce_equals_gemm_add_quantize(kind, choice):
    if choice.cfg == 5 and kind == "nvfp4":
        pytest.skip("two K atoms per stage do not fit every kind")
    if kind.startswith("w8a16") and not choice.swap:
        pytest.skip("mixed kinds keep the weight as operand A")
    m, n, k = 8, 1024, 1024
    x, w, kw, _, _ = operands(kind, m, n, k, seed=3)
    plan = Plan(tc={m: choice})
    ar = CM.OneShotAllReduce(None, _dev(), max_bytes=m * n * 2, local=True)
    want = L.gemm(x, w, out_dtype=torch.bfloat16, plan=plan, **kw)
    resid = (torch.randn(m, n, generator=torch.Generator().manual_seed(9)) * want.float().abs().mean().item()).to(torch.bfloat16).to(DEV)
    for call in range(3):  # the flag counters only grow: later calls must work like the first; buffers alternate
        ar.gemm_push(call, x, w, out_dtype=torch.bfloat16, plan=plan, **kw)
        out, q, s = ar.reduce_local(call, m, n, torch.bfloat16, residual=resid if call else None, quantize=True)
        ref = want if call == 0 else (want.float() + resid.float()).to(torch.bfloat16)  # one rounding, like an elementwise add
        q_ref, s_ref = L.quantize_fp8(ref)
        assert torch.equal(out, ref), (kind, choice, call)
        assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref), (kind, choice, call)
    assert int(ar._done.item()) == 0  # the completion counter of the push returns to zero
    assert N.device_status() == 0


def test_single_rank_step_same_bits_with_and_without_push():
    """A decode step on one GPU through the push kernels equals the same step with plain gemm(), elementwise residual
    add and the stand-alone quantizer, bit for bit - FP8 (fused quantizer in the consumer) and bf16."""
    shape = TP.LayerShape(hidden=1024, qkv=1536, inter=2048)
    x = (torch.randn(4, 1024, generator=torch.Generator().manual_seed(5)) * 0.1).to(torch.bfloat16).to(DEV)
    for kind in ("fp8", "bf16"):
        plain = TP.DecodeStep(kind, 2, 1, 0, _dev(), shape=shape, residual=True).run(x)
        ar = CM.OneShotAllReduce(None, _dev(), max_bytes=4 * 1024 * 2, local=True)
        step = TP.DecodeStep(kind, 2, 1, 0, _dev(), shape=shape, residual=True, comm=ar, push=True)
        pushed = step.run(x)
        assert step.reduces == 4 and torch.isfinite(pushed.float()).all()
        assert torch.equal(pushed, plain), kind
        graph = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(graph):
                y = step.run(x)
        torch.cuda.current_stream().wait_stream(s)
        for _ in range(3):
            y.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y, plain), kind
    assert N.device_status() == 0


def test_wait_for_a_missing_signal_runs_out_and_reports():
    """llg_reduce_local is told of two ranks, but nobody ever signals for the second: with the limit set to about a
    millisecond the wait gives up, the kernel returns, llg_device_status() reads 16 once and then 0, and the next GEMM
    is correct. Nothing traps and nothing hangs."""
    dev = _dev()
    m, n = 4, 512
    recv = torch.zeros(2 * m * n, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(2 * N.AR_MAX_CTAS * 2, dtype=torch.int32, device=dev)
    flags.view(N.AR_MAX_CTAS * 2, 2)[:m, 0] = 1  # rank 0 "has signalled" every row; rank 1 never will
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    N.lib.llg_set_wait_limit(2_000_000)
    try:
        N.check(N.lib.llg_reduce_local(C.c_void_p(recv.data_ptr()), m * n * 2, C.c_void_p(flags.data_ptr()), C.c_void_p(out.data_ptr()),
                                       None, None, 0, None, m, n, 1, 1e-12, 2, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
    finally:
        N.lib.llg_set_wait_limit(0)
    assert N.device_status() == 16
    assert N.device_status() == 0
    x, w, kw, xd, wd = operands("bf16", 4, 256, 512)
    y = L.gemm(x, w, out_dtype=torch.float32, plan=Plan(tc={4: TcChoice(cfg=0, swap=True, stages=4, ksplit=2)}))
    ref = xd @ wd.T
    assert float(np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()) < 2e-5
    assert N.device_status() == 0
