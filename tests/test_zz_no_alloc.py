"""The allocation-free split-K entry point, llg_tc_gemm_static_ws, called through the C ABI.

Some hosts of this library cannot give it a workspace tensor: a serving process that split the whole GPU into its own
memory pools at start-up, or a latency-critical loop / plugin sandbox in which cudaMalloc is off limits because it
stalls the device. For them the library keeps a small fixed scratch array of its own. This test checks that the
variant returns exactly what the regular entry point (caller-provided workspace) returns, on two calls in a row - the
second one finds the first one's leftovers in the shared scratch - and that a problem larger than the scratch is
refused with a clear message. Collected last on purpose, so a failure here cannot hide the other tests under -x.
"""
import ctypes as C

import pytest
import torch

import lowlat_gemm as L
from lowlat_gemm import _native as N, _ops

from _cases import operands

pytestmark = pytest.mark.gpu


def _args(x, w, kw, y, ws, cnt, ksplit, kind_id=2, cfg=0):
    return _ops.fill_tc_args(y, w.view(torch.uint8), x.view(torch.uint8), None, None, kw["w_scale"].float().contiguous(),
                             kw["x_scale"].float().contiguous(), None, None, 1.0, kind_id, True, True, cfg, 4, ksplit, ws, cnt)


def _bare(a):
    """The same call without workspace and counters: the variant must not need them."""
    a.ws, a.ws_elems, a.counters, a.counters_elems = None, 0, None, 0
    return a


def test_static_workspace_entry_matches_regular_entry_twice():
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    for m, n, k, ksplit in [(4, 336, 4096, 8), (16, 1000, 2048, 3)]:
        x, w, kw, _, _ = operands("fp8", m, n, k, seed=m)
        ws, cnt = L._workspace(dev, ksplit * n * m, 64)
        want = torch.empty(m, n, device=dev, dtype=torch.float32)
        N.check(N.lib.llg_tc_gemm(C.byref(_args(x, w, kw, want, ws, cnt, ksplit)), stream))
        outs = [torch.full((m, n), float("nan"), device=dev, dtype=torch.float32) for _ in range(2)]
        N.check(N.lib.llg_tc_gemm_static_ws(C.byref(_bare(_args(x, w, kw, torch.empty_like(want), ws, cnt, ksplit))), stream))
        calls = [_bare(_args(x, w, kw, outs[call], ws, cnt, ksplit)) for call in range(2)]  # descriptors built beforehand
        torch.cuda.synchronize()  # the first call on the device has looked the scratch address up; from here on ...
        free_before = torch.cuda.mem_get_info(dev)[0]
        for a in calls:
            N.check(N.lib.llg_tc_gemm_static_ws(C.byref(a), stream))
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before  # ... a call takes no device memory from anyone
        for call in range(2):
            assert torch.equal(outs[call], want), (m, n, k, ksplit, call)  # same kernel, same summation order: same bits
    assert N.device_status() == 0


def test_static_workspace_rejects_oversized_problem():
    dev = torch.device("cuda", torch.cuda.current_device())
    x, w, kw, _, _ = operands("fp8", 16, 16384, 256, seed=1)
    y = torch.empty(16, 16384, device=dev, dtype=torch.float32)
    ws, cnt = L._workspace(dev, 0, 0)
    a = _args(x, w, kw, y, ws, cnt, 8)  # 8 * 16384 * 16 partials = 2 Mi > 1 Mi
    rc = N.lib.llg_tc_gemm_static_ws(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = N.lib.llg_last_error().decode()
    assert msg.startswith("lowlat_gemm: static workspace too small") and "2097152" in msg and "1048576" in msg
