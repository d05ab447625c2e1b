"""All-reduce over peer-mapped ("symmetric") memory for the row-parallel boundaries of a tensor-parallel decode layer.

Two forms, both with plain peer loads / stores and one-way counter signals only - no multicast, no NVLS:
  pull  the GEMM writes its partial into this rank's symmetric buffer; one small kernel (`llg_allreduce_oneshot`, or
        `llg_allreduce_quant_fp8` with the next projection's quantizer fused in) reads every rank's partial over NVLink
        and adds them in rank order;
  push  the GEMM itself stores every finished output element into every rank's buffer from its epilogue
        (`llg_tc_gemm_push`) and signals once it is done; the consumer (`llg_reduce_local`) adds the local copies in
        rank order, optionally adds the residual, stores the new hidden state and quantizes it for the next projection.
        The transfer overlaps the GEMM's remaining tiles and no load crosses NVLink on the critical path.
Both give every rank the same bits, run after run. The reference has nothing comparable (no multi-GPU code); the
baseline these replace is `torch.distributed.all_reduce` (NCCL).

torch is used for what it is here for: allocating and exchanging the peer mappings
(`torch.distributed._symmetric_memory`).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _native as N

_DT = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}


class OneShotAllReduce:
    """Two alternating symmetric buffers (consecutive all-reduces must not share one) plus the flag words."""

    def __init__(self, group, device: torch.device, max_bytes: int, ctas: int = 16, buffers: int = 2, local: bool = False):
        """max_bytes: largest payload of one all-reduce. Every buffer holds one such region per rank (the push form
        collects rank s's partial in region s; the pull form uses region 0). local=True builds a single-rank instance
        on ordinary device memory (no process group needed): the same kernels then serve a one-GPU step."""
        self.device, self.ctas, self.max_bytes = device, ctas, (max_bytes + 15) // 16 * 16
        if ctas > N.AR_MAX_CTAS:
            raise ValueError(f"at most {N.AR_MAX_CTAS} CTAs per all-reduce")
        if local:
            self.group, self.rank, self.world = None, 0, 1
            self.bufs = [torch.empty(self.max_bytes, dtype=torch.uint8, device=device) for _ in range(buffers)]
            self.flags = torch.zeros(2 * N.AR_MAX_CTAS, dtype=torch.int32, device=device)
            self._host_buf_ptrs = [[b.data_ptr()] for b in self.bufs]
            self._host_flag_ptrs = [self.flags.data_ptr()]
            self._handles = []
        else:
            import torch.distributed._symmetric_memory as symm

            self.group = group if group is not None else dist.group.WORLD
            self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
            if self.world > 8:
                raise ValueError("one-shot all-reduce supports at most 8 ranks")
            self.bufs = [symm.empty(self.max_bytes * self.world, dtype=torch.uint8, device=device) for _ in range(buffers)]
            # per rank: [AR_MAX_CTAS][world] arrival counters (the peers add to them) + as many consumed counts (private)
            self.flags = symm.empty(2 * N.AR_MAX_CTAS * self.world, dtype=torch.int32, device=device)
            self.flags.zero_()
            handles = [symm.rendezvous(b, self.group) for b in self.bufs]
            fh = symm.rendezvous(self.flags, self.group)
            self._host_buf_ptrs = [list(h.buffer_ptrs) for h in handles]
            self._host_flag_ptrs = list(fh.buffer_ptrs)
            self._handles = handles + [fh]
        # device arrays of peer pointers, index = rank (the pull kernels read them)
        self._buf_ptrs = [torch.tensor(p, dtype=torch.int64, device=device) for p in self._host_buf_ptrs]
        self._flag_ptrs = torch.tensor(self._host_flag_ptrs, dtype=torch.int64, device=device)
        self._done = torch.zeros(1, dtype=torch.int32, device=device)  # push form: CTAs of the running GEMM that finished
        torch.cuda.synchronize(device)
        if not local:
            dist.barrier(self.group)

    def view(self, index: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """This rank's symmetric buffer `index` as a tensor: pass it as `out=` to the GEMM that produces the partial."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.max_bytes:
            raise ValueError(f"all-reduce buffer holds {self.max_bytes} bytes, need {nbytes}")
        return self.bufs[index % len(self.bufs)][:nbytes].view(dtype).view(*shape)

    def reduce(self, index: int, out: torch.Tensor) -> torch.Tensor:
        """out = sum over ranks of buffer `index` (same shape and dtype as the view the partial was written to)."""
        nbytes = out.numel() * out.element_size()
        if nbytes % 16 or not out.is_contiguous():
            raise ValueError("all-reduce payload must be contiguous and a multiple of 16 bytes")
        with torch.cuda.device(self.device):
            N.check(N.lib.llg_allreduce_oneshot(
                C.c_void_p(self._buf_ptrs[index % len(self.bufs)].data_ptr()), C.c_void_p(self._flag_ptrs.data_ptr()),
                C.c_void_p(out.data_ptr()), nbytes, _DT[out.dtype], self.rank, self.world, self.ctas,
                C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        return out

    def reduce_quantize_fp8(self, index: int, rows: int, cols: int, dtype: torch.dtype, out: torch.Tensor | None = None,
                            min_scale: float = 1e-12):
        """(q, scale) = quantize_fp8(sum over ranks of buffer `index`), one kernel (`llg_allreduce_quant_fp8`): the
        16-bit sum is formed and quantized in registers, bit-identical to reduce() followed by quantize_fp8(). With
        `out` ([rows, cols], contiguous, `dtype`) the 16-bit sum is stored as well. rows <= 64, cols % 8 == 0."""
        q = torch.empty(rows, cols, device=self.device, dtype=torch.float8_e4m3fn)
        scale = torch.empty(rows, device=self.device, dtype=torch.float32)
        if out is not None and (not out.is_contiguous() or out.dtype != dtype or tuple(out.shape) != (rows, cols)):
            raise ValueError("out must be a contiguous [rows, cols] tensor of the partials' dtype")
        with torch.cuda.device(self.device):
            N.check(N.lib.llg_allreduce_quant_fp8(
                C.c_void_p(self._buf_ptrs[index % len(self.bufs)].data_ptr()), C.c_void_p(self._flag_ptrs.data_ptr()),
                C.c_void_p(out.data_ptr() if out is not None else 0), C.c_void_p(q.data_ptr()), q.stride(0),
                C.c_void_p(scale.data_ptr()), rows, cols, _DT[dtype], float(min_scale), self.rank, self.world,
                C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        return q, scale

    # ---- push form ---------------------------------------------------------------------------------------------------

    def _region(self, index: int, src: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for v in shape:
            n *= v
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.max_bytes:
            raise ValueError(f"all-reduce buffer holds {self.max_bytes} bytes per rank, need {nbytes}")
        buf = self.bufs[index % len(self.bufs)]
        return buf[src * self.max_bytes: src * self.max_bytes + nbytes].view(dtype).view(*shape)

    def gemm_push(self, index: int, x: torch.Tensor, w: torch.Tensor, *, out_dtype: torch.dtype, plan=None, prefetch=None,
                  prefetch_bytes: int = 0, **scales) -> None:
        """The row-parallel projection x @ w^T of all-reduce `index`, with its result stored into every rank's receive
        buffer by the GEMM's own epilogue (tensor-core engine; same keyword arguments as gemm() for the scales)."""
        from . import _ops, api

        mine = self._region(index, self.rank, (x.reshape(-1, x.shape[-1]).shape[0], w.shape[0]), out_dtype)
        pr = api._problem(x, w, scales.get("x_block_scale"), scales.get("w_block_scale"), None, mine)
        plan = plan or api.get_plan(pr.kind, pr.n, pr.k, pr.device)
        launch = api.tc_launch_for(pr, api.tc_choice_for(pr.kind, pr.m, pr.n, pr.k, plan, pr.device), prefetch=prefetch,
                                   prefetch_bytes=prefetch_bytes, **scales)
        args = _ops.fill_tc_args(*launch.op_args())
        push = N.PushArgs()
        push.world, push.rank, push.rows = self.world, self.rank, pr.m
        off = self.rank * self.max_bytes
        for d in range(self.world):
            push.dst[d] = self._host_buf_ptrs[index % len(self.bufs)][d] + off
            push.flags[d] = self._host_flag_ptrs[d]
        push.done = self._done.data_ptr()
        with torch.cuda.device(self.device):
            N.check(N.lib.llg_tc_gemm_push(C.byref(args), C.byref(push), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))

    def reduce_local(self, index: int, rows: int, cols: int, dtype: torch.dtype, *, residual: torch.Tensor | None = None,
                     want_out: bool = True, quantize: bool = False, min_scale: float = 1e-12):
        """Consumer of gemm_push(index, ...): (out, q, scale) with out = round(sum over ranks) (+ residual, one more
        rounding) when want_out, and (q, scale) = quantize_fp8(out) when quantize - all in one kernel, bit-identical to
        all_reduce, elementwise add and quantize_fp8 run one after the other."""
        if not (want_out or quantize):
            raise ValueError("nothing to compute")
        out = torch.empty(rows, cols, device=self.device, dtype=dtype) if want_out else None
        q = torch.empty(rows, cols, device=self.device, dtype=torch.float8_e4m3fn) if quantize else None
        scale = torch.empty(rows, device=self.device, dtype=torch.float32) if quantize else None
        if residual is not None and (not residual.is_contiguous() or residual.dtype != dtype or tuple(residual.shape) != (rows, cols)):
            raise ValueError("residual must be a contiguous [rows, cols] tensor of the partials' dtype")
        with torch.cuda.device(self.device):
            N.check(N.lib.llg_reduce_local(
                C.c_void_p(self.bufs[index % len(self.bufs)].data_ptr()), self.max_bytes, C.c_void_p(self.flags.data_ptr()),
                C.c_void_p(out.data_ptr() if want_out else 0), C.c_void_p(residual.data_ptr() if residual is not None else 0),
                C.c_void_p(q.data_ptr() if quantize else 0), q.stride(0) if quantize else 0,
                C.c_void_p(scale.data_ptr() if quantize else 0), rows, cols, _DT[dtype], float(min_scale), self.world,
                C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        return out, q, scale
