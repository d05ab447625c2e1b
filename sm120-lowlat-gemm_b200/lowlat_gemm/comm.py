"""One-shot all-reduce over peer-mapped ("symmetric") memory for the row-parallel boundaries of a tensor-parallel
decode layer: the GEMM writes its partial straight into this rank's symmetric buffer, one small kernel
(`llg_allreduce_oneshot`) then reads every rank's partial over NVLink and adds them in rank order. Plain peer loads and
one-way counter signals only - no multicast, no NVLS. The reference has nothing comparable (no multi-GPU code); the
baseline this replaces is `torch.distributed.all_reduce` (NCCL).

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

    def __init__(self, group, device: torch.device, max_bytes: int, ctas: int = 16, buffers: int = 2):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("one-shot all-reduce supports at most 8 ranks")
        self.device, self.ctas, self.max_bytes = device, ctas, (max_bytes + 15) // 16 * 16
        self.bufs = [symm.empty(self.max_bytes, dtype=torch.uint8, device=device) for _ in range(buffers)]
        if ctas > N.AR_MAX_CTAS:
            raise ValueError(f"at most {N.AR_MAX_CTAS} CTAs per all-reduce")
        # per rank: [AR_MAX_CTAS][world] arrival counters (the peers add to them) + as many consumed counts (private)
        self.flags = symm.empty(2 * N.AR_MAX_CTAS * self.world, dtype=torch.int32, device=device)
        self.flags.zero_()
        handles = [symm.rendezvous(b, self.group) for b in self.bufs]
        fh = symm.rendezvous(self.flags, self.group)
        # device arrays of peer pointers, index = rank
        self._buf_ptrs = [torch.tensor(list(h.buffer_ptrs), dtype=torch.int64, device=device) for h in handles]
        self._flag_ptrs = torch.tensor(list(fh.buffer_ptrs), dtype=torch.int64, device=device)
        self._handles = handles + [fh]
        torch.cuda.synchronize(device)
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
