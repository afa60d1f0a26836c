"""Data-parallel sharding of one matmul forward + backward across the GPUs of a box.

One process per GPU (``torch.distributed``; NCCL on GPUs, gloo in CPU tests).  The
path shards by ROWS of A (the batch dimension for a batched product, which is the
same thing once the batch is folded into M):

    rank g holds   A_g = A[rows_g, :],  dC_g = dC[rows_g, :]          (never exchanged)
    replicated     B                    (broadcast once into every GPU's own memory)
    forward        C_g  = A_g . B                                     no communication
    backward       dA_g = dC_g . B^T                                  no communication
                   dB   = sum_g A_g^T . dC_g                          ONE all-reduce

The all-reduce of the dB partials is issued on a side stream right after the dB GEMM
and overlaps the dA GEMM.  ``gather_output`` all-gathers C only for callers that need
it on every device.  Kernels only ever read the GPU's own memory.

torch is used for process groups, streams and device buffers only; the GEMMs are the
library's (``rp_matmul_ex`` through the C ABI), injected as ``gemm`` so that the
host-side logic can be exercised on CPU ranks with a stand-in.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable

import torch
import torch.distributed as dist

from . import _lib

_TORCH_CODE = {torch.float32: _lib.F32, torch.float64: _lib.F64, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def row_partition(rows: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of this rank's rows: an even split, remainder to the first ranks."""
    base, extra = divmod(rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def cuda_gemm(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, trans_a=False, trans_b=False, accumulate=False,
              max_sms: int = 0) -> None:
    """c (+)= op(a) . op(b) on c's device and the current torch stream, through the C ABI.
    2-D tensors with a unit stride in one dimension; op() is expressed as swapped strides (no copy)."""
    if not c.is_cuda:
        raise RuntimeError("recpulse_b200: CUDA tensors only (no CPU path)")
    lib = _lib.load()
    av = a.t() if trans_a else a
    bv = b.t() if trans_b else b
    m, k = av.shape
    k2, n = bv.shape
    assert k == k2 and c.shape == (m, n) and c.stride(1) == 1
    g = _lib.RpbGemm()
    g.m, g.n, g.k, g.batch, g.reduce = m, n, k, 1, 1
    g.a_row, g.a_col = av.stride(0), av.stride(1)
    g.b_row, g.b_col = bv.stride(0), bv.stride(1)
    g.c_row = c.stride(0)
    g.accumulate = int(accumulate)
    g.max_sms = int(max_sms)
    stream = torch.cuda.current_stream(c.device).cuda_stream
    rc = lib.rp_matmul_ex(C.c_void_p(c.data_ptr()), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.byref(g),
                          _TORCH_CODE[c.dtype], c.device.index, C.c_void_p(stream))
    if rc != 0:
        raise RuntimeError("rp_matmul_ex failed")


class RowShardedMatmul:
    """Forward + backward of C = A.B with A's rows split over the ranks of ``group``."""

    def __init__(self, b: torch.Tensor, group=None, gemm: Callable = cuda_gemm, src: int = 0, comm_sms: int = 16):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.gemm = gemm
        self.comm_sms = comm_sms
        self.b = b
        if self.world > 1:
            dist.broadcast(self.b, src=src, group=group)        # replicate B into local memory once
        self._side = torch.cuda.Stream(b.device) if b.is_cuda else None

    def forward(self, a_rows: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((a_rows.shape[0], self.b.shape[1]), dtype=a_rows.dtype, device=a_rows.device)
        self.gemm(out, a_rows, self.b)
        return out

    def backward(self, a_rows, dc_rows, da_out=None, db_out=None):
        """Returns (dA_rows, dB).  dB is complete (summed over ranks) when this returns on the
        current stream's timeline."""
        if da_out is None:
            da_out = torch.empty_like(a_rows)
        if db_out is None:
            db_out = torch.empty_like(self.b)
        self.gemm(db_out, a_rows, dc_rows, trans_a=True)         # partial dB first ...
        work = None
        if self.world > 1:
            if self._side is not None:
                self._side.wait_stream(torch.cuda.current_stream(db_out.device))
                with torch.cuda.stream(self._side):
                    work = dist.all_reduce(db_out, group=self.group, async_op=True)
            else:
                work = dist.all_reduce(db_out, group=self.group, async_op=True)
        # ... so its reduction hides behind dA.  The GEMM kernels are persistent and fill every SM, which
        # would leave the collective's thread blocks waiting for the GEMM to end; while a reduction is in
        # flight the dA GEMM therefore leaves `comm_sms` SMs free.
        if work is not None and self.comm_sms and self.gemm is cuda_gemm:
            sms = torch.cuda.get_device_properties(da_out.device).multi_processor_count
            self.gemm(da_out, dc_rows, self.b, trans_b=True, max_sms=max(2, sms - self.comm_sms))
        else:
            self.gemm(da_out, dc_rows, self.b, trans_b=True)
        if work is not None:
            work.wait()
            if self._side is not None:
                torch.cuda.current_stream(db_out.device).wait_stream(self._side)
        return da_out, db_out

    def gather_output(self, c_rows: torch.Tensor) -> torch.Tensor:
        """All-gather C (equal row counts per rank) for callers that need it on every device."""
        if self.world == 1:
            return c_rows
        full = torch.empty((c_rows.shape[0] * self.world, c_rows.shape[1]), dtype=c_rows.dtype, device=c_rows.device)
        dist.all_gather_into_tensor(full, c_rows.contiguous(), group=self.group)
        return full
