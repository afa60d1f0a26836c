"""Python caller of the library's sharded entry points (``RpbShard`` in include/recpulse_b200.h).

The sharding itself -- NCCL communicator, replication of B, the float32 reduction of the dB
partials overlapped with the dA GEMM, the optional all-gather of C -- lives in the shared
library (csrc/shard.cu) behind the C ABI.  This module only does what a launcher does:

    rank g holds   A_g = A[rows_g, :],  dC_g = dC[rows_g, :]          (never exchanged)
    replicated     B                    (rp_shard_replicate, once)
    forward        C_g  = A_g . B                                     no communication
    backward       dA_g = dC_g . B^T                                  no communication
                   dB   = sum_g A_g^T . dC_g                          one reduction per step

it carries the 128-byte rendezvous id from rank 0 to the other ranks (over whatever
``torch.distributed`` group the launcher already has; gloo is enough) and passes device
pointers of torch tensors through ctypes.  No torch collective is on the data path.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib

_TORCH_CODE = {torch.float32: _lib.F32, torch.float64: _lib.F64, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
SLICE_ONLY = 1


def row_partition(rows: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of this rank's rows (``rpb_shard_rows``): an even split, remainder to the first ranks."""
    b, e = C.c_longlong(), C.c_longlong()
    _lib.load().rpb_shard_rows(rows, world, rank, C.byref(b), C.byref(e))
    return b.value, e.value


def db_slice(k: int, n: int, dtype_code: int, world: int, rank: int, db_wire: int = 0, flags: int = SLICE_ONLY) -> tuple[int, int]:
    """Elements of dB that `rank` holds after a backward with `flags` (``rpb_shard_db_slice_of``)."""
    b, e = C.c_longlong(), C.c_longlong()
    if _lib.load().rpb_shard_db_slice_of(k, n, dtype_code, world, rank, db_wire, flags, C.byref(b), C.byref(e)) != 0:
        raise ValueError("rpb_shard_db_slice_of: bad arguments")
    return b.value, e.value


def exchange_unique_id(group=None, make=None) -> bytes:
    """Rank 0 of `group` makes the rendezvous id (``rpb_shard_unique_id``, or `make()` in tests) and every
    rank returns the same 128 bytes."""
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    box = [None]
    if rank == 0:
        if make is not None:
            box[0] = bytes(make())
        else:
            buf = C.create_string_buffer(128)
            if _lib.load().rpb_shard_unique_id(buf) != 0:
                raise RuntimeError("rpb_shard_unique_id failed")
            box[0] = buf.raw
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    if not isinstance(box[0], (bytes, bytearray)) or len(box[0]) != 128:
        raise RuntimeError("unique id exchange failed")
    return bytes(box[0])


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class RowShardedMatmul:
    """Forward + backward of C = A.B with A's rows split over ranks, through the C ABI.

    `unique_id` comes from :func:`exchange_unique_id`; `b` is this rank's device buffer for B
    (filled on rank `src`, overwritten elsewhere by the replication)."""

    def __init__(self, b: torch.Tensor, rank: int = 0, world: int = 1, unique_id: bytes | None = None, src: int = 0,
                 comm_sms: int | None = None, db_wire: int | None = None):
        if not b.is_cuda:
            raise RuntimeError("recpulse_b200: CUDA tensors only (no CPU path)")
        self.lib = _lib.load()
        self.rank, self.world, self.b = rank, world, b
        self.device = b.device.index
        self.code = _TORCH_CODE[b.dtype]
        self.handle = self.lib.rpb_shard_create(unique_id, rank, world, self.device)
        if not self.handle:
            raise RuntimeError("rpb_shard_create failed")
        if comm_sms is not None or db_wire is not None:
            self.lib.rpb_shard_configure(self.handle, -1 if comm_sms is None else comm_sms, 0 if db_wire is None else db_wire)
        if world > 1:
            self._check(self.lib.rp_shard_replicate(self.handle, _ptr(b), b.numel() * b.element_size(), src, self._stream()),
                        "rp_shard_replicate")

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.b.device).cuda_stream)

    @staticmethod
    def _check(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed")

    def forward(self, a_rows: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        rows, k = a_rows.shape
        n = self.b.shape[1]
        if out is None:
            out = torch.empty((rows, n), dtype=a_rows.dtype, device=a_rows.device)
        assert a_rows.is_contiguous() and out.is_contiguous() and self.b.is_contiguous()
        self._check(self.lib.rp_matmul_rowsharded_forward(self.handle, _ptr(out), _ptr(a_rows), _ptr(self.b), rows, k, n,
                                                          self.code, self._stream()), "rp_matmul_rowsharded_forward")
        return out

    def backward(self, a_rows, dc_rows, da_out=None, db_out=None, flags: int = 0):
        """Returns (dA_rows, dB); dB is the sum over all ranks, complete in the current stream's order."""
        rows, k = a_rows.shape
        n = self.b.shape[1]
        if da_out is None:
            da_out = torch.empty_like(a_rows)
        if db_out is None:
            db_out = torch.empty_like(self.b)
        assert a_rows.is_contiguous() and dc_rows.is_contiguous() and da_out.is_contiguous() and db_out.is_contiguous()
        self._check(self.lib.rp_matmul_rowsharded_backward(self.handle, _ptr(da_out), _ptr(db_out), _ptr(a_rows), _ptr(self.b),
                                                           _ptr(dc_rows), rows, k, n, self.code, flags, self._stream()),
                    "rp_matmul_rowsharded_backward")
        return da_out, db_out

    def gather_output(self, c_rows: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """All-gather of C (equal row counts per rank) for callers that need it on every device."""
        rows, n = c_rows.shape
        if out is None:
            out = torch.empty((rows * self.world, n), dtype=c_rows.dtype, device=c_rows.device)
        self._check(self.lib.rp_matmul_gather_rows(self.handle, _ptr(out), _ptr(c_rows), rows, n, self.code, self._stream()),
                    "rp_matmul_gather_rows")
        return out

    def close(self):
        if self.handle:
            self.lib.rpb_shard_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
