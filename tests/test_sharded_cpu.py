"""Host-side logic of the row-sharded forward + backward on two CPU ranks (gloo).  The GEMM is
injected: here the oracle stands in for the CUDA library, which is the only thing the product runs."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cpu_gemm(c, a, b, trans_a=False, trans_b=False, accumulate=False):
    av = a.t() if trans_a else a
    bv = b.t() if trans_b else b
    r = av.double() @ bv.double()
    c.copy_((c.double() + r if accumulate else r).to(c.dtype))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from recpulse_b200.sharded import RowShardedMatmul, row_partition
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    m, k, n = 37, 24, 16                       # rows do not divide evenly
    A = torch.randn(m, k, generator=g, dtype=torch.float64); B = torch.randn(k, n, generator=g, dtype=torch.float64)
    dC = torch.randn(m, n, generator=g, dtype=torch.float64)
    r0, r1 = row_partition(m, world, rank)
    b_local = B.clone() if rank == 0 else torch.zeros_like(B)     # only rank 0 holds B at first
    op = RowShardedMatmul(b_local, gemm=_cpu_gemm)
    assert torch.equal(op.b, B)                                    # replicated by the broadcast
    c = op.forward(A[r0:r1])
    da, db = op.backward(A[r0:r1], dC[r0:r1])
    ok = (torch.allclose(c, A[r0:r1] @ B) and torch.allclose(da, dC[r0:r1] @ B.t())
          and torch.allclose(db, A.t() @ dC))                      # dB is the sum over ranks
    # even split for the optional gather of C
    m2 = 8 * world
    A2 = torch.randn(m2, k, generator=g, dtype=torch.float64)
    s0, s1 = row_partition(m2, world, rank)
    full = op.gather_output(op.forward(A2[s0:s1]))
    ok = ok and torch.allclose(full, A2 @ B)
    q.put((rank, bool(ok), (r0, r1)))
    dist.destroy_process_group()


def test_row_partition_covers_all_rows():
    sys.path.insert(0, ROOT)
    from recpulse_b200.sharded import row_partition
    for rows in (1, 7, 64, 65536, 100003):
        for world in (1, 2, 3, 4, 8):
            spans = [row_partition(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_forward_backward_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), results
    spans = sorted(s for _, _, s in results)
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == 37


def test_cuda_gemm_refuses_cpu_tensors():
    sys.path.insert(0, ROOT)
    from recpulse_b200.sharded import cuda_gemm
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        cuda_gemm(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2))
