"""The sharded entry points on two real GPUs (NCCL issued by the library itself): as two processes, and as
two threads of one process.  Skipped on boxes with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHILD = os.path.join(ROOT, "tests", "sharded_child.py")


def _two_gpus():
    import torch
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.gpu
def test_two_process_row_sharded_forward_backward():
    if not _two_gpus():
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", CHILD],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SHARDED OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.gpu
def test_two_threads_of_one_process():
    if not _two_gpus():
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, CHILD, "--threads"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SHARDED OK (threads)" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


@pytest.mark.gpu
def test_single_rank_shard_needs_no_nccl():
    """world == 1: the same entry points on one GPU, no communicator."""
    import torch
    from recpulse_b200 import sharded
    g = torch.Generator().manual_seed(3)
    m, k, n = 300, 256, 384
    A = (torch.randn(m, k, generator=g) / 16).to(torch.bfloat16); B = torch.randn(k, n, generator=g).to(torch.bfloat16)
    dC = torch.randn(m, n, generator=g).to(torch.bfloat16)
    op = sharded.RowShardedMatmul(B.cuda())
    c = op.forward(A.cuda()); da, db = op.backward(A.cuda(), dC.cuda())
    full = op.gather_output(c)
    torch.cuda.synchronize()
    rel = lambda x, ref: float((x.double().cpu() - ref).norm() / ref.norm())
    assert rel(c, A.double() @ B.double()) < 4e-3 and rel(da, dC.double() @ B.double().t()) < 4e-3
    assert rel(db, A.double().t() @ dC.double()) < 4e-3 and torch.equal(full, c)
    op.close()
