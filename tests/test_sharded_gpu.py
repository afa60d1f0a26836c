"""Row-sharded forward + backward on two real GPUs (NCCL), through the library's CUDA GEMMs.
Skipped on boxes with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, %r)
import torch, torch.distributed as dist
from recpulse_b200.sharded import RowShardedMatmul, row_partition
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
g = torch.Generator(device="cpu").manual_seed(11)
m, k, n = 1000, 512, 768
A = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16); B = torch.randn(k, n, generator=g).to(torch.bfloat16)
dC = torch.randn(m, n, generator=g).to(torch.bfloat16)
r0, r1 = row_partition(m, world, rank)
b_local = B.to(dev) if rank == 0 else torch.zeros(k, n, dtype=torch.bfloat16, device=dev)
op = RowShardedMatmul(b_local)
a_rows = A[r0:r1].to(dev); dc_rows = dC[r0:r1].to(dev)
c = op.forward(a_rows)
da, db = op.backward(a_rows, dc_rows)
torch.cuda.synchronize()
def rel(x, ref):
    return float((x.double().cpu() - ref).norm() / ref.norm())
Ad, Bd, Gd = A.double(), B.double(), dC.double()
errs = (rel(c, Ad[r0:r1] @ Bd), rel(da, Gd[r0:r1] @ Bd.t()), rel(db, Ad.t() @ Gd))
assert all(e < 1e-2 for e in errs), errs
m2 = 256 * world
A2 = torch.randn(m2, k, generator=g).to(torch.bfloat16)
s0, s1 = row_partition(m2, world, rank)
full = op.gather_output(op.forward(A2[s0:s1].to(dev)))
assert full.shape == (m2, n) and rel(full, A2.double() @ Bd) < 1e-2
dist.barrier()
if rank == 0:
    print("SHARDED OK", errs)
dist.destroy_process_group()
''' % ROOT


@pytest.mark.gpu
def test_two_gpu_row_sharded_forward_backward(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SHARDED OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
