"""One rank of the two-GPU test of the sharded entry points (launched by tests/test_sharded_gpu.py with
torch.distributed.run, or as threads of one process with --threads).  torch.distributed (gloo) only carries
the 128-byte rendezvous id; every collective on the data path is issued by the library."""
import ctypes as C
import os
import sys
import threading

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from recpulse_b200 import _lib, sharded  # noqa: E402


def rel(x, ref):
    return float((x.double().cpu() - ref).norm() / ref.norm())


def run_rank(rank, world, uid, log):
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(11)
    m, k, n = 1000, 512, 768                       # rows do not divide evenly; dB is 1.5 MiB in float32
    A = (torch.randn(m, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    B = torch.randn(k, n, generator=g).to(torch.bfloat16)
    dC = torch.randn(m, n, generator=g).to(torch.bfloat16)
    Ad, Bd, Gd = A.double(), B.double(), dC.double()
    r0, r1 = sharded.row_partition(m, world, rank)
    b_local = B.to(dev) if rank == 0 else torch.zeros(k, n, dtype=torch.bfloat16, device=dev)
    op = sharded.RowShardedMatmul(b_local, rank=rank, world=world, unique_id=uid)
    torch.cuda.synchronize(dev)
    assert torch.equal(op.b.cpu(), B), "B was not replicated"
    a_rows = A[r0:r1].to(dev); dc_rows = dC[r0:r1].to(dev)
    before = lib.rpb_shard_collective_count()
    c = op.forward(a_rows)
    da, db = op.backward(a_rows, dc_rows)
    torch.cuda.synchronize(dev)
    assert lib.rpb_shard_collective_count() > before, "no collective was issued by the library"
    db_ref = Ad.t() @ Gd
    errs = (rel(c, Ad[r0:r1] @ Bd), rel(da, Gd[r0:r1] @ Bd.t()), rel(db, db_ref))
    assert all(e < 4e-3 for e in errs), errs
    # dB was summed in float32 and rounded once: most elements are exactly the rounded float64 sum,
    # and none is further than one bfloat16 step from it
    exact = db_ref.to(torch.bfloat16)
    same = float((db.cpu() == exact).double().mean())
    assert same > 0.98, same
    assert float(((db.double().cpu() - db_ref).abs() / db_ref.abs().clamp_min(1e-3)).max()) < 2 ** -7
    # reduce-scattered only: this rank's slice equals the same elements of the gathered result
    db2 = torch.full_like(db, float("nan"))
    op.backward(a_rows, dc_rows, db_out=db2, flags=sharded.SLICE_ONLY)
    torch.cuda.synchronize(dev)
    s0, s1 = sharded.db_slice(k, n, _lib.BF16, world, rank)
    assert (s1 - s0) * world == k * n
    assert torch.equal(db2.flatten()[s0:s1].cpu(), db.flatten()[s0:s1].cpu())
    # the operand-type wire (one all-reduce in bfloat16) stays inside the path's tolerance too
    lib.rpb_shard_configure(op.handle, 16, 1)
    _, db3 = op.backward(a_rows, dc_rows)
    torch.cuda.synchronize(dev)
    assert rel(db3, db_ref) < 1e-2
    lib.rpb_shard_configure(op.handle, 16, 0)
    # small dB (float32 all-reduce route) and float32 operands (all-reduced in place)
    k2, n2 = 64, 512
    A2 = torch.randn(m, k2, generator=g).to(torch.float16); G2 = torch.randn(m, n2, generator=g).to(torch.float16)
    B2 = (torch.randn(k2, n2, generator=g) / 8).to(torch.float16)
    op2 = sharded.RowShardedMatmul(B2.to(dev), rank=rank, world=world, unique_id=None if world == 1 else uid2[0])
    _, db4 = op2.backward(A2[r0:r1].to(dev), G2[r0:r1].to(dev))
    torch.cuda.synchronize(dev)
    assert rel(db4, A2.double().t() @ G2.double()) < 6e-4
    # all-gather of C for callers that want it everywhere
    mg = 256 * world
    Ag = torch.randn(mg, k, generator=g).to(torch.bfloat16)
    t0, t1 = sharded.row_partition(mg, world, rank)
    full = op.gather_output(op.forward(Ag[t0:t1].to(dev)))
    torch.cuda.synchronize(dev)
    assert full.shape == (mg, n) and rel(full, Ag.double() @ Bd) < 4e-3
    # the same step from host buffers: B from rank 0's host memory only, dB back as one slice per rank
    rows = r1 - r0
    hA = A[r0:r1].contiguous().pin_memory(); hG = dC[r0:r1].contiguous().pin_memory()
    hB = B.contiguous().pin_memory() if rank == 0 else None
    hC = torch.empty(rows, n, dtype=torch.bfloat16).pin_memory(); hdA = torch.empty(rows, k, dtype=torch.bfloat16).pin_memory()
    hdB = torch.full((k, n), float("nan"), dtype=torch.bfloat16).pin_memory()
    b0, b1 = C.c_longlong(), C.c_longlong()
    p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
    rc = lib.rp_matmul_rowsharded_fwdbwd_host(op.handle, p(hC), p(hdA), p(hdB), p(hA), p(hB), p(hG), rows, k, n, _lib.BF16, 256,
                                              C.byref(b0), C.byref(b1))
    assert rc == 0 and (b0.value, b1.value) == (s0, s1)
    assert rel(hC, Ad[r0:r1] @ Bd) < 4e-3 and rel(hdA, Gd[r0:r1] @ Bd.t()) < 4e-3
    assert torch.equal(hdB.flatten()[s0:s1], db.flatten()[s0:s1].cpu())
    assert lib.rpb_device_status(rank) == 0
    op2.close(); op.close()
    log.append((rank, errs))


uid2 = [None]


def main():
    if "--threads" in sys.argv:
        # one process, one thread per GPU: the form a single RecPulse process would use
        world = 2
        lib = _lib.load()
        ids = []
        for _ in range(2):
            buf = C.create_string_buffer(128)
            assert lib.rpb_shard_unique_id(buf) == 0
            ids.append(buf.raw)
        uid2[0] = ids[1]
        log, errors = [], []

        def guarded(r):
            try:
                run_rank(r, world, ids[0], log)
            except BaseException as e:          # noqa: BLE001
                errors.append((r, repr(e)))
        threads = [threading.Thread(target=guarded, args=(r,)) for r in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        assert not errors and len(log) == world, (errors, log)
        print("SHARDED OK (threads)", sorted(log))
        return
    import torch.distributed as dist
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    uid = sharded.exchange_unique_id()
    uid2[0] = sharded.exchange_unique_id()
    log = []
    run_rank(rank, world, uid, log)
    dist.barrier()
    if rank == 0:
        print("SHARDED OK", log)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
