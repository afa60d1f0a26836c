"""Host side of the sharded path on two CPU ranks (gloo): what a launcher does before any GPU work --
the rendezvous id reaches every rank unchanged, the ranks' row spans and dB slices (computed by the
library's own arithmetic, rpb_shard_rows / rpb_shard_db_slice_of) tile the problem, and the entry points
refuse bad arguments and a box without a GPU instead of falling back to anything."""
import ctypes as C
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BF16, F32 = 3, 0


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    from recpulse_b200 import sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    uid = sharded.exchange_unique_id(make=lambda: bytes(range(128)))     # rank 0's bytes, everywhere
    rows = sharded.row_partition(37, world, rank)                        # rows do not divide evenly
    big = sharded.db_slice(8192, 8192, BF16, world, rank)                # reduce-scattered: a slice each
    small = sharded.db_slice(64, 512, BF16, world, rank)                 # below 1 MiB: all-reduced, everything
    f32 = sharded.db_slice(8192, 8192, F32, world, rank)                 # float32 operands: all-reduced in place
    whole = sharded.db_slice(8192, 8192, BF16, world, rank, flags=0)     # all-gathered afterwards
    q.put((rank, uid, rows, big, small, f32, whole))
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


def test_db_slices_tile_the_gradient():
    sys.path.insert(0, ROOT)
    from recpulse_b200.sharded import db_slice
    for world in (2, 4, 8):
        spans = [db_slice(8192, 8192, BF16, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 8192 * 8192
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    # three ranks do not divide 1024 x 1000 into 16-byte multiples: no slicing
    assert db_slice(1024, 1000, BF16, 3, 1) == (0, 1024 * 1000)
    # the operand-type wire never slices
    assert db_slice(8192, 8192, BF16, 8, 3, db_wire=1) == (0, 8192 * 8192)
    with pytest.raises(ValueError):
        db_slice(0, 8, BF16, 2, 0)


def test_two_rank_rendezvous_and_partition_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, uid0, rows0, big0, small0, f0, w0), (_, uid1, rows1, big1, small1, f1, w1) = results
    assert uid0 == uid1 == bytes(range(128))
    assert rows0 == (0, 19) and rows1 == (19, 37)
    assert big0 == (0, 8192 * 4096) and big1 == (8192 * 4096, 8192 * 8192)
    assert small0 == small1 == (0, 64 * 512)
    assert f0 == f1 == w0 == w1 == (0, 8192 * 8192)


def test_shard_entry_points_refuse_bad_arguments_and_missing_gpus():
    sys.path.insert(0, ROOT)
    import recpulse_b200 as rpb
    lib = rpb.load()
    uid = bytes(128)
    assert not lib.rpb_shard_create(uid, 2, 2, 0)          # rank outside the world
    assert not lib.rpb_shard_create(None, 0, 2, 0)         # several ranks need an id
    assert not lib.rpb_shard_create(uid, 0, 1, -1)         # host "device"
    if not torch.cuda.is_available():
        assert not lib.rpb_shard_create(None, 0, 1, 0)     # no GPU: no shard, and no CPU stand-in
    buf = C.c_void_p(0)
    assert lib.rp_matmul_rowsharded_forward(None, buf, buf, buf, 4, 4, 4, BF16, None) == -1
    assert lib.rp_matmul_rowsharded_backward(None, buf, buf, buf, buf, buf, 4, 4, 4, BF16, 0, None) == -1
    assert lib.rp_matmul_gather_rows(None, buf, buf, 4, 4, BF16, None) == -1
    assert lib.rp_shard_replicate(None, buf, 16, 0, None) == -1
    assert lib.rp_matmul_rowsharded_fwdbwd_host(None, buf, buf, buf, buf, buf, buf, 4, 4, 4, BF16, 0, None, None) == -1
    assert lib.rpb_shard_rank(None) == -1 and lib.rpb_shard_world(None) == -1


def test_python_caller_refuses_cpu_tensors():
    sys.path.insert(0, ROOT)
    from recpulse_b200.sharded import RowShardedMatmul
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        RowShardedMatmul(torch.zeros(2, 2))
