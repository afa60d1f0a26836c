"""GPU parity of the raw GEMM entry points (rp_matmul, matmul_kernel_device, rp_matmul_ex)
against the CPU oracle, through the C ABI.  Sizes are kept where the oracle's naive loop
finishes in seconds; full-size workloads are covered by test_full_size_gpu.py."""
import ctypes as C
import os

import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib
from oracle import oracle as O
from helpers import CODE, check_close, f64, rand_operand

pytestmark = pytest.mark.gpu


UMMA = (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_SPLITK)


@pytest.fixture(scope="module")
def lib():
    lib = rpb.load()
    yield lib
    lib.rpb_force_kernel(0)
    assert lib.rpb_device_status(0) == 0


def dev(arr, dtype):
    return rpb.Tensor.from_numpy(np.ascontiguousarray(arr), dtype=dtype)


def store(logical, transposed, pad):
    """Lay a [..., r, c] array out in memory: optionally transposed storage, optionally padded rows.
    Returns (buffer, row_stride, col_stride, matrix_elems) with strides in elements of the LOGICAL matrix."""
    x = np.swapaxes(logical, -1, -2) if transposed else logical
    rows, cols = x.shape[-2:]
    ld = cols + pad
    buf = np.zeros(x.shape[:-1] + (ld,), x.dtype)
    buf[..., :cols] = x
    rs, cs = (1, ld) if transposed else (ld, 1)
    return buf, rs, cs, rows * ld


def run_ex(lib, dtype, a, b, ta=False, tb=False, pad_a=0, pad_b=0, c_init=None, expect=None, oracle=True, bias=None,
           gates=False):
    """a: [batch|1, reduce|1, m, k] bits, b: [batch|1, reduce|1, k, n] bits (size-1 dims broadcast)."""
    batch = max(a.shape[0], b.shape[0]); reduce = max(a.shape[1], b.shape[1])
    m, k = a.shape[2:]; n = b.shape[3]
    abuf, a_rs, a_cs, a_mat = store(a, ta, pad_a)
    bbuf, b_rs, b_cs, b_mat = store(b, tb, pad_b)
    g = rpb.RpbGemm()
    g.m, g.n, g.k, g.batch, g.reduce = m, n, k, batch, reduce
    g.a_row, g.a_col, g.b_row, g.b_col = a_rs, a_cs, b_rs, b_cs
    g.a_reduce = a_mat if a.shape[1] > 1 else 0
    g.a_batch = a_mat * a.shape[1] if a.shape[0] > 1 else 0
    g.b_reduce = b_mat if b.shape[1] > 1 else 0
    g.b_batch = b_mat * b.shape[1] if b.shape[0] > 1 else 0
    g.c_row, g.c_batch = n, m * n
    g.accumulate = int(c_init is not None)
    g.epilogue = 1 if gates else 0
    tbias = dev(bias, dtype) if bias is not None else None
    g.bias = tbias.data_ptr if tbias is not None else None
    ta_, tb_ = dev(abuf, dtype), dev(bbuf, dtype)
    c0 = c_init if c_init is not None else np.zeros((batch, m, n), O.storage(CODE[dtype]))
    tc = dev(c0, dtype)
    rc = lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta_.data_ptr), C.c_void_p(tb_.data_ptr), C.byref(g),
                          CODE[dtype], 0, None)
    assert rc == 0
    got = tc.to_numpy()
    if expect is not None:
        assert lib.rpb_last_kernel() in expect, lib.rpb_last_kernel()
    # reference: per batch, sum over the summed problems, unrounded, then one rounding
    a64 = np.broadcast_to(f64(a, dtype), (batch, reduce, m, k))
    b64 = np.broadcast_to(f64(b, dtype), (batch, reduce, k, n))
    ref64 = np.matmul(a64, b64).sum(axis=1)                     # BLAS per (batch, summed problem), then the sum
    if bias is not None:
        ref64 = ref64 + f64(bias, dtype)[None, None, :]
    if c_init is not None:
        ref64 = ref64 + f64(c_init, dtype)
    if gates:                                                   # LSTM gate epilogue: tanh on the third column quarter
        q = n // 4
        act = 1 / (1 + np.exp(-ref64)); act[..., 2 * q:3 * q] = np.tanh(ref64[..., 2 * q:3 * q])
        ref64 = act
    ref = O.narrow(ref64.astype(np.float32), CODE[dtype]) if dtype in ("float16", "bfloat16") else ref64.astype(
        O.storage(CODE[dtype]))
    check_close(got, ref, dtype, k * reduce, what=f"{dtype} m{m} k{k} n{n} b{batch} r{reduce} ta{ta} tb{tb}")
    if reduce == 1 and c_init is None and bias is None and oracle and not gates:
        # same-dtype reference of the path: the oracle's restatement of rp_matmul
        for bi in range(batch):
            o = O.rp_matmul(np.ascontiguousarray(a[min(bi, a.shape[0] - 1), 0]),
                            np.ascontiguousarray(b[min(bi, b.shape[0] - 1), 0]), CODE[dtype])
            check_close(got[bi], o, dtype, k, what=f"vs oracle {dtype} m{m} k{k} n{n}")
    return got


SHAPES_SMALL = [(1, 1, 1), (3, 4, 5), (1, 7, 1), (16, 32, 8), (33, 65, 17), (64, 64, 64), (100, 130, 70), (128, 784, 256)]


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", SHAPES_SMALL)
def test_simt_all_dtypes_all_layouts(lib, dtype, shape):
    lib.rpb_force_kernel(_lib.KERNEL_SIMT)
    m, k, n = shape
    rng = np.random.default_rng(1000 * CODE[dtype] + SHAPES_SMALL.index(shape))       # the same inputs in every process
    a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
    for ta, tb in [(False, False), (True, False), (False, True), (True, True)]:
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=3 if ta else 0, pad_b=5 if tb else 0, expect=(_lib.KERNEL_SIMT,))
    lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_simt_large_tile_and_splitk(lib, dtype):
    rng = np.random.default_rng(5)
    for (m, k, n) in [(512, 96, 640), (64, 2048, 64), (700, 300, 520)]:
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        run_ex(lib, dtype, a, b, expect=(_lib.KERNEL_SIMT, _lib.KERNEL_DMMA, _lib.KERNEL_TF32X3))


@pytest.mark.parametrize("layout", [(False, False), (True, False), (False, True), (True, True)])
def test_fp64_tensor_core_kernel(lib, layout):
    """mma.sync f64 kernel: all operand orientations, ragged and odd extents, long K (split over CTAs),
    batches, summed problems and the accumulate epilogue.  Leading dimensions stay even (16 bytes)."""
    ta, tb = layout
    dtype = "float64"
    rng = np.random.default_rng(43)
    for (m, k, n) in [(128, 16, 128), (256, 64, 384), (100, 130, 70), (129, 35, 131), (64, 2048, 64), (300, 17, 260)]:
        a = rand_operand(rng, (1, 1, m, k), dtype, dist="uniform"); b = rand_operand(rng, (1, 1, k, n), dtype, dist="uniform")
        pa = (m % 2) if ta else (k % 2)          # make the stored leading dimension even
        pb = (k % 2) if tb else (n % 2)
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=pa, pad_b=pb, expect=(_lib.KERNEL_DMMA,))
    a = rand_operand(rng, (3, 2, 96, 40), dtype); b = rand_operand(rng, (3, 2, 40, 72), dtype)
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=(_lib.KERNEL_DMMA,))
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, c_init=rand_operand(rng, (3, 96, 72), dtype), expect=(_lib.KERNEL_DMMA,))


@pytest.mark.parametrize("layout", [(False, False), (True, True)])
def test_fp64_balanced_schedule(lib, layout, monkeypatch):
    """More tiles than SMs with a sparse last wave: (tile, K block) units are dealt evenly to one CTA per SM and
    the tiles cut between two CTAs are summed by a fix-up kernel.  Ragged edges, batches, bias, C += AB; the
    result is reproducible and agrees with the one-CTA-per-tile schedule to rounding."""
    ta, tb = layout
    dtype = "float64"
    rng = np.random.default_rng(101)
    m, k, n = 1700, 300, 1500                       # 14 x 12 = 168 tiles of 128 x 128, 10 K blocks
    a = rand_operand(rng, (1, 1, m, k), dtype, dist="uniform"); b = rand_operand(rng, (1, 1, k, n), dtype, dist="uniform")
    got = run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=(_lib.KERNEL_DMMA,), oracle=False)
    again = run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=(_lib.KERNEL_DMMA,), oracle=False)
    assert np.array_equal(got, again)
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, oracle=False, bias=rand_operand(rng, (n,), dtype))
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, oracle=False, c_init=rand_operand(rng, (1, m, n), dtype))
    a2 = rand_operand(rng, (2, 2, 1100, 200), dtype); b2 = rand_operand(rng, (2, 2, 200, 1300), dtype)
    run_ex(lib, dtype, a2, b2, ta=ta, tb=tb, oracle=False)      # 2 x 99 tiles, 2 summed problems of 7 K blocks
    monkeypatch.setenv("RPB_DMMA_BALANCED", "0")
    plain = run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=(_lib.KERNEL_DMMA,), oracle=False)
    assert np.max(np.abs(plain - got)) <= 1e-12 * np.sqrt(k)


@pytest.mark.parametrize("layout", [(False, False), (True, False), (False, True), (True, True)])
def test_fp32_3xtf32_kernel(lib, layout):
    """float32 on tensor cores (3xTF32): must meet the same fp32 bound as the strict-fp32 reference,
    in every operand orientation, with ragged extents, K splits, batches and accumulation."""
    ta, tb = layout
    dtype = "float32"
    rng = np.random.default_rng(47)
    for (m, k, n) in [(64, 32, 64), (128, 784, 256), (64, 512, 2048), (100, 132, 68), (129, 37, 131), (32, 4096, 64),
                      (1500, 100, 1300)]:
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        pa = (-m % 4) if ta else (-k % 4)        # stored leading dimension a multiple of 4 floats
        pb = (-k % 4) if tb else (-n % 4)
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=pa, pad_b=pb, expect=(_lib.KERNEL_TF32X3,) + UMMA)
    a = rand_operand(rng, (3, 2, 96, 40), dtype); b = rand_operand(rng, (3, 2, 40, 72), dtype)
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=(_lib.KERNEL_TF32X3,))
    run_ex(lib, dtype, a, b, ta=ta, tb=tb, c_init=rand_operand(rng, (3, 96, 72), dtype), expect=(_lib.KERNEL_TF32X3,))


@pytest.mark.parametrize("layout", [(False, False), (True, False), (False, True), (True, True)])
def test_fp32_tcgen05_3xtf32_kernel(lib, layout):
    """float32 on tcgen05 (kind::tf32, hi/lo split in shared memory): one-CTA and two-CTA tiles, every
    operand orientation, ragged extents, K split, batches, summed problems, accumulate."""
    ta, tb = layout
    dtype = "float32"
    lib.rpb_force_kernel(_lib.KERNEL_UMMA)
    rng = np.random.default_rng(71)
    try:
        for (m, k, n) in [(128, 32, 128), (128, 784, 256), (64, 512, 2048), (100, 132, 68), (129, 36, 132), (64, 4096, 64),
                          (1500, 100, 1300), (512, 1024, 768), (2048, 512, 1024)]:
            a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
            pa = (-m % 4) if ta else (-k % 4)
            pb = (-k % 4) if tb else (-n % 4)
            run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=pa, pad_b=pb, expect=UMMA)
        a = rand_operand(rng, (3, 2, 96, 40), dtype); b = rand_operand(rng, (3, 2, 40, 72), dtype)
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=UMMA)
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, c_init=rand_operand(rng, (3, 96, 72), dtype), expect=UMMA)
    finally:
        lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_batch_reduce_accumulate_semantics(lib, dtype):
    rng = np.random.default_rng(11)
    m, k, n = 24, 40, 16
    a = rand_operand(rng, (3, 2, m, k), dtype); b = rand_operand(rng, (3, 2, k, n), dtype, scale=0.2)
    run_ex(lib, dtype, a, b)
    # broadcast B over the batch, and over the summed problems
    run_ex(lib, dtype, a, rand_operand(rng, (1, 1, k, n), dtype, scale=0.2))
    run_ex(lib, dtype, rand_operand(rng, (1, 2, m, k), dtype), b)
    c0 = rand_operand(rng, (3, m, n), dtype)
    run_ex(lib, dtype, a, b, c_init=c0)
    run_ex(lib, dtype, a, b, ta=True, tb=True, c_init=c0)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("layout", [(False, False), (True, False), (False, True), (True, True)])
def test_umma_layouts_and_ragged_edges(lib, dtype, layout):
    """All four operand-major combinations (forward NN, dA = dC.B^T, dB = A^T.dC, and both
    transposed), tile-aligned and ragged M/N/K.  Strides stay multiples of 8 elements (16 bytes)."""
    ta, tb = layout
    rng = np.random.default_rng(17)
    for (m, k, n) in [(128, 64, 256), (128, 128, 64), (256, 512, 512), (136, 200, 72), (8, 8, 8), (264, 72, 520),
                      (1000, 328, 136), (64, 512, 2048)]:
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=UMMA)
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=8, pad_b=16, expect=UMMA)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_umma_splitk_batch_reduce_accumulate(lib, dtype):
    rng = np.random.default_rng(23)
    # skinny, long K -> split over CTAs
    a = rand_operand(rng, (1, 1, 64, 4096), dtype); b = rand_operand(rng, (1, 1, 4096, 128), dtype, scale=1 / 64)
    run_ex(lib, dtype, a, b, expect=(_lib.KERNEL_UMMA_SPLITK,))
    run_ex(lib, dtype, a, b, ta=True, tb=False, expect=(_lib.KERNEL_UMMA_SPLITK,))
    c0 = rand_operand(rng, (1, 64, 128), dtype)
    run_ex(lib, dtype, a, b, c_init=c0, expect=(_lib.KERNEL_UMMA_SPLITK,))
    # batched, broadcast, summed problems, accumulate into C
    m, k, n = 72, 136, 200
    a = rand_operand(rng, (5, 3, m, k), dtype); b = rand_operand(rng, (5, 3, k, n), dtype, scale=0.1)
    run_ex(lib, dtype, a, b, expect=UMMA)
    run_ex(lib, dtype, a, b, ta=True, tb=True, expect=UMMA)
    run_ex(lib, dtype, a, rand_operand(rng, (1, 1, k, n), dtype, scale=0.1), expect=UMMA)
    run_ex(lib, dtype, rand_operand(rng, (1, 3, m, k), dtype), b, expect=UMMA)
    c0 = rand_operand(rng, (5, m, n), dtype)
    run_ex(lib, dtype, a, b, c_init=c0, expect=UMMA)
    # the broadcast-batched fp16 workload, reduced: A[16,512,64] x B[1,64,512]
    a = rand_operand(rng, (16, 1, 512, 64), dtype); b = rand_operand(rng, (1, 1, 64, 512), dtype, scale=1 / 8)
    run_ex(lib, dtype, a, b, expect=UMMA)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_umma_tail_split_and_bias(lib, dtype):
    """Tile counts just above one wave: the tiles of the sparse last wave are cut along K and summed by
    tail_reduce_kernel (with and without a bias); checked against a float64 product (the oracle's naive
    loop would take minutes at this size)."""
    rng = np.random.default_rng(73)
    for (m, k, n) in [(1280, 6144, 4096), (2304, 6400, 2104)]:     # >= 96 K blocks per tile: the tail split is on
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        if dtype == "float32":
            lib.rpb_force_kernel(_lib.KERNEL_UMMA)
        try:
            run_ex(lib, dtype, a, b, expect=UMMA, oracle=False)
            run_ex(lib, dtype, a, b, tb=True, expect=UMMA, oracle=False, bias=rand_operand(rng, (n,), dtype))
        finally:
            lib.rpb_force_kernel(0)


PLANS = ["64,1,0", "128,1,0", "256,1,0", "64,1,1", "128,1,1",          # every tile shape, unsplit
         "64,3,0", "128,2,0", "256,4,0", "64,2,1", "128,4,1"]          # and with K slices


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("plan", PLANS)
def test_every_tile_plan_gives_the_same_product(lib, dtype, plan, monkeypatch):
    """The planner picks among one-CTA tiles 128 x {64, 128, 256}, pair tiles 256 x {128, 256} and K slices;
    RPB_UMMA_PLAN pins each in turn.  Ragged M/N/K, both B orientations, plus bias (unsplit) and C += AB."""
    monkeypatch.setenv("RPB_UMMA_PLAN", plan)
    rng = np.random.default_rng(2000 + 100 * CODE[dtype] + PLANS.index(plan))          # the same inputs in every process
    m, k, n = 520, 1160, 776                       # ragged against every tile; 19 / 37 K blocks
    a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
    split = int(plan.split(",")[1]) > 1
    kinds = (_lib.KERNEL_UMMA_SPLITK,) if split else (_lib.KERNEL_UMMA,)
    lib.rpb_force_kernel(_lib.KERNEL_UMMA)         # float32 of this size would otherwise take the mma.sync kernel
    try:
        run_ex(lib, dtype, a, b, expect=kinds, oracle=False)
        run_ex(lib, dtype, a, b, tb=True, expect=kinds, oracle=False)
        run_ex(lib, dtype, a, b, ta=True, expect=kinds, oracle=False, bias=rand_operand(rng, (n,), dtype))
        run_ex(lib, dtype, a, b, c_init=rand_operand(rng, (1, m, n), dtype), expect=UMMA, oracle=False)
    finally:
        lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("plan", ["128,1,2", "128,3,2"])
def test_double_width_pair_tile(lib, dtype, plan, monkeypatch):
    """The 256 x 512 pair tile (two accumulators sharing the A tile; RPB_UMMA_PLAN's third field = 2), which the
    planner takes for large 16-bit problems.  K of one, three and many blocks (shorter than, between and beyond the
    lead of the first accumulator), ragged M/N/K with a last tile whose second accumulator is almost empty, every
    operand orientation, batches, bias, C += AB, float32 output; and the same bits as the 256 x 256 tile."""
    rng = np.random.default_rng(4100 + CODE[dtype] + len(plan) + int(plan[4]))
    split = int(plan.split(",")[1]) > 1
    kinds = (_lib.KERNEL_UMMA_SPLITK,) if split else (_lib.KERNEL_UMMA,)
    shapes = [(256, 64, 512), (768, 192, 1536), (520, 1160, 776), (1024, 4096, 1024)]
    for (m, k, n) in shapes:
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        outs = {}
        for pl in (plan, "128,%s,1" % plan.split(",")[1]):
            monkeypatch.setenv("RPB_UMMA_PLAN", pl)
            outs[pl] = [run_ex(lib, dtype, a, b, ta=ta, tb=tb, expect=kinds if k >= 256 or not split else None, oracle=(m <= 768))
                        for ta, tb in ((False, False), (True, False), (False, True), (True, True))]
        for x, y in zip(*outs.values()):
            assert np.array_equal(x, y), (m, k, n)
    monkeypatch.setenv("RPB_UMMA_PLAN", plan)
    m, k, n = 520, 1160, 776
    a = rand_operand(rng, (3, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
    run_ex(lib, dtype, a, b, expect=kinds, oracle=False)                                              # batched A, shared B
    run_ex(lib, dtype, a[:1], b, tb=True, expect=kinds, oracle=False, bias=rand_operand(rng, (n,), dtype))
    run_ex(lib, dtype, a[:1], b, c_init=rand_operand(rng, (1, m, n), dtype), expect=UMMA, oracle=False)   # register epilogue
    # float32 output of the unrounded sums
    ta_, tb_ = dev(a[0, 0], dtype), dev(b[0, 0], dtype)
    out = dev(np.full((m, n), np.nan, np.float32), "float32")
    g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n); g.c_float32 = 1
    assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta_.data_ptr), C.c_void_p(tb_.data_ptr), C.byref(g),
                            CODE[dtype], 0, None) == 0
    ref = f64(a[0, 0], dtype) @ f64(b[0, 0], dtype)
    got = out.to_numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-6 * np.sqrt(k) * np.sqrt(np.mean(ref * ref))
    assert lib.rpb_device_status(0) == 0


@pytest.mark.parametrize("plan", ["64,1,0", "128,1,1", "128,1,2"])
def test_rendezvous_of_the_ctas_changes_no_bit_and_cannot_hang(lib, plan, monkeypatch):
    """Launches of several waves of whole tiles keep their CTAs (pairs) in step with a counter they all wait on at
    tile starts and every few K blocks.  The product must be the same bits with and without it.  The wait is soft
    (a unit that has waited ~30 us switches it off for the launch), so two such launches on two streams at once --
    whose CTAs may keep one another from starting -- must both finish with the right bits and a clean status, and
    so must a launch replayed from a CUDA graph."""
    import torch
    dtype = "bfloat16"
    monkeypatch.setenv("RPB_UMMA_PLAN", plan)
    rng = np.random.default_rng(6100 + len(plan) + int(plan[0]))
    m, k, n = 4104, 328, 4232                       # 14+ waves of any tile shape, ragged edges, 6 K blocks
    a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
    ta, tb = dev(a, dtype), dev(b, dtype)
    g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)

    def run(tc, stream=None):
        assert lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                CODE[dtype], 0, C.c_void_p(stream) if stream else None) == 0
    blank = lambda: dev(np.zeros((m, n), np.uint16), dtype)
    outs = {}
    for setting in ("0", "-1", "-2", "-32"):        # off; tile starts only, every 2 / 32 K blocks (negative: short tiles too)
        monkeypatch.setenv("RPB_TILE_SYNC", setting)
        tc = blank(); run(tc)
        outs[setting] = tc.to_numpy()
        assert lib.rpb_device_status(0) == 0
    for setting in ("-1", "-2", "-32"):
        assert np.array_equal(outs[setting], outs["0"]), setting
    ref = f64(a, dtype) @ f64(b, dtype)
    check_close(outs["0"], O.narrow(ref.astype(np.float32), CODE[dtype]), dtype, k, f"plan {plan}")
    # two streams at once, several rounds
    monkeypatch.setenv("RPB_TILE_SYNC", "-2")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    c1, c2 = blank(), blank()
    torch.cuda.synchronize()
    for _ in range(4):
        run(c1, s1.cuda_stream); run(c2, s2.cuda_stream)
    torch.cuda.synchronize()
    assert lib.rpb_device_status(0) == 0
    assert np.array_equal(c1.to_numpy(), outs["0"]) and np.array_equal(c2.to_numpy(), outs["0"])
    # captured once, replayed three times (the counter is zeroed by a memset node of the graph)
    c3 = blank()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        run(c3, torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert lib.rpb_device_status(0) == 0
    assert np.array_equal(c3.to_numpy(), outs["0"])
    del graph
    assert lib.rpb_scratch_reset(0) == 0


def test_placement_aware_tile_order_changes_no_bit(lib, monkeypatch):
    """On a full grid of CTA pairs the library learns where the hardware places the clusters (the first such launch
    records every cluster's SM) and from then on deals the tiles of each wave so that the pairs of one GPC take a
    3 x 3 block of them.  Which pair computes a tile must not change a bit of it: launches before and after the
    permutation exists are compared with RPB_PLACE=0, ragged edges and a last wave that is not full included."""
    dtype = "bfloat16"
    rng = np.random.default_rng(7300)
    for (m, k, n) in ((16384, 264, 8192), (20000, 136, 6152)):       # 1024 and 948 double-width tiles, column groups of 6
        a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
        ta, tb = dev(a, dtype), dev(b, dtype)
        g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)

        def run():
            tc = dev(np.zeros((m, n), np.uint16), dtype)
            assert lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                    CODE[dtype], 0, None) == 0
            assert lib.rpb_last_kernel() == _lib.KERNEL_UMMA
            return tc.to_numpy()
        monkeypatch.setenv("RPB_PLACE", "0")
        plain = run()
        monkeypatch.delenv("RPB_PLACE")
        for _ in range(4):
            assert np.array_equal(run(), plain)
        ref = f64(a, dtype) @ f64(b, dtype)
        check_close(plain, O.narrow(ref.astype(np.float32), CODE[dtype]), dtype, k, f"{m}x{k}x{n}")
    assert lib.rpb_device_status(0) == 0


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_gate_epilogue_in_every_kernel_family(lib, dtype):
    """RpbGemm.epilogue = LSTM gates: applied inside the tcgen05 kernel's register epilogue when that writes C directly,
    and by one pass over C behind every other plan (mma.sync and general-stride kernels, K slices, balanced fp64
    schedule, packed operands); always after bias and "C += AB"."""
    rng = np.random.default_rng(131)
    cases = [((64, 512, 2048), None), ((128, 64, 1024), None), ((40, 36, 24), None), ((64, 4096, 64), None),
             ((1700, 300, 1500), None), ((520, 1160, 776), "128,2,0"), ((520, 1160, 776), "128,1,1")]
    for (m, k, n), plan in cases:
        if plan and dtype == "float64":
            continue
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        bias = rand_operand(rng, (n,), dtype); c0 = rand_operand(rng, (1, m, n), dtype)
        if plan:
            os.environ["RPB_UMMA_PLAN"] = plan
            lib.rpb_force_kernel(_lib.KERNEL_UMMA)
        try:
            run_ex(lib, dtype, a, b, gates=True)
            run_ex(lib, dtype, a, b, gates=True, bias=bias, c_init=c0)
            run_ex(lib, dtype, a, b, tb=True, gates=True, c_init=c0)
        finally:
            os.environ.pop("RPB_UMMA_PLAN", None)
            lib.rpb_force_kernel(0)
    lib.rpb_force_kernel(_lib.KERNEL_SIMT)
    a = rand_operand(rng, (2, 1, 33, 20), dtype); b = rand_operand(rng, (2, 1, 20, 16), dtype)
    run_ex(lib, dtype, a, b, gates=True, expect=(_lib.KERNEL_SIMT,))
    lib.rpb_force_kernel(0)
    g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), 4, 4, 6); g.epilogue = 1          # n % 4 != 0 is refused
    t = dev(np.zeros((4, 6), O.storage(CODE[dtype])), dtype)
    assert lib.rp_matmul_ex(C.c_void_p(t.data_ptr), C.c_void_p(t.data_ptr), C.c_void_p(t.data_ptr), C.byref(g), CODE[dtype], 0, None) == -1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "float64"])
def test_conv2d_gemm_loops_as_single_launches(lib, dtype):
    """conv2d in the reference multiplies per image (ops/ops.c:4761-4770 forward, :4536-4550 input gradient,
    :4575-4617 weight gradient with materialised transposes and an rp_add per image).  Through rp_matmul_ex each
    loop is ONE launch: the weight is a broadcast batch operand, transposes are stride swaps, and the weight
    gradient is a summed problem over the images."""
    rng = np.random.default_rng(151)
    n_img, c_out, ck, pix = 6, 40, 72, 96                  # images, output channels, C_in*kH*kW, out_H*out_W
    w = rand_operand(rng, (1, 1, c_out, ck), dtype, scale=1 / np.sqrt(ck))
    col = rand_operand(rng, (n_img, 1, ck, pix), dtype)
    gout = rand_operand(rng, (n_img, 1, c_out, pix), dtype)
    # forward: out[n] = W . col[n]
    run_ex(lib, dtype, w, col, oracle=False)
    # input gradient: dcol[n] = W^T . dout[n]  (W read transposed, no wt_buf)
    wt = np.ascontiguousarray(np.swapaxes(w, -1, -2))
    run_ex(lib, dtype, wt, gout, ta=True, oracle=False)
    # weight gradient: dW = sum_n dout[n] . col[n]^T  (col read transposed, images as summed problems, no col_t_buf)
    g_r = np.ascontiguousarray(np.swapaxes(gout, 0, 1)); colt_r = np.ascontiguousarray(np.swapaxes(np.swapaxes(col, -1, -2), 0, 1))
    run_ex(lib, dtype, g_r, colt_r, tb=True, oracle=False)
    # ... and accumulated into an existing weight gradient in the same epilogue (the reference's rp_add)
    run_ex(lib, dtype, g_r, colt_r, tb=True, oracle=False, c_init=rand_operand(rng, (1, c_out, ck), dtype))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_unaligned_half_operands_take_the_general_path(lib, dtype):
    rng = np.random.default_rng(29)
    a = rand_operand(rng, (1, 1, 33, 65), dtype); b = rand_operand(rng, (1, 1, 65, 17), dtype, scale=0.1)
    run_ex(lib, dtype, a, b, expect=(_lib.KERNEL_SIMT,))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_large_unaligned_half_operands_are_packed_for_the_tensor_cores(lib, dtype):
    """Odd leading dimensions (a vocabulary of 50257, a padded view) cannot be described to the TMA engine;
    above ~0.5 GFLOP the offending operands are packed once and the tcgen05 kernel still runs."""
    rng = np.random.default_rng(83)
    for (m, k, n, ta, tb, pa, pb) in [(520, 1001, 1003, False, False, 0, 0), (1000, 999, 520, True, True, 3, 5),
                                      (640, 1024, 1030, False, False, 0, 0)]:
        a = rand_operand(rng, (1, 1, m, k), dtype); b = rand_operand(rng, (1, 1, k, n), dtype, scale=1 / np.sqrt(k))
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=pa, pad_b=pb, expect=UMMA, oracle=False)
    # batched, summed problems, broadcast B, accumulate: the packed copies keep the batch structure
    a = rand_operand(rng, (3, 2, 300, 333), dtype); b = rand_operand(rng, (1, 2, 333, 520), dtype, scale=0.05)
    run_ex(lib, dtype, a, b, expect=UMMA, oracle=False)
    run_ex(lib, dtype, a, b, tb=True, c_init=rand_operand(rng, (3, 300, 520), dtype), expect=UMMA, oracle=False)


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_rp_matmul_and_matmul_kernel_device(lib, dtype):
    rng = np.random.default_rng(31)
    for (m, k, n) in [(2, 3, 2), (64, 512, 256), (128, 784, 256)]:
        a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
        ta, tb = dev(a, dtype), dev(b, dtype)
        tc = dev(np.zeros((m, n), O.storage(CODE[dtype])), dtype)
        args = (C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), m, k, n, CODE[dtype])
        assert lib.rp_matmul(*args, 0) == 0
        check_close(tc.to_numpy(), O.rp_matmul(a, b, CODE[dtype]), dtype, k, "rp_matmul")
        tc2 = dev(np.zeros((m, n), O.storage(CODE[dtype])), dtype)
        assert lib.matmul_kernel_device(C.c_void_p(tc2.data_ptr), *args[1:]) == 0
        assert np.array_equal(tc2.to_numpy(), tc.to_numpy())
    # reference tests/unit/test_functional.py:281-302 known answer
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3); b = np.arange(1, 7, dtype=np.float32).reshape(3, 2)
    ta, tb, tc = dev(a, "float32"), dev(b, "float32"), dev(np.zeros((2, 2), np.float32), "float32")
    assert lib.rp_matmul(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), 2, 3, 2, 0, 0) == 0
    assert np.array_equal(tc.to_numpy(), np.array([[22, 28], [49, 64]], np.float32))


def test_host_buffer_entry_point(lib):
    rng = np.random.default_rng(37)
    a = rand_operand(rng, (96, 160), "bfloat16"); b = rand_operand(rng, (160, 64), "bfloat16", scale=0.1)
    c = np.zeros((96, 64), np.uint16)
    assert lib.rp_matmul_host(c.ctypes.data_as(C.c_void_p), a.ctypes.data_as(C.c_void_p),
                              b.ctypes.data_as(C.c_void_p), 96, 160, 64, O.BF16, 0) == 0
    check_close(c, O.rp_matmul(a, b, O.BF16), "bfloat16", 160, "rp_matmul_host")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32", "float64"])
def test_streamed_host_forward_backward(lib, dtype):
    """rp_matmul_fwdbwd_host: row chunks streamed through three streams; ragged last chunk; optional outputs."""
    rng = np.random.default_rng(53)
    m, k, n = 1000, 136, 264
    a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
    dc = rand_operand(rng, (m, n), dtype)
    st = O.storage(CODE[dtype])
    c = np.zeros((m, n), st); da = np.zeros((m, k), st); db = np.zeros((k, n), st)
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    for chunk in (0, 256, 300, 4096):
        c[:] = 0; da[:] = 0; db[:] = 0
        assert lib.rp_matmul_fwdbwd_host(p(c), p(da), p(db), p(a), p(b), p(dc), m, k, n, CODE[dtype], 0, chunk) == 0
        check_close(c, O.rp_matmul(a, b, CODE[dtype]), dtype, k, f"C chunk={chunk}")
        oda, odb = O.matmul_backward(a, b, dc, CODE[dtype])
        check_close(da, oda, dtype, n, f"dA chunk={chunk}")
        check_close(db, odb, dtype, m, f"dB chunk={chunk}")
    # forward only, and backward-of-B only
    c[:] = 0
    assert lib.rp_matmul_fwdbwd_host(p(c), None, None, p(a), p(b), None, m, k, n, CODE[dtype], 0, 0) == 0
    check_close(c, O.rp_matmul(a, b, CODE[dtype]), dtype, k, "forward only")
    db[:] = 0
    assert lib.rp_matmul_fwdbwd_host(None, None, p(db), p(a), p(b), p(dc), m, k, n, CODE[dtype], 0, 0) == 0
    check_close(db, O.matmul_backward(a, b, dc, CODE[dtype])[1], dtype, m, "dB only")
    assert lib.rp_matmul_fwdbwd_host(None, None, p(db), p(a), p(b), None, m, k, n, CODE[dtype], 0, 0) == -1
    assert lib.rpb_release_host_pipeline(0) == 0


def test_results_do_not_depend_on_scheduling(lib):
    rng = np.random.default_rng(41)
    a = rand_operand(rng, (1, 1, 64, 4096), "bfloat16"); b = rand_operand(rng, (1, 1, 4096, 128), "bfloat16", scale=1 / 64)
    first = run_ex(lib, "bfloat16", a, b)
    for _ in range(3):
        assert np.array_equal(run_ex(lib, "bfloat16", a, b), first)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("plan", ["64,1,0", "128,1,0", "256,1,0", "64,1,1", "128,1,1"])
def test_balanced_schedule_gives_the_same_product(lib, dtype, plan, monkeypatch):
    """The balanced schedule deals tiles x K-blocks evenly over the CTAs (pairs): tiles are cut along K, the head
    piece goes through an fp32 scratch tile and the neighbour finishes it in its epilogue.  Forced here on ragged
    shapes with few SMs (max_sms), so that every CTA cuts tiles at both ends of its range, for every tile shape;
    checked against float64 and for run-to-run determinism."""
    monkeypatch.setenv("RPB_UMMA_PLAN", plan)
    monkeypatch.setenv("RPB_BALANCED", "2")
    rng = np.random.default_rng(3000 + 100 * CODE[dtype] + PLANS.index(plan))
    lib.rpb_force_kernel(_lib.KERNEL_UMMA)
    try:
        for (m, k, n, sms) in [(1000, 1160, 1544, 6), (1300, 2056, 1100, 20), (2048, 1024, 2048, 14)]:
            a = rand_operand(rng, (m, k), dtype, scale=1 / np.sqrt(k)); b = rand_operand(rng, (k, n), dtype)
            bias = rand_operand(rng, (n,), dtype)
            ref = f64(a, dtype) @ f64(b, dtype) + f64(bias, dtype)
            ta, tb, tbias = dev(a, dtype), dev(b, dtype), dev(bias, dtype)
            outs = []
            for trial in range(2):
                tc = dev(np.zeros((m, n), O.storage(CODE[dtype])), dtype)
                g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)
                g.max_sms = sms; g.bias = tbias.data_ptr
                assert lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                        CODE[dtype], 0, None) == 0
                assert lib.rpb_last_kernel() == _lib.KERNEL_UMMA
                outs.append(tc.to_numpy())
            assert np.array_equal(outs[0], outs[1])
            got = f64(outs[0], dtype)
            if dtype == "float32":      # the path's float32 bound: max |err| / (sqrt(K) rms)
                err = np.abs(got - ref).max() / (np.sqrt(k) * np.sqrt(np.mean(ref * ref)))
                assert err <= 1e-5, (m, k, n, sms, err)
            else:
                err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
                assert err <= {"bfloat16": 4e-3, "float16": 6e-4}[dtype], (m, k, n, sms, err)
        # transposed operands (the backward GEMMs' layouts) on the balanced path
        m, k, n = 1536, 1280, 1024
        at = rand_operand(rng, (k, m), dtype, scale=1 / np.sqrt(k)); bt = rand_operand(rng, (n, k), dtype)
        ref = f64(at, dtype).T @ f64(bt, dtype).T
        tc = dev(np.zeros((m, n), O.storage(CODE[dtype])), dtype); ta, tb = dev(at, dtype), dev(bt, dtype)
        g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)
        g.a_row, g.a_col, g.b_row, g.b_col, g.max_sms = 1, m, 1, k, 10
        assert lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g), CODE[dtype], 0, None) == 0
        got = f64(tc.to_numpy(), dtype)
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= {"bfloat16": 4e-3, "float16": 6e-4, "float32": 2e-5}[dtype]
    finally:
        lib.rpb_force_kernel(0)
    assert lib.rpb_device_status(0) == 0


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_two_slice_tail_is_finished_inside_the_kernel(lib, dtype):
    """A last wave that fills between a quarter and a half of the CTA pairs: its tiles are cut into TWO K slices that
    run side by side, and per epilogue warp the slice that arrives second adds the first one's fp32 sums and writes
    C (no reduction launch).  Ragged M, N and K, with a bias; float64 reference; identical bits on every run although
    the arrival order is not fixed."""
    rng = np.random.default_rng(91)
    m, k, n = 2000, 6200, 3300                       # 8 x 13 = 104 tiles of 256 x 256 on 74 pairs: 30 tail tiles
    a = rand_operand(rng, (m, k), dtype, scale=1 / np.sqrt(k)); b = rand_operand(rng, (k, n), dtype)
    bias = rand_operand(rng, (n,), dtype)
    pad = (-n) % 8
    bp = np.zeros((k, n + pad), b.dtype); bp[:, :n] = b          # row stride a multiple of 16 bytes
    ref = f64(a, dtype) @ f64(b, dtype) + f64(bias, dtype)
    ap = np.zeros((m, k + (-k) % 8), a.dtype); ap[:, :k] = a
    ta, tb, tbias = dev(ap, dtype), dev(bp, dtype), dev(bias, dtype)
    if dtype == "float32":
        lib.rpb_force_kernel(_lib.KERNEL_UMMA)
    try:
        outs = []
        for trial in range(3):
            tc = dev(np.zeros((m, n + pad), O.storage(CODE[dtype])), dtype)
            g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)
            g.a_row = ap.shape[1]; g.b_row = n + pad; g.c_row = n + pad; g.bias = tbias.data_ptr
            before = lib.rpb_launch_count()
            assert lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                    CODE[dtype], 0, None) == 0
            assert lib.rpb_last_kernel() == _lib.KERNEL_UMMA
            if dtype != "float32":                     # the float32 planner may choose another tile shape
                assert lib.rpb_launch_count() - before == 1, "the tail was not finished inside the GEMM kernel"
            outs.append(tc.to_numpy()[:, :n])
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
        got = f64(outs[0], dtype)
        if dtype == "float32":
            assert np.abs(got - ref).max() / (np.sqrt(k) * np.sqrt(np.mean(ref * ref))) <= 1e-5
        else:
            assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= {"bfloat16": 4e-3, "float16": 6e-4}[dtype]
    finally:
        lib.rpb_force_kernel(0)
    assert lib.rpb_device_status(0) == 0
