"""Parity at the full sizes of the benchmark workloads, where the oracle's naive loop cannot run the
whole product: sampled rows / columns against the oracle, plus size-independent identities that touch
every output tile (column sums of C, linearity of the accumulate epilogue)."""
import ctypes as C

import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib
from oracle import oracle as O
from helpers import CODE, check_close, f64, rand_operand

pytestmark = pytest.mark.gpu


def T(bits, dtype, grad=False):
    return rpb.Tensor.from_numpy(np.ascontiguousarray(bits), dtype=dtype, requires_grad=grad)


def fwd_bwd(a, b, dc, dtype):
    A = T(a, dtype, True); B = T(b, dtype, True)
    y = A.op_matmul(B)
    kern = rpb.load().rpb_last_kernel()
    y.backward(T(dc, dtype))
    return y.to_numpy(), A.grad.to_numpy(), B.grad.to_numpy(), kern


def sampled_check(a, b, dc, c, da, db, dtype, rng, rows=3):
    m, k = a.shape; n = b.shape[1]
    code = CODE[dtype]
    ri = rng.choice(m, rows, replace=False)
    # C[rows] = A[rows] . B ; dA[rows] = dC[rows] . B^T
    check_close(c[ri], O.rp_matmul(a[ri], b, code), dtype, k, "C rows")
    check_close(da[ri], O.rp_matmul(dc[ri], np.ascontiguousarray(b.T), code), dtype, n, "dA rows")
    # dB[cols of A] = A[:, cols]^T . dC
    ci = rng.choice(k, rows, replace=False)
    check_close(db[ci], O.rp_matmul(np.ascontiguousarray(a[:, ci].T), dc, code), dtype, m, "dB rows")


def column_sum_identity(a, b, c, dtype, tol):
    """1^T C = (1^T A) B: every tile of C contributes.  The rounding noise of M summed outputs is about
    2^-8/sqrt(12) * sqrt(M) * rms(C) per column (4-5 sigma over thousands of columns stays below 2e-2 of
    sqrt(M) * rms(C)); one wrong 128-row tile would show up at ~0.1."""
    lhs = f64(c, dtype).sum(axis=0)
    rhs = f64(a, dtype).sum(axis=0) @ f64(b, dtype)
    scale = np.sqrt(a.shape[0]) * np.sqrt(np.mean(f64(c, dtype) ** 2))
    assert np.abs(lhs - rhs).max() / scale < tol


def test_bf16_square_4096():
    dtype = "bfloat16"; rng = np.random.default_rng(0)
    a = rand_operand(rng, (4096, 4096), dtype, scale=1 / 64); b = rand_operand(rng, (4096, 4096), dtype, scale=1 / 64)
    dc = rand_operand(rng, (4096, 4096), dtype)
    c, da, db, kern = fwd_bwd(a, b, dc, dtype)
    assert kern in (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_SPLITK)
    sampled_check(a, b, dc, c, da, db, dtype, rng)
    column_sum_identity(a, b, c, dtype, 2e-2)
    column_sum_identity(dc, np.ascontiguousarray(b.T), da, dtype, 2e-2)


def test_bf16_row_shard_8192():
    """One rank's share of the row-sharded 65536 x 8192 x 8192 GEMM at 8 GPUs."""
    dtype = "bfloat16"; rng = np.random.default_rng(1)
    a = rand_operand(rng, (8192, 8192), dtype, scale=1 / np.sqrt(8192)); b = rand_operand(rng, (8192, 8192), dtype)
    dc = rand_operand(rng, (8192, 8192), dtype)
    c, da, db, kern = fwd_bwd(a, b, dc, dtype)
    assert kern == _lib.KERNEL_UMMA
    sampled_check(a, b, dc, c, da, db, dtype, rng, rows=2)
    column_sum_identity(a, b, c, dtype, 2e-2)
    column_sum_identity(np.ascontiguousarray(a.T), dc, db, dtype, 2e-2)


def test_fp16_broadcast_batched_full():
    """A[64,512,64] x B[1,64,512] -> C[64,512,512]; dB summed over the batch.  Small enough for the
    oracle to run in full."""
    dtype = "float16"; rng = np.random.default_rng(2)
    a = rand_operand(rng, (64, 512, 64), dtype); b = rand_operand(rng, (1, 64, 512), dtype, scale=1 / 8)
    dc = rand_operand(rng, (64, 512, 512), dtype)
    c, da, db, kern = fwd_bwd(a, b, dc, dtype)
    assert c.shape == (64, 512, 512) and da.shape == a.shape and db.shape == b.shape
    check_close(c, O.bmm(a, b, CODE[dtype]), dtype, 64, "bmm C")
    oda, odb = O.bmm_backward(a, b, dc, CODE[dtype])
    check_close(da, oda, dtype, 512, "bmm dA")
    check_close(db, odb, dtype, 64 * 512, "bmm dB")


def test_fp64_2048():
    dtype = "float64"; rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (2048, 2048)); b = rng.uniform(-1, 1, (2048, 2048)); dc = rng.uniform(-1, 1, (2048, 2048))
    c, da, db, _ = fwd_bwd(a, b, dc, dtype)
    sampled_check(a, b, dc, c, da, db, dtype, rng, rows=4)
    # against numpy's fp64 product for the whole matrices (independent summation order)
    for got, ref in ((c, a @ b), (da, dc @ b.T), (db, a.T @ dc)):
        rms = np.sqrt(np.mean(ref ** 2))
        assert (np.abs(got - ref) / np.maximum(np.abs(ref), rms)).max() <= 1e-12


def test_fp32_mlp_and_lstm_full():
    """The two float32 workloads in full (the oracle finishes them in about a second)."""
    dtype = "float32"; rng = np.random.default_rng(0)
    for (m, k, n) in [(128, 784, 256), (64, 512, 2048)]:
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = rng.uniform(-1 / np.sqrt(k), 1 / np.sqrt(k), (k, n)).astype(np.float32)
        dy = rng.standard_normal((m, n)).astype(np.float32)
        c, da, db, _ = fwd_bwd(x, w, dy, dtype)
        check_close(c, O.rp_matmul(x, w, O.F32), dtype, k, "C")
        oda, odb = O.matmul_backward(x, w, dy, O.F32)
        check_close(da, oda, dtype, n, "dX"); check_close(db, odb, dtype, m, "dW")
        # the other reading of "normalised by sqrt(K)": max|err| / (sqrt(K) max|A| max|B|)
        assert np.abs(c - O.rp_matmul(x, w, O.F32)).max() / (np.sqrt(k) * np.abs(x).max() * np.abs(w).max()) <= 1e-5


def test_accumulate_is_linear_at_full_size():
    """C = A.B twice with accumulate equals 2 A.B up to one rounding: exercises the '+= C' epilogue on
    every tile of a large output."""
    dtype = "bfloat16"; rng = np.random.default_rng(5)
    lib = rpb.load()
    m, k, n = 2048, 1024, 4096
    a = rand_operand(rng, (m, k), dtype, scale=1 / 32); b = rand_operand(rng, (k, n), dtype)
    ta, tb = T(a, dtype), T(b, dtype)
    out1 = T(np.zeros((m, n), np.uint16), dtype); out2 = T(np.zeros((m, n), np.uint16), dtype)
    g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)
    args = lambda o: (C.c_void_p(o.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g), CODE[dtype], 0, None)
    assert lib.rp_matmul_ex(*args(out1)) == 0
    assert lib.rp_matmul_ex(*args(out2)) == 0
    g.accumulate = 1
    assert lib.rp_matmul_ex(*args(out2)) == 0
    x1 = f64(out1.to_numpy(), dtype); x2 = f64(out2.to_numpy(), dtype)
    assert np.linalg.norm(x2 - 2 * x1) / np.linalg.norm(2 * x1) < 4e-3
    assert lib.rpb_device_status(0) == 0


def test_bf16_row_sharded_65536_full():
    """The benchmark's own shape on one GPU: 65536 x 8192 x 8192 forward + backward through rp_matmul_ex.  512 row
    tiles per column group, A and C larger than 2^31 bytes' worth of offsets, 256 two-CTA tile rows.  Inputs are
    generated on the device (the bits that are checked are copied back, so both sides see the same values);
    sampled rows of C and dA against the oracle, sampled entries of dB against float64, and the three column-sum
    identities over every tile."""
    import torch
    dtype = "bfloat16"
    lib = rpb.load()
    m, k, n = 65536, 8192, 8192
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    A = (torch.randn((m, k), generator=gen, device="cuda") / np.sqrt(k)).to(torch.bfloat16)
    B = torch.randn((k, n), generator=gen, device="cuda").to(torch.bfloat16)
    dC = torch.randn((m, n), generator=gen, device="cuda").to(torch.bfloat16)
    Cc = torch.empty((m, n), device="cuda", dtype=torch.bfloat16); dA = torch.empty_like(A); dB = torch.empty_like(B)

    def gemm(c, a, b, mm, kk, nn, a_strides, b_strides):
        g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), mm, kk, nn)
        g.a_row, g.a_col = a_strides; g.b_row, g.b_col = b_strides
        assert lib.rp_matmul_ex(C.c_void_p(c.data_ptr()), C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.byref(g),
                                CODE[dtype], 0, None) == 0
        assert lib.rpb_last_kernel() == _lib.KERNEL_UMMA
    gemm(Cc, A, B, m, k, n, (k, 1), (n, 1))
    gemm(dA, dC, B, m, n, k, (n, 1), (1, n))            # B^T through swapped strides
    gemm(dB, A, dC, k, m, n, (1, k), (n, 1))            # A^T through swapped strides
    torch.cuda.synchronize()
    assert lib.rpb_device_status(0) == 0
    bits = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    rng = np.random.default_rng(9)
    # rows from the first tile, the last tile and past the 2^31-byte offset of A and C
    ri = np.array([5, 40000, m - 1])
    idx = torch.as_tensor(ri, device="cuda")
    b_bits = bits(B)
    check_close(bits(Cc[idx]), O.rp_matmul(bits(A[idx]), b_bits, CODE[dtype]), dtype, k, "C rows")
    check_close(bits(dA[idx]), O.rp_matmul(bits(dC[idx]), np.ascontiguousarray(b_bits.T), CODE[dtype]), dtype, n, "dA rows")
    ii = torch.as_tensor(rng.integers(0, k, 64), device="cuda"); jj = torch.as_tensor(rng.integers(0, n, 64), device="cuda")
    want = (A[:, ii].double() * dC[:, jj].double()).sum(dim=0)
    got = dB[ii, jj].double()
    assert float((got - want).norm() / want.norm()) <= 4e-3
    colsum = lambda t: t.sum(dim=0, dtype=torch.float64)
    rms = lambda t: float(t.float().pow(2).mean().sqrt())
    Bd = B.double()
    assert float((colsum(Cc) - colsum(A) @ Bd).abs().max()) / (np.sqrt(m) * rms(Cc)) < 2e-2
    assert float((colsum(dA) - colsum(dC) @ Bd.t()).abs().max()) / (np.sqrt(m) * rms(dA)) < 2e-2
    rs = dC.sum(dim=1, dtype=torch.float64)
    rhs = torch.zeros(k, device="cuda", dtype=torch.float64)
    for s in range(0, m, 4096):
        rhs += A[s:s + 4096].double().t() @ rs[s:s + 4096]
    assert float((dB.sum(dim=1, dtype=torch.float64) - rhs).abs().max()) / (np.sqrt(n) * rms(dB)) < 2e-2
