"""The oracle (oracle/matmul_oracle.c) pinned against the reference.

Three pins: known-answer vectors from the reference's own tests, fixtures made
by the unmodified reference (tests/golden/make_golden.py), and -- when the
compiled reference is present -- the reference's ``rp_matmul`` called directly.
"""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as O

CODE = {"float32": O.F32, "float64": O.F64, "float16": O.F16, "bfloat16": O.BF16}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _views(case):
    m, k, n, ta, tb, twice = [int(v) for v in case["meta"]]
    a = case["a"].T if ta else case["a"]
    b = case["b"].T if tb else case["b"]
    return a, b, case["w"], twice


def test_golden_cases_present(golden):
    assert len(golden) == 44
    assert {d for (_, d) in golden} == set(CODE)


@pytest.mark.parametrize("dtype", list(CODE))
def test_forward_bit_exact_vs_reference_fixtures(golden, dtype):
    for (name, dt), case in golden.items():
        if dt != dtype:
            continue
        a, b, w, _ = _views(case)
        c = O.op_matmul(a, b, CODE[dtype])
        assert np.array_equal(c, case["c"]), name


@pytest.mark.parametrize("dtype", list(CODE))
def test_backward_bit_exact_vs_reference_fixtures(golden, dtype):
    for (name, dt), case in golden.items():
        if dt != dtype:
            continue
        a, b, w, twice = _views(case)
        da, db = O.matmul_backward(a, b, w, CODE[dtype])
        if twice:   # second pass accumulates into the first (ops.c:6781-6789)
            da, db = O.matmul_backward(a, b, w, CODE[dtype], acc_da=da, acc_db=db)
        m, k, n, ta, tb, _ = [int(v) for v in case["meta"]]
        # the reference stores the grad of a transposed *view* on the leaf, i.e. in
        # the leaf's own layout: d(leaf) = (d view)^T
        exp_da = case["da"].T if ta else case["da"]
        exp_db = case["db"].T if tb else case["db"]
        assert np.array_equal(da, exp_da), name
        assert np.array_equal(db, exp_db), name


def test_known_answers_from_reference_tests():
    # tests/unit/test_functional.py:281-302 (fp32 2x3 . 3x2 and identity)
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    b = np.arange(1, 7, dtype=np.float32).reshape(3, 2)
    assert np.array_equal(O.rp_matmul(a, b, O.F32), np.array([[22, 28], [49, 64]], np.float32))
    eye = np.eye(3, dtype=np.float32)
    assert np.array_equal(O.rp_matmul(a, eye, O.F32), a)
    # tests/autograd/test_matmul_autograd.py:14-120 (fp64; dA = 1.B^T, dB = A^T.1)
    a64 = np.arange(1, 7, dtype=np.float64).reshape(2, 3)
    b64 = np.array([1, 0, 0, 1, 1, 0], np.float64).reshape(3, 2)
    ones = np.ones((2, 2))
    da, db = O.matmul_backward(a64, b64, ones, O.F64)
    assert np.abs(da - ones @ b64.T).max() < 1e-10
    assert np.abs(db - a64.T @ ones).max() < 1e-10
    # non-square 2x4 . 4x3 (test_matmul_autograd.py:230-287)
    a = np.arange(8, dtype=np.float64).reshape(2, 4); b = np.arange(12, dtype=np.float64).reshape(4, 3)
    assert np.abs(O.rp_matmul(a, b, O.F64) - a @ b).max() < 1e-10


@pytest.mark.parametrize("shape", [(3, 4, 5), (16, 32, 8), (1, 7, 1), (64, 64, 64)])
def test_fp64_vs_numpy_like_reference_stress(shape):
    # tests/stress/stress_torch_parity.py:86-95 tolerances
    m, k, n = shape
    rng = np.random.default_rng(1)
    a = rng.uniform(-1, 1, (m, k)); b = rng.uniform(-1, 1, (k, n))
    np.testing.assert_allclose(O.rp_matmul(a, b, O.F64), a @ b, rtol=1e-9, atol=1e-10)


def test_half_rounding_is_half_up_not_rne():
    lib = O.lib()
    # 1 + 2^-8 sits exactly between two bf16 values; RNE -> 0x3F80, half-up -> 0x3F81
    assert lib.orc_fp32_to_bf16(1.00390625) == 0x3F81
    # 1 + 2^-11 is the fp16 tie; half-up -> 0x3C01
    assert lib.orc_fp32_to_fp16(1.00048828125) == 0x3C01
    for h in (0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0xFBFF, 0x8000, 0x7C00):
        assert lib.orc_fp32_to_fp16(lib.orc_fp16_to_fp32(h)) == h
    for h in (0x0001, 0x0080, 0x3F80, 0x7F7F, 0xFF7F, 0x8000, 0x7F80):
        assert lib.orc_fp32_to_bf16(lib.orc_bf16_to_fp32(h)) == h


def test_bmm_broadcast_definition():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((4, 5, 6)).astype(np.float32)
    b = rng.standard_normal((1, 6, 7)).astype(np.float32)
    dc = rng.standard_normal((4, 5, 7)).astype(np.float32)
    c = O.bmm(a, b, O.F32)
    for i in range(4):
        assert np.array_equal(c[i], O.rp_matmul(a[i], b[0], O.F32))
    da, db = O.bmm_backward(a, b, dc, O.F32)
    assert da.shape == a.shape and db.shape == b.shape
    np.testing.assert_allclose(db[0], np.einsum("bmk,bmn->kn", a, dc), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(da, np.einsum("bmn,kn->bmk", dc, b[0]), rtol=1e-4, atol=1e-5)
    # halves: one rounding at the end of the batch sum
    ah = O.narrow(a, O.F16); bh = O.narrow(b, O.F16); dh = O.narrow(dc, O.F16)
    _, dbh = O.bmm_backward(ah, bh, dh, O.F16)
    ref = np.einsum("bmk,bmn->kn", O.to_f64(ah, O.F16), O.to_f64(dh, O.F16))
    assert np.abs(O.to_f64(dbh, O.F16)[0] - ref).max() <= 2.0 ** -10 * np.abs(ref).max() * 1.01


def test_against_compiled_reference_rp_matmul():
    so = os.path.join(ROOT, "oracle", "_ref", "recpulse_cuda.so")
    if not os.path.exists(so):
        pytest.skip("compiled reference not present")
    # importing python first resolves the extension's libpython symbols
    ref = ctypes.CDLL(so, mode=ctypes.RTLD_LOCAL)
    ref.rp_matmul.restype = ctypes.c_int
    rng = np.random.default_rng(7)
    for dtype in (O.F32, O.F64, O.F16, O.BF16):
        for (m, k, n) in [(5, 9, 4), (31, 257, 19), (128, 784, 16)]:
            a = O.narrow(rng.standard_normal((m, k)), dtype)
            b = O.narrow(rng.uniform(-1, 1, (k, n)) / np.sqrt(k), dtype)
            exp = np.empty((m, n), O.storage(dtype))
            rc = ref.rp_matmul(exp.ctypes.data_as(ctypes.c_void_p), a.ctypes.data_as(ctypes.c_void_p),
                               b.ctypes.data_as(ctypes.c_void_p), m, k, n, dtype, -1)
            assert rc == 0
            assert np.array_equal(O.rp_matmul(a, b, dtype), exp), (dtype, m, k, n)


@pytest.mark.parametrize("dtype", list(CODE))
def test_linear_composition_bit_exact_vs_reference_fixtures(linear_golden, dtype):
    """x @ W + b and its three gradients as the reference composes them (module.py:110-114)."""
    seen = 0
    for (name, dt), case in linear_golden.items():
        if dt != dtype:
            continue
        seen += 1
        code = CODE[dtype]
        assert np.array_equal(O.linear_forward(case["x"], case["w"], case["b"], code), case["y"]), name
        dx, dw = O.matmul_backward(case["x"], case["w"], case["g"], code)
        assert np.array_equal(dx, case["dx"]) and np.array_equal(dw, case["dw"]), name
        assert np.array_equal(O.bias_grad(case["g"], code), case["db"]), name
    assert seen == 3


@pytest.mark.parametrize("dtype", list(CODE))
def test_lstm_gates_composition_bit_exact_vs_reference_fixtures(lstm_gates_golden, dtype):
    """The gate block of LSTMCell.forward (module.py:289-300) and its five gradients, as run by the reference:
    forward, then dY -> gradient of the pre-activations -> the two matmul backwards and the bias gradient."""
    seen = 0
    for (name, dt), case in lstm_gates_golden.items():
        if dt != dtype:
            continue
        seen += 1
        code = CODE[dtype]
        y = O.lstm_gates_forward(case["x"], case["w"], case["h"], case["u"], case["b"], code)
        assert np.array_equal(y, case["y"]), name
        dpre = O.lstm_gates_grad(case["g"], case["y"], code)
        dx, dw = O.matmul_backward(case["x"], case["w"], dpre, code)
        dh, du = O.matmul_backward(case["h"], case["u"], dpre, code)
        assert np.array_equal(dx, case["dx"]) and np.array_equal(dw, case["dw"]), name
        assert np.array_equal(dh, case["dh"]) and np.array_equal(du, case["du"]), name
        assert np.array_equal(O.bias_grad(dpre, code), case["db"]), name
    assert seen == 3


@pytest.mark.parametrize("dtype", list(CODE))
def test_gru_cell_composition_bit_exact_vs_reference_fixtures(gru_cell_golden, dtype):
    """GRUCell.forward (recpulse/module.py:329-348) op by op, and its backward to all six leaves, against the
    unmodified reference's own run: every bit of h' and of every gradient."""
    code = CODE[dtype]
    seen = 0
    for (name, dt), case in gru_cell_golden.items():
        if dt != dtype:
            continue
        seen += 1
        bi, bh = case.get("bi"), case.get("bh")
        hn = O.gru_cell_forward(case["x"], case["wi"], case["h"], case["wh"], bi, bh, code)
        assert np.array_equal(hn, case["hn"]), name
        dx, dwi, dh, dwh, dbi, dbh = O.gru_cell_backward(case["g"], case["x"], case["wi"], case["h"], case["wh"], bi, bh, code)
        for got, key in ((dx, "dx"), (dwi, "dwi"), (dh, "dh"), (dwh, "dwh")):
            assert np.array_equal(got, case[key]), (name, key)
        if bi is not None:
            assert np.array_equal(dbi, case["dbi"]) and np.array_equal(dbh, case["dbh"]), name
    assert seen == 4


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_conv2d_restatement_bit_exact_vs_reference_fixtures(conv2d_golden, dtype):
    """op_conv2d + backward (ops/ops.c:4480-4770: per-image im2col, rp_matmul, col2im, rp_add) against the
    unmodified reference's CPU run.  float32 / float64: the reference's host conv2d does not handle the 16-bit types."""
    code = CODE[dtype]
    seen = 0
    for (name, dt), case in conv2d_golden.items():
        if dt != dtype:
            continue
        seen += 1
        mt = [int(v) for v in case["meta"]]
        st, pd, dl = tuple(mt[7:9]), tuple(mt[9:11]), tuple(mt[11:13])
        assert np.array_equal(O.conv2d_forward(case["x"], case["w"], st, pd, dl, code), case["y"]), name
        dx, dw = O.conv2d_backward(case["x"], case["w"], case["g"], st, pd, dl, code)
        assert np.array_equal(dx, case["dx"]) and np.array_equal(dw, case["dw"]), name
    assert seen == 4
