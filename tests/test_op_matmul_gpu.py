"""GPU parity of op_matmul + backward_matmul_fn (the autograd node) through the C ABI,
against fixtures produced by the unmodified reference and against the oracle."""
import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib
from oracle import oracle as O
from helpers import CODE, check_close, rand_operand

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = rpb.load()
    yield lib
    lib.rpb_force_kernel(0)
    assert lib.rpb_device_status(0) == 0


def T(bits, dtype, grad=False):
    return rpb.Tensor.from_numpy(np.ascontiguousarray(bits), dtype=dtype, requires_grad=grad)


@pytest.mark.parametrize("family", [_lib.KERNEL_SIMT, 0])
@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_reference_fixtures_forward_backward(lib, golden, dtype, family):
    lib.rpb_force_kernel(family)
    for (name, dt), case in golden.items():
        if dt != dtype:
            continue
        m, k, n, ta, tb, twice = [int(v) for v in case["meta"]]
        a = T(case["a"], dtype, grad=True); b = T(case["b"], dtype, grad=True); w = T(case["w"], dtype)
        av = a.transpose(0, 1) if ta else a                 # views collect their own grads
        bv = b.transpose(0, 1) if tb else b
        y = av.op_matmul(bv)
        assert y.shape == (m, n) and y.dtype == dtype
        check_close(y.to_numpy(), case["c"], dtype, k, f"{name} fwd")
        y.backward(w)
        if twice:
            y2 = av.op_matmul(bv)
            y2.backward(w)                                  # accumulates into the existing grads
        da = av.grad.to_numpy(); db = bv.grad.to_numpy()
        # fixtures hold the leaf-layout grads; the gradient of a transposed view is their transpose
        exp_da = case["da"].T if ta else case["da"]; exp_db = case["db"].T if tb else case["db"]
        check_close(da, exp_da, dtype, n, f"{name} dA")
        check_close(db, exp_db, dtype, m, f"{name} dB")
    lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16", "float64"])
def test_mlp_and_lstm_gate_shapes(lib, dtype):
    """The float32 MLP-layer GEMM X[128,784].W[784,256] and the LSTM gate GEMM H[64,512].W[512,2048],
    the latter also with W given as the stride-swapped view of a [2048,512] buffer."""
    rng = np.random.default_rng(0)
    for (m, k, n, tview) in [(128, 784, 256, False), (64, 512, 2048, False), (64, 512, 2048, True)]:
        x = rand_operand(rng, (m, k), dtype)
        w = O.narrow(rng.uniform(-1, 1, (k, n)) / np.sqrt(k), CODE[dtype])
        dy = rand_operand(rng, (m, n), dtype)
        X = T(x, dtype, grad=True)
        if tview:
            Wbuf = T(np.ascontiguousarray(w.T), dtype, grad=True)
            W = Wbuf.transpose(0, 1)
        else:
            W = T(w, dtype, grad=True)
        y = X.op_matmul(W)
        check_close(y.to_numpy(), O.rp_matmul(x, w, CODE[dtype]), dtype, k, "fwd")
        y.backward(T(dy, dtype))
        da, db = O.matmul_backward(x, w, dy, CODE[dtype])
        check_close(X.grad.to_numpy(), da, dtype, n, "dX")
        gw = W.grad.to_numpy()
        check_close(gw, db, dtype, m, "dW")


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
def test_batched_and_broadcast_batched(lib, dtype):
    rng = np.random.default_rng(4)
    # A[8,512,64] x B[1,64,512] (broadcast over the batch); dB is summed over the batch
    a = rand_operand(rng, (8, 96, 64), dtype); b = rand_operand(rng, (1, 64, 128), dtype, scale=1 / 8)
    dc = rand_operand(rng, (8, 96, 128), dtype)
    A = T(a, dtype, grad=True); B = T(b, dtype, grad=True)
    y = A.op_matmul(B)
    assert y.shape == (8, 96, 128)
    check_close(y.to_numpy(), O.bmm(a, b, CODE[dtype]), dtype, 64, "bmm fwd")
    y.backward(T(dc, dtype))
    da, db = O.bmm_backward(a, b, dc, CODE[dtype])
    check_close(A.grad.to_numpy(), da, dtype, 128, "bmm dA")
    assert B.grad.shape == (1, 64, 128)
    check_close(B.grad.to_numpy(), db, dtype, 8 * 96, "bmm dB (summed over batch)")
    # 2-D weight against a 3-D batch (Linear applied to [batch, seq, features])
    b2 = rand_operand(rng, (64, 128), dtype, scale=1 / 8)
    A = T(a, dtype, grad=True); B = T(b2, dtype, grad=True)
    y = A.op_matmul(B)
    check_close(y.to_numpy(), O.bmm(a, b2[None], CODE[dtype]), dtype, 64, "3d x 2d fwd")
    y.backward(T(dc, dtype))
    da, db = O.bmm_backward(a, b2[None], dc, CODE[dtype])
    assert B.grad.shape == (64, 128)
    check_close(B.grad.to_numpy(), db[0], dtype, 8 * 96, "3d x 2d dB")
    # both batched, two leading dims, one of them broadcast in A
    a4 = rand_operand(rng, (1, 3, 40, 24), dtype); b4 = rand_operand(rng, (2, 3, 24, 32), dtype, scale=0.2)
    dc4 = rand_operand(rng, (2, 3, 40, 32), dtype)
    A = T(a4, dtype, grad=True); B = T(b4, dtype, grad=True)
    y = A.op_matmul(B)
    assert y.shape == (2, 3, 40, 32)
    from helpers import f64
    ref = np.einsum("xymk,xykn->xymn", np.broadcast_to(f64(a4, dtype), (2, 3, 40, 24)), f64(b4, dtype))
    assert np.linalg.norm(f64(y.to_numpy(), dtype) - ref) / np.linalg.norm(ref) < {"float32": 1e-5, "float16": 2e-3, "bfloat16": 1e-2}[dtype]
    y.backward(T(dc4, dtype))
    ref_da = np.einsum("xymn,xykn->ymk", f64(dc4, dtype), f64(b4, dtype))[None]
    ref_db = np.einsum("ymk,xymn->xykn", f64(a4, dtype)[0], f64(dc4, dtype))
    got_da = f64(A.grad.to_numpy(), dtype); got_db = f64(B.grad.to_numpy(), dtype)
    assert A.grad.shape == (1, 3, 40, 24) and B.grad.shape == (2, 3, 24, 32)
    tol = {"float32": 1e-5, "float16": 2e-3, "bfloat16": 1e-2}[dtype]
    assert np.linalg.norm(got_da - ref_da) / np.linalg.norm(ref_da) < tol
    assert np.linalg.norm(got_db - ref_db) / np.linalg.norm(ref_db) < tol


def test_errors_match_reference_behaviour(lib):
    a = T(np.zeros((2, 3), np.float32), "float32"); b = T(np.zeros((4, 5), np.float32), "float32")
    with pytest.raises(RuntimeError, match="op_matmul operation failed"):
        a.op_matmul(b)                                       # stress_edge_cases.py:41-42
    b64 = T(np.zeros((3, 5), np.float64), "float64")
    with pytest.raises(RuntimeError):
        a.op_matmul(b64)
    v = T(np.zeros((3,), np.float32), "float32")
    with pytest.raises(RuntimeError):
        v.op_matmul(b)


def test_no_grad_no_node_and_refcounts(lib):
    a = T(np.ones((4, 4), np.float32), "float32"); b = T(np.ones((4, 4), np.float32), "float32")
    y = a.op_matmul(b)
    assert not y._t.metadata                                 # ops.c:6851: node only if an input requires grad
    assert np.array_equal(y.to_numpy(), np.full((4, 4), 4, np.float32))
    a = T(np.ones((4, 4), np.float32), "float32", grad=True)
    before = (a._t.refcount, b._t.refcount)
    y = a.op_matmul(b)
    assert y._t.metadata and y._t.metadata.contents.requires_grad and not y._t.metadata.contents.is_leaf
    assert (a._t.refcount, b._t.refcount) == (before[0] + 1, before[1] + 1)   # grad_fn_attach retains inputs
    y.backward(T(np.ones((4, 4), np.float32), "float32"))
    assert (a._t.refcount, b._t.refcount) == before          # node freed, inputs released
    assert a.grad is not None and b.grad is None             # only inputs that require grad get one
    assert np.array_equal(a.grad.to_numpy(), np.full((4, 4), 4, np.float32))


@pytest.mark.parametrize("family", [_lib.KERNEL_SIMT, 0])
@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_linear_node_vs_reference_fixtures(lib, linear_golden, dtype, family):
    """op_linear (bias in the GEMM epilogue, bias gradient on the device) against the reference's
    op_matmul + op_add composition."""
    lib.rpb_force_kernel(family)
    for (name, dt), case in linear_golden.items():
        if dt != dtype:
            continue
        m, k = case["x"].shape; n = case["w"].shape[1]
        x = T(case["x"], dtype, True); w = T(case["w"], dtype, True); b = T(case["b"], dtype, True)
        y = x.op_linear(w, b)
        check_close(y.to_numpy(), case["y"], dtype, k, f"{name} y")
        y.backward(T(case["g"], dtype))
        check_close(x.grad.to_numpy(), case["dx"], dtype, n, f"{name} dx")
        check_close(w.grad.to_numpy(), case["dw"], dtype, m, f"{name} dw")
        assert b.grad.shape == (n,)
        check_close(b.grad.to_numpy(), case["db"], dtype, m, f"{name} dbias")
    lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_linear_node_larger_shapes_and_accumulation(lib, dtype):
    rng = np.random.default_rng(61)
    for lead, k, n in [((512,), 256, 384), ((4, 96), 64, 128), ((1000,), 136, 264), ((64,), 4096, 136)]:
        x = rand_operand(rng, lead + (k,), dtype); w = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
        b = rand_operand(rng, (n,), dtype); g = rand_operand(rng, lead + (n,), dtype)
        X = T(x, dtype, True); W = T(w, dtype, True); B = T(b, dtype, True)
        y = X.op_linear(W, B)
        assert y.shape == lead + (n,)
        check_close(y.to_numpy(), O.linear_forward(x, w, b, CODE[dtype]), dtype, k, "y")
        y.backward(T(g, dtype))
        rows = int(np.prod(lead))
        check_close(B.grad.to_numpy(), O.bias_grad(g, CODE[dtype]), dtype, rows, "dbias")
        dx, dw = O.matmul_backward(x.reshape(rows, k), w, g.reshape(rows, n), CODE[dtype])
        check_close(X.grad.to_numpy().reshape(rows, k), dx, dtype, n, "dx")
        check_close(W.grad.to_numpy(), dw, dtype, rows, "dw")
        # a second use of the same parameters accumulates into the existing grads (weight sharing)
        y2 = X.op_linear(W, B)
        y2.backward(T(g, dtype))
        from helpers import f64
        got = f64(B.grad.to_numpy(), dtype); ref = 2 * f64(O.bias_grad(g, CODE[dtype]), dtype)
        tol = {"float32": 1e-5, "float64": 1e-12, "float16": 2e-3, "bfloat16": 1e-2}[dtype]
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < tol
    # bias of the wrong length or dtype is rejected
    with pytest.raises(RuntimeError):
        T(x, dtype).op_linear(T(w, dtype), T(rand_operand(rng, (n + 1,), dtype), dtype))


def test_colsum_entry_point(lib):
    import ctypes as C
    rng = np.random.default_rng(67)
    for dtype in ("float32", "bfloat16", "float64"):
        for rows, cols, pad in [(1, 5, 0), (33, 70, 2), (5000, 130, 6), (70000, 64, 0)]:
            x = rand_operand(rng, (rows, cols + pad), dtype)
            tin = T(x, dtype); tout = T(np.zeros((cols,), O.storage(CODE[dtype])), dtype)
            assert lib.rp_colsum_ex(C.c_void_p(tout.data_ptr), C.c_void_p(tin.data_ptr), rows, cols, cols + pad, CODE[dtype],
                                    0, 0, None) == 0
            check_close(tout.to_numpy(), O.bias_grad(np.ascontiguousarray(x[:, :cols]), CODE[dtype]), dtype, rows, "colsum")


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_gate_node_two_products_one_output(lib, dtype):
    """op_linear2: x.W_ih + h.W_hh + b as one node (LSTMCell / GRUCell gate pre-activations,
    recpulse/module.py:289, 334-335), against the reference composition matmul, matmul, add, add."""
    from helpers import f64
    rng = np.random.default_rng(79)
    for (bsz, e, hdim, n) in [(64, 64, 256, 1024), (5, 24, 40, 72), (128, 512, 512, 2048)]:
        x = rand_operand(rng, (bsz, e), dtype); w = rand_operand(rng, (e, n), dtype, scale=1 / np.sqrt(e))
        h = rand_operand(rng, (bsz, hdim), dtype); u = rand_operand(rng, (hdim, n), dtype, scale=1 / np.sqrt(hdim))
        b = rand_operand(rng, (n,), dtype); g = rand_operand(rng, (bsz, n), dtype)
        X, W, H, U, B = (T(v, dtype, True) for v in (x, w, h, u, b))
        y = X.op_linear2(W, H, U, B)
        assert y.shape == (bsz, n)
        ref = f64(x, dtype) @ f64(w, dtype) + f64(h, dtype) @ f64(u, dtype) + f64(b, dtype)
        got = f64(y.to_numpy(), dtype)
        tol = {"float32": 2e-6, "float64": 1e-13, "float16": 1e-3, "bfloat16": 6e-3}[dtype]
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < tol
        # the reference's own composition (each op rounds to the storage dtype) is no closer to the exact result
        comp = O.linear_forward(x, w, np.zeros_like(b), CODE[dtype])
        y.backward(T(g, dtype))
        dx, dw = O.matmul_backward(x, w, g, CODE[dtype]); dh, du = O.matmul_backward(h, u, g, CODE[dtype])
        check_close(X.grad.to_numpy(), dx, dtype, n, "dx"); check_close(W.grad.to_numpy(), dw, dtype, bsz, "dw")
        check_close(H.grad.to_numpy(), dh, dtype, n, "dh"); check_close(U.grad.to_numpy(), du, dtype, bsz, "du")
        check_close(B.grad.to_numpy(), O.bias_grad(g, CODE[dtype]), dtype, bsz, "dbias")
        del comp
    with pytest.raises(RuntimeError):
        T(x, dtype).op_linear2(T(w, dtype), T(h, dtype), T(rand_operand(rng, (hdim, n + 8), dtype), dtype))


@pytest.mark.parametrize("family", [_lib.KERNEL_SIMT, 0])
@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_lstm_gates_node_vs_reference_fixtures(lib, lstm_gates_golden, dtype, family):
    """op_lstm_gates against the reference's own run of LSTMCell's gate block (matmul, matmul, add, add, chunk,
    sigmoid / tanh) and of its backward down to all five leaves."""
    lib.rpb_force_kernel(family)
    try:
        for (name, dt), case in lstm_gates_golden.items():
            if dt != dtype:
                continue
            m, kx = case["x"].shape; kh = case["h"].shape[1]; n = case["w"].shape[1]
            x = T(case["x"], dtype, True); w = T(case["w"], dtype, True); h = T(case["h"], dtype, True)
            u = T(case["u"], dtype, True); b = T(case["b"], dtype, True)
            y = x.op_lstm_gates(w, h, u, b)
            check_close(y.to_numpy(), case["y"], dtype, kx + kh, f"{name} y", tight=False)
            y.backward(T(case["g"], dtype))
            check_close(x.grad.to_numpy(), case["dx"], dtype, n, f"{name} dx", tight=False)
            check_close(w.grad.to_numpy(), case["dw"], dtype, m, f"{name} dw", tight=False)
            check_close(h.grad.to_numpy(), case["dh"], dtype, n, f"{name} dh", tight=False)
            check_close(u.grad.to_numpy(), case["du"], dtype, m, f"{name} du", tight=False)
            check_close(b.grad.to_numpy(), case["db"], dtype, m, f"{name} dbias", tight=False)
    finally:
        lib.rpb_force_kernel(0)


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_lstm_gates_node_cell_sizes(lib, dtype):
    """LSTM cell sizes (batch 64 / 128, hidden 256 / 512) against the oracle's restatement of the composition;
    no bias as well; a column count that is not a multiple of 4 is refused."""
    rng = np.random.default_rng(83)
    for (bsz, e, hdim, bias) in [(64, 64, 256, True), (128, 512, 512, True), (33, 40, 24, False)]:
        n = 4 * hdim
        x = rand_operand(rng, (bsz, e), dtype); w = rand_operand(rng, (e, n), dtype, scale=1 / np.sqrt(e))
        h = rand_operand(rng, (bsz, hdim), dtype); u = rand_operand(rng, (hdim, n), dtype, scale=1 / np.sqrt(hdim))
        b = rand_operand(rng, (n,), dtype) if bias else None
        g = rand_operand(rng, (bsz, n), dtype)
        X = T(x, dtype, True); W = T(w, dtype, True); H = T(h, dtype, True); U = T(u, dtype, True)
        B = T(b, dtype, True) if bias else None
        y = X.op_lstm_gates(W, H, U, B)
        ref_y = O.lstm_gates_forward(x, w, h, u, b, CODE[dtype])
        check_close(y.to_numpy(), ref_y, dtype, e + hdim, "gates")
        got_y = y.to_numpy()
        y.backward(T(g, dtype))
        dpre = O.lstm_gates_grad(g, got_y, CODE[dtype])          # from the node's own output: isolates the backward
        dx, dw = O.matmul_backward(x, w, dpre, CODE[dtype])
        dh, du = O.matmul_backward(h, u, dpre, CODE[dtype])
        check_close(X.grad.to_numpy(), dx, dtype, n, "dx"); check_close(W.grad.to_numpy(), dw, dtype, bsz, "dw")
        check_close(H.grad.to_numpy(), dh, dtype, n, "dh"); check_close(U.grad.to_numpy(), du, dtype, bsz, "du")
        if bias:
            check_close(B.grad.to_numpy(), O.bias_grad(dpre, CODE[dtype]), dtype, bsz, "dbias")
    with pytest.raises(RuntimeError):
        T(x, dtype).op_lstm_gates(T(rand_operand(rng, (x.shape[1], 6), dtype), dtype), T(h, dtype),
                                  T(rand_operand(rng, (h.shape[1], 6), dtype), dtype))


def test_lstm_gate_passes_on_strided_rows(lib):
    """rp_lstm_gates_ex / rp_lstm_gates_grad_ex on matrices whose rows are further apart than n."""
    import ctypes as C
    rng = np.random.default_rng(89)
    for dtype in ("float32", "bfloat16", "float64"):
        rows, n, pad = 37, 24, 8
        pre = rand_operand(rng, (rows, n + pad), dtype); g = rand_operand(rng, (rows, n + pad), dtype)
        t = T(pre, dtype)
        assert lib.rp_lstm_gates_ex(C.c_void_p(t.data_ptr), rows, n, n + pad, CODE[dtype], 0, None) == 0
        out = t.to_numpy()
        from helpers import f64
        p64 = f64(pre, dtype)[:, :n]
        ref = 1 / (1 + np.exp(-p64)); ref[:, n // 2:3 * n // 4] = np.tanh(p64[:, n // 2:3 * n // 4])
        tol = {"float32": 1e-6, "float64": 1e-14, "bfloat16": 8e-3}[dtype]
        assert np.max(np.abs(f64(out, dtype)[:, :n] - ref)) < tol
        assert np.array_equal(out[:, n:], pre[:, n:])              # the padding is not touched
        tg = T(g, dtype); td = T(np.zeros((rows, n), O.storage(CODE[dtype])), dtype)
        assert lib.rp_lstm_gates_grad_ex(C.c_void_p(td.data_ptr), C.c_void_p(tg.data_ptr), C.c_void_p(t.data_ptr), rows, n,
                                         n, n + pad, n + pad, CODE[dtype], 0, None) == 0
        exp = O.lstm_gates_grad(np.ascontiguousarray(g[:, :n]), np.ascontiguousarray(out[:, :n]), CODE[dtype])
        check_close(td.to_numpy(), exp, dtype, 1, "gate grad")
        assert lib.rp_lstm_gates_ex(C.c_void_p(t.data_ptr), rows, 6, 8, CODE[dtype], 0, None) == -1   # n % 4 != 0
