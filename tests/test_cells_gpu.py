"""The callers next to the matmul path: the GRU cell as one node, conv2d as im2col + single GEMM launches, and the
kernels' bounded wait exercised by itself."""
import ctypes as C

import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib
from oracle import oracle as O
from helpers import CODE, check_close, f64, rand_operand

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    lib = rpb.load()
    yield lib
    lib.rpb_force_kernel(0)
    assert lib.rpb_device_status(0) == 0


def T(bits, dtype, grad=False):
    return rpb.Tensor.from_numpy(np.ascontiguousarray(bits), dtype=dtype, requires_grad=grad)


def chain_close(got, ref, exact, dtype, k, what):
    """For results behind a CHAIN of nodes.  float32 / float64: the path's bound against the reference.  16-bit types:
    the reference rounds after every one of its dozen nodes, this library once per stored tensor, so on a handful of
    elements the two can differ by more than 1e-2 while both sit inside 1e-2 of the exact (float64) chain; accepted
    is 1e-2 against the reference, or -- where the reference itself is that far from exact -- 1e-2 against the exact
    chain for both."""
    if dtype in ("float32", "float64"):
        return check_close(got, ref, dtype, k, what, tight=False)
    g, r = f64(got, dtype), f64(ref, dtype)
    rel = lambda a, b: float(np.linalg.norm(a - b) / (np.linalg.norm(b) or 1.0))
    if rel(g, r) <= 1e-2:
        return
    assert rel(g, exact) <= 1e-2 and rel(r, exact) <= 1e-2, (what, rel(g, r), rel(g, exact), rel(r, exact))


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_gru_cell_node_vs_reference_fixtures(lib, gru_cell_golden, dtype):
    """op_gru_cell against the reference's own run of GRUCell.forward and its backward down to all six leaves."""
    for (name, dt), case in gru_cell_golden.items():
        if dt != dtype:
            continue
        m, kx, hidden, bias = [int(v) for v in case["meta"]]
        x = T(case["x"], dtype, True); wi = T(case["wi"], dtype, True); h = T(case["h"], dtype, True); wh = T(case["wh"], dtype, True)
        bi = T(case["bi"], dtype, True) if bias else None; bh = T(case["bh"], dtype, True) if bias else None
        hn = x.op_gru_cell(wi, h, wh, bi, bh)
        assert hn.shape == (m, hidden)
        w64 = lambda key: f64(case[key], dtype) if key in case else None
        ex_hn = O.gru_cell_forward(w64("x"), w64("wi"), w64("h"), w64("wh"), w64("bi"), w64("bh"), O.F64)
        ex = O.gru_cell_backward(w64("g"), w64("x"), w64("wi"), w64("h"), w64("wh"), w64("bi"), w64("bh"), O.F64)
        chain_close(hn.to_numpy(), case["hn"], ex_hn, dtype, kx + hidden, f"{name} h'")
        hn.backward(T(case["g"], dtype))
        for t, key, kk, e in ((x, "dx", 3 * hidden, ex[0]), (wi, "dwi", m, ex[1]), (h, "dh", 3 * hidden, ex[2]), (wh, "dwh", m, ex[3])):
            chain_close(t.grad.to_numpy(), case[key], e, dtype, kk, f"{name} {key}")
        if bias:
            chain_close(bi.grad.to_numpy(), case["dbi"], ex[4], dtype, m, f"{name} dbi")
            chain_close(bh.grad.to_numpy(), case["dbh"], ex[5], dtype, m, f"{name} dbh")


@pytest.mark.parametrize("dtype", ["float32", "float64", "float16", "bfloat16"])
def test_gru_cell_node_cell_sizes(lib, dtype):
    """Sizes of a real cell (batch 64, input 96, hidden 128), gradient accumulation into existing grads, and a second
    step that reuses the weights (their gradients accumulate in the GEMM epilogues)."""
    rng = np.random.default_rng(71)
    m, kx, hd = 64, 96, 128
    x = rand_operand(rng, (m, kx), dtype); h = rand_operand(rng, (m, hd), dtype, scale=0.5)
    wi = rand_operand(rng, (kx, 3 * hd), dtype, scale=1 / np.sqrt(kx)); wh = rand_operand(rng, (hd, 3 * hd), dtype, scale=1 / np.sqrt(hd))
    bi = rand_operand(rng, (3 * hd,), dtype, scale=0.1); bh = rand_operand(rng, (3 * hd,), dtype, scale=0.1)
    g = rand_operand(rng, (m, hd), dtype)
    code = CODE[dtype]
    X, WI, H, WH, BI, BH = (T(v, dtype, True) for v in (x, wi, h, wh, bi, bh))
    hn = X.op_gru_cell(WI, H, WH, BI, BH)
    if dtype in ("float16", "bfloat16"):
        assert lib.rpb_last_kernel() in (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_SPLITK, _lib.KERNEL_SIMT)
    w64 = [f64(v, dtype) for v in (x, wi, h, wh, bi, bh)]
    chain_close(hn.to_numpy(), O.gru_cell_forward(x, wi, h, wh, bi, bh, code), O.gru_cell_forward(*w64, O.F64), dtype, kx + hd, "h'")
    hn.backward(T(g, dtype))
    ref = O.gru_cell_backward(g, x, wi, h, wh, bi, bh, code)
    ex = O.gru_cell_backward(f64(g, dtype), *w64, O.F64)
    for t, r, e, kk, what in ((X, ref[0], ex[0], 3 * hd, "dx"), (WI, ref[1], ex[1], m, "dwi"), (H, ref[2], ex[2], 3 * hd, "dh"),
                              (WH, ref[3], ex[3], m, "dwh"), (BI, ref[4], ex[4], m, "dbi"), (BH, ref[5], ex[5], m, "dbh")):
        chain_close(t.grad.to_numpy(), r, e, dtype, kk, what)
    # a second step from h' with the same weights: every leaf's gradient is accumulated, not replaced
    first = [f64(t.grad.to_numpy(), dtype) for t in (WI, WH, BI, BH, H)]
    hn2 = X.op_gru_cell(WI, H, WH, BI, BH)
    hn2.backward(T(g, dtype))
    for t, f in zip((WI, WH, BI, BH, H), first):
        now = f64(t.grad.to_numpy(), dtype)
        assert np.linalg.norm(now - 2 * f) / np.linalg.norm(2 * f) < (1e-2 if dtype in ("float16", "bfloat16") else 1e-5)
    # shape errors
    with pytest.raises(RuntimeError):
        X.op_gru_cell(WI, H, T(rand_operand(rng, (hd, 3 * hd + 3), dtype), dtype), BI, BH)
    with pytest.raises(RuntimeError):
        X.op_gru_cell(WI, T(rand_operand(rng, (m + 1, hd), dtype), dtype), WH, None, None)


def _conv_struct(meta):
    n, c, hh, ww, oc, kh, kw, sh, sw, ph, pw, dh, dw = [int(v) for v in meta]
    cv = _lib.RpbConv2d(n, c, hh, ww, oc, kh, kw, sh, sw, ph, pw, dh, dw)
    return cv, (n, c, hh, ww, oc, kh, kw), (sh, sw), (ph, pw), (dh, dw)


def _run_conv(lib, dtype, x, w, g, cv):
    oh, ow = C.c_int(), C.c_int()
    assert lib.rp_conv2d_out_shape(C.byref(cv), C.byref(oh), C.byref(ow)) == 0
    cols = lib.rp_conv2d_col_elems(C.byref(cv))
    st = O.storage(CODE[dtype])
    tx, tw, tg = T(x, dtype), T(w, dtype), T(g, dtype)
    col = T(np.zeros(cols, st), dtype); dcol = T(np.zeros(cols, st), dtype)
    y = T(np.zeros((cv.N, cv.C_out, oh.value, ow.value), st), dtype)
    dx = T(np.full(x.shape, 7, st), dtype); dw = T(np.full(w.shape, 7, st), dtype)      # stale contents must not leak
    p = lambda t: C.c_void_p(t.data_ptr)
    before = lib.rpb_launch_count()
    assert lib.rp_conv2d_forward_ex(p(y), p(tx), p(tw), p(col), C.byref(cv), CODE[dtype], 0, None) == 0
    fwd_launches = lib.rpb_launch_count() - before
    assert lib.rp_conv2d_backward_ex(p(dx), 0, p(dw), 0, p(tg), p(tw), p(col), p(dcol), C.byref(cv), CODE[dtype], 0, None) == 0
    return y.to_numpy(), dx.to_numpy(), dw.to_numpy(), fwd_launches


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_conv2d_vs_reference_fixtures(lib, conv2d_golden, dtype):
    """rp_conv2d_forward_ex / rp_conv2d_backward_ex against the unmodified reference's CPU op_conv2d + backward."""
    for (name, dt), case in conv2d_golden.items():
        if dt != dtype:
            continue
        cv, (n, c, hh, ww, oc, kh, kw), st, pd, dl = _conv_struct(case["meta"])
        y, dx, dw, launches = _run_conv(lib, dtype, case["x"], case["w"], case["g"], cv)
        assert launches <= 3, launches                     # one im2col pass + one GEMM (+ a K-slice reduction), not N of each
        kk = c * kh * kw
        check_close(y, case["y"], dtype, kk, f"{name} y")
        check_close(dx, case["dx"], dtype, oc * kh * kw, f"{name} dx")
        check_close(dw, case["dw"], dtype, n * y.shape[2] * y.shape[3], f"{name} dw")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
def test_conv2d_layer_sizes(lib, dtype):
    """A CIFAR-sized layer (16 images, 32 -> 64 channels, 3 x 3, 16 x 16 pixels) against a float64 convolution built
    from the same bits; weight-gradient accumulation in the GEMM epilogue."""
    rng = np.random.default_rng(83)
    n, c, hh, ww, oc, kh, kw = 16, 32, 16, 16, 64, 3, 3
    x = rand_operand(rng, (n, c, hh, ww), dtype); w = rand_operand(rng, (oc, c, kh, kw), dtype, scale=1 / np.sqrt(c * kh * kw))
    cv = _lib.RpbConv2d(n, c, hh, ww, oc, kh, kw, 1, 1, 1, 1, 1, 1)
    g = rand_operand(rng, (n, oc, hh, ww), dtype)
    y, dx, dw, _ = _run_conv(lib, dtype, x, w, g, cv)
    x64, w64, g64 = f64(x, dtype), f64(w, dtype), f64(g, dtype)
    ry = O.conv2d_forward(x64[:2], w64, (1, 1), (1, 1), (1, 1), O.F64)            # two images: the numpy loops are slow
    rdx, _ = O.conv2d_backward(x64[:2], w64, g64[:2], (1, 1), (1, 1), (1, 1), O.F64)
    tol = {"bfloat16": 4e-3, "float16": 6e-4, "float32": 2e-6}[dtype]
    rel = lambda a, b: np.linalg.norm(a - b) / np.linalg.norm(b)
    assert rel(f64(y, dtype)[:2], ry) < tol and rel(f64(dx, dtype)[:2], rdx) < tol
    # dW over all 16 images through an einsum of the same im2col arithmetic
    xp = np.pad(x64, ((0, 0), (0, 0), (1, 1), (1, 1)))
    rdw = np.zeros(w64.shape)
    for i in range(kh):
        for j in range(kw):
            rdw[:, :, i, j] = np.einsum("nohw,nchw->oc", g64, xp[:, :, i:i + hh, j:j + ww])
    assert rel(f64(dw, dtype), rdw) < tol
    assert lib.rp_conv2d_col_elems(C.byref(_lib.RpbConv2d(1, 1, 2, 2, 1, 5, 5, 1, 1, 0, 0, 1, 1))) == -1      # kernel larger than image


def test_bounded_wait_gives_up_and_reports(lib):
    """The kernels' wait on a barrier, alone: nobody ever signals it, the limit (about half a millisecond) runs out,
    the kernel returns normally, and the device's status word carries the code until it is read once."""
    assert lib.rpb_device_status(0) == 0
    assert lib.rpb_selftest_bounded_wait(0, 1000000) == 0
    assert lib.rpb_device_status(0) == 9
    assert lib.rpb_device_status(0) == 0
    # the context is intact: a GEMM right after runs and is correct
    rng = np.random.default_rng(5)
    a = rand_operand(rng, (128, 256), "bfloat16", scale=1 / 16); b = rand_operand(rng, (256, 128), "bfloat16")
    out = np.zeros((128, 128), np.uint16)
    assert lib.rp_matmul_host(out.ctypes.data_as(C.c_void_p), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p),
                              128, 256, 128, O.BF16, 0) == 0
    check_close(out, O.rp_matmul(a, b, O.BF16), "bfloat16", 256, "GEMM after the self-test")
    # a synchronous entry point reports a kernel that gave up instead of returning garbage silently
    assert lib.rpb_selftest_bounded_wait(0, 1000000) == 0
    assert lib.rp_matmul_host(out.ctypes.data_as(C.c_void_p), a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p),
                              128, 256, 128, O.BF16, 0) == -1
    assert lib.rpb_device_status(0) == 0
    lib.rpb_set_wait_limit_ms(500); lib.rpb_set_wait_limit_ms(0)
    assert lib.rpb_selftest_bounded_wait(0, 0) == -1 and lib.rpb_selftest_bounded_wait(0, 10 ** 12) == -1
