"""ctypes/numpy front end of ``liboracle.so`` (oracle/matmul_oracle.c).

TEST INFRASTRUCTURE ONLY.  The shipped library never imports this module.
Half-precision arrays are carried as ``uint16`` bit patterns so that the
reference's round-half-up narrowing (core/half_precision.h:50-97) is the only
conversion ever applied.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

F32, F64, F16, BF16 = 0, 1, 2, 3
DTYPE_NAMES = {F32: "float32", F64: "float64", F16: "float16", BF16: "bfloat16"}
_NP = {F32: np.float32, F64: np.float64, F16: np.uint16, BF16: np.uint16}
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile liboracle.so (and the reference, when its tree is present)."""
    subprocess.run(["make", "-s", "-C", _HERE, "all"], check=True)
    return os.path.join(_HERE, "liboracle.so")


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
        _LIB = C.CDLL(path)
        _LIB.orc_fp16_to_fp32.restype = C.c_float
        _LIB.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        _LIB.orc_bf16_to_fp32.restype = C.c_float
        _LIB.orc_bf16_to_fp32.argtypes = [C.c_uint16]
        _LIB.orc_fp32_to_fp16.restype = C.c_uint16
        _LIB.orc_fp32_to_fp16.argtypes = [C.c_float]
        _LIB.orc_fp32_to_bf16.restype = C.c_uint16
        _LIB.orc_fp32_to_bf16.argtypes = [C.c_float]
    return _LIB


def storage(dtype: int):
    return _NP[dtype]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _ints(v):
    return None if v is None else (C.c_int * len(v))(*[int(x) for x in v])


def narrow(x: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 -> storage bits of ``dtype`` with the reference's rounding."""
    if dtype == F32:
        return np.ascontiguousarray(x, np.float32)
    if dtype == F64:
        return np.ascontiguousarray(x, np.float64)
    src = np.ascontiguousarray(x, np.float32)
    out = np.empty(src.shape, np.uint16)
    lib().orc_narrow(_p(src), _p(out), C.c_size_t(src.size), dtype)
    return out


def widen(x: np.ndarray, dtype: int) -> np.ndarray:
    """storage bits -> float32 (f16/bf16), or the array itself as float."""
    if dtype in (F32, F64):
        return np.asarray(x)
    src = np.ascontiguousarray(x, np.uint16)
    out = np.empty(src.shape, np.float32)
    lib().orc_widen(_p(src), _p(out), C.c_size_t(src.size), dtype)
    return out


def to_f64(x: np.ndarray, dtype: int) -> np.ndarray:
    return widen(x, dtype).astype(np.float64)


def rp_matmul(a: np.ndarray, b: np.ndarray, dtype: int) -> np.ndarray:
    """Packed 2-D product, functional.c:978-1002 (host branch)."""
    a = np.ascontiguousarray(a, _NP[dtype]); b = np.ascontiguousarray(b, _NP[dtype])
    m, k = a.shape; k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), _NP[dtype])
    rc = lib().orc_rp_matmul(_p(c), _p(a), _p(b), m, k, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_rp_matmul failed")
    return c


def _elem_strides(x: np.ndarray):
    return [s // x.itemsize for s in x.strides]


def op_matmul(a: np.ndarray, b: np.ndarray, dtype: int) -> np.ndarray:
    """Forward on (possibly strided) 2-D numpy views, ops.c:6816-6847."""
    m, k = a.shape; _, n = b.shape
    c = np.empty((m, n), _NP[dtype])
    rc = lib().orc_op_matmul(_p(c), _p(a), _ints(_elem_strides(a)), _p(b),
                             _ints(_elem_strides(b)), m, k, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_op_matmul failed")
    return c


def matmul_backward(a, b, dc, dtype, need_da=True, need_db=True, acc_da=None, acc_db=None):
    """ops.c:6759-6814.  ``acc_*``: existing grads to accumulate into (copied)."""
    m, k = a.shape; _, n = b.shape
    dc = np.ascontiguousarray(dc, _NP[dtype])
    accumulate = int(acc_da is not None or acc_db is not None)
    da = (acc_da.copy() if acc_da is not None else np.empty((m, k), _NP[dtype])) if need_da else None
    db = (acc_db.copy() if acc_db is not None else np.empty((k, n), _NP[dtype])) if need_db else None
    rc = lib().orc_matmul_backward(_p(da), _p(db), _p(a), _ints(_elem_strides(a)), _p(b),
                                   _ints(_elem_strides(b)), _p(dc), m, k, n, dtype, accumulate)
    if rc != 0:
        raise RuntimeError("orc_matmul_backward failed")
    return da, db


def _batch_stride(x):
    return 0 if x.shape[0] == 1 else x.shape[1] * x.shape[2]


def bmm(a: np.ndarray, b: np.ndarray, dtype: int) -> np.ndarray:
    """[Ba,m,k] x [Bb,k,n] with Ba/Bb in {1, batch}: loop of reference 2-D products."""
    a = np.ascontiguousarray(a, _NP[dtype]); b = np.ascontiguousarray(b, _NP[dtype])
    batch = max(a.shape[0], b.shape[0]); m, k = a.shape[1:]; n = b.shape[2]
    c = np.empty((batch, m, n), _NP[dtype])
    rc = lib().orc_bmm(_p(c), _p(a), _p(b), batch, C.c_size_t(_batch_stride(a)),
                       C.c_size_t(_batch_stride(b)), m, k, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_bmm failed")
    return c


def bmm_backward(a, b, dc, dtype):
    a = np.ascontiguousarray(a, _NP[dtype]); b = np.ascontiguousarray(b, _NP[dtype])
    dc = np.ascontiguousarray(dc, _NP[dtype])
    batch = dc.shape[0]; m, k = a.shape[1:]; n = b.shape[2]
    da = np.empty(a.shape, _NP[dtype]); db = np.empty(b.shape, _NP[dtype])
    rc = lib().orc_bmm_backward(_p(da), _p(db), _p(a), _p(b), _p(dc), batch,
                                C.c_size_t(_batch_stride(a)), C.c_size_t(_batch_stride(b)),
                                m, k, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_bmm_backward failed")
    return da, db


def linear_forward(x, w, bias, dtype):
    """RecPulse's Linear.forward composition: op_add(op_matmul(x, w), bias)."""
    x = np.ascontiguousarray(x, _NP[dtype]); w = np.ascontiguousarray(w, _NP[dtype])
    bias = np.ascontiguousarray(bias, _NP[dtype]).reshape(-1)
    lead = x.shape[:-1]
    k = x.shape[-1]; n = w.shape[1]
    m = int(np.prod(lead))
    y = np.empty((m, n), _NP[dtype])
    rc = lib().orc_linear_forward(_p(y), _p(x.reshape(m, k)), _p(w), _p(bias), m, k, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_linear_forward failed")
    return y.reshape(lead + (n,))


def bias_grad(dy, dtype):
    """Sum of dY over every leading index (reduce_grad_to_shape)."""
    dy = np.ascontiguousarray(dy, _NP[dtype])
    n = dy.shape[-1]; rows = dy.size // n
    out = np.empty((n,), _NP[dtype])
    rc = lib().orc_bias_grad(_p(out), _p(dy), C.c_longlong(rows), n, dtype)
    if rc != 0:
        raise RuntimeError("orc_bias_grad failed")
    return out


def lstm_gates_forward(x, w, h, u, bias, dtype):
    """Activated LSTM gates as RecPulse's LSTMCell.forward composes them (recpulse/module.py:289-300)."""
    x = np.ascontiguousarray(x, _NP[dtype]); w = np.ascontiguousarray(w, _NP[dtype])
    h = np.ascontiguousarray(h, _NP[dtype]); u = np.ascontiguousarray(u, _NP[dtype])
    m, kx = x.shape; kh = h.shape[1]; n = w.shape[1]
    b = None if bias is None else np.ascontiguousarray(bias, _NP[dtype]).reshape(-1)
    y = np.empty((m, n), _NP[dtype])
    rc = lib().orc_lstm_gates_forward(_p(y), _p(x), _p(w), _p(h), _p(u), _p(b) if b is not None else None, m, kx, kh, n, dtype)
    if rc != 0:
        raise RuntimeError("orc_lstm_gates_forward failed")
    return y


def lstm_gates_grad(dy, y, dtype):
    """Gradient of the gate pre-activations from the activated output (sigmoid / tanh backward)."""
    dy = np.ascontiguousarray(dy, _NP[dtype]); y = np.ascontiguousarray(y, _NP[dtype])
    n = y.shape[-1]; rows = y.size // n
    out = np.empty(y.shape, _NP[dtype])
    rc = lib().orc_lstm_gates_grad(_p(out), _p(dy), _p(y), C.c_longlong(rows), n, dtype)
    if rc != 0:
        raise RuntimeError("orc_lstm_gates_grad failed")
    return out


def gru_cell_forward(x, w_ih, h, w_hh, b_ih, b_hh, dtype):
    """One GRU cell step as RecPulse's GRUCell.forward composes it (recpulse/module.py:329-348)."""
    x = np.ascontiguousarray(x, _NP[dtype]); w_ih = np.ascontiguousarray(w_ih, _NP[dtype])
    h = np.ascontiguousarray(h, _NP[dtype]); w_hh = np.ascontiguousarray(w_hh, _NP[dtype])
    m, kx = x.shape; hd = h.shape[1]
    bi = None if b_ih is None else np.ascontiguousarray(b_ih, _NP[dtype]).reshape(-1)
    bh = None if b_hh is None else np.ascontiguousarray(b_hh, _NP[dtype]).reshape(-1)
    out = np.empty((m, hd), _NP[dtype])
    rc = lib().orc_gru_cell_forward(_p(out), _p(x), _p(w_ih), _p(h), _p(w_hh), _p(bi), _p(bh), m, kx, hd, dtype)
    if rc != 0:
        raise RuntimeError("orc_gru_cell_forward failed")
    return out


def gru_cell_backward(g, x, w_ih, h, w_hh, b_ih, b_hh, dtype):
    """(dx, dw_ih, dh, dw_hh, db_ih, db_hh) of the same composition for the upstream gradient g of h'."""
    x = np.ascontiguousarray(x, _NP[dtype]); w_ih = np.ascontiguousarray(w_ih, _NP[dtype])
    h = np.ascontiguousarray(h, _NP[dtype]); w_hh = np.ascontiguousarray(w_hh, _NP[dtype])
    g = np.ascontiguousarray(g, _NP[dtype])
    m, kx = x.shape; hd = h.shape[1]
    bi = None if b_ih is None else np.ascontiguousarray(b_ih, _NP[dtype]).reshape(-1)
    bh = None if b_hh is None else np.ascontiguousarray(b_hh, _NP[dtype]).reshape(-1)
    dx = np.empty_like(x); dwi = np.empty_like(w_ih); dh = np.empty_like(h); dwh = np.empty_like(w_hh)
    dbi = None if bi is None else np.empty_like(bi); dbh = None if bh is None else np.empty_like(bh)
    rc = lib().orc_gru_cell_backward(_p(dx), _p(dwi), _p(dh), _p(dwh), _p(dbi), _p(dbh), _p(g), _p(x), _p(w_ih), _p(h), _p(w_hh),
                                     _p(bi), _p(bh), m, kx, hd, dtype)
    if rc != 0:
        raise RuntimeError("orc_gru_cell_backward failed")
    return dx, dwi, dh, dwh, dbi, dbh


def _conv_geometry(x_shape, w_shape, stride, pad, dil):
    n, c, hh, ww = x_shape; oc, c2, kh, kw = w_shape
    assert c == c2
    oh = (hh + 2 * pad[0] - dil[0] * (kh - 1) - 1) // stride[0] + 1          # ops/ops.c:4739-4740
    ow = (ww + 2 * pad[1] - dil[1] * (kw - 1) - 1) // stride[1] + 1
    return n, c, hh, ww, oc, kh, kw, oh, ow


def _im2col(img, kh, kw, stride, pad, dil, oh, ow):
    """functional/functional_host.c im2col: col[(c kH + kh) kW + kw, oh out_W + ow], zeros outside the image."""
    c, hh, ww = img.shape
    col = np.zeros((c * kh * kw, oh * ow), img.dtype)
    for ch in range(c):
        for i in range(kh):
            for j in range(kw):
                row = (ch * kh + i) * kw + j
                for a in range(oh):
                    hi = a * stride[0] + i * dil[0] - pad[0]
                    if hi < 0 or hi >= hh:
                        continue
                    for b in range(ow):
                        wi = b * stride[1] + j * dil[1] - pad[1]
                        if 0 <= wi < ww:
                            col[row, a * ow + b] = img[ch, hi, wi]
    return col


def conv2d_forward(x, w, stride, pad, dil, dtype):
    """op_conv2d without bias (ops/ops.c:4735-4770): per image im2col, then rp_matmul(weight, col).  float32 / float64."""
    assert dtype in (F32, F64)
    n, c, hh, ww, oc, kh, kw, oh, ow = _conv_geometry(x.shape, w.shape, stride, pad, dil)
    w2 = np.ascontiguousarray(w.reshape(oc, c * kh * kw))
    out = np.empty((n, oc, oh, ow), _NP[dtype])
    for i in range(n):
        out[i] = rp_matmul(w2, _im2col(x[i], kh, kw, stride, pad, dil, oh, ow), dtype).reshape(oc, oh, ow)
    return out


def conv2d_backward(x, w, gout, stride, pad, dil, dtype):
    """(dx, dw) of the same (ops/ops.c:4480-4620): per image W^T . dout through col2im in (c, kh, kw, oh, ow) order
    (functional_host.c:1291-1313), and dW = sum over images, in image order, of dout . col^T, each product rounded
    and added by rp_add."""
    assert dtype in (F32, F64)
    n, c, hh, ww, oc, kh, kw, oh, ow = _conv_geometry(x.shape, w.shape, stride, pad, dil)
    w2 = np.ascontiguousarray(w.reshape(oc, c * kh * kw))
    wt = np.ascontiguousarray(w2.T)
    dx = np.zeros(x.shape, _NP[dtype]); dw = np.zeros((oc, c * kh * kw), _NP[dtype])
    for i in range(n):
        g2 = np.ascontiguousarray(gout[i].reshape(oc, oh * ow))
        dcol = rp_matmul(wt, g2, dtype)
        gim = np.zeros((c, hh, ww), _NP[dtype])
        for ch in range(c):
            for a in range(kh):
                for b in range(kw):
                    row = (ch * kh + a) * kw + b
                    for p in range(oh):
                        hi = p * stride[0] + a * dil[0] - pad[0]
                        if hi < 0 or hi >= hh:
                            continue
                        for q in range(ow):
                            wi = q * stride[1] + b * dil[1] - pad[1]
                            if 0 <= wi < ww:
                                gim[ch, hi, wi] = gim[ch, hi, wi] + dcol[row, p * ow + q]
        dx[i] = dx[i] + gim
        col = _im2col(x[i], kh, kw, stride, pad, dil, oh, ow)
        dw = dw + rp_matmul(g2, np.ascontiguousarray(col.T), dtype)
    return dx, dw.reshape(w.shape)
