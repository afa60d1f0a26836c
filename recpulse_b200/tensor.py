"""Python mirror of the part of ``recpulse_cuda.Tensor`` that the matmul path touches.

Same method names and argument meaning as RecPulse's CPython binding
(python/tensor_python.c): ``from_numpy``, ``requires_grad_``, ``transpose``,
``op_matmul``, ``backward``, ``grad``, ``to_numpy``, ``shape`` / ``dtype`` /
``device``.  Every call goes through the C ABI of librecpulse_b200.so on a CUDA
device; there is no host implementation.

float16 / bfloat16 data crosses the numpy boundary as ``uint16`` bit patterns
(numpy has no bfloat16), so no conversion happens behind the caller's back.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

_NP = {_lib.F32: np.float32, _lib.F64: np.float64, _lib.F16: np.uint16, _lib.BF16: np.uint16}


def _device_id(device) -> int:
    if isinstance(device, int):
        return device
    if device == "cuda":
        return 0
    if isinstance(device, str) and device.startswith("cuda:"):
        return int(device[5:])
    raise ValueError(f"recpulse_b200 handles CUDA tensors only, got device={device!r}")


def _ints(v):
    return (C.c_int * len(v))(*[int(x) for x in v])


class Tensor:
    """Owns one reference to a C ``Tensor`` struct."""

    def __init__(self, ptr, keepalive=None):
        if not ptr:
            raise RuntimeError("NULL tensor")
        self._p = ptr
        self._keep = keepalive

    def __del__(self):
        p, self._p = getattr(self, "_p", None), None
        if p:
            _lib.load().rpb_tensor_release(p)

    # -- construction -------------------------------------------------------------
    @staticmethod
    def from_numpy(arr: np.ndarray, dtype: str | None = None, device="cuda:0", requires_grad=False) -> "Tensor":
        """``arr``: float32/float64 values, or uint16 bit patterns with dtype='float16'|'bfloat16'."""
        if dtype is None:
            dtype = {np.dtype(np.float32): "float32", np.dtype(np.float64): "float64",
                     np.dtype(np.float16): "float16"}[arr.dtype]
        code = _lib.DTYPE_CODE[dtype]
        if arr.dtype == np.float16:
            arr = arr.view(np.uint16)
        arr = np.ascontiguousarray(arr, _NP[code])
        p = _lib.load().rpb_tensor_from_host(arr.ctypes.data_as(C.c_void_p), code, arr.ndim, _ints(arr.shape),
                                             _device_id(device), bool(requires_grad))
        if not p:
            raise RuntimeError("from_numpy failed")
        return Tensor(p)

    # -- attributes ---------------------------------------------------------------
    @property
    def _t(self):
        return self._p.contents

    @property
    def shape(self):
        return tuple(self._t.shape[i] for i in range(self._t.ndim))

    @property
    def strides(self):
        return tuple(self._t.strides[i] for i in range(self._t.ndim))

    @property
    def ndim(self):
        return self._t.ndim

    @property
    def dtype(self):
        return _lib.DTYPE_NAME[self._t.dtype]

    @property
    def device_id(self):
        return self._t.device_id

    @property
    def device(self):
        return f"cuda:{self._t.device_id}"

    @property
    def data_ptr(self):
        return self._t.data

    @property
    def requires_grad(self):
        return bool(self._t.metadata) and self._t.metadata.contents.requires_grad

    def requires_grad_(self, flag=True):
        if not self._t.metadata:
            raise RuntimeError("create the tensor with requires_grad=True (no Meta attached)")
        self._t.metadata.contents.requires_grad = bool(flag)
        return self

    @property
    def grad(self):
        """Borrowed view of the accumulated gradient (None before backward)."""
        if not self._t.metadata or not self._t.metadata.contents.grad:
            return None
        g = self._t.metadata.contents.grad
        g.contents.refcount += 1
        return Tensor(g, keepalive=self)

    # -- views --------------------------------------------------------------------
    def as_strided(self, shape, strides, offset=0) -> "Tensor":
        p = _lib.load().rpb_tensor_view(self._p, len(shape), _ints(shape), _ints(strides), offset)
        if not p:
            raise RuntimeError("view failed")
        return Tensor(p, keepalive=self)

    def transpose(self, d0, d1) -> "Tensor":
        shape, strides = list(self.shape), list(self.strides)
        shape[d0], shape[d1] = shape[d1], shape[d0]
        strides[d0], strides[d1] = strides[d1], strides[d0]
        return self.as_strided(shape, strides)

    def expand(self, shape) -> "Tensor":
        old, st = self.shape, self.strides
        pad = len(shape) - len(old)
        strides = [0] * pad + [0 if (o == 1 and s != 1) else t for o, s, t in zip(old, shape[pad:], st)]
        return self.as_strided(list(shape), strides)

    # -- the path -----------------------------------------------------------------
    def op_matmul(self, other: "Tensor") -> "Tensor":
        if not isinstance(other, Tensor):
            raise TypeError("op_matmul expects a Tensor")
        p = _lib.load().op_matmul(self._p, other._p)
        if not p:
            raise RuntimeError("op_matmul operation failed")     # python/tensor_python.c:2293-2297
        return Tensor(p, keepalive=(self, other))

    def op_linear(self, weight: "Tensor", bias: "Tensor | None") -> "Tensor":
        """y = self . weight + bias as one node (bias added in the GEMM epilogue)."""
        p = _lib.load().op_linear(self._p, weight._p, bias._p if bias is not None else None)
        if not p:
            raise RuntimeError("op_linear operation failed")
        return Tensor(p, keepalive=(self, weight, bias))

    def op_linear2(self, weight: "Tensor", h: "Tensor", u: "Tensor", bias: "Tensor | None" = None) -> "Tensor":
        """y = self . weight + h . u + bias as one node (LSTM / GRU gate pre-activations)."""
        p = _lib.load().op_linear2(self._p, weight._p, h._p, u._p, bias._p if bias is not None else None)
        if not p:
            raise RuntimeError("op_linear2 operation failed")
        return Tensor(p, keepalive=(self, weight, h, u, bias))

    def op_lstm_gates(self, weight: "Tensor", h: "Tensor", u: "Tensor", bias: "Tensor | None" = None) -> "Tensor":
        """Activated LSTM gates act(self . weight + h . u + bias), columns i, f, g, o (sigmoid, sigmoid, tanh,
        sigmoid), as one node; the composition of recpulse/module.py:289-300."""
        p = _lib.load().op_lstm_gates(self._p, weight._p, h._p, u._p, bias._p if bias is not None else None)
        if not p:
            raise RuntimeError("op_lstm_gates operation failed")
        return Tensor(p, keepalive=(self, weight, h, u, bias))

    def op_gru_cell(self, w_ih: "Tensor", h: "Tensor", w_hh: "Tensor", b_ih: "Tensor | None" = None,
                    b_hh: "Tensor | None" = None) -> "Tensor":
        """h' of one GRU cell step for input `self` and state `h`, as one node; the composition of
        recpulse/module.py:329-348."""
        p = _lib.load().op_gru_cell(self._p, w_ih._p, h._p, w_hh._p, b_ih._p if b_ih is not None else None,
                                    b_hh._p if b_hh is not None else None)
        if not p:
            raise RuntimeError("op_gru_cell operation failed")
        return Tensor(p, keepalive=(self, w_ih, h, w_hh, b_ih, b_hh))

    def backward(self, grad_output: "Tensor") -> None:
        """Run this node's backward with an explicit upstream gradient and free the node."""
        if _lib.load().rpb_backward_node(self._p, grad_output._p) != 0:
            raise RuntimeError("backward operation failed")      # python/tensor_python.c:1349-1362

    def zero_grad(self) -> None:
        _lib.load().rpb_tensor_zero_grad(self._p)

    def copy_from_numpy(self, arr: np.ndarray) -> None:
        """New values into the SAME device buffer (what a captured CUDA graph keeps reading)."""
        arr = np.ascontiguousarray(arr.view(np.uint16) if arr.dtype == np.float16 else arr, _NP[self._t.dtype])
        if arr.shape != self.shape or _lib.load().rpb_tensor_write_host(self._p, arr.ctypes.data_as(C.c_void_p)) != 0:
            raise RuntimeError("copy_from_numpy failed")

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.shape, _NP[self._t.dtype])
        if _lib.load().rpb_tensor_to_host(self._p, out.ctypes.data_as(C.c_void_p)) != 0:
            raise RuntimeError("to_numpy failed")
        return out


def from_numpy(arr, dtype=None, device="cuda:0", requires_grad=False) -> Tensor:
    return Tensor.from_numpy(arr, dtype, device, requires_grad)
