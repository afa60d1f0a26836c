"""ctypes binding of librecpulse_b200.so (the C ABI declared in include/recpulse_b200.h).

There is no Python or CPU implementation behind this module: when the shared
library is missing and cannot be built, importing fails with an error.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

F32, F64, F16, BF16 = 0, 1, 2, 3
DTYPE_CODE = {"float32": F32, "float64": F64, "float16": F16, "bfloat16": BF16}
DTYPE_NAME = {v: k for k, v in DTYPE_CODE.items()}
DTYPE_SIZE = {F32: 4, F64: 8, F16: 2, BF16: 2}

KERNEL_NONE, KERNEL_SIMT, KERNEL_UMMA, KERNEL_UMMA_SPLITK, KERNEL_DMMA, KERNEL_TF32X3 = 0, 1, 2, 3, 4, 5


class Meta(C.Structure):
    pass


class GradFn(C.Structure):
    pass


class CTensor(C.Structure):
    pass


Meta._fields_ = [("is_leaf", C.c_bool), ("requires_grad", C.c_bool), ("is_frozen", C.c_bool),
                 ("grad_fn", C.POINTER(GradFn)), ("grad", C.POINTER(CTensor))]
CTensor._fields_ = [("dtype", C.c_int), ("data", C.c_void_p), ("ndim", C.c_int), ("size", C.c_size_t),
                    ("shape", C.POINTER(C.c_int)), ("strides", C.POINTER(C.c_int)), ("device_id", C.c_int),
                    ("owns_data", C.c_bool), ("refcount", C.c_int), ("base_tensor", C.POINTER(CTensor)),
                    ("data_offset", C.c_size_t), ("metadata", C.POINTER(Meta))]
GradFn._fields_ = [("backward", C.c_void_p), ("inputs", C.POINTER(C.POINTER(CTensor))), ("num_inputs", C.c_int),
                   ("saved_data", C.c_void_p), ("owner", C.POINTER(CTensor))]


class RpbConv2d(C.Structure):
    _fields_ = [(f, C.c_int) for f in ("N", "C_in", "H", "W", "C_out", "kH", "kW", "stride_h", "stride_w", "pad_h", "pad_w",
                                       "dilation_h", "dilation_w")]


class RpbGemm(C.Structure):
    _fields_ = [("m", C.c_int), ("n", C.c_int), ("k", C.c_int), ("batch", C.c_int), ("reduce", C.c_int),
                ("a_row", C.c_longlong), ("a_col", C.c_longlong), ("a_batch", C.c_longlong), ("a_reduce", C.c_longlong),
                ("b_row", C.c_longlong), ("b_col", C.c_longlong), ("b_batch", C.c_longlong), ("b_reduce", C.c_longlong),
                ("c_row", C.c_longlong), ("c_batch", C.c_longlong), ("accumulate", C.c_int), ("bias", C.c_void_p), ("max_sms", C.c_int), ("epilogue", C.c_int), ("c_float32", C.c_int)]


# every symbol include/recpulse_b200.h declares: name -> (restype, argtypes)
TP = C.POINTER(CTensor)
SYMBOLS = {
    "matmul_kernel_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "rp_matmul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "op_matmul": (TP, [TP, TP]),
    "backward_matmul_fn": (None, [C.POINTER(GradFn), TP]),
    "op_linear": (TP, [TP, TP, TP]),
    "backward_linear_fn": (None, [C.POINTER(GradFn), TP]),
    "op_linear2": (TP, [TP, TP, TP, TP, TP]),
    "backward_linear2_fn": (None, [C.POINTER(GradFn), TP]),
    "op_lstm_gates": (TP, [TP, TP, TP, TP, TP]),
    "backward_lstm_gates_fn": (None, [C.POINTER(GradFn), TP]),
    "rp_lstm_gates_ex": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
    "rp_lstm_gates_grad_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong, C.c_longlong,
                                        C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
    "op_gru_cell": (TP, [TP, TP, TP, TP, TP, TP]),
    "backward_gru_cell_fn": (None, [C.POINTER(GradFn), TP]),
    "rp_gru_gates_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong, C.c_int,
                                  C.c_int, C.c_void_p]),
    "rp_gru_gates_grad_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_longlong, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
    "rp_conv2d_out_shape": (C.c_int, [C.POINTER(RpbConv2d), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rp_conv2d_col_elems": (C.c_longlong, [C.POINTER(RpbConv2d)]),
    "rp_conv2d_forward_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(RpbConv2d), C.c_int, C.c_int,
                                       C.c_void_p]),
    "rp_conv2d_backward_ex": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.POINTER(RpbConv2d), C.c_int, C.c_int, C.c_void_p]),
    "rp_colsum_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int,
                               C.c_void_p]),
    "rpb_gemm_packed": (None, [C.POINTER(RpbGemm), C.c_int, C.c_int, C.c_int]),
    "rp_matmul_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(RpbGemm), C.c_int, C.c_int, C.c_void_p]),
    "rp_matmul_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "rp_matmul_fwdbwd_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "rpb_release_host_pipeline": (C.c_int, [C.c_int]),
    "rp_matmul_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.POINTER(C.c_int)]),
    "rpb_last_kernel": (C.c_int, []),
    "rpb_umma_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                                C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "rpb_launch_count": (C.c_ulonglong, []),
    "rpb_force_kernel": (None, [C.c_int]),
    "rpb_device_status": (C.c_int, [C.c_int]),
    "rpb_version": (C.c_char_p, []),
    "rpb_trace_enable": (C.c_int, [C.c_int]),
    "rpb_trace_read": (C.c_int, [C.POINTER(C.c_ulonglong), C.c_int]),
    "rpb_set_wait_limit_ms": (None, [C.c_int]),
    "rpb_selftest_bounded_wait": (C.c_int, [C.c_int, C.c_longlong]),
    "rpb_tensor_from_host": (TP, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_bool]),
    "rpb_tensor_empty": (TP, [C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int]),
    "rpb_tensor_view": (TP, [TP, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_size_t]),
    "rpb_tensor_to_host": (C.c_int, [TP, C.c_void_p]),
    "rpb_tensor_write_host": (C.c_int, [TP, C.c_void_p]),
    "rpb_tensor_zero_grad": (None, [TP]),
    "rpb_tensor_release": (None, [TP]),
    "rpb_backward_node": (C.c_int, [TP, TP]),
    "rpb_shard_unique_id": (C.c_int, [C.c_void_p]),
    "rpb_shard_create": (C.c_void_p, [C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "rpb_shard_destroy": (None, [C.c_void_p]),
    "rpb_shard_rank": (C.c_int, [C.c_void_p]),
    "rpb_shard_world": (C.c_int, [C.c_void_p]),
    "rpb_shard_configure": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "rpb_shard_rows": (None, [C.c_longlong, C.c_int, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "rpb_shard_collective_count": (C.c_ulonglong, []),
    "rpb_shard_db_slice_of": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_longlong),
                                        C.POINTER(C.c_longlong)]),
    "rp_shard_replicate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "rp_matmul_rowsharded_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                                               C.c_int, C.c_void_p]),
    "rp_matmul_rowsharded_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "rp_matmul_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p]),
    "rp_matmul_rowsharded_fwdbwd_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                   C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int,
                                                   C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "rpb_node_stream": (None, [C.c_void_p, C.c_int]),
    "rpb_node_synchronize": (C.c_int, [C.c_int]),
    "rpb_scratch_reserve": (C.c_int, [C.c_int, C.c_size_t]),
    "rpb_scratch_reset": (C.c_int, [C.c_int]),
    "rpb_mem_info": (C.c_int, [C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
}

_LIB = None


def lib_path() -> str:
    return _build.LIB


def load(global_scope: bool = False) -> C.CDLL:
    """Load (building first if stale) the shared library.

    ``global_scope=True`` puts its symbols in the process's global scope, which is
    how the library takes over ``rp_matmul`` / ``op_matmul`` inside an unmodified
    ``recpulse_cuda.so`` imported afterwards.
    """
    global _LIB
    if _LIB is None or global_scope:
        path = _build.build()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `python -m recpulse_b200.build`")
        mode = C.RTLD_GLOBAL if global_scope else C.DEFAULT_MODE
        lib = C.CDLL(path, mode=mode)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)      # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB
