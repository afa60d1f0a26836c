"""CPU-side checks: the shared library builds, loads and exports the whole C ABI;
host-side argument checks that need no GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = rpb.load()
    header = open(os.path.join(ROOT, "include", "recpulse_b200.h")).read()
    body = header[header.index("drop-in entry points"):]
    declared = set(re.findall(r"\b([a-z_0-9]+)\s*\(", re.sub(r"/\*.*?\*/", "", body, flags=re.S)))
    declared = {d for d in declared if d.startswith(("rp_", "rpb_", "op_", "matmul_", "backward_"))}
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.rpb_version()


def test_struct_layout_matches_reference_abi():
    # core/tensor.h:27-42 on LP64: dtype@0 data@8 ndim@16 size@24 shape@32 strides@40 device_id@48
    # owns_data@52 refcount@56 base_tensor@64 data_offset@72 metadata@80, sizeof 88
    T = _lib.CTensor
    assert (T.dtype.offset, T.data.offset, T.ndim.offset, T.size.offset) == (0, 8, 16, 24)
    assert (T.shape.offset, T.strides.offset, T.device_id.offset, T.owns_data.offset) == (32, 40, 48, 52)
    assert (T.refcount.offset, T.base_tensor.offset, T.data_offset.offset, T.metadata.offset) == (56, 64, 72, 80)
    assert C.sizeof(T) == 88
    assert C.sizeof(_lib.Meta) == 24 and _lib.Meta.grad_fn.offset == 8 and _lib.Meta.grad.offset == 16
    assert C.sizeof(_lib.GradFn) == 40


def test_packed_descriptor():
    lib = rpb.load()
    g = rpb.RpbGemm()
    lib.rpb_gemm_packed(C.byref(g), 3, 4, 5)
    assert (g.m, g.k, g.n, g.batch, g.reduce) == (3, 4, 5, 1, 1)
    assert (g.a_row, g.a_col, g.b_row, g.b_col, g.c_row, g.accumulate) == (4, 1, 5, 1, 5, 0)


def test_argument_errors_without_gpu():
    lib = rpb.load()
    buf = np.zeros(16, np.float32).ctypes.data_as(C.c_void_p)
    # rp_matmul's checks, functional/functional.c:979
    assert lib.rp_matmul(None, buf, buf, 2, 2, 2, 0, 0) == -1
    assert lib.rp_matmul(buf, buf, buf, 0, 2, 2, 0, 0) == -1
    assert lib.rp_matmul(buf, buf, buf, 2, -1, 2, 0, 0) == -1
    # host memory is not this library's business and no reference is loaded here
    assert lib.rp_matmul(buf, buf, buf, 2, 2, 2, 0, -1) == -1
    g = rpb.RpbGemm()
    lib.rpb_gemm_packed(C.byref(g), 2, 2, 2)
    assert lib.rp_matmul_ex(buf, buf, buf, C.byref(g), 0, -1, None) == -1
    assert lib.op_matmul(None, None) is None or not lib.op_matmul(None, None)


def test_op_matmul_rejects_bad_operands_on_host_structs():
    # shape / dtype / device checks happen before any CUDA call (ops/ops.c:6817-6820)
    lib = rpb.load()

    def host_struct(shape, dtype=0, device=-1):
        t = _lib.CTensor()
        t.dtype = dtype; t.ndim = len(shape); t.device_id = device
        t.shape = (C.c_int * len(shape))(*shape)
        strides = [int(np.prod(shape[i + 1:])) for i in range(len(shape))]
        t.strides = (C.c_int * len(shape))(*strides)
        t.size = int(np.prod(shape))
        return t

    a, b = host_struct([2, 3]), host_struct([4, 5])
    assert not lib.op_matmul(C.byref(a), C.byref(b))           # inner dimension mismatch
    a, b = host_struct([2, 3]), host_struct([3, 5], dtype=1)
    assert not lib.op_matmul(C.byref(a), C.byref(b))           # dtype mismatch
    a, b = host_struct([2, 3], device=0), host_struct([3, 5], device=-1)
    assert not lib.op_matmul(C.byref(a), C.byref(b))           # cpu @ cuda
    a, b = host_struct([3]), host_struct([3, 5])
    assert not lib.op_matmul(C.byref(a), C.byref(b))           # 1-D operand
    a, b = host_struct([2, 3]), host_struct([3, 5])
    assert not lib.op_matmul(C.byref(a), C.byref(b))           # host tensors: no CPU path here


def test_tile_plan_model_on_the_host():
    """rpb_umma_plan is pure host arithmetic: the decisions the measurements behind the model call for."""
    import ctypes as C
    from recpulse_b200 import _lib
    lib = _lib.load()

    def plan(m, n, k, dtype=3, reduce=1, batch=1, sms=148):          # 3 = DTYPE_BFLOAT16, 0 = DTYPE_FLOAT32
        bn, sl, pr = C.c_int(), C.c_int(), C.c_int()
        assert lib.rpb_umma_plan(m, n, k, reduce, batch, dtype, sms, C.byref(bn), C.byref(sl), C.byref(pr)) == 0
        return bn.value, sl.value, pr.value

    assert plan(65536, 8192, 8192) == (128, 1, 2)        # the row-sharded workload: double-width pair tiles, no K slices
    assert plan(8192, 8192, 65536) == (128, 1, 2)        # its dB
    assert plan(8192, 8192, 8192, sms=132) == (128, 1, 2)    # with SMs left to a collective
    assert plan(4096, 4096, 4096) == (128, 1, 1)         # 3.46 waves of 256 x 256 tiles, the last one cut along K: stays
    assert plan(2048, 2048, 4096) == (128, 1, 1)         # one wave: halving the tile count would idle half the SMs
    assert plan(65536, 2048, 512, dtype=0)[2] == 1       # float32 never takes the double-width tile
    bn, sl, pr = plan(1024, 1024, 1024)                  # few tiles, short K: narrow one-CTA tiles, un-split
    assert (sl, pr) == (1, 0) and bn in (64, 128)
    assert plan(4096, 4096, 64) == (256, 1, 0)           # K of one block: the pair's hand-offs do not pay
    bn, sl, pr = plan(64, 512, 32768)                    # skinny weight gradient: K slices fill the SMs
    assert sl >= 8 and pr == 0
    bn, sl, pr = plan(128, 8192, 4096)                   # one row of tiles: no pair (m < 256)
    assert pr == 0
    assert plan(65536, 2048, 512, dtype=0)[2] == 1       # fp32 (3xTF32) large output: pair tiles
    assert lib.rpb_umma_plan(0, 8, 8, 1, 1, 3, 148, None, None, None) == -1
    assert lib.rpb_umma_plan(8, 8, 8, 1, 1, 1, 148, None, None, None) == -1      # float64 has no tcgen05 plan


def test_new_entry_points_refuse_bad_arguments_without_gpu():
    """GRU / conv2d passes, the stream-ordered node switch and the diagnostics: argument errors need no GPU."""
    lib = rpb.load()
    buf = np.zeros(64, np.float32).ctypes.data_as(C.c_void_p)
    # GRU passes: host "device", hidden <= 0, row stride shorter than a row
    assert lib.rp_gru_gates_ex(buf, buf, buf, buf, 4, 4, 4, 0, -1, None) == -1
    assert lib.rp_gru_gates_ex(buf, buf, buf, buf, 4, 0, 4, 0, 0, None) == -1
    assert lib.rp_gru_gates_ex(buf, buf, buf, buf, 4, 4, 3, 0, 0, None) == -1
    assert lib.rp_gru_gates_grad_ex(buf, buf, None, 0, None, buf, buf, buf, 4, 4, 4, 0, 0, None) == -1
    # conv2d geometry (ops/ops.c:4739-4740): kernel larger than the padded image, zero stride
    cv = _lib.RpbConv2d(2, 3, 7, 6, 4, 3, 3, 1, 1, 1, 1, 1, 1)
    oh, ow = C.c_int(), C.c_int()
    assert lib.rp_conv2d_out_shape(C.byref(cv), C.byref(oh), C.byref(ow)) == 0 and (oh.value, ow.value) == (7, 6)
    assert lib.rp_conv2d_col_elems(C.byref(cv)) == 2 * 27 * 42
    cv2 = _lib.RpbConv2d(3, 2, 9, 8, 5, 2, 3, 2, 1, 0, 1, 1, 2)
    assert lib.rp_conv2d_out_shape(C.byref(cv2), C.byref(oh), C.byref(ow)) == 0 and (oh.value, ow.value) == (4, 6)
    assert lib.rp_conv2d_col_elems(C.byref(_lib.RpbConv2d(1, 1, 2, 2, 1, 5, 5, 1, 1, 0, 0, 1, 1))) == -1
    assert lib.rp_conv2d_col_elems(C.byref(_lib.RpbConv2d(1, 1, 8, 8, 1, 3, 3, 0, 1, 0, 0, 1, 1))) == -1
    assert lib.rp_conv2d_forward_ex(buf, buf, buf, None, C.byref(cv), 0, 0, None) == -1
    assert lib.rp_conv2d_backward_ex(None, 0, None, 0, buf, buf, buf, buf, C.byref(cv), 0, 0, None) == -1
    # node switch and wait limit are plain host state
    lib.rpb_node_stream(None, 0); lib.rpb_node_stream(None, 1)
    lib.rpb_set_wait_limit_ms(250); lib.rpb_set_wait_limit_ms(0)
    assert lib.rpb_trace_read((C.c_ulonglong * 4)(), 4) == -1          # tracing is off
    assert lib.rpb_selftest_bounded_wait(0, 0) == -1
    assert lib.op_gru_cell(None, None, None, None, None, None) is None or not lib.op_gru_cell(None, None, None, None, None, None)
