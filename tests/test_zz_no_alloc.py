"""rp_matmul_noalloc: the GEMM variant for callers that cannot let the library allocate
(their own pool owns the device memory, or they are in a section where cudaMalloc's device-wide
stall is not acceptable).  Its K-split partial tiles live in a fixed array inside the library
instead of a cudaMalloc'ed buffer.  Checked here against the regular entry point (rp_matmul_ex),
twice in a row, because the built-in array keeps the previous call's contents.

This file is collected last on purpose, so a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest

import recpulse_b200 as rpb
from recpulse_b200 import _lib
from oracle import oracle as O
from helpers import CODE, HALF_FROB_TIGHT, check_close, f64, rand_operand

pytestmark = pytest.mark.gpu


def _regular(lib, ta, tb, m, k, n, dtype):
    out = rpb.Tensor.from_numpy(np.zeros((m, n), np.uint16), dtype=dtype)
    g = rpb.RpbGemm()
    lib.rpb_gemm_packed(C.byref(g), m, k, n)
    assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                            CODE[dtype], 0, None) == 0
    return out.to_numpy()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_noalloc_matches_regular_entry_point_on_consecutive_calls(dtype):
    lib = rpb.load()
    rng = np.random.default_rng(2)
    # two different problems back to back: the second must not see the first one's partial tiles
    for (m, k, n) in [(64, 4096, 128), (200, 1024, 136)]:
        a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / np.sqrt(k))
        ta = rpb.Tensor.from_numpy(a, dtype=dtype); tb = rpb.Tensor.from_numpy(b, dtype=dtype)
        ref = _regular(lib, ta, tb, m, k, n, dtype)
        want = O.rp_matmul(a, b, CODE[dtype])                 # the reference's own algorithm on the same bits
        free_before = None
        for call in range(2):
            out = rpb.Tensor.from_numpy(np.full((m, n), 0x7FC0, np.uint16), dtype=dtype)    # NaN-filled output
            status = C.c_int(-1)
            rc = lib.rp_matmul_noalloc(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr),
                                       m, k, n, CODE[dtype], 0, None, C.byref(status))
            assert rc == 0 and status.value == 0
            assert lib.rpb_last_kernel() == _lib.KERNEL_UMMA_SPLITK          # the scratch-using kernel ran
            got = out.to_numpy()
            g64, r64 = f64(got, dtype), f64(ref, dtype)
            assert np.isfinite(g64).all()
            err = np.linalg.norm(g64 - r64) / np.linalg.norm(r64)
            assert err <= HALF_FROB_TIGHT[dtype], (dtype, m, k, n, call, err)
            check_close(got, want, dtype, k, f"rp_matmul_noalloc vs oracle, call {call}")
            # nothing was allocated: after the first call on the device (which loads the kernel and resolves the
            # built-in buffers) the free device memory does not move
            free_now, total = C.c_size_t(), C.c_size_t()
            assert lib.rpb_mem_info(0, C.byref(free_now), C.byref(total)) == 0
            if call == 1:
                assert free_now.value == free_before, (free_before, free_now.value)
            free_before = free_now.value


def test_noalloc_rejects_what_it_cannot_hold():
    lib = rpb.load()
    dtype = "bfloat16"
    a = rpb.Tensor.from_numpy(np.zeros((4096, 128), np.uint16), dtype=dtype)
    b = rpb.Tensor.from_numpy(np.zeros((128, 4096), np.uint16), dtype=dtype)
    out = rpb.Tensor.from_numpy(np.zeros((4096, 4096), np.uint16), dtype=dtype)
    # 2 splits x 4096 x 4096 x 4 bytes = 128 MiB > 16 MiB
    assert lib.rp_matmul_noalloc(C.c_void_p(out.data_ptr), C.c_void_p(a.data_ptr), C.c_void_p(b.data_ptr),
                                 4096, 128, 4096, CODE[dtype], 0, None, None) == -1
    # unsupported dtype and layout are refused too
    assert lib.rp_matmul_noalloc(C.c_void_p(out.data_ptr), C.c_void_p(a.data_ptr), C.c_void_p(b.data_ptr),
                                 64, 64, 64, CODE["float32"], 0, None, None) == -1
    assert lib.rp_matmul_noalloc(C.c_void_p(out.data_ptr), C.c_void_p(a.data_ptr), C.c_void_p(b.data_ptr),
                                 64, 60, 64, CODE[dtype], 0, None, None) == -1
