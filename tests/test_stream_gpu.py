"""Float32 outputs of 16-bit GEMMs, the scratch buffer's behaviour around stream capture, and the nodes run
stream-ordered (no synchronisation per call, replay from a CUDA graph)."""
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
    lib.rpb_node_stream(None, 1)
    assert lib.rpb_device_status(0) == 0


def dev(arr, dtype):
    return rpb.Tensor.from_numpy(np.ascontiguousarray(arr), dtype=dtype)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("shape", [(520, 1160, 776), (64, 4096, 128), (304, 200, 136), (2048, 512, 1024)])
def test_float32_output_is_the_unrounded_sum(lib, dtype, shape, monkeypatch):
    """RpbGemm.c_float32: the dB partials of the sharded path.  Checked against float64 at float32 accuracy,
    with A^T read through swapped strides (the dB form), one-slice and K-sliced plans, TMA and register stores."""
    m, k, n = shape
    rng = np.random.default_rng(m + k + n)
    at = rand_operand(rng, (k, m), dtype, scale=1 / np.sqrt(k)); b = rand_operand(rng, (k, n), dtype)
    ref = f64(at, dtype).T @ f64(b, dtype)
    ta, tb = dev(at, dtype), dev(b, dtype)
    for plan in (None, "128,1,0", "64,3,0"):
        if plan:
            monkeypatch.setenv("RPB_UMMA_PLAN", plan)
        out = dev(np.full((m, n), np.nan, np.float32), "float32")
        g = rpb.RpbGemm()
        lib.rpb_gemm_packed(C.byref(g), m, k, n)
        g.a_row, g.a_col = 1, m                      # A stored transposed
        g.c_float32 = 1
        assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                CODE[dtype], 0, None) == 0
        assert lib.rpb_last_kernel() in (_lib.KERNEL_UMMA, _lib.KERNEL_UMMA_SPLITK)
        got = out.to_numpy().astype(np.float64)
        assert np.isfinite(got).all()
        # fp32 accumulation of exact 16-bit products: far inside one 16-bit rounding step
        assert np.abs(got - ref).max() <= 2e-6 * np.sqrt(k) * np.sqrt(np.mean(ref * ref)) + 1e-30, (plan, shape)
        # "C += AB" keeps a float32 running sum (gradients accumulated over row chunks before their one rounding)
        g.accumulate = 1
        assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                                CODE[dtype], 0, None) == 0
        twice = out.to_numpy().astype(np.float64)
        assert np.abs(twice - 2 * ref).max() <= 4e-6 * np.sqrt(k) * np.sqrt(np.mean(ref * ref)) + 1e-30, (plan, shape)
    monkeypatch.delenv("RPB_UMMA_PLAN", raising=False)
    # what it cannot do is refused, not approximated
    g.accumulate = 0
    tbias = dev(rand_operand(rng, (n,), dtype), dtype)
    g.bias = tbias.data_ptr
    assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                            CODE[dtype], 0, None) == -1
    g.bias = None
    assert lib.rp_matmul_ex(C.c_void_p(out.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr), C.byref(g),
                            CODE["float32"], 0, None) == -1


def test_scratch_used_in_a_capture_cannot_grow(lib):
    """A graph holds the scratch buffer's address: after a capture that used it, a call that needs a larger
    buffer is refused (-1) instead of freeing it under the graph; rpb_scratch_reset lifts the pin."""
    import torch
    dtype = "bfloat16"
    assert lib.rpb_scratch_reset(0) == 0
    rng = np.random.default_rng(3)
    m, k, n = 64, 4096, 128                                  # K-sliced: partial tiles go through the scratch
    a = rand_operand(rng, (m, k), dtype, scale=1 / 64); b = rand_operand(rng, (k, n), dtype)
    ta, tb, tc = dev(a, dtype), dev(b, dtype), dev(np.zeros((m, n), np.uint16), dtype)
    g = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g), m, k, n)
    call = lambda stream: lib.rp_matmul_ex(C.c_void_p(tc.data_ptr), C.c_void_p(ta.data_ptr), C.c_void_p(tb.data_ptr),
                                           C.byref(g), CODE[dtype], 0, C.c_void_p(stream) if stream else None)
    assert call(None) == 0 and lib.rpb_last_kernel() == _lib.KERNEL_UMMA_SPLITK      # warm: the scratch exists (32 MiB)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        assert call(torch.cuda.current_stream().cuda_stream) == 0
    graph.replay(); torch.cuda.synchronize()
    check_close(tc.to_numpy(), O.rp_matmul(a, b, CODE[dtype]), dtype, k, "replayed K-sliced GEMM")
    # a problem whose partial tiles need more than the buffer holds: refused while the pin stands
    m2, k2, n2 = 2048, 8192, 2048
    big_a = dev(np.zeros((m2, k2), np.uint16), dtype); big_b = dev(np.zeros((k2, n2), np.uint16), dtype)
    big_c = dev(np.zeros((m2, n2), np.uint16), dtype)
    g2 = rpb.RpbGemm(); lib.rpb_gemm_packed(C.byref(g2), m2, k2, n2)
    import os
    os.environ["RPB_UMMA_PLAN"] = "256,4,0"                  # 4 K slices of 2048 x 2048 fp32 = 64 MiB of scratch
    try:
        big = lambda: lib.rp_matmul_ex(C.c_void_p(big_c.data_ptr), C.c_void_p(big_a.data_ptr), C.c_void_p(big_b.data_ptr),
                                       C.byref(g2), CODE[dtype], 0, None)
        assert big() == -1
        graph.replay(); torch.cuda.synchronize()             # the graph still owns a live buffer
        check_close(tc.to_numpy(), O.rp_matmul(a, b, CODE[dtype]), dtype, k, "replay after the refusal")
        del graph
        assert lib.rpb_scratch_reset(0) == 0
        assert big() == 0
        torch.cuda.synchronize()
    finally:
        del os.environ["RPB_UMMA_PLAN"]
    assert lib.rpb_scratch_reserve(0, 96 << 20) == 0
    assert lib.rpb_device_status(0) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_nodes_run_stream_ordered_without_synchronising(lib, dtype):
    """rpb_node_stream(stream, 0): op_matmul + backward queue their work and return; results are the same as
    in the default synchronous mode once the stream is synchronised."""
    import torch
    rng = np.random.default_rng(11)
    m, k, n = 128, 784, 256
    a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / 28); dc = rand_operand(rng, (m, n), dtype)

    def fwd_bwd():
        A = rpb.Tensor.from_numpy(a, dtype=dtype, requires_grad=True); B = rpb.Tensor.from_numpy(b, dtype=dtype, requires_grad=True)
        y = A.op_matmul(B)
        y.backward(rpb.Tensor.from_numpy(dc, dtype=dtype))
        return y, A, B

    y0, A0, B0 = fwd_bwd()
    want = (y0.to_numpy(), A0.grad.to_numpy(), B0.grad.to_numpy())
    s = torch.cuda.Stream()
    lib.rpb_node_stream(C.c_void_p(s.cuda_stream), 0)
    try:
        y1, A1, B1 = fwd_bwd()
        assert lib.rpb_node_synchronize(0) == 0
        got = (y1.to_numpy(), A1.grad.to_numpy(), B1.grad.to_numpy())
    finally:
        lib.rpb_node_stream(None, 1)
    for g_, w_ in zip(got, want):
        assert np.array_equal(g_, w_)
    check_close(got[0], O.rp_matmul(a, b, CODE[dtype]), dtype, k, "C")


def test_node_step_replayed_from_a_graph(lib):
    """The capture recipe for a launch-bound step: warm the shapes, switch the nodes to a capturing stream without
    synchronisation, capture op_matmul + backward once (outputs and gradients become allocations of the graph)
    and replay it with new input values written into the same leaf tensors."""
    import torch
    dtype = "float32"
    rng = np.random.default_rng(13)
    m, k, n = 64, 512, 2048
    a = rand_operand(rng, (m, k), dtype); b = rand_operand(rng, (k, n), dtype, scale=1 / 23); dc = rand_operand(rng, (m, n), dtype)
    A = rpb.Tensor.from_numpy(a, dtype=dtype, requires_grad=True); B = rpb.Tensor.from_numpy(b, dtype=dtype, requires_grad=True)
    G = rpb.Tensor.from_numpy(dc, dtype=dtype)
    y = A.op_matmul(B); y.backward(G)                         # warm-up in the default mode: sizes the scratch
    A.zero_grad(); B.zero_grad(); del y
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    lib.rpb_node_stream(C.c_void_p(s.cuda_stream), 0)
    try:
        with torch.cuda.graph(graph, stream=s):
            y = A.op_matmul(B)
            y.backward(G)
    finally:
        lib.rpb_node_stream(None, 1)
    for trial in range(2):
        a2 = rand_operand(rng, (m, k), dtype)
        A.copy_from_numpy(a2)                                 # new values, same device buffer
        graph.replay(); torch.cuda.synchronize()
        check_close(y.to_numpy(), O.rp_matmul(a2, b, CODE[dtype]), dtype, k, f"C replay {trial}")
        oda, odb = O.matmul_backward(a2, b, dc, CODE[dtype])
        check_close(A.grad.to_numpy(), oda, dtype, n, f"dA replay {trial}")
        check_close(B.grad.to_numpy(), odb, dtype, m, f"dB replay {trial}")
    assert lib.rpb_device_status(0) == 0
    del graph
    assert lib.rpb_scratch_reset(0) == 0
