"""Child process of test_dropin_gpu.py: the UNMODIFIED reference extension (compiled from its
own sources into oracle/_ref/) with librecpulse_b200.so placed in front of it, exactly as a
RecPulse user would run it.  Replays the reference's matmul tests on the GPU and compares
GPU results with the reference's own CPU path in the same process.  Prints 'DROPIN OK'."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
interpose = "--no-interpose" not in sys.argv
if interpose:
    import recpulse_b200
    lib = recpulse_b200.load(global_scope=True)     # same effect as LD_PRELOAD
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
import recpulse_cuda as rp  # noqa: E402


def launches():
    return lib.rpb_launch_count() if interpose else 0


def t(x, dtype, device, grad=False):
    if dtype == "bfloat16":
        r = rp.from_numpy(np.ascontiguousarray(x, np.float32)).to(dtype="bfloat16")
    else:
        r = rp.from_numpy(np.ascontiguousarray(x.astype({"float32": np.float32, "float64": np.float64,
                                                          "float16": np.float16}[dtype])))
    if device != "cpu":
        r = r.to(device=device)
    if grad:
        r.requires_grad_(True)
    return r


def npy(x):
    return np.asarray(x.to(device="cpu").to(dtype="float64").to_numpy(), np.float64)


rng = np.random.default_rng(0)
n0 = launches()

# stress_torch_parity.py:86-95 -- fp64 shapes, GPU vs numpy, rtol 1e-9 atol 1e-10
for (m, k, n) in [(3, 4, 5), (16, 32, 8), (1, 7, 1), (64, 64, 64)]:
    a = rng.uniform(-1, 1, (m, k)); b = rng.uniform(-1, 1, (k, n))
    y = t(a, "float64", "cuda").op_matmul(t(b, "float64", "cuda"))
    np.testing.assert_allclose(npy(y), a @ b, rtol=1e-9, atol=1e-10)

# test_functional.py:281-302 known answer
y = t(np.arange(1, 7.).reshape(2, 3), "float32", "cuda").op_matmul(t(np.arange(1, 7.).reshape(3, 2), "float32", "cuda"))
assert np.array_equal(npy(y), [[22, 28], [49, 64]])

# stress_gradcheck.py:214-243 -- grads CPU vs CUDA, incl. a transposed (non-contiguous) A, 1e-7
def grads(device, dtype, transposed):
    a = rng0.uniform(-1, 1, (4, 3) if transposed else (3, 4)); b = rng0.uniform(-1, 1, (4, 2)); w = rng0.uniform(.5, 1.5, (3, 2))
    A = t(a, dtype, device, True); B = t(b, dtype, device, True); W = t(w, dtype, device)
    At = A.transpose(0, 1) if transposed else A
    loss = At.op_matmul(B).op_mul(W).op_sum_all()
    loss.backward()
    return npy(A.grad), npy(B.grad)

for transposed in (False, True):
    rng0 = np.random.default_rng(5); gc = grads("cpu", "float64", transposed)
    rng0 = np.random.default_rng(5); gg = grads("cuda", "float64", transposed)
    for c, g in zip(gc, gg):
        assert np.abs(c - g).max() < 1e-7

# stress_torch_parity.py:150-171 -- tanh MLP x@W1 -> tanh -> @W2 -> mse, grads CPU vs CUDA
def mlp(device, dtype):
    r = np.random.default_rng(9)
    x = r.standard_normal((32, 20)); w1 = r.standard_normal((20, 16)) * .3; w2 = r.standard_normal((16, 4)) * .3
    tgt = r.standard_normal((32, 4))
    X = t(x, dtype, device); W1 = t(w1, dtype, device, True); W2 = t(w2, dtype, device, True); T = t(tgt, dtype, device)
    loss = X.op_matmul(W1).op_tanh().op_matmul(W2).op_mse_loss(T)
    loss.backward()
    return npy(W1.grad), npy(W2.grad), float(npy(loss).ravel()[0])

c = mlp("cpu", "float64"); g = mlp("cuda", "float64")
for x, y in zip(c[:2], g[:2]):
    np.testing.assert_allclose(y, x, rtol=1e-7, atol=1e-10)
c = mlp("cpu", "float32"); g = mlp("cuda", "float32")
for x, y in zip(c[:2], g[:2]):
    assert np.linalg.norm(x - y) / np.linalg.norm(x) < 1e-4

# half precision: two chained matmuls, CPU reference vs this library on the GPU.  (The reference's own
# tanh/mse backward kernels fail to launch for half types on the GPU, with or without this library,
# so the chain uses only matmul, mul and sum.)
def chain(device, dtype):
    r = np.random.default_rng(13)
    x = r.standard_normal((32, 24)); w1 = r.standard_normal((24, 16)) * .3; w2 = r.standard_normal((16, 8)) * .3
    wt = r.uniform(.5, 1.5, (32, 8))
    X = t(x, dtype, device); W1 = t(w1, dtype, device, True); W2 = t(w2, dtype, device, True); Wt = t(wt, dtype, device)
    loss = X.op_matmul(W1).op_matmul(W2).op_mul(Wt).op_sum_all()
    loss.backward()
    return npy(W1.grad), npy(W2.grad)

for dtype, tol in (("float16", 1e-2), ("bfloat16", 4e-2)):
    c = chain("cpu", dtype); g = chain("cuda", dtype)
    for x, y in zip(c, g):
        assert np.linalg.norm(x - y) / np.linalg.norm(x) < tol, (dtype, np.linalg.norm(x - y) / np.linalg.norm(x))

# test_half_precision_full.py:743-811 -- dtype / shape of half matmul + backward on CUDA
for dtype in ("float16", "bfloat16"):
    A = t(rng.standard_normal((8, 16)), dtype, "cuda", True); B = t(rng.standard_normal((16, 8)), dtype, "cuda", True)
    y = A.op_matmul(B)
    assert y.dtype == dtype and y.shape == (8, 8)
    y.op_sum_all().backward()
    assert A.grad.dtype == dtype and A.grad.shape == (8, 16) and B.grad.shape == (16, 8)

# grad accumulation over two uses of the same weight (LSTM-style weight sharing across steps)
def shared(device):
    r = np.random.default_rng(3)
    W = t(r.standard_normal((12, 12)) * .3, "float64", device, True)
    h = t(r.standard_normal((5, 12)), "float64", device)
    for _ in range(3):
        h = h.op_matmul(W).op_tanh()
    h.op_sum_all().backward()
    return npy(W.grad)

np.testing.assert_allclose(shared("cuda"), shared("cpu"), rtol=1e-7, atol=1e-10)

# stress_edge_cases.py:41-42, 193-194
for bad in (lambda: t(np.zeros((2, 3)), "float32", "cuda").op_matmul(t(np.zeros((4, 5)), "float32", "cuda")),
            lambda: t(np.zeros((2, 3)), "float32", "cpu").op_matmul(t(np.zeros((3, 5)), "float32", "cuda"))):
    try:
        bad()
        raise SystemExit("expected RuntimeError")
    except RuntimeError:
        pass

# new capability through the unchanged binding: broadcast-batched matmul
if interpose:
    a = rng.standard_normal((4, 6, 8)); b = rng.standard_normal((1, 8, 5))
    A = t(a, "float32", "cuda", True); B = t(b, "float32", "cuda", True)
    y = A.op_matmul(B)
    assert y.shape == (4, 6, 5)
    np.testing.assert_allclose(npy(y), a.astype(np.float32).astype(np.float64) @ b.astype(np.float32).astype(np.float64), rtol=1e-4, atol=1e-5)
    y.op_sum_all().backward()
    assert B.grad.shape == (1, 8, 5)
    np.testing.assert_allclose(npy(B.grad)[0], a.astype(np.float32).astype(np.float64).sum(0).sum(0)[:, None] * np.ones((8, 5)), rtol=1e-4, atol=1e-4)
    assert launches() - n0 >= 40, launches() - n0         # the GEMMs really ran in this library
    assert lib.rpb_device_status(0) == 0
print("DROPIN OK", launches() - n0)
