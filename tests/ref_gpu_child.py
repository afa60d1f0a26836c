"""Child process of the same-dtype parity test: one matmul forward + backward in float16 / bfloat16 on the GPU
through the reference's own CPython binding -- either the UNMODIFIED reference alone (its cuBLAS path,
functional/functional_device.cu:1029-1057) or the same binding with librecpulse_b200.so loaded in front of it --
on seeded inputs that the reference itself narrows, so both runs multiply identical bits.

    python tests/ref_gpu_child.py OUT.npz DTYPE M K N [--interpose]
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
out_path, dtype, m, k, n = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), int(sys.argv[5])
interpose = "--interpose" in sys.argv
lib = None
if interpose:
    import recpulse_b200
    lib = recpulse_b200.load(global_scope=True)          # same effect as LD_PRELOAD
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
import recpulse_cuda as rp  # noqa: E402


def t(x, grad=False):
    if dtype == "bfloat16":
        r = rp.from_numpy(np.ascontiguousarray(x, np.float32)).to(dtype="bfloat16")
    else:
        r = rp.from_numpy(np.ascontiguousarray(x.astype(np.float16)))
    r = r.to(device="cuda")
    if grad:
        r.requires_grad_(True)
    return r


def f32(x):
    return np.asarray(x.to(device="cpu").to(dtype="float32").to_numpy(), np.float32)


rng = np.random.default_rng(1000 + m + k + n)
a = rng.standard_normal((m, k), dtype=np.float32) / np.float32(np.sqrt(k))
b = rng.standard_normal((k, n), dtype=np.float32)
w = rng.standard_normal((m, n), dtype=np.float32)
A, B, W = t(a, True), t(b, True), t(w)
n0 = lib.rpb_launch_count() if lib else 0
y = A.op_matmul(B)
loss = y.op_mul(W).op_sum_all()          # its backward hands W to backward_matmul_fn unchanged
loss.backward()
launches = (lib.rpb_launch_count() - n0) if lib else 0
if interpose:
    assert launches >= 3, "the library's kernels did not run"
    assert lib.rpb_device_status(0) == 0
np.savez(out_path, c=f32(y), da=f32(A.grad), db=f32(B.grad), launches=launches)
print("REF_GPU_CHILD OK", dtype, m, k, n, "interposed" if interpose else "reference", launches)
