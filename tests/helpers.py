"""Shared helpers of the parity tests: seeded inputs, error metrics, C-ABI shortcuts."""
from __future__ import annotations

import ctypes as C

import numpy as np

from oracle import oracle as O

CODE = {"float32": O.F32, "float64": O.F64, "float16": O.F16, "bfloat16": O.BF16}

# Tolerances of the path's contract.
FP64_REL = 1e-12        # max |x-ref| / max(|ref|, rms(ref))
FP32_SQRTK = 1e-5       # max |x-ref| / (sqrt(K) * rms(ref))  (the stricter of the two normalisations)
HALF_FROB = 1e-2        # ||x-ref||_F / ||ref||_F, same dtype
# What fp32 accumulation + one rounding should actually achieve (asserted too).
HALF_FROB_TIGHT = {"bfloat16": 4e-3, "float16": 6e-4}


def rand_operand(rng, shape, dtype, scale=1.0, dist="normal"):
    """Seeded values narrowed ONCE on the host to storage bits of `dtype`."""
    x = rng.standard_normal(shape) if dist == "normal" else rng.uniform(-1, 1, shape)
    return O.narrow(x * scale, CODE[dtype])


def f64(x, dtype):
    return O.to_f64(np.asarray(x), CODE[dtype])


def check_close(got, ref, dtype, k, what="", tight=True):
    """`tight=False` for results that sit behind several roundings of the 16-bit type in the reference's
    composition (a chain of nodes), where only the path's stated tolerance applies."""
    g = f64(got, dtype); r = f64(ref, dtype)
    assert g.shape == r.shape, (what, g.shape, r.shape)
    err = np.abs(g - r)
    rms = float(np.sqrt(np.mean(r * r))) or 1.0
    if dtype == "float64":
        rel = float((err / np.maximum(np.abs(r), rms)).max())
        assert rel <= FP64_REL, f"{what}: fp64 rel err {rel:.3e}"
    elif dtype == "float32":
        e1 = float(err.max() / (np.sqrt(k) * rms))
        assert e1 <= FP32_SQRTK, f"{what}: fp32 err/(sqrt(K)*rms) {e1:.3e}"
    else:
        fro = float(np.linalg.norm(g - r) / (np.linalg.norm(r) or 1.0))
        assert fro <= HALF_FROB, f"{what}: {dtype} rel Frobenius {fro:.3e}"
        assert not tight or fro <= HALF_FROB_TIGHT[dtype], f"{what}: {dtype} rel Frobenius {fro:.3e} (tight bound)"


def gemm_ex(lib, a_dev, b_dev, c_dev, g, dtype, device=0, stream=None):
    rc = lib.rp_matmul_ex(C.c_void_p(c_dev), C.c_void_p(a_dev), C.c_void_p(b_dev), C.byref(g), CODE[dtype], device,
                          C.c_void_p(stream) if stream else None)
    assert rc == 0, "rp_matmul_ex failed"
