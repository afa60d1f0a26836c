"""Randomised shapes, strides, batches and flags through rp_matmul_ex, every dtype, against a float64
reference of the widened inputs (rounded once to the storage dtype).  Seeded: the same cases every run."""
import numpy as np
import pytest

import recpulse_b200 as rpb
from test_gemm_gpu import run_ex
from helpers import rand_operand

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32", "float64"])
def test_random_problems(dtype):
    lib = rpb.load()
    rng = np.random.default_rng({"bfloat16": 101, "float16": 102, "float32": 103, "float64": 104}[dtype])
    align = {"bfloat16": 8, "float16": 8, "float32": 4, "float64": 2}[dtype]
    for case in range(40):
        m = int(rng.integers(1, 400)); k = int(rng.integers(1, 700)); n = int(rng.integers(1, 400))
        if rng.random() < 0.6:        # mostly tensor-core-addressable extents, sometimes anything
            m, k, n = [max(align, (v // align) * align) for v in (m, k, n)]
        batch = int(rng.choice([1, 1, 2, 5])); reduce = int(rng.choice([1, 1, 1, 3]))
        a_b = batch if rng.random() < 0.8 else 1; b_b = batch if rng.random() < 0.7 else 1
        a_r = reduce if rng.random() < 0.8 else 1; b_r = reduce if rng.random() < 0.8 else 1
        ta = bool(rng.random() < 0.5); tb = bool(rng.random() < 0.5)
        pad_a = int(rng.choice([0, 0, align, 3])); pad_b = int(rng.choice([0, 0, align, 5]))
        a = rand_operand(rng, (a_b, a_r, m, k), dtype); b = rand_operand(rng, (b_b, b_r, k, n), dtype, scale=1 / np.sqrt(k * reduce))
        c0 = rand_operand(rng, (max(a_b, b_b), m, n), dtype) if rng.random() < 0.3 else None
        run_ex(lib, dtype, a, b, ta=ta, tb=tb, pad_a=pad_a, pad_b=pad_b, c_init=c0)
    assert lib.rpb_device_status(0) == 0
