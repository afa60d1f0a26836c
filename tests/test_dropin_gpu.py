"""Drop-in check: the unmodified RecPulse extension with this library loaded in front of it."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "recpulse_cuda.so")


@pytest.mark.gpu
def test_reference_binding_runs_on_this_library():
    if not os.path.exists(REF_SO):
        pytest.skip("compiled reference (oracle/_ref/recpulse_cuda.so) not present")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "dropin_child.py")], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and "DROPIN OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_host_tensors_pass_through_to_the_reference():
    """Without a GPU: with the library interposed, CPU tensors still reach RecPulse's own host code."""
    if not os.path.exists(REF_SO):
        pytest.skip("compiled reference not present")
    code = (
        "import sys, numpy as np; sys.path.insert(0, %r); import recpulse_b200; lib = recpulse_b200.load(global_scope=True);"
        "sys.path.insert(0, %r); import recpulse_cuda as rp;"
        "a = rp.from_numpy(np.arange(6, dtype=np.float64).reshape(2, 3)); a.requires_grad_(True);"
        "b = rp.from_numpy(np.arange(6, dtype=np.float64).reshape(3, 2));"
        "y = a.op_matmul(b); y.op_sum_all().backward();"
        "assert y.to_numpy().tolist() == [[10.0, 13.0], [28.0, 40.0]], y.to_numpy();"
        "assert a.grad.to_numpy().tolist() == [[1.0, 5.0, 9.0]] * 2;"
        "assert lib.rpb_launch_count() == 0; print('PASS')" % (ROOT, os.path.dirname(REF_SO)))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,shape", [("bfloat16", (1024, 1024, 1024)), ("float16", (1024, 1024, 1024)),
                                         ("bfloat16", (2048, 4096, 1024)), ("float16", (1536, 2048, 3072)),
                                         ("bfloat16", (4096, 4096, 4096))])
def test_same_dtype_parity_against_the_reference_gpu_path(tmp_path, dtype, shape):
    """float16 / bfloat16 forward and both gradients against the reference ON THE GPU in the same dtype (its cuBLAS
    calls, functional/functional_device.cu:1029-1057), through the reference's own binding in two child processes:
    alone, and with this library in front.  Relative Frobenius error <= 1e-2 for C, dA and dB."""
    import numpy as np
    if not os.path.exists(REF_SO):
        pytest.skip("compiled reference (oracle/_ref/recpulse_cuda.so) not present")
    m, k, n = shape
    outs = {}
    for mode in ("reference", "interposed"):
        path = str(tmp_path / f"{mode}.npz")
        cmd = [sys.executable, os.path.join(ROOT, "tests", "ref_gpu_child.py"), path, dtype, str(m), str(k), str(n)]
        if mode == "interposed":
            cmd.append("--interpose")
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0 and "REF_GPU_CHILD OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
        outs[mode] = np.load(path)
    assert int(outs["interposed"]["launches"]) >= 3 and int(outs["reference"]["launches"]) == 0
    for key in ("c", "da", "db"):
        ref = outs["reference"][key].astype(np.float64); got = outs["interposed"][key].astype(np.float64)
        assert np.isfinite(ref).all() and np.isfinite(got).all(), key
        err = np.linalg.norm(got - ref) / np.linalg.norm(ref)
        assert err <= 1e-2, (dtype, shape, key, err)
