"""The public header compiles as plain C11 and a C program links against the library (CPU); on a GPU the
same program multiplies through rp_matmul_host and the autograd node."""
import os
import subprocess

import pytest

import recpulse_b200 as rpb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    rpb.load()
    exe = str(tmp_path / "abi_check")
    libdir = os.path.join(ROOT, "recpulse_b200")
    cmd = ["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "c", "abi_check.c"), "-o", exe, "-L", libdir, "-lrecpulse_b200",
           "-Wl,-rpath," + libdir, "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_c11_and_program_links(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "sm_100a" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_c_program_runs_the_path(tmp_path):
    exe = _build(tmp_path)
    r = subprocess.run([exe, "run"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "C ABI OK" in r.stdout, r.stdout + r.stderr
