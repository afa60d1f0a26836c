"""Generate tests/golden/{matmul,linear,lstm_gates,gru_cell,conv2d}_golden.npz from the UNMODIFIED reference.

Run in a container where the reference tree is mounted and compiled by
``make -C oracle ref`` (produces oracle/_ref/recpulse_cuda.so):

    python tests/golden/make_golden.py

Every case runs the reference's own CPU ``op_matmul`` + ``backward()`` through
its CPython binding (python/tensor_python.c) and stores inputs and outputs as
raw storage bits (float16/bfloat16 as uint16), so the fixtures can be replayed
without the reference.  The upstream gradient dC is injected as
``loss = sum(y * w)``, whose backward hands ``w`` to ``backward_matmul_fn``
unchanged (1 * w is exact in every dtype).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
import recpulse_cuda as rp  # noqa: E402

DT = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "bfloat16": np.float32}


def to_rp(x64, dtype):
    """float64 numpy -> CPU reference tensor of `dtype`, narrowed by the reference itself."""
    if dtype == "bfloat16":
        return rp.from_numpy(np.ascontiguousarray(x64, np.float32)).to(dtype="bfloat16")
    return rp.from_numpy(np.ascontiguousarray(x64.astype(DT[dtype])))


def bits(t):
    """reference tensor -> numpy storage bits."""
    dt = t.dtype
    if dt == "bfloat16":
        f = t.to(dtype="float32").to_numpy()
        return (np.ascontiguousarray(f).view(np.uint32) >> 16).astype(np.uint16)
    a = np.ascontiguousarray(t.to_numpy())
    return a.view(np.uint16) if dt == "float16" else a


def run_case(name, dtype, m, k, n, rng, ta=False, tb=False, twice=False, scale=1.0):
    a64 = rng.uniform(-1, 1, (k, m) if ta else (m, k)) * scale
    b64 = rng.uniform(-1, 1, (n, k) if tb else (k, n)) * scale
    w64 = rng.uniform(-1, 1, (m, n))
    a = to_rp(a64, dtype); b = to_rp(b64, dtype); w = to_rp(w64, dtype)
    a.requires_grad_(True); b.requires_grad_(True)
    av = a.transpose(0, 1) if ta else a
    bv = b.transpose(0, 1) if tb else b
    y = av.op_matmul(bv)
    loss = y.op_mul(w).op_sum_all()
    keep = [y, loss]
    if twice:            # second use of the same leaves: grads accumulate through rp_add
        y2 = av.op_matmul(bv)
        l2 = y2.op_mul(w).op_sum_all()
        loss = loss.op_add(l2)
        keep += [y2, l2, loss]
    loss.backward()
    out = {
        "a": bits(a), "b": bits(b), "w": bits(w), "c": bits(y),
        "da": bits(a.grad), "db": bits(b.grad),
        "meta": np.array([m, k, n, int(ta), int(tb), int(twice)], np.int64),
    }
    return {f"{name}/{dtype}/{key}": val for key, val in out.items()}


def run_linear(name, dtype, m, k, n, rng):
    """x @ W + b exactly as recpulse/module.py:110-114 composes it, with loss = sum(y * w)."""
    x64 = rng.uniform(-1, 1, (m, k)); w64 = rng.uniform(-1, 1, (k, n)) / np.sqrt(k)
    b64 = rng.uniform(-1, 1, (n,)); g64 = rng.uniform(-1, 1, (m, n))
    x = to_rp(x64, dtype); w = to_rp(w64, dtype); b = to_rp(b64, dtype); g = to_rp(g64, dtype)
    for t in (x, w, b):
        t.requires_grad_(True)
    y = x.op_matmul(w).op_add(b)
    loss = y.op_mul(g).op_sum_all()
    loss.backward()
    out = {"x": bits(x), "w": bits(w), "b": bits(b), "g": bits(g), "y": bits(y),
           "dx": bits(x.grad), "dw": bits(w.grad), "db": bits(b.grad)}
    return {f"{name}/{dtype}/{key}": val for key, val in out.items()}


def run_lstm_gates(name, dtype, m, kx, kh, hidden, rng):
    """The gate block of LSTMCell.forward (recpulse/module.py:289-300) with one bias, loss = sum(act * g)."""
    n = 4 * hidden
    x64 = rng.uniform(-1, 1, (m, kx)); w64 = rng.uniform(-1, 1, (kx, n)) / np.sqrt(kx)
    h64 = rng.uniform(-1, 1, (m, kh)); u64 = rng.uniform(-1, 1, (kh, n)) / np.sqrt(kh)
    b64 = rng.uniform(-1, 1, (n,)); g64 = rng.uniform(-1, 1, (m, n))
    x = to_rp(x64, dtype); w = to_rp(w64, dtype); h = to_rp(h64, dtype); u = to_rp(u64, dtype); b = to_rp(b64, dtype)
    for t in (x, w, h, u, b):
        t.requires_grad_(True)
    gates = x.op_matmul(w).op_add(h.op_matmul(u)).op_add(b)
    i_g, f_g, g_g, o_g = gates.chunk(4, 1)
    acts = [i_g.op_sigmoid(), f_g.op_sigmoid(), g_g.op_tanh(), o_g.op_sigmoid()]
    gs = [to_rp(g64[:, q * hidden:(q + 1) * hidden], dtype) for q in range(4)]
    keep = [gates, i_g, f_g, g_g, o_g] + acts + gs
    loss = None
    for a, g in zip(acts, gs):
        term = a.op_mul(g).op_sum_all()
        keep.append(term)
        loss = term if loss is None else loss.op_add(term)
        keep.append(loss)
    loss.backward()
    out = {"x": bits(x), "w": bits(w), "h": bits(h), "u": bits(u), "b": bits(b),
           "g": np.concatenate([bits(g) for g in gs], axis=1), "y": np.concatenate([bits(a) for a in acts], axis=1),
           "dx": bits(x.grad), "dw": bits(w.grad), "dh": bits(h.grad), "du": bits(u.grad), "db": bits(b.grad)}
    return {f"{name}/{dtype}/{key}": val for key, val in out.items()}


def run_gru_cell(name, dtype, m, kx, hidden, rng, bias=True):
    """One step of GRUCell.forward (recpulse/module.py:329-348), op by op as the module composes it,
    with loss = sum(h_next * g)."""
    n = 3 * hidden
    x64 = rng.uniform(-1, 1, (m, kx)); wi64 = rng.uniform(-1, 1, (kx, n)) / np.sqrt(kx)
    h64 = rng.uniform(-1, 1, (m, hidden)); wh64 = rng.uniform(-1, 1, (hidden, n)) / np.sqrt(hidden)
    bi64 = rng.uniform(-1, 1, (n,)); bh64 = rng.uniform(-1, 1, (n,)); g64 = rng.uniform(-1, 1, (m, hidden))
    x = to_rp(x64, dtype); wi = to_rp(wi64, dtype); h = to_rp(h64, dtype); wh = to_rp(wh64, dtype)
    bi = to_rp(bi64, dtype); bh = to_rp(bh64, dtype); g = to_rp(g64, dtype)
    leaves = [x, wi, h, wh] + ([bi, bh] if bias else [])
    for t in leaves:
        t.requires_grad_(True)
    gi = x.op_matmul(wi); gh = h.op_matmul(wh)
    if bias:
        gi = gi.op_add(bi); gh = gh.op_add(bh)
    i_r, i_z, i_n = gi.chunk(3, 1)
    h_r, h_z, h_n = gh.chunk(3, 1)
    r = i_r.op_add(h_r).op_sigmoid()
    z = i_z.op_add(h_z).op_sigmoid()
    nn = i_n.op_add(r.op_mul(h_n)).op_tanh()
    h_next = z.op_rsub_scalar(1.0).op_mul(nn).op_add(z.op_mul(h))
    loss = h_next.op_mul(g).op_sum_all()
    loss.backward()
    out = {"x": bits(x), "wi": bits(wi), "h": bits(h), "wh": bits(wh), "g": bits(g), "hn": bits(h_next),
           "dx": bits(x.grad), "dwi": bits(wi.grad), "dh": bits(h.grad), "dwh": bits(wh.grad),
           "meta": np.array([m, kx, hidden, int(bias)], np.int64)}
    if bias:
        out.update({"bi": bits(bi), "bh": bits(bh), "dbi": bits(bi.grad), "dbh": bits(bh.grad)})
    return {f"{name}/{dtype}/{key}": val for key, val in out.items()}


def run_conv2d(name, dtype, n, c, hh, ww, oc, kh, kw, stride, pad, dil, rng):
    """op_conv2d without bias + backward (ops/ops.c:4480-4770) on the CPU, loss = sum(y * g).  float32 / float64 only:
    the reference's host conv2d leaves its transposed buffers unset for the 16-bit types."""
    x64 = rng.uniform(-1, 1, (n, c, hh, ww)); w64 = rng.uniform(-1, 1, (oc, c, kh, kw)) / np.sqrt(c * kh * kw)
    x = to_rp(x64, dtype); w = to_rp(w64, dtype)
    x.requires_grad_(True); w.requires_grad_(True)
    y = x.op_conv2d(w, None, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1])
    g = to_rp(rng.uniform(-1, 1, tuple(y.shape)), dtype)
    loss = y.op_mul(g).op_sum_all()
    loss.backward()
    out = {"x": bits(x), "w": bits(w), "g": bits(g), "y": bits(y), "dx": bits(x.grad), "dw": bits(w.grad),
           "meta": np.array([n, c, hh, ww, oc, kh, kw, *stride, *pad, *dil], np.int64)}
    return {f"{name}/{dtype}/{key}": val for key, val in out.items()}


def main():
    rng = np.random.default_rng(20240607)
    store = {}
    shapes = [(3, 4, 5), (16, 32, 8), (1, 7, 1), (64, 64, 64), (33, 65, 17), (2, 300, 3)]
    for dtype in DT:
        for (m, k, n) in shapes:
            store.update(run_case(f"nn_{m}x{k}x{n}", dtype, m, k, n, rng))
        store.update(run_case("ta_12x20x9", dtype, 12, 20, 9, rng, ta=True))
        store.update(run_case("tb_12x20x9", dtype, 12, 20, 9, rng, tb=True))
        store.update(run_case("tatb_24x40x16", dtype, 24, 40, 16, rng, ta=True, tb=True))
        store.update(run_case("acc_10x14x6", dtype, 10, 14, 6, rng, twice=True))
        store.update(run_case("big_40x130x50", dtype, 40, 130, 50, rng, scale=4.0))
    np.savez_compressed(os.path.join(HERE, "matmul_golden.npz"), **store)
    print("cases:", len(store) // 7)
    lin = {}
    rng = np.random.default_rng(20240608)
    for dtype in DT:
        for (m, k, n) in [(5, 7, 3), (32, 48, 16), (17, 33, 40)]:
            lin.update(run_linear(f"linear_{m}x{k}x{n}", dtype, m, k, n, rng))
    np.savez_compressed(os.path.join(HERE, "linear_golden.npz"), **lin)
    print("linear cases:", len(lin) // 8)
    gates = {}
    rng = np.random.default_rng(20240609)
    for dtype in DT:
        for (m, kx, kh, hidden) in [(3, 5, 4, 2), (16, 24, 8, 8), (9, 33, 17, 5)]:
            gates.update(run_lstm_gates(f"gates_{m}x{kx}x{kh}x{hidden}", dtype, m, kx, kh, hidden, rng))
    np.savez_compressed(os.path.join(HERE, "lstm_gates_golden.npz"), **gates)
    print("lstm gate cases:", len(gates) // 12)
    gru = {}
    rng = np.random.default_rng(20240610)
    for dtype in DT:
        for (m, kx, hidden, bias) in [(3, 5, 2, True), (16, 24, 8, True), (9, 33, 5, False), (7, 12, 16, True)]:
            gru.update(run_gru_cell(f"gru_{m}x{kx}x{hidden}_{'b' if bias else 'nb'}", dtype, m, kx, hidden, rng, bias))
    np.savez_compressed(os.path.join(HERE, "gru_cell_golden.npz"), **gru)
    print("gru cell cases:", sum(1 for k in gru if k.endswith("/meta")))
    conv = {}
    rng = np.random.default_rng(20240611)
    for dtype in ("float32", "float64"):
        conv.update(run_conv2d("conv_3x3_same", dtype, 2, 3, 7, 6, 4, 3, 3, (1, 1), (1, 1), (1, 1), rng))
        conv.update(run_conv2d("conv_2x3_strided_dilated", dtype, 3, 2, 9, 8, 5, 2, 3, (2, 1), (0, 1), (1, 2), rng))
        conv.update(run_conv2d("conv_1x1", dtype, 2, 8, 5, 5, 16, 1, 1, (1, 1), (0, 0), (1, 1), rng))
        conv.update(run_conv2d("conv_5x5_stride2", dtype, 4, 3, 12, 12, 8, 5, 5, (2, 2), (2, 2), (1, 1), rng))
    np.savez_compressed(os.path.join(HERE, "conv2d_golden.npz"), **conv)
    print("conv2d cases:", sum(1 for k in conv if k.endswith("/meta")))


if __name__ == "__main__":
    main()
