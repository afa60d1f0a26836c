#!/usr/bin/env python
"""Benchmark of the matmul forward + backward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one forward + backward of one matmul: C = A.B, dB = A^T.dC, dA = dC.B^T (both inputs
require grad).  The default workload is the row-sharded large GEMM, bf16 A[65536,8192] x B[8192,8192]
with fp32 accumulation: A's rows are split evenly over the N ranks (strong scaling, total work
fixed), B is replicated, the dB partials are all-reduced over NCCL overlapped with the dA GEMM.
Other workloads (--workload square4096 | bmm_fp16 | mlp_fp32 | lstm_fp32 | fp64_2048) run on one GPU.

Inputs are seeded synthetic data with the shapes and distributions of the named workload and
are larger than L2 (126 MB), so no L2 flush is needed between iterations.

One JSON line is printed by rank 0.  `value` times the kernels with inputs resident in HBM
(CUDA events on the launching stream, max over ranks); `e2e` times the same step through the C ABI
starting from pinned HOST buffers (H2D of A, B, dC and D2H of C, dA, dB inside the timed region);
`roofline` is the tcgen05 GEMM kernel against the measured cuBLAS bf16 peak; `cpu_baseline` is the
reference's own CPU matmul (compiled from its sources, oracle/_ref) on a bounded slab.
`--impl reference` times only that CPU implementation.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "matmul fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (dtype, batch, m, k, n, broadcast_b, shards)
    "rowsharded_65536x8192x8192": ("bfloat16", 1, 65536, 8192, 8192, False, True),
    "square4096": ("bfloat16", 1, 4096, 4096, 4096, False, False),
    "bmm_fp16": ("float16", 64, 512, 64, 512, True, True),
    "mlp_fp32": ("float32", 1, 128, 784, 256, False, False),
    "lstm_fp32": ("float32", 1, 64, 512, 2048, False, False),
    "fp64_2048": ("float64", 1, 2048, 2048, 2048, False, False),
}
DEFAULT_WORKLOAD = "rowsharded_65536x8192x8192"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    p.add_argument("--e2e-steps", type=int, default=3)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-graph", action="store_true", help="do not replay the step from a CUDA graph on launch-bound workloads")
    p.add_argument("--compare", action="store_true", help="also time torch.matmul (cuBLAS, warm handle) on the same step")
    p.add_argument("--comm-sms", type=int, default=16, help="SMs the dA GEMM leaves to the dB all-reduce (N > 1)")
    p.add_argument("--rows", type=int, default=0, help="override the row count M of the workload (profiling cases)")
    return p.parse_args()


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE forward-GEMM launch, from the ncu
# captures summarised under profiles/.  The default workload is too large to capture under the size rule,
# so its figure is the 8192-row capture scaled by the row count (A, C and the per-row-block re-reads of B
# all grow with the rows).
NCU_TRAFFIC_BYTES = {
    "rowsharded_65536x8192x8192": lambda rows: 1.2109e9 * rows / 8192.0,      # 1.083 GB read + 0.128 GB written
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"tflops": d["bf16_tflops_sustained"], "tflops_burst": d["bf16_tflops"], "hbm": d["hbm_gbs"], "src": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm": 6650.0, "src": "fallback"}


# --------------------------------------------------------------------------- CPU reference arm

def cpu_reference_matmul():
    """(callable(C, A, B, m, k, n, dtype_code) -> rc, kind): the reference's own rp_matmul on host
    memory when it was compiled from its sources, else the C oracle port."""
    so = os.path.join(ROOT, "oracle", "_ref", "recpulse_cuda.so")
    if os.path.exists(so):
        ref = C.CDLL(so)
        ref.rp_matmul.restype = C.c_int
        ref.rp_matmul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        return (lambda c, a, b, m, k, n, dt: ref.rp_matmul(c, a, b, m, k, n, dt, -1)), "reference"
    from oracle import oracle as O
    lib = O.lib()
    return (lambda c, a, b, m, k, n, dt: lib.orc_rp_matmul(c, a, b, m, k, n, dt)), "port"


def cpu_sample(workload, budget_s, steps=1, warmup=0):
    """Times fwd + dA + dB of a row slab of the workload on the reference's serial CPU loop.
    Returns (tflops, description, kind, per-step seconds)."""
    import numpy as np
    from oracle import oracle as O
    dtype, batch, m, k, n, _, _ = WORKLOADS[workload]
    code = {"float32": O.F32, "float64": O.F64, "float16": O.F16, "bfloat16": O.BF16}[dtype]
    fn, kind = cpu_reference_matmul()
    rng = np.random.default_rng(0)
    b = O.narrow(rng.standard_normal((k, n)), code)
    bt = np.ascontiguousarray(b.T)
    p = lambda x: x.ctypes.data_as(C.c_void_p)

    def run(rows):
        a = O.narrow(rng.standard_normal((rows, k)) / np.sqrt(k), code)
        dc = O.narrow(rng.standard_normal((rows, n)), code)
        at = np.ascontiguousarray(a.T)
        c = np.empty((rows, n), a.dtype); da = np.empty((rows, k), a.dtype); db = np.empty((k, n), a.dtype)
        t0 = time.perf_counter()
        assert fn(p(c), p(a), p(b), rows, k, n, code) == 0          # C  = A . B
        assert fn(p(da), p(dc), p(bt), rows, n, k, code) == 0       # dA = dC . B^T (B^T packed, as ops.c:6771 does)
        assert fn(p(db), p(at), p(dc), k, rows, n, code) == 0       # dB = A^T . dC
        return time.perf_counter() - t0

    total_rows = batch * m
    t1 = run(1)                                                     # probe: one row
    per_step_budget = budget_s / max(1, steps + warmup)
    rows = int(max(1, min(total_rows, per_step_budget / max(t1, 1e-6))))
    for _ in range(warmup):
        run(rows)
    times = [run(rows) for _ in range(steps)]
    dt = sum(times) / len(times)
    flops = 3 * 2.0 * rows * k * n
    desc = f"fwd+dA+dB of a {rows}-row slab ({rows}x{k}x{n} {dtype}) of {workload}, serial reference loop"
    return flops / dt / 1e12, desc, kind, dt


def run_reference_arm(args, rank):
    if rank != 0:
        return
    budget = 150.0
    tflops, desc, kind, dt = cpu_sample(args.workload, budget, steps=args.steps, warmup=args.warmup)
    dtype = WORKLOADS[args.workload][0]
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": {"bfloat16": "bf16", "float16": "f16", "float32": "f32", "float64": "f64"}[dtype],
        "data": "synthetic", "config": {"workload": args.workload, "sample": desc},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": 1, "kind": kind, "sample": desc},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_gpu_as_shipped(dtype_name, m, k, n, steps, fill=None):
    """The unmodified reference (oracle/_ref) on the GPU, as shipped: op_matmul + backward_matmul_fn through
    its own C entry points (cuBLAS handle created and destroyed per call, transposes materialised,
    cudaMalloc + memset per output).  `fill` = device pointers (A, B, dC) whose contents are copied into the
    reference's tensors, so it multiplies the same values as the other arms.  Returns ms per step, or None."""
    so = os.path.join(ROOT, "oracle", "_ref", "recpulse_cuda.so")
    if not os.path.exists(so):
        return None
    from recpulse_b200._lib import CTensor, GradFn, Meta
    ref = C.CDLL(so)
    libc = C.CDLL(None)
    libc.calloc.restype = C.c_void_p
    libc.calloc.argtypes = [C.c_size_t, C.c_size_t]
    TP = C.POINTER(CTensor)
    ref.zeros_tensor.restype = TP
    ref.zeros_tensor.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_void_p]
    ref.op_matmul.restype = TP
    ref.op_matmul.argtypes = [TP, TP]
    ref.backward_matmul_fn.restype = None
    ref.backward_matmul_fn.argtypes = [C.POINTER(GradFn), TP]
    ref.free_tensor.restype = None
    ref.free_tensor.argtypes = [TP]
    code = {"float32": 0, "float64": 1, "float16": 2, "bfloat16": 3}[dtype_name]

    def make(shape, grad):
        meta = None
        if grad:
            meta = libc.calloc(1, C.sizeof(Meta))
            mm = C.cast(meta, C.POINTER(Meta)).contents
            mm.is_leaf = True; mm.requires_grad = True
        return ref.zeros_tensor(code, 0, 2, (C.c_int * 2)(*shape), meta)

    a, b, g = make((m, k), True), make((k, n), True), make((m, n), False)
    if not a or not b or not g:
        return None
    if fill:
        ref.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        es = {"float32": 4, "float64": 8, "float16": 2, "bfloat16": 2}[dtype_name]
        for t, src, cnt in ((a, fill[0], m * k), (b, fill[1], k * n), (g, fill[2], m * n)):
            ref.cudaMemcpy(t.contents.data, src, cnt * es, 3)          # device to device

    def step():
        out = ref.op_matmul(a, b)
        ref.backward_matmul_fn(out.contents.metadata.contents.grad_fn, g)
        ref.free_tensor(out)
        for t in (a, b):                                   # drop the grads so every step allocates like the first
            mt = t.contents.metadata.contents
            if mt.grad:
                ref.free_tensor(mt.grad)
                mt.grad = None

    import torch
    step(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps * 1e3
    for t in (a, b, g):
        ref.free_tensor(t)
    return dt


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- GPU arm

def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import recpulse_b200
    from recpulse_b200 import _lib
    from recpulse_b200.sharded import RowShardedMatmul, cuda_gemm, row_partition

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the matmul path has no CPU implementation)")
    lib = recpulse_b200.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if args.gpus != world and rank == 0 and world > 1:
        print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE {world}; using WORLD_SIZE", file=sys.stderr)
    n_gpus = world

    dtype_name, batch, m, k, n, bcast_b, shards = WORKLOADS[args.workload]
    if args.rows:
        batch, m = 1, args.rows
    tdtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "float64": torch.float64}[dtype_name]
    es = torch.empty((), dtype=tdtype).element_size()
    rows_total = batch * m            # a broadcast-batched product folds its batch into the rows of A
    if world > 1 and not shards:
        raise SystemExit(f"workload {args.workload} is single-GPU (replicas only)")
    r0, r1 = row_partition(rows_total, world, rank)
    rows = r1 - r0

    gen = torch.Generator(device=dev); gen.manual_seed(1234 + rank)
    a_scale = 1.0 / np.sqrt(k) if dtype_name == "bfloat16" else 1.0
    A = (torch.randn((rows, k), generator=gen, device=dev, dtype=torch.float32) * a_scale).to(tdtype)
    gen_b = torch.Generator(device=dev); gen_b.manual_seed(99)
    Bm = (torch.randn((k, n), generator=gen_b, device=dev, dtype=torch.float32) * (0.125 if bcast_b else 1.0)).to(tdtype)
    dC = torch.randn((rows, n), generator=gen, device=dev, dtype=torch.float32).to(tdtype)
    Cc = torch.empty((rows, n), device=dev, dtype=tdtype)
    dA = torch.empty((rows, k), device=dev, dtype=tdtype)
    dB = torch.empty((k, n), device=dev, dtype=tdtype)

    op = RowShardedMatmul(Bm, gemm=cuda_gemm, comm_sms=args.comm_sms)

    def step():
        op.forward(A, out=Cc)
        op.backward(A, dC, da_out=dA, db_out=dB)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    if lib.rpb_device_status(local_rank) != 0:
        raise SystemExit("bench.py: a bounded wait inside the tcgen05 kernel ran out during warm-up")

    # ---- timed region: K steps, kernels only, inputs resident in HBM
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = lib.rpb_launch_count()
    stream = torch.cuda.current_stream(dev)
    resident = (2 * rows * k + 2 * k * n + 2 * rows * n) * es
    flush = None
    if resident < (512 << 20):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB of L2
    # Launch-bound workloads (a few microseconds of GPU work per launch) are replayed from a CUDA graph, the way
    # a training loop would run them: the host cost of issuing each launch disappears from the timed region.
    graph = None
    launches_per_step = None
    if flush is not None and world == 1 and not args.no_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        n0 = lib.rpb_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
        launches_per_step = lib.rpb_launch_count() - n0
        torch.cuda.synchronize(dev)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(dev)
    step_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    # per-launch events for the roofline of the dominant kernel (forward GEMM of every step)
    fwd_ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        if flush is not None:
            flush.fill_(i & 1)                      # evict the operands from L2 (outside the timed events)
        step_ev[i][0].record(stream)
        if graph is not None:
            graph.replay()
            fwd_ev[i].record(stream)
        else:
            op.forward(A, out=Cc)
            fwd_ev[i].record(stream)
            op.backward(A, dC, da_out=dA, db_out=dB)
        step_ev[i][1].record(stream)
    barrier()
    elapsed_ms = sum(a.elapsed_time(b) for a, b in step_ev)
    launches = lib.rpb_launch_count() - launches0
    if graph is not None:
        launches = launches_per_step * args.steps          # counted while capturing; each replay re-issues them
    clocks = sampler.stop() if rank == 0 else None
    fwd_ms = sum(step_ev[i][0].elapsed_time(fwd_ev[i]) for i in range(args.steps)) / args.steps
    if graph is not None:
        fwd_ms = elapsed_ms / args.steps        # the replayed step is one unit: the roofline below is per STEP
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    if lib.rpb_device_status(local_rank) != 0:
        raise SystemExit("bench.py: a bounded wait inside the tcgen05 kernel ran out")

    flops_step = 3 * 2.0 * rows_total * k * n
    ms_per_step = elapsed_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e12

    # ---- optional: the same three GEMMs through torch.matmul (cuBLAS with a warm handle), for context only
    cublas = None
    if args.compare and world == 1:
        def cublas_step():
            torch.matmul(A, Bm, out=Cc); torch.matmul(A.t(), dC, out=dB); torch.matmul(dC, Bm.t(), out=dA)
        for _ in range(3):
            cublas_step()
        tot = 0.0
        for i in range(args.steps):
            if flush is not None:
                flush.fill_(i & 1)
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record(stream); cublas_step(); c1.record(stream)
            torch.cuda.synchronize(dev)
            tot += c0.elapsed_time(c1)
        cublas = {"tflops": flops_step / (tot / args.steps * 1e-3) / 1e12, "ms_per_step": tot / args.steps,
                  "what": "torch.matmul x3 (cuBLAS, warm handle, outputs preallocated)"}
        ref_ms = reference_gpu_as_shipped(dtype_name, rows, k, n, min(args.steps, 5), fill=(A.data_ptr(), Bm.data_ptr(), dC.data_ptr()))
        if ref_ms:
            cublas["reference_as_shipped_ms_per_step"] = ref_ms
            cublas["reference_as_shipped_tflops"] = flops_step / (ref_ms * 1e-3) / 1e12
        # the same step through this library's autograd node (allocation + synchronisation included)
        import recpulse_b200 as rpb
        dn = dtype_name
        def to_lib(t, grad):                                         # same operand values as the kernel-only arm
            host = t.contiguous().view(torch.int16 if es == 2 else t.dtype).cpu().numpy()
            return rpb.Tensor.from_numpy(host.view(np.uint16) if es == 2 else host, dtype=dn, requires_grad=grad)
        hA, hB, hG = to_lib(A, True), to_lib(Bm, True), to_lib(dC, False)
        def node_step():
            y = hA.op_matmul(hB); y.backward(hG)
            for t in (hA, hB):
                mt = t._t.metadata.contents
                if mt.grad:
                    lib.rpb_tensor_release(mt.grad); mt.grad = None
        node_step(); torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(min(args.steps, 5)):
            node_step()
        torch.cuda.synchronize(dev)
        cublas["this_library_node_ms_per_step"] = (time.perf_counter() - t0) / min(args.steps, 5) * 1e3

    # ---- end to end from pinned host buffers through the C ABI
    e2e = None
    if not args.no_e2e:
        hA = torch.empty((rows, k), dtype=tdtype).pin_memory(); hA.copy_(A)
        hB = torch.empty((k, n), dtype=tdtype).pin_memory(); hB.copy_(Bm)
        hdC = torch.empty((rows, n), dtype=tdtype).pin_memory(); hdC.copy_(dC)
        hC = torch.empty((rows, n), dtype=tdtype).pin_memory()
        hdA = torch.empty((rows, k), dtype=tdtype).pin_memory()
        hdB = torch.empty((k, n), dtype=tdtype).pin_memory()

        code = {"float32": 0, "float64": 1, "float16": 2, "bfloat16": 3}[dtype_name]
        ptr = lambda t: C.c_void_p(t.data_ptr())

        def e2e_step():
            # the library's host-buffer entry point: chunked H2D of A and dC, GEMMs and D2H of C and dA
            # overlapped on three streams, dB as one GEMM at the end; returns when the host buffers are filled
            rc = lib.rp_matmul_fwdbwd_host(ptr(hC), ptr(hdA), ptr(hdB), ptr(hA), ptr(hB), ptr(hdC), rows, k, n, code,
                                           local_rank, 0)
            if rc != 0:
                raise SystemExit("bench.py: rp_matmul_fwdbwd_host failed")
            if world > 1:                          # dB partials of the ranks are summed on the host-visible copy
                dB.copy_(hdB, non_blocking=True)
                dist.all_reduce(dB)
                hdB.copy_(dB, non_blocking=True)
                torch.cuda.synchronize(dev)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        e2e_ms = (time.perf_counter() - t0) / args.e2e_steps * 1e3
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        h2d = (rows * k + k * n + rows * n) * es
        d2h = (rows * n + rows * k + k * n) * es
        e2e = {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "steps": args.e2e_steps,
               "pcie_gbs_each_way": max(h2d, d2h) / (e2e_ms * 1e-3) / 1e9,
               "api": "rp_matmul_fwdbwd_host (C ABI, pinned host buffers, wall clock around the synchronous call)"}

    if rank == 0:
        pk = peaks()
        half = dtype_name in ("bfloat16", "float16")
        flops_fwd = 2.0 * rows * k * n                               # one launch of the dominant kernel on this rank
        bytes_unit = (rows * k + k * n + rows * n) * es              # algorithmic bytes of that launch
        unit = "forward GEMM launch"
        if graph is not None:                                        # whole replayed step: three GEMMs
            flops_fwd *= 3; bytes_unit *= 3; unit = "fwd+bwd step replayed from a CUDA graph"
        traffic_fn = NCU_TRAFFIC_BYTES.get(args.workload)
        traffic = traffic_fn(rows) if traffic_fn else None
        if half and args.workload != "bmm_fp16":
            achieved = flops_fwd / (fwd_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "rpb_umma::gemm_kernel (" + unit + ")", "achieved": achieved,
                    "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                    "peak_source": pk["src"] + " cuBLAS bf16, sustained", "traffic": traffic,
                    "traffic_note": "ncu DRAM bytes of one forward launch at 8192 rows, scaled by rows" if traffic else None,
                    "algorithmic_bytes": bytes_unit,
                    "avg_launch_ms": fwd_ms}
        else:
            achieved = bytes_unit / (fwd_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": unit, "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                    "frac": achieved / pk["hbm"], "peak_source": pk["src"] + " copy bandwidth", "traffic": None,
                    "avg_launch_ms": fwd_ms}
        cpu = None
        if n_gpus == 1 and not args.no_cpu_baseline:
            tf, desc, kind, _ = cpu_sample(args.workload, 20.0)
            cpu = {"value": tf, "unit": UNIT, "cores": 1, "kind": kind, "sample": desc}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"bfloat16": "bf16", "float16": "f16", "float32": "f32", "float64": "f64"}[dtype_name],
            "data": "synthetic",
            "config": {"workload": args.workload, "m": rows_total, "k": k, "n": n, "rows_per_gpu": rows,
                       "parallelism": f"rows of A over {n_gpus} GPU(s), B replicated, dB all-reduced" if n_gpus > 1 else "single GPU",
                       "l2": "inputs larger than L2, no flush" if flush is None else "L2 flushed (256 MB write) before every step, outside the timed events",
                       "accumulate": "fp32", "cuda_graph": graph is not None},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roof, "cpu_baseline": cpu,
            "pct_of_nominal_dense_peak": value / (2250.0 * n_gpus) if half else None,
        }
        if cublas:
            line["cublas_same_step"] = cublas
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
