#!/usr/bin/env python
"""Benchmark of the matmul forward + backward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one forward + backward of one matmul: C = A.B, dB = A^T.dC, dA = dC.B^T (both inputs
require grad).  The default workload is the row-sharded large GEMM, bf16 A[65536,8192] x B[8192,8192]
with fp32 accumulation: A's rows are split evenly over the N ranks (strong scaling, total work
fixed), B is replicated, the dB partials are reduced over NCCL by the library itself (float32 on
the wire, one rounding) while the dA GEMM runs.  Every data-path call goes through the C ABI of
librecpulse_b200.so; torch supplies device buffers, streams and the launcher's process group
(barriers, the max over ranks of the timings, the rendezvous id).

Inputs are seeded synthetic data with the shapes and distributions of the named workload.  Workloads
larger than L2 (126 MB) need no flush between iterations; the small ones are flushed before every
step and replayed from a CUDA graph.

One JSON line is printed by rank 0:
  value        kernels only, inputs resident in HBM (CUDA events on the launching stream, max over ranks)
  e2e          the same step through the C ABI from pinned HOST buffers, copies inside the timed region
  roofline     the forward GEMM launches against the measured cuBLAS bf16 peaks (burst and sustained)
  parity_check sampled rows of C and dA against the CPU oracle, sampled entries of (the reduced) dB
               against float64 dot products, and the column-sum identities over every tile; a failed
               check makes the run exit non-zero
  workloads    the other configurations: at N = 1 bf16 4096^3, the fp16 broadcast-batched product, fp64
               2048^3 and the two float32 layer GEMMs; at N > 1 the batch-sharded fp16 product and the
               default workload with the all-gather of C inside the step
  cpu_baseline the reference's own CPU matmul (compiled from its sources) on a bounded slab
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
SHORT = {"bfloat16": "bf16", "float16": "f16", "float32": "f32", "float64": "f64"}
CODE = {"float32": 0, "float64": 1, "float16": 2, "bfloat16": 3}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(WORKLOADS))
    p.add_argument("--e2e-steps", type=int, default=10)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-parity", action="store_true", help="skip the output check after the timed region")
    p.add_argument("--no-workloads", action="store_true", help="time only --workload, not the other configurations")
    p.add_argument("--no-graph", action="store_true", help="do not replay the step from a CUDA graph on launch-bound workloads")
    p.add_argument("--compare", action="store_true", help="also time the reference as shipped and the node path on the same step")
    p.add_argument("--comm-sms", type=int, default=-1, help="SMs the dA GEMM leaves to the dB reduction (N > 1); -1: the library chooses 16 or 32")
    p.add_argument("--db-wire", type=int, default=0, help="0: dB partials cross NVLink in float32; 1: in the operand type")
    p.add_argument("--rows", type=int, default=0, help="override the row count M of the workload (profiling cases)")
    return p.parse_args()


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE forward launch of the tcgen05 GEMM at
# K = N = 8192, from ncu captures at two row counts: the figure grows linearly with the rows (A and C are
# streamed once per column group, B is re-read once per row block), so a launch of `rows` rows is the line
# through the two captures.  (rows, bytes) pairs; None until both captures exist.  Captured with the 256 x 512
# pair tile the planner takes for this workload (the 256 x 256 tile read 1.2061e9 / 2.2903e9 bytes).
NCU_TRAFFIC_POINTS = {
    "rowsharded_65536x8192x8192": ((8192, 0.9560e9), (16384, 1.9076e9)),
}


def traffic_estimate(workload, rows):
    pts = NCU_TRAFFIC_POINTS.get(workload)
    if not pts or not pts[0]:
        return None, None
    (r0, b0), second = pts
    if second:
        r1, b1 = second
        slope = (b1 - b0) / (r1 - r0)
        return b0 + slope * (rows - r0), f"line through the ncu captures at {r0} and {r1} rows"
    return b0 * rows / r0, f"ncu capture at {r0} rows scaled by rows"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"sustained": d["bf16_tflops_sustained"], "burst": d["bf16_tflops"], "hbm": d["hbm_gbs"],
                "sm_max_mhz": d.get("sm_max_mhz", 1965.0), "src": "measured"}
    return {"sustained": 1400.0, "burst": 1590.0, "hbm": 6650.0, "sm_max_mhz": 1965.0, "src": "fallback"}


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
        "vs_baseline": None, "dtype": SHORT[dtype],
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
    code = CODE[dtype_name]

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
    """nvidia-smi in query mode only, every 20 ms, so that a timed region of a few tens of milliseconds is
    covered by more than a couple of samples."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def stop(self, busy_watts=350.0):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, watts, reasons, capped = [], [], [], set(), 0
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                s, m_, w = float(f[0]), float(f[1]), float(f[2])
            except ValueError:
                continue
            sm.append(s); mx.append(m_); watts.append(w)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
                    capped += name == "sw_power_cap"
        # samples taken while the GPU was working (the sampler also runs over the set-up around the region)
        busy = [s for s, w in zip(sm, watts) if w >= busy_watts] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(busy) if watts else 0,
                "power_w_max": max(watts) if watts else None, "power_w_median_under_load":
                statistics.median([w for w in watts if w >= busy_watts]) if any(w >= busy_watts for w in watts) else None,
                "power_cap_share": capped / len(sm) if sm else None}


def numa_pin(torch, local_rank):
    """Pins this process to the CPUs of its GPU's NUMA node before any pinned host buffer is allocated,
    so that the buffers land in the memory next to the GPU's PCIe root.  Returns what it found."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        node = int(open(base + "/numa_node").read().strip())
        cpus = open(base + "/local_cpulist").read().strip()
        info = {"pci": bdf, "numa_node": node, "local_cpulist": cpus}
        if node >= 0 and cpus:
            ids = set()
            for part in cpus.split(","):
                lo, _, hi = part.partition("-")
                ids.update(range(int(lo), int(hi or lo) + 1))
            allowed = ids & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["pinned_cpus"] = len(allowed)
        return info
    except Exception as e:                                      # noqa: BLE001 (diagnostic only)
        return {"error": repr(e)[:120]}


# --------------------------------------------------------------------------- one workload on the GPU(s)

class Runner:
    """Buffers of one workload on this rank and its fwd+bwd step through the C ABI."""

    def __init__(self, env, workload, rows_override=0, gather=False):
        torch, np = env["torch"], env["np"]
        self.env, self.name, self.gather = env, workload, gather
        dtype_name, batch, m, k, n, bcast_b, shards = WORKLOADS[workload]
        if rows_override:
            batch, m = 1, rows_override
        self.dtype_name, self.k, self.n, self.bcast_b = dtype_name, k, n, bcast_b
        self.tdtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
                       "float64": torch.float64}[dtype_name]
        self.es = torch.empty((), dtype=self.tdtype).element_size()
        self.rows_total = batch * m        # a broadcast-batched product folds its batch into the rows of A
        world, rank, dev = env["world"], env["rank"], env["dev"]
        if world > 1 and not shards:
            raise SystemExit(f"workload {workload} is single-GPU (replicas only)")
        from recpulse_b200.sharded import RowShardedMatmul, row_partition
        self.r0, self.r1 = row_partition(self.rows_total, world, rank)
        rows = self.rows = self.r1 - self.r0
        gen = torch.Generator(device=dev); gen.manual_seed(1234 + rank)
        a_scale = 1.0 / np.sqrt(k) if dtype_name == "bfloat16" else 1.0
        self.A = (torch.randn((rows, k), generator=gen, device=dev, dtype=torch.float32) * a_scale).to(self.tdtype)
        gen_b = torch.Generator(device=dev); gen_b.manual_seed(99)
        Bm = (torch.randn((k, n), generator=gen_b, device=dev, dtype=torch.float32) * (0.125 if bcast_b else 1.0)).to(self.tdtype)
        if rank != 0 and world > 1:
            Bm.zero_()                      # only rank 0 holds B before the replication
        self.dC = torch.randn((rows, n), generator=gen, device=dev, dtype=torch.float32).to(self.tdtype)
        self.Cc = torch.empty((rows, n), device=dev, dtype=self.tdtype)
        self.dA = torch.empty((rows, k), device=dev, dtype=self.tdtype)
        self.dB = torch.empty((k, n), device=dev, dtype=self.tdtype)
        self.Cfull = torch.empty((rows * world, n), device=dev, dtype=self.tdtype) if gather else None
        uid = env["new_uid"]() if world > 1 else None
        self.op = RowShardedMatmul(Bm, rank=rank, world=world, unique_id=uid, comm_sms=env["args"].comm_sms,
                                   db_wire=env["args"].db_wire)
        self.B = self.op.b
        self.flops_step = 3 * 2.0 * self.rows_total * k * n
        self.resident = (2 * rows * k + 2 * k * n + 2 * rows * n) * self.es

    def forward(self):
        self.op.forward(self.A, out=self.Cc)
        if self.gather:
            self.op.gather_output(self.Cc, out=self.Cfull)

    def backward(self):
        self.op.backward(self.A, self.dC, da_out=self.dA, db_out=self.dB)

    def step(self):
        self.forward()
        self.backward()

    def close(self):
        self.op.close()


def time_workload(env, run, steps, warmup, with_clocks=True):
    """K timed steps of `run` (CUDA events on the launching stream, max over ranks)."""
    torch, dist, lib, dev = env["torch"], env["dist"], env["lib"], env["dev"]
    world, rank, local_rank = env["world"], env["rank"], env["local_rank"]
    args = env["args"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(3, warmup)):
        run.step()
    barrier()
    if lib.rpb_device_status(local_rank) != 0:
        raise SystemExit("bench.py: a bounded wait inside the tcgen05 kernel ran out during warm-up")

    stream = torch.cuda.current_stream(dev)
    flush = None
    if run.resident < (512 << 20):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # > 126 MB of L2
    # Launch-bound workloads (a few microseconds of GPU work per launch) are replayed from a CUDA graph, the way
    # a training loop would run them: the host cost of issuing each launch disappears from the timed region.
    graph, launches_per_step = None, None
    if flush is not None and world == 1 and not args.no_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        n0 = lib.rpb_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run.step()
        launches_per_step = lib.rpb_launch_count() - n0
        torch.cuda.synchronize(dev)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(dev)
    sampler = None
    if rank == 0 and with_clocks:
        sampler = ClockSampler(local_rank).start()
        time.sleep(0.15)
    launches0 = lib.rpb_launch_count()
    coll0 = lib.rpb_shard_collective_count()
    step_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    fwd_ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]      # end of the forward launch of every step
    barrier()
    for i in range(steps):
        if flush is not None:
            flush.fill_(i & 1)                      # evict the operands from L2 (outside the timed events)
        step_ev[i][0].record(stream)
        if graph is not None:
            graph.replay()
            fwd_ev[i].record(stream)
        else:
            run.forward()
            fwd_ev[i].record(stream)
            run.backward()
        step_ev[i][1].record(stream)
    barrier()
    elapsed_ms = sum(a.elapsed_time(b) for a, b in step_ev)
    launches = lib.rpb_launch_count() - launches0
    if graph is not None:
        launches = launches_per_step * steps          # counted while capturing; each replay re-issues them
    clocks = sampler.stop() if sampler else None
    fwd_ms = sum(step_ev[i][0].elapsed_time(fwd_ev[i]) for i in range(steps)) / steps
    if graph is not None:
        fwd_ms = elapsed_ms / steps             # the replayed step is one unit: the roofline is per STEP
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    if lib.rpb_device_status(local_rank) != 0:
        raise SystemExit("bench.py: a bounded wait inside the tcgen05 kernel ran out")
    ms_per_step = elapsed_ms / steps
    return {"ms_per_step": ms_per_step, "value": run.flops_step / (ms_per_step * 1e-3) / 1e12, "fwd_ms": fwd_ms,
            "graph": graph is not None, "flushed": flush is not None, "launches": int(launches), "clocks": clocks,
            "collectives": int(lib.rpb_shard_collective_count() - coll0), "_flush": flush, "_stream": stream}


def roofline_of(run, timing, pk, n_gpus):
    """The dominant kernel of the timed region against the measured peaks.  Tensor-bound workloads: the forward
    GEMM launch (all three GEMMs of a graph-replayed step) against the cuBLAS bf16 peaks; the denominator of
    `frac` is the burst peak when the sampled SM clock stayed near its maximum and the sustained one when the
    power cap held the clock down.  Memory-bound workloads: algorithmic bytes against the measured copy rate."""
    rows, k, n, es = run.rows, run.k, run.n, run.es
    flops = 2.0 * rows * k * n
    bytes_unit = (rows * k + k * n + rows * n) * es
    unit = "forward GEMM launch"
    if timing["graph"]:
        flops *= 3; bytes_unit *= 3; unit = "fwd+bwd step replayed from a CUDA graph"
    fwd_ms = timing["fwd_ms"]
    clocks = timing["clocks"] or {}
    mhz, mhz_max = clocks.get("sm_mhz"), clocks.get("sm_max_mhz") or pk["sm_max_mhz"]
    tensor_bound = run.dtype_name == "bfloat16" or (run.dtype_name == "float16" and not run.bcast_b)
    if tensor_bound:
        achieved = flops / (fwd_ms * 1e-3) / 1e12
        capped = bool(mhz and mhz < 0.85 * mhz_max)
        traffic, note = traffic_estimate(run.name, rows)
        return {"bound": "tensor", "kernel": "rpb_umma::gemm_kernel (" + unit + ")", "achieved": achieved,
                "peak": pk["sustained"] if capped else pk["burst"], "unit": "TFLOP/s",
                "frac": achieved / (pk["sustained"] if capped else pk["burst"]),
                "frac_burst": achieved / pk["burst"], "frac_sustained": achieved / pk["sustained"],
                "regime": ("power-capped clock: sustained peak" if capped else "clock near maximum: burst peak") +
                          (f" (median {mhz:.0f} of {mhz_max:.0f} MHz under load)" if mhz else " (no clock samples)"),
                "peak_source": pk["src"] + " cuBLAS bf16 8192^3 (burst = best of 10, sustained = 4 s loop)",
                "ms_x_sm_mhz": fwd_ms * mhz if mhz else None,
                "traffic": traffic, "traffic_note": note, "algorithmic_bytes": bytes_unit, "avg_launch_ms": fwd_ms,
                "pct_of_nominal_dense_peak": achieved / 2250.0}
    achieved = bytes_unit / (fwd_ms * 1e-3) / 1e9
    if run.dtype_name == "float64":
        tf = flops / (fwd_ms * 1e-3) / 1e12
        return {"bound": "fp64 pipe", "kernel": "rpb_dmma::gemm_kernel (" + unit + ")", "achieved": tf, "peak": 40.0,
                "unit": "TFLOP/s", "frac": tf / 40.0, "peak_source": "nominal fp64 (no measured fp64 peak on record)",
                "traffic": None, "avg_launch_ms": fwd_ms}
    return {"bound": "hbm", "kernel": unit, "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
            "frac": achieved / pk["hbm"], "peak_source": pk["src"] + " copy bandwidth", "traffic": None,
            "algorithmic_bytes": bytes_unit, "avg_launch_ms": fwd_ms}


def torch_matmul_same_step(env, run, timing, steps):
    """The same three GEMMs through torch.matmul (cuBLAS, warm handle, outputs preallocated): context only."""
    torch, dev = env["torch"], env["dev"]
    A, Bm, dC, Cc, dA, dB = run.A, run.B, run.dC, run.Cc, run.dA, run.dB
    flush, stream = timing["_flush"], timing["_stream"]

    def cublas_step():
        torch.matmul(A, Bm, out=Cc); torch.matmul(A.t(), dC, out=dB); torch.matmul(dC, Bm.t(), out=dA)
    for _ in range(3):
        cublas_step()
    tot = 0.0
    for i in range(steps):
        if flush is not None:
            flush.fill_(i & 1)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record(stream); cublas_step(); c1.record(stream)
        torch.cuda.synchronize(dev)
        tot += c0.elapsed_time(c1)
    ms = tot / steps
    return {"tflops": run.flops_step / (ms * 1e-3) / 1e12, "ms_per_step": ms,
            "what": "torch.matmul x3 (cuBLAS, warm handle, outputs preallocated, eager)"}


# --------------------------------------------------------------------------- parity of what was timed

def parity_check(env, run, sample_rows=2, entries=64):
    """Checks the outputs the timed steps left in the buffers.  Rows of C and dA of this rank against the CPU
    oracle on the same bits; sampled entries of dB (summed over all ranks) against float64 dot products; and
    the column-sum identities 1^T C = (1^T A) B, 1^T dA = (1^T dC) B^T, dB 1 = A^T (dC 1), which every output
    tile contributes to.  Returns the record; `ok` is the AND over all ranks."""
    torch, np, dist, dev = env["torch"], env["np"], env["dist"], env["dev"]
    world, rank = env["world"], env["rank"]
    from oracle import oracle as O
    code = {"float32": O.F32, "float64": O.F64, "float16": O.F16, "bfloat16": O.BF16}[run.dtype_name]
    half = run.es == 2
    tol = {"bfloat16": 4e-3, "float16": 6e-4, "float32": 1e-5, "float64": 1e-12}[run.dtype_name]
    t0 = time.perf_counter()

    def bits(t):                                    # device tensor -> numpy storage bits
        t = t.contiguous()
        return t.view(torch.int16).cpu().numpy().view(np.uint16) if half else t.cpu().numpy()

    def err(got, ref, k):                           # the path's metric for this dtype
        g, r = O.to_f64(got, code), O.to_f64(ref, code)
        if run.dtype_name == "float64":
            rms = float(np.sqrt(np.mean(r * r))) or 1.0
            return float((np.abs(g - r) / np.maximum(np.abs(r), rms)).max())
        if run.dtype_name == "float32":
            rms = float(np.sqrt(np.mean(r * r))) or 1.0
            return float(np.abs(g - r).max() / (np.sqrt(k) * rms))
        return float(np.linalg.norm(g - r) / (np.linalg.norm(r) or 1.0))

    rng = np.random.default_rng(7 + rank)
    rows, k, n = run.rows, run.k, run.n
    # keep the oracle's share to a few seconds: one row costs 2 k n flops at ~0.2 GFLOP/s
    take = max(1, min(sample_rows, rows, int(2.0e9 / (2.0 * k * n)) or 1))
    ri = np.sort(rng.choice(rows, take, replace=False))
    idx = torch.as_tensor(ri, device=dev)
    b_bits = bits(run.B)
    c_err = err(bits(run.Cc[idx]), O.rp_matmul(bits(run.A[idx]), b_bits, code), k)
    da_err = err(bits(run.dA[idx]), O.rp_matmul(bits(run.dC[idx]), np.ascontiguousarray(b_bits.T), code), n)
    # dB entries: partial float64 dot products of this rank's rows, summed over the ranks
    gen = np.random.default_rng(99)                 # the same entries on every rank
    ii = torch.as_tensor(gen.integers(0, k, entries), device=dev); jj = torch.as_tensor(gen.integers(0, n, entries), device=dev)
    part = (run.A[:, ii].double() * run.dC[:, jj].double()).sum(dim=0)
    # identities in float64 on the device (chunked by torch's reduction; nothing of size rows x n is materialised in fp64)
    colsum = lambda t: t.sum(dim=0, dtype=torch.float64)
    rowsum = lambda t: t.sum(dim=1, dtype=torch.float64)
    Bd = run.B.double()
    id_c = (colsum(run.Cc) - colsum(run.A) @ Bd).abs().max() / (np.sqrt(rows) * run.Cc.float().pow(2).mean().sqrt().double())
    id_da = (colsum(run.dA) - colsum(run.dC) @ Bd.t()).abs().max() / (np.sqrt(rows) * run.dA.float().pow(2).mean().sqrt().double())
    db_rhs = torch.zeros(k, device=dev, dtype=torch.float64)
    rs = rowsum(run.dC)
    step_rows = max(1, (256 << 20) // (k * 8))
    for s in range(0, rows, step_rows):
        db_rhs += run.A[s:s + step_rows].double().t() @ rs[s:s + step_rows]
    if world > 1:
        dist.all_reduce(part); dist.all_reduce(db_rhs)
    got = run.dB[ii, jj].double()
    db_entry_err = float(((got - part).norm() / part.norm()).item())
    id_db = float(((rowsum(run.dB) - db_rhs).abs().max() /
                   (np.sqrt(n) * run.dB.float().pow(2).mean().sqrt().double())).item())
    id_tol = 2e-2 if half else 1e-4
    rec = {"rows": int(take), "row_index": [int(x) for x in ri], "max_rel": max(c_err, da_err, db_entry_err),
           "c_rows_vs_oracle": c_err, "da_rows_vs_oracle": da_err, "db_entries_vs_float64": db_entry_err,
           "db_entries": entries, "tolerance": tol,
           "column_sum_identity": {"c": float(id_c.item()), "da": float(id_da.item()), "db": id_db, "tolerance": id_tol},
           "what": "rows of C and dA vs the CPU oracle on the same bits; dB entries (summed over ranks) vs float64; "
                   "1^T C = (1^T A) B and its dA / dB forms over every tile",
           "seconds": None}
    ok = (c_err <= tol and da_err <= tol and db_entry_err <= tol and float(id_c.item()) <= id_tol and
          float(id_da.item()) <= id_tol and id_db <= id_tol)
    if world > 1:
        flag = torch.tensor([1.0 if ok else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        worst = torch.tensor([rec["max_rel"]], device=dev, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        ok = bool(flag.item() > 0.5); rec["max_rel"] = float(worst.item()); rec["ranks_checked"] = world
    rec["ok"] = bool(ok)
    rec["seconds"] = time.perf_counter() - t0
    return rec


# --------------------------------------------------------------------------- end to end from host buffers

def e2e_measure(env, run, steps):
    torch, dist, lib, dev = env["torch"], env["dist"], env["lib"], env["dev"]
    world, rank, local_rank = env["world"], env["rank"], env["local_rank"]
    rows, k, n, es = run.rows, run.k, run.n, run.es
    td = run.tdtype
    hA = torch.empty((rows, k), dtype=td).pin_memory(); hA.copy_(run.A)
    hdC = torch.empty((rows, n), dtype=td).pin_memory(); hdC.copy_(run.dC)
    hB = None
    if rank == 0:
        hB = torch.empty((k, n), dtype=td).pin_memory(); hB.copy_(run.B)
    hC = torch.empty((rows, n), dtype=td).pin_memory()
    hdA = torch.empty((rows, k), dtype=td).pin_memory()
    hdB = torch.empty((k, n), dtype=td).pin_memory()
    code = CODE[run.dtype_name]
    ptr = lambda t: None if t is None else C.c_void_p(t.data_ptr())
    b0, b1 = C.c_longlong(0), C.c_longlong(k * n)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def e2e_step():
        # the library's host-buffer entry point: chunked H2D of A and dC, GEMMs and D2H of C and dA overlapped
        # on three streams; N > 1: B is uploaded by rank 0 only and replicated over NVLink, dB is reduced on the
        # devices and every rank copies back its slice.  Returns when the host buffers are filled.
        if world > 1:
            rc = lib.rp_matmul_rowsharded_fwdbwd_host(run.op.handle, ptr(hC), ptr(hdA), ptr(hdB), ptr(hA), ptr(hB), ptr(hdC),
                                                      rows, k, n, code, 0, C.byref(b0), C.byref(b1))
        else:
            rc = lib.rp_matmul_fwdbwd_host(ptr(hC), ptr(hdA), ptr(hdB), ptr(hA), ptr(hB), ptr(hdC), rows, k, n, code,
                                           local_rank, 0)
        if rc != 0:
            raise SystemExit("bench.py: the host-buffer entry point failed")

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) / steps * 1e3
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    db_elems = b1.value - b0.value
    h2d = (rows * k + rows * n + (k * n if rank == 0 else 0)) * es
    d2h = (rows * n + rows * k + db_elems) * es
    # what one PCIe link does on this box at this rank count: H2D alone, D2H alone and both at once, all ranks together
    probe = {}
    nbytes = min(hA.numel() * es, 512 << 20)
    src = hA.view(torch.uint8).flatten()[:nbytes]; dst_h = hC.view(torch.uint8).flatten()[:nbytes]
    dbuf = torch.empty(nbytes, dtype=torch.uint8, device=dev); dbuf2 = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    for name in ("h2d", "d2h", "both"):
        barrier()
        t0 = time.perf_counter()
        for _ in range(4):
            if name in ("h2d", "both"):
                with torch.cuda.stream(s1):
                    dbuf.copy_(src, non_blocking=True)
            if name in ("d2h", "both"):
                with torch.cuda.stream(s2):
                    dst_h.copy_(dbuf2, non_blocking=True)
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        rate = torch.tensor([4 * nbytes / dt / 1e9], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(rate)                   # aggregate over the ranks
        probe[name + "_gbs_all_ranks"] = float(rate.item())
    tot_h2d = torch.tensor([float(h2d), float(d2h)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tot_h2d)
    return {"value": run.flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(tot_h2d[0].item()),
            "d2h_bytes_per_step": int(tot_h2d[1].item()), "h2d_bytes_this_rank": int(h2d), "d2h_bytes_this_rank": int(d2h),
            "ms_per_step": e2e_ms, "steps": steps,
            "pcie_gbs_each_way_per_rank": max(h2d, d2h) / (e2e_ms * 1e-3) / 1e9,
            "pcie_gbs_each_way_all_ranks": max(float(tot_h2d[0].item()), float(tot_h2d[1].item())) / (e2e_ms * 1e-3) / 1e9,
            "pcie_probe": probe, "numa": env["numa"],
            "api": ("rp_matmul_rowsharded_fwdbwd_host" if world > 1 else "rp_matmul_fwdbwd_host") +
                   " (C ABI, pinned host buffers, wall clock around the synchronous call, max over ranks)"}


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
    from recpulse_b200 import sharded

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the matmul path has no CPU implementation)")
    lib = recpulse_b200.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = numa_pin(torch, local_rank)              # before any pinned host buffer exists
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if args.gpus != world and rank == 0 and world > 1:
        print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE {world}; using WORLD_SIZE", file=sys.stderr)
    n_gpus = world
    env = {"torch": torch, "np": np, "dist": dist, "lib": lib, "dev": dev, "world": world, "rank": rank,
           "local_rank": local_rank, "args": args, "numa": numa, "new_uid": lambda: sharded.exchange_unique_id()}
    pk = peaks()

    run = Runner(env, args.workload, rows_override=args.rows)
    timing = time_workload(env, run, args.steps, args.warmup)
    value, ms_per_step = timing["value"], timing["ms_per_step"]
    roof = roofline_of(run, timing, pk, n_gpus) if rank == 0 else None

    parity = None
    if not args.no_parity:
        parity = parity_check(env, run)

    compare = None
    if world == 1:
        compare = torch_matmul_same_step(env, run, timing, args.steps)
        if args.compare:
            ref_ms = reference_gpu_as_shipped(run.dtype_name, run.rows, run.k, run.n, min(args.steps, 5),
                                              fill=(run.A.data_ptr(), run.B.data_ptr(), run.dC.data_ptr()))
            if ref_ms:
                compare["reference_as_shipped_ms_per_step"] = ref_ms
                compare["reference_as_shipped_tflops"] = run.flops_step / (ref_ms * 1e-3) / 1e12

    e2e = None
    if not args.no_e2e:
        e2e = e2e_measure(env, run, args.e2e_steps)

    # ---- the other configurations
    workloads = {}
    if not args.no_workloads and args.workload == DEFAULT_WORKLOAD and not args.rows:
        if world == 1:
            names = ["square4096", "bmm_fp16", "fp64_2048", "mlp_fp32", "lstm_fp32"]
            for name in names:
                r2 = Runner(env, name)
                t2 = time_workload(env, r2, max(args.steps, 20), args.warmup)
                rec = {"value": t2["value"], "unit": UNIT, "ms_per_step": t2["ms_per_step"], "dtype": SHORT[r2.dtype_name],
                       "shape": [r2.rows_total, r2.k, r2.n], "cuda_graph": t2["graph"], "l2_flushed": t2["flushed"],
                       "gpu_launches": t2["launches"], "roofline": roofline_of(r2, t2, pk, 1), "clocks": t2["clocks"],
                       "torch_matmul_same_step": torch_matmul_same_step(env, r2, t2, max(args.steps, 20))}
                if not args.no_parity:
                    rec["parity_check"] = parity_check(env, r2)
                workloads[name] = rec
                r2.close()
                del t2
                lib.rpb_scratch_reset(local_rank)   # the replayed graph is gone: the scratch it pinned may grow again
        else:
            r2 = Runner(env, "bmm_fp16")
            t2 = time_workload(env, r2, max(args.steps, 20), args.warmup, with_clocks=False)
            rec = {"value": t2["value"], "unit": UNIT, "ms_per_step": t2["ms_per_step"], "dtype": "f16",
                   "shape": [r2.rows_total, r2.k, r2.n], "rows_per_gpu": r2.rows, "collectives": t2["collectives"],
                   "what": "batch folded into the rows of A and split over the ranks; dB (64 x 512) all-reduced in float32"}
            if not args.no_parity:
                rec["parity_check"] = parity_check(env, r2)
            workloads["bmm_fp16"] = rec
            r2.close()
            r3 = Runner(env, DEFAULT_WORKLOAD, gather=True)
            t3 = time_workload(env, r3, args.steps, args.warmup, with_clocks=False)
            workloads["rowsharded_with_allgather_of_C"] = {
                "value": t3["value"], "unit": UNIT, "ms_per_step": t3["ms_per_step"], "collectives": t3["collectives"],
                "without_allgather": value,
                "what": "the default workload with C all-gathered onto every GPU inside the step (1 GiB over NVLink)"}
            r3.close()

    ok = True
    if parity is not None:
        ok = parity["ok"] and all(w.get("parity_check", {}).get("ok", True) for w in workloads.values())

    if rank == 0:
        cpu = None
        if n_gpus == 1 and not args.no_cpu_baseline:
            tf, desc, kind, _ = cpu_sample(args.workload, 20.0)
            cpu = {"value": tf, "unit": UNIT, "cores": 1, "kind": kind, "sample": desc}
        half = run.es == 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": SHORT[run.dtype_name], "data": "synthetic",
            "config": {"workload": args.workload, "m": run.rows_total, "k": run.k, "n": run.n, "rows_per_gpu": run.rows,
                       "parallelism": (f"rows of A over {n_gpus} GPU(s), B replicated, dB reduce-scattered in float32 + all-gathered"
                                       if n_gpus > 1 else "single GPU"),
                       "collective": "NCCL (issued by librecpulse_b200 through its C ABI)" if n_gpus > 1 else None,
                       "collectives_in_timed_region": timing["collectives"],
                       "l2": "inputs larger than L2, no flush" if not timing["flushed"] else
                             "L2 flushed (256 MB write) before every step, outside the timed events",
                       "accumulate": "fp32", "cuda_graph": timing["graph"]},
            "clocks": timing["clocks"], "e2e": e2e, "gpu_launches": timing["launches"], "roofline": roof,
            "cpu_baseline": cpu, "parity_check": parity, "workloads": workloads or None,
            "pct_of_nominal_dense_peak": value / (2250.0 * n_gpus) if half else None,
        }
        if compare:
            line["torch_matmul_same_step"] = compare
        print(json.dumps(line), flush=True)
    run.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("bench.py: parity check failed")


if __name__ == "__main__":
    main()
