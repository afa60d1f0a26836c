/*
 * Forward + backward of one matmul for operands that live in HOST memory:
 *   C = A.B,  dA = dC.B^T,  dB = A^T.dC     (packed row-major, all six matrices on the host)
 *
 * RecPulse reaches the GPU with whole-tensor synchronous copies (core/tensor_device.cu:295-372) and only
 * then multiplies.  Here the rows of A and dC are streamed in chunks: while chunk i+1 crosses PCIe
 * host-to-device, chunk i is multiplied (C_i and dA_i depend on row chunk i only) and chunk i-1's results
 * travel device-to-host on a third stream, so both PCIe directions and the tensor cores are busy at once.
 * A and dC land in full-size device buffers, so dB is ONE GEMM over all rows at the end (a single
 * rounding, exactly like the resident path).  Device buffers are cached per device between calls.
 */
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda_runtime.h>

#include "rpb_common.h"
#include "shard_internal.h"

extern "C" int rpb_take_status(int device_id);   /* gemm_dispatch.cu */

namespace {

struct HostPipe {
    char* buf = nullptr;
    size_t bytes = 0;
    cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
    static constexpr int MAX_CHUNKS = 1024;
    cudaEvent_t in_done[MAX_CHUNKS] = {};
    cudaEvent_t mm_done[MAX_CHUNKS] = {};
    cudaEvent_t b_ready = nullptr, db_done = nullptr;
    bool ready = false;
};
HostPipe g_pipe[64];
std::mutex g_pipe_mutex[64];         /* per device: a sharded call waits inside for the other ranks' GPUs */

#define HP_CUDA(call)                                                                           \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess) {                                                                \
            fprintf(stderr, "recpulse_b200: %s failed: %s\n", #call, cudaGetErrorString(e_));   \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

int pipe_setup(HostPipe& p, size_t need, int chunks) {
    if (!p.ready) {
        HP_CUDA(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
        HP_CUDA(cudaStreamCreateWithFlags(&p.s_mm, cudaStreamNonBlocking));
        HP_CUDA(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
        HP_CUDA(cudaEventCreateWithFlags(&p.b_ready, cudaEventDisableTiming));
        HP_CUDA(cudaEventCreateWithFlags(&p.db_done, cudaEventDisableTiming));
        p.ready = true;
    }
    for (int i = 0; i < chunks; ++i) {
        if (!p.in_done[i]) HP_CUDA(cudaEventCreateWithFlags(&p.in_done[i], cudaEventDisableTiming));
        if (!p.mm_done[i]) HP_CUDA(cudaEventCreateWithFlags(&p.mm_done[i], cudaEventDisableTiming));
    }
    if (need > p.bytes) {
        if (p.buf) HP_CUDA(cudaFree(p.buf));
        p.buf = nullptr; p.bytes = 0;
        HP_CUDA(cudaMalloc(&p.buf, need));
        p.bytes = need;
    }
    return 0;
}

/* `sh` == nullptr: one GPU.  Otherwise this rank's rows of a product sharded over sh's ranks: B comes from rank
 * 0's host buffer (one upload per box, then NVLink), dB is reduced on the devices and only this rank's slice
 * [*db_begin, *db_end) of its elements is copied back. */
int fwdbwd_host(RpbShard* sh, void* C, void* dA, void* dB, const void* A, const void* B, const void* dC,
                int m, int k, int n, DType dtype, int device_id, int chunk_rows, long long* db_begin, long long* db_end) {
    const size_t es = rpb_dtype_size((int)dtype);
    const int world = rpb_shard_world_of(sh), rank = rpb_shard_rank_of(sh);
    const bool b_local = world == 1 || rank == 0;          /* this rank uploads B */
    if (!A || (b_local && !B) || m <= 0 || k <= 0 || n <= 0 || !es || device_id < 0 || device_id >= 64) return -1;
    if (!C && !dA && !dB) return -1;
    const bool bwd = dA || dB;
    if (bwd && !dC) { fprintf(stderr, "recpulse_b200: backward needs dC\n"); return -1; }
    int prev = -1;
    HP_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) HP_CUDA(cudaSetDevice(device_id));
    std::lock_guard<std::mutex> lock(g_pipe_mutex[device_id]);
    HostPipe& p = g_pipe[device_id];

    if (chunk_rows <= 0) {
        /* about 64 MB of A per chunk, at least 8 chunks on large inputs, multiples of 256 rows */
        long long r = (64ll << 20) / ((long long)k * es);
        if (r > m / 8) r = m / 8;
        r = (r / 256) * 256;
        chunk_rows = (int)(r < 256 ? (m < 256 ? m : 256) : r);
    }
    int chunks = (m + chunk_rows - 1) / chunk_rows;
    if (chunks > HostPipe::MAX_CHUNKS) { chunk_rows = (m + HostPipe::MAX_CHUNKS - 1) / HostPipe::MAX_CHUNKS; chunks = (m + chunk_rows - 1) / chunk_rows; }

    const size_t a_b = up256(es * m * k), b_b = up256(es * k * n), c_b = up256(es * m * n);
    const size_t need = a_b + b_b + (C ? c_b : 0) + (bwd ? c_b : 0) + (dA ? a_b : 0) + (dB ? b_b : 0);
    int rc = pipe_setup(p, need, chunks);
    if (rc) { if (prev != device_id) cudaSetDevice(prev); return -1; }
    char* q = p.buf;
    char* dAm = q; q += a_b;                         /* A        */
    char* dBm = q; q += b_b;                         /* B        */
    char* dCm = C ? q : nullptr; if (C) q += c_b;    /* C        */
    char* dGm = bwd ? q : nullptr; if (bwd) q += c_b;/* dC       */
    char* ddA = dA ? q : nullptr; if (dA) q += a_b;  /* dA       */
    char* ddB = dB ? q : nullptr;                    /* dB       */

    auto fail = [&](const char* what) {
        fprintf(stderr, "recpulse_b200: rp_matmul_fwdbwd_host: %s failed: %s\n", what, cudaGetErrorString(cudaGetLastError()));
        cudaDeviceSynchronize();
        if (prev != device_id) cudaSetDevice(prev);
        return -1;
    };

    if (b_local && cudaMemcpyAsync(dBm, B, es * k * n, cudaMemcpyHostToDevice, p.s_in) != cudaSuccess) return fail("copy of B");
    if (world > 1 && rpb_shard_broadcast_bytes(sh, dBm, es * k * n, 0, p.s_in)) return fail("broadcast of B");
    if (cudaEventRecord(p.b_ready, p.s_in) != cudaSuccess) return fail("event");
    if (cudaStreamWaitEvent(p.s_mm, p.b_ready, 0) != cudaSuccess) return fail("wait");

    for (int i = 0; i < chunks; ++i) {
        const int r0 = i * chunk_rows;
        const int rows = (m - r0 < chunk_rows) ? m - r0 : chunk_rows;
        const size_t offA = es * (size_t)r0 * k, offC = es * (size_t)r0 * n;
        if (cudaMemcpyAsync(dAm + offA, (const char*)A + offA, es * rows * k, cudaMemcpyHostToDevice, p.s_in) != cudaSuccess)
            return fail("copy of A rows");
        if (bwd && cudaMemcpyAsync(dGm + offC, (const char*)dC + offC, es * rows * n, cudaMemcpyHostToDevice, p.s_in) != cudaSuccess)
            return fail("copy of dC rows");
        cudaEventRecord(p.in_done[i], p.s_in);
        cudaStreamWaitEvent(p.s_mm, p.in_done[i], 0);
        RpbGemm g;
        if (C) {                                     /* C_i = A_i . B */
            rpb_gemm_packed(&g, rows, k, n);
            if (rp_matmul_ex(dCm + offC, dAm + offA, dBm, &g, dtype, device_id, p.s_mm)) return fail("forward GEMM");
        }
        if (dA) {                                    /* dA_i = dC_i . B^T : B read through swapped strides */
            rpb_gemm_packed(&g, rows, n, k);
            g.b_row = 1; g.b_col = n;
            if (rp_matmul_ex(ddA + offA, dGm + offC, dBm, &g, dtype, device_id, p.s_mm)) return fail("dA GEMM");
        }
        cudaEventRecord(p.mm_done[i], p.s_mm);
        cudaStreamWaitEvent(p.s_out, p.mm_done[i], 0);
        if (C && cudaMemcpyAsync((char*)C + offC, dCm + offC, es * rows * n, cudaMemcpyDeviceToHost, p.s_out) != cudaSuccess)
            return fail("copy of C rows");
        if (dA && cudaMemcpyAsync((char*)dA + offA, ddA + offA, es * rows * k, cudaMemcpyDeviceToHost, p.s_out) != cudaSuccess)
            return fail("copy of dA rows");
    }
    long long s_begin = 0, s_end = (long long)k * n;
    if (dB) {                                        /* dB = A^T . dC over all rows (of all ranks), one rounding */
        if (world > 1) {
            rpb_shard_db_slice(sh, k, n, (int)dtype, RPB_SHARD_SLICE_ONLY, &s_begin, &s_end);
            if (rpb_shard_db_begin(sh, ddB, dAm, dGm, m, k, n, (int)dtype, RPB_SHARD_SLICE_ONLY, p.s_mm) ||
                rpb_shard_db_end(sh, p.s_mm)) return fail("dB GEMM + reduction");
        } else {
            RpbGemm g;
            rpb_gemm_packed(&g, k, m, n);
            g.a_row = 1; g.a_col = k;
            if (rp_matmul_ex(ddB, dAm, dGm, &g, dtype, device_id, p.s_mm)) return fail("dB GEMM");
        }
        cudaEventRecord(p.db_done, p.s_mm);
        cudaStreamWaitEvent(p.s_out, p.db_done, 0);
        if (cudaMemcpyAsync((char*)dB + es * s_begin, ddB + es * s_begin, es * (size_t)(s_end - s_begin), cudaMemcpyDeviceToHost,
                            p.s_out) != cudaSuccess) return fail("copy of dB");
    }
    if (db_begin) *db_begin = s_begin;
    if (db_end) *db_end = s_end;
    cudaError_t e1 = cudaStreamSynchronize(p.s_out);
    cudaError_t e2 = cudaStreamSynchronize(p.s_mm);
    cudaError_t e3 = cudaStreamSynchronize(p.s_in);
    if (prev != device_id) cudaSetDevice(prev);
    if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess) {
        fprintf(stderr, "recpulse_b200: rp_matmul_fwdbwd_host: %s\n", cudaGetErrorString(e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3)));
        return -1;
    }
    return rpb_take_status(device_id) ? -1 : 0;
}

}  // namespace

extern "C" {

int rp_matmul_fwdbwd_host(void* C, void* dA, void* dB, const void* A, const void* B, const void* dC,
                          int m, int k, int n, DType dtype, int device_id, int chunk_rows) {
    return fwdbwd_host(nullptr, C, dA, dB, A, B, dC, m, k, n, dtype, device_id, chunk_rows, nullptr, nullptr);
}

int rp_matmul_rowsharded_fwdbwd_host(RpbShard* shard, void* C_rows, void* dA_rows, void* dB, const void* A_rows, const void* B,
                                     const void* dC_rows, long long rows, int k, int n, DType dtype, int chunk_rows,
                                     long long* db_begin, long long* db_end) {
    if (!shard || rows <= 0 || rows > 0x7fffffffLL) return -1;
    return fwdbwd_host(shard, C_rows, dA_rows, dB, A_rows, B, dC_rows, (int)rows, k, n, dtype, rpb_shard_device_of(shard),
                       chunk_rows, db_begin, db_end);
}

/* Frees the device buffers that rp_matmul_fwdbwd_host keeps between calls on `device_id`. */
int rpb_release_host_pipeline(int device_id) {
    if (device_id < 0 || device_id >= 64) return -1;
    std::lock_guard<std::mutex> lock(g_pipe_mutex[device_id]);
    HostPipe& p = g_pipe[device_id];
    if (!p.buf) return 0;
    int prev = -1;
    HP_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) HP_CUDA(cudaSetDevice(device_id));
    cudaFree(p.buf);
    p.buf = nullptr; p.bytes = 0;
    if (prev != device_id) cudaSetDevice(prev);
    return 0;
}

}  // extern "C"
