/*
 * The matmul path sharded over the GPUs of one box, behind the C ABI.
 *
 * RecPulse's only multi-GPU primitive is a whole-tensor device-to-device copy (tensor_copy_device,
 * core/tensor_device.cu:295-372: cudaDeviceEnablePeerAccess + cudaMemcpyPeer, reached from tensor_to,
 * core/tensor.c:82-144).  This file is the layer that primitive would grow into for the matmul path:
 *
 *     rank g holds   A_g = A[rows_g, :],  dC_g = dC[rows_g, :]        never exchanged
 *     replicated     B        copied once into every GPU's own memory (rp_shard_replicate)
 *     forward        C_g  = A_g . B                                   no communication
 *     backward       dA_g = dC_g . B^T                                no communication
 *                    dB   = sum_g A_g^T . dC_g                        one reduction per step
 *
 * One RpbShard per (thread or process, GPU): an NCCL communicator, a side stream for the collectives and a
 * float32 staging buffer.  The dB partials leave the GEMM as UNROUNDED float32 sums (RpbGemm.c_float32), are
 * reduce-scattered in float32 over NVLink, rounded ONCE to the operand type by the rank that owns the slice
 * and all-gathered in the operand type: dB keeps the single rounding it has on one GPU, and the wire carries
 * 4 + 2 bytes per element instead of the 8 of a float32 all-reduce.  The collective runs on the side stream
 * while the dA GEMM runs on the caller's stream; the persistent GEMM kernel leaves `comm_sms` SMs to it.
 * Every kernel reads its own GPU's memory only.
 *
 * NCCL is resolved at run time (dlopen): a process that already carries libnccl.so.2 shares it, and the
 * library still loads where NCCL is absent (single-GPU use, symbol checks on a CPU box).
 */
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include <dlfcn.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rpb_common.h"
#include "shard_internal.h"

namespace {

/* The part of NCCL's public C interface this file uses (nccl.h: ncclUniqueId is 128 opaque bytes; the
 * enumerator values below are the ones nccl.h has carried since 2.10). */
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclSuccess = 0 };
enum { ncclInt8 = 0, ncclFloat16 = 6, ncclFloat32 = 7, ncclFloat64 = 8, ncclBfloat16 = 9 };
enum { ncclSum = 0 };

struct Nccl {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
};
Nccl g_nccl;
std::mutex g_nccl_mutex;

int load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return 0;
    void* h = nullptr;
    if (const char* path = getenv("RPB_NCCL_LIB")) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);       /* the copy the process already uses */
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) {
        fprintf(stderr, "recpulse_b200: NCCL not found (%s); set RPB_NCCL_LIB to libnccl.so.2\n", dlerror());
        return -1;
    }
    Nccl n;
    n.handle = h;
#define RPB_SYM(field, name)                                                                   \
    *reinterpret_cast<void**>(&n.field) = dlsym(h, name);                                      \
    if (!n.field) { fprintf(stderr, "recpulse_b200: %s missing from NCCL\n", name); return -1; }
    RPB_SYM(GetUniqueId, "ncclGetUniqueId")
    RPB_SYM(CommInitRank, "ncclCommInitRank")
    RPB_SYM(CommDestroy, "ncclCommDestroy")
    RPB_SYM(Broadcast, "ncclBroadcast")
    RPB_SYM(AllReduce, "ncclAllReduce")
    RPB_SYM(ReduceScatter, "ncclReduceScatter")
    RPB_SYM(AllGather, "ncclAllGather")
    RPB_SYM(GetErrorString, "ncclGetErrorString")
    RPB_SYM(GetVersion, "ncclGetVersion")
#undef RPB_SYM
    g_nccl = n;
    return 0;
}

#define SH_CUDA(call)                                                                           \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess) {                                                                \
            fprintf(stderr, "recpulse_b200: %s failed: %s\n", #call, cudaGetErrorString(e_));   \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)
#define SH_NCCL(call)                                                                           \
    do {                                                                                        \
        ncclResult_t r_ = (call);                                                               \
        if (r_ != ncclSuccess) {                                                                \
            fprintf(stderr, "recpulse_b200: %s failed: %s\n", #call, g_nccl.GetErrorString(r_)); \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

int nccl_type(int dtype) {
    switch (dtype) {
        case DTYPE_FLOAT32: return ncclFloat32;
        case DTYPE_FLOAT64: return ncclFloat64;
        case DTYPE_FLOAT16: return ncclFloat16;
        case DTYPE_BFLOAT16: return ncclBfloat16;
    }
    return -1;
}

/* dst[i] = round(src[i]) for the slice a rank owns after the float32 reduce-scatter: the one rounding of dB */
template <typename T>
__global__ void round_slice_kernel(T* __restrict__ dst, const float* __restrict__ src, size_t count) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < count; i += stride) {
        if (i + 4 <= count) {
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            if constexpr (sizeof(T) == 2) {
                T o[4];
                if constexpr (std::is_same<T, __nv_bfloat16>::value) {
                    o[0] = __float2bfloat16_rn(v.x); o[1] = __float2bfloat16_rn(v.y);
                    o[2] = __float2bfloat16_rn(v.z); o[3] = __float2bfloat16_rn(v.w);
                } else {
                    o[0] = __float2half_rn(v.x); o[1] = __float2half_rn(v.y);
                    o[2] = __float2half_rn(v.z); o[3] = __float2half_rn(v.w);
                }
                *reinterpret_cast<uint2*>(dst + i) = *reinterpret_cast<const uint2*>(o);
            }
        } else {
            for (size_t j = i; j < count; ++j) {
                if constexpr (std::is_same<T, __nv_bfloat16>::value) dst[j] = __float2bfloat16_rn(src[j]);
                else dst[j] = __float2half_rn(src[j]);
            }
        }
    }
}

int launch_round(void* dst, const float* src, size_t count, int dtype, int blocks_cap, cudaStream_t s) {
    size_t want = (count / 4 + 255) / 256;
    int blocks = (int)(want < (size_t)blocks_cap ? (want ? want : 1) : (size_t)blocks_cap);
    if (dtype == DTYPE_BFLOAT16)
        round_slice_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(dst), src, count);
    else
        round_slice_kernel<__half><<<blocks, 256, 0, s>>>(reinterpret_cast<__half*>(dst), src, count);
    SH_CUDA(cudaGetLastError());
    return 0;
}

std::atomic<unsigned long long> g_collectives{0};

}  // namespace

struct RpbShard {
    int rank = 0, world = 1, device = 0;
    ncclComm_t comm = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_ready = nullptr, ev_done = nullptr;
    float* stage = nullptr;            /* float32 dB partials [k][n] */
    size_t stage_bytes = 0;
    int sm_count = 0;
    int comm_sms = -1;                 /* SMs the dA GEMM leaves to the collective's thread blocks; -1: chosen per call */
    int db_wire = 0;                   /* 0: float32 reduce-scatter + rounded all-gather; 1: all-reduce in the operand type */
    bool pending = false;              /* a dB reduction is in flight on the side stream */
};

namespace {
struct DeviceGuard {
    int prev = -1; bool moved = false;
    int enter(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) return -1;
        if (prev != device) { if (cudaSetDevice(device) != cudaSuccess) return -1; moved = true; }
        return 0;
    }
    ~DeviceGuard() { if (moved) cudaSetDevice(prev); }
};

int ensure_stage(RpbShard* s, size_t bytes) {
    if (bytes <= s->stage_bytes) return 0;
    if (s->stage) SH_CUDA(cudaFree(s->stage));
    s->stage = nullptr; s->stage_bytes = 0;
    SH_CUDA(cudaMalloc(reinterpret_cast<void**>(&s->stage), bytes));
    s->stage_bytes = bytes;
    return 0;
}
}  // namespace

/* ---- internal interface (shard_internal.h): used by the host-buffer pipeline */

int rpb_shard_rank_of(const RpbShard* s) { return s ? s->rank : 0; }
int rpb_shard_world_of(const RpbShard* s) { return s ? s->world : 1; }
int rpb_shard_device_of(const RpbShard* s) { return s ? s->device : -1; }

int rpb_shard_broadcast_bytes(RpbShard* s, void* buf, size_t bytes, int root, cudaStream_t stream) {
    if (!s || s->world == 1) return 0;
    SH_NCCL(g_nccl.Broadcast(buf, buf, bytes, ncclInt8, root, s->comm, stream));
    g_collectives++;
    return 0;
}

/* How dB travels.  0: all-reduce in the operand type (float32 / float64 operands, or db_wire == 1);
 * 1: float32 all-reduce + rounding (small dB); 2: float32 reduce-scatter, rounding of the owned slice, and an
 * all-gather in the operand type unless only the slice is wanted. */
static int db_route_of(int world, int db_wire, int k, int n, int dtype) {
    const size_t es = rpb_dtype_size(dtype);
    const size_t count = (size_t)k * n;
    if (world == 1 || es != 2 || db_wire != 0) return 0;
    const size_t chunk = count / (size_t)world;
    const bool even = count % (size_t)world == 0 && (chunk * es) % 16 == 0;
    return (even && count * sizeof(float) >= (size_t(1) << 20)) ? 2 : 1;
}
static int db_route(const RpbShard* s, int k, int n, int dtype) { return db_route_of(s->world, s->db_wire, k, n, dtype); }

extern "C" int rpb_shard_db_slice_of(int k, int n, DType dtype, int world, int rank, int db_wire, int flags, long long* begin,
                                     long long* end) {
    if (k <= 0 || n <= 0 || world < 1 || rank < 0 || rank >= world || !rpb_dtype_size((int)dtype)) return -1;
    long long b = 0, e = (long long)k * n;
    if ((flags & RPB_SHARD_SLICE_ONLY) && db_route_of(world, db_wire, k, n, (int)dtype) == 2) {
        const long long chunk = e / world;
        b = chunk * rank; e = b + chunk;
    }
    if (begin) *begin = b;
    if (end) *end = e;
    return 0;
}

void rpb_shard_db_slice(const RpbShard* s, int k, int n, int dtype, int flags, long long* begin, long long* end) {
    if (!s) { if (begin) *begin = 0; if (end) *end = (long long)k * n; return; }
    rpb_shard_db_slice_of(k, n, (DType)dtype, s->world, s->rank, s->db_wire, flags, begin, end);
}

/* dB = sum over ranks of A_rows^T . dC_rows.  The partial GEMM runs on `stream`, the reduction on the side
 * stream; rpb_shard_db_end makes `stream` wait for it.  RPB_SHARD_SLICE_ONLY: no all-gather, only this rank's
 * slice of dB (elements [rank * k*n/world, (rank+1) * k*n/world)) is valid afterwards. */
int rpb_shard_db_begin(RpbShard* s, void* dB, const void* A_rows, const void* dC_rows, long long rows, int k, int n,
                       int dtype, int flags, cudaStream_t stream) {
    const size_t es = rpb_dtype_size(dtype);
    const size_t count = (size_t)k * n;
    const int route = db_route(s, k, n, dtype);
    const bool f32_wire = route != 0;
    RpbGemm g;
    memset(&g, 0, sizeof(g));
    g.m = k; g.n = n; g.k = (int)rows; g.batch = g.reduce = 1;
    g.a_row = 1; g.a_col = k;                 /* A^T read through swapped strides */
    g.b_row = n; g.b_col = 1;
    g.c_row = n;
    void* target = dB;
    if (f32_wire) {
        if (ensure_stage(s, count * sizeof(float))) return -1;
        target = s->stage;
        g.c_float32 = 1;
    }
    if (rows > 0) {
        if (rp_matmul_ex(target, A_rows, dC_rows, &g, (DType)dtype, s->device, stream)) return -1;
    } else {
        SH_CUDA(cudaMemsetAsync(target, 0, count * (f32_wire ? 4 : es), stream));   /* a rank without rows adds zeros */
    }
    if (s->world == 1) return 0;
    SH_CUDA(cudaEventRecord(s->ev_ready, stream));
    SH_CUDA(cudaStreamWaitEvent(s->side, s->ev_ready, 0));
    const size_t chunk = count / (size_t)s->world;
    if (route == 2) {
        float* mine = s->stage + (size_t)s->rank * chunk;
        SH_NCCL(g_nccl.ReduceScatter(s->stage, mine, chunk, ncclFloat32, ncclSum, s->comm, s->side));
        char* out = reinterpret_cast<char*>(dB) + (size_t)s->rank * chunk * es;
        if (launch_round(out, mine, chunk, dtype, 8 * (s->comm_sms > 0 ? s->comm_sms : 16), s->side)) return -1;
        g_collectives++;
        if (!(flags & RPB_SHARD_SLICE_ONLY)) {
            SH_NCCL(g_nccl.AllGather(out, dB, chunk, nccl_type(dtype), s->comm, s->side));
            g_collectives++;
        }
    } else if (route == 1) {
        /* small (a broadcast-batched B of a few hundred KB): one all-reduce has the lower latency */
        SH_NCCL(g_nccl.AllReduce(s->stage, s->stage, count, ncclFloat32, ncclSum, s->comm, s->side));
        if (launch_round(dB, s->stage, count, dtype, 8 * (s->comm_sms > 0 ? s->comm_sms : 16), s->side)) return -1;
        g_collectives++;
    } else {
        SH_NCCL(g_nccl.AllReduce(dB, dB, count, nccl_type(dtype), ncclSum, s->comm, s->side));
        g_collectives++;
    }
    SH_CUDA(cudaEventRecord(s->ev_done, s->side));
    s->pending = true;
    return 0;
}

int rpb_shard_db_end(RpbShard* s, cudaStream_t stream) {
    if (!s->pending) return 0;
    s->pending = false;
    SH_CUDA(cudaStreamWaitEvent(stream, s->ev_done, 0));
    return 0;
}

extern "C" {

int rpb_shard_unique_id(void* id_out) {
    if (!id_out) return -1;
    if (load_nccl()) return -1;
    ncclUniqueId id;
    SH_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out, &id, sizeof(id));
    return 0;
}

RpbShard* rpb_shard_create(const void* unique_id, int rank, int world, int device_id) {
    if (world < 1 || rank < 0 || rank >= world || device_id < 0 || (world > 1 && !unique_id)) {
        fprintf(stderr, "recpulse_b200: rpb_shard_create: bad arguments (rank %d of %d, device %d)\n", rank, world, device_id);
        return nullptr;
    }
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || device_id >= ndev) {
        cudaGetLastError();
        fprintf(stderr, "recpulse_b200: rpb_shard_create: no CUDA device %d\n", device_id);
        return nullptr;
    }
    DeviceGuard guard;
    if (guard.enter(device_id)) return nullptr;
    RpbShard* s = new RpbShard();
    s->rank = rank; s->world = world; s->device = device_id;
    auto fail = [&]() -> RpbShard* { rpb_shard_destroy(s); return nullptr; };
    if (cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, device_id) != cudaSuccess) return fail();
    if (cudaStreamCreateWithFlags(&s->side, cudaStreamNonBlocking) != cudaSuccess) return fail();
    if (cudaEventCreateWithFlags(&s->ev_ready, cudaEventDisableTiming) != cudaSuccess) return fail();
    if (cudaEventCreateWithFlags(&s->ev_done, cudaEventDisableTiming) != cudaSuccess) return fail();
    if (const char* e = getenv("RPB_SHARD_COMM_SMS")) s->comm_sms = atoi(e);
    if (const char* e = getenv("RPB_SHARD_DB_WIRE")) s->db_wire = !strcmp(e, "operand") ? 1 : 0;
    if (world > 1) {
        if (load_nccl()) return fail();
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        ncclResult_t r = g_nccl.CommInitRank(&s->comm, world, id, rank);
        if (r != ncclSuccess) {
            fprintf(stderr, "recpulse_b200: ncclCommInitRank failed: %s\n", g_nccl.GetErrorString(r));
            s->comm = nullptr;
            return fail();
        }
    }
    return s;
}

void rpb_shard_destroy(RpbShard* s) {
    if (!s) return;
    DeviceGuard guard;
    guard.enter(s->device);
    if (s->side) cudaStreamSynchronize(s->side);
    if (s->comm) g_nccl.CommDestroy(s->comm);
    if (s->stage) cudaFree(s->stage);
    if (s->ev_ready) cudaEventDestroy(s->ev_ready);
    if (s->ev_done) cudaEventDestroy(s->ev_done);
    if (s->side) cudaStreamDestroy(s->side);
    delete s;
}

int rpb_shard_rank(const RpbShard* s) { return s ? s->rank : -1; }
int rpb_shard_world(const RpbShard* s) { return s ? s->world : -1; }
unsigned long long rpb_shard_collective_count(void) { return g_collectives.load(); }

int rpb_shard_configure(RpbShard* s, int comm_sms, int db_wire) {
    if (!s || comm_sms < -1 || db_wire < 0 || db_wire > 1) return -1;
    s->comm_sms = comm_sms;
    s->db_wire = db_wire;
    return 0;
}

void rpb_shard_rows(long long rows, int world, int rank, long long* begin, long long* end) {
    if (world < 1 || rank < 0 || rank >= world || rows < 0) { if (begin) *begin = 0; if (end) *end = 0; return; }
    const long long base = rows / world, extra = rows % world;
    const long long b = rank * base + (rank < extra ? rank : extra);
    if (begin) *begin = b;
    if (end) *end = b + base + (rank < extra ? 1 : 0);
}

int rp_shard_replicate(RpbShard* s, void* buf, size_t bytes, int root, void* stream) {
    if (!s || !buf || !bytes || root < 0 || root >= s->world) return -1;
    DeviceGuard guard;
    if (guard.enter(s->device)) return -1;
    return rpb_shard_broadcast_bytes(s, buf, bytes, root, reinterpret_cast<cudaStream_t>(stream));
}

int rp_matmul_rowsharded_forward(RpbShard* s, void* C_rows, const void* A_rows, const void* B, long long rows, int k, int n,
                                 DType dtype, void* stream) {
    if (!s || !C_rows || !A_rows || !B || rows < 0 || rows > 0x7fffffffLL || k <= 0 || n <= 0 || !rpb_dtype_size((int)dtype)) return -1;
    if (rows == 0) return 0;
    RpbGemm g;
    rpb_gemm_packed(&g, (int)rows, k, n);
    return rp_matmul_ex(C_rows, A_rows, B, &g, dtype, s->device, stream);
}

int rp_matmul_rowsharded_backward(RpbShard* s, void* dA_rows, void* dB, const void* A_rows, const void* B, const void* dC_rows,
                                  long long rows, int k, int n, DType dtype, int flags, void* stream) {
    if (!s || !dC_rows || rows < 0 || rows > 0x7fffffffLL || k <= 0 || n <= 0 || !rpb_dtype_size((int)dtype)) return -1;
    if ((dB && !A_rows) || (dA_rows && !B) || (!dA_rows && !dB)) return -1;
    DeviceGuard guard;
    if (guard.enter(s->device)) return -1;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    /* the dB partials first, so that their reduction travels while the dA GEMM runs */
    if (dB && rpb_shard_db_begin(s, dB, A_rows, dC_rows, rows, k, n, (int)dtype, flags, st)) return -1;
    if (dA_rows && rows > 0) {
        RpbGemm g;
        rpb_gemm_packed(&g, (int)rows, n, k);
        g.b_row = 1; g.b_col = n;             /* B^T read through swapped strides */
        /* the GEMM kernels are persistent and fill every SM; a collective launched beside one would wait for it
         * to end, so while a reduction is in flight the GEMM leaves comm_sms SMs free */
        int cs = s->comm_sms;
        if (cs < 0) {
            /* 16 SMs let a 2-4 rank reduction finish inside the dA GEMM.  When the rows per rank get few (8 ranks of the
             * 65536-row workload) the exchange outlasts the GEMM and is what the step waits for: NCCL then needs all of
             * its thread blocks resident.  Measured at 8 GPUs, 8192 rows per rank: 2.72 ms per step with 16 SMs left free,
             * 2.41 with 32, 2.44 with 48.  Model: the GEMM at 1.3 PFLOP/s against the exchanged bytes at 260 GB/s. */
            const double es = (double)rpb_dtype_size((int)dtype);
            const double t_gemm = 2.0 * (double)rows * k * n / 1.3e15;
            const double t_comm = (double)(s->world - 1) / s->world * (double)k * n * (4.0 + es) / 260e9;
            cs = t_comm > t_gemm ? 32 : 16;
        }
        if (s->pending && cs > 0 && s->sm_count - cs >= 2) g.max_sms = s->sm_count - cs;
        if (rp_matmul_ex(dA_rows, dC_rows, B, &g, dtype, s->device, stream)) return -1;
    }
    return rpb_shard_db_end(s, st);
}

int rp_matmul_gather_rows(RpbShard* s, void* C_full, const void* C_rows, long long rows, int n, DType dtype, void* stream) {
    const size_t es = rpb_dtype_size((int)dtype);
    if (!s || !C_full || !C_rows || rows <= 0 || n <= 0 || !es) return -1;
    DeviceGuard guard;
    if (guard.enter(s->device)) return -1;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (s->world == 1) {
        if (C_full != C_rows) SH_CUDA(cudaMemcpyAsync(C_full, C_rows, (size_t)rows * n * es, cudaMemcpyDeviceToDevice, st));
        return 0;
    }
    SH_NCCL(g_nccl.AllGather(C_rows, C_full, (size_t)rows * n, nccl_type((int)dtype), s->comm, st));
    g_collectives++;
    return 0;
}

}  // extern "C"
