/*
 * Kernel selection and launch for librecpulse_b200: the raw-pointer entry points
 * (matmul_kernel_device, rp_matmul, rp_matmul_ex, rp_matmul_host) and the per-device
 * state they share (TMA descriptor encoder, scratch buffer for K-split partial
 * tiles, device status word).
 */
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include <dlfcn.h>
#include <link.h>

#include "gemm_dmma.cuh"
#include "gemm_simt.cuh"
#include "gemm_tf32x3.cuh"
#include "reduce_cols.cuh"
#include "gate_act.cuh"
#include "gemm_umma.cuh"
#include "rpb_common.h"

namespace {

constexpr int MAX_DEVICES = 64;
constexpr int BAL_MAX_UNITS = 1024;       /* CTAs (pairs) a balanced launch may use: far above any SM count */
constexpr int PLACE_MAX = 128;            /* units (CTA pairs) the placement-aware tile order knows about */
constexpr int SYNC_CTRS = 8;              /* launches that overlap on the device (other streams) do not share a rendezvous counter */

struct DeviceState {
    std::atomic<bool> ready{false};
    int sm_count = 0;
    int cc_major = 0;
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    cudaEvent_t scratch_free = nullptr;   /* recorded after the last reader of scratch */
    cudaStream_t scratch_stream = nullptr;
    bool scratch_used = false;
    bool scratch_pinned = false;          /* handed out inside a stream capture: a graph holds its address */
    int* status = nullptr;                /* this device's word of g_status_words (mapped host memory) */
    int* bal_flags = nullptr;             /* hand-off counters of the balanced schedule: [slot][rank][ready, done], all
                                           * zero between launches (the kernel clears what it used) */
    std::atomic<bool> bal_dirty{false};   /* a kernel gave up part-way: clear the counters before the next use */
    /* placement-aware tile order of the pair kernels (Args.wave_slot): state 0 = eligible launches record where the
     * hardware puts the clusters, 2 = permutation ready, 3 = the placement does not fit the scheme */
    std::mutex place_mu;
    int place_state = 0;
    int* place_smid = nullptr;            /* mapped host memory, PLACE_MAX ints, -1 until a kernel wrote them */
    unsigned char place_slot[PLACE_MAX];
    int* sync_ctrs = nullptr;             /* rendezvous of a launch's CTAs: SYNC_CTRS counters (one per launch, taken in turn), 128 bytes apart */
    std::atomic<unsigned int> sync_serial{0};
    std::mutex mu;                        /* guards the scratch fields: per device, because growing the scratch waits
                                           * for this device, whose work may in turn wait for another thread's GPU */
};

/* Kernel status words, one per device, in page-locked host memory that every device can address (the host
 * pointer is the device pointer under unified addressing).  A tcgen05 kernel whose bounded wait ran out
 * stores a code there; the host reads the word after the synchronisation it does anyway, without a copy. */
int* g_status_words = nullptr;

DeviceState g_dev[MAX_DEVICES];
std::mutex g_mutex;
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_force{-1};
thread_local int t_last_kernel = RPB_KERNEL_NONE;
thread_local bool t_act_fused = false;      /* set by the launcher whose epilogue applied RpbProblem.act */

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

#define RPB_CUDA(call)                                                                          \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess) {                                                                \
            fprintf(stderr, "recpulse_b200: %s failed: %s\n", #call, cudaGetErrorString(e_));   \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

/* The dynamic shared-memory limit of a kernel is set once per device, not once per launch.  `done` is a
 * static array owned by the launcher of that one kernel instantiation. */
template <typename K>
cudaError_t smem_attr_once(K kern, int bytes, std::atomic<bool>* done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < MAX_DEVICES && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess && dev >= 0 && dev < MAX_DEVICES) done[dev].store(true, std::memory_order_release);
    return e;
}

/* Encoded tensor maps are reused while the same operand (address, extents, strides, box) comes back,
 * which is the common case in a training loop: encoding costs about a microsecond per map. */
struct MapKey {
    const void* base; unsigned long long d[4], s[3]; unsigned box[4]; int dt, rank, swz;
    bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
    static constexpr int N = 64;
    MapKey key[N]; CUtensorMap map[N]; bool used[N] = {}; int next = 0;
    std::mutex mu;
    bool get(const MapKey& k, CUtensorMap* out) {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < N; ++i) if (used[i] && key[i] == k) { *out = map[i]; return true; }
        return false;
    }
    void put(const MapKey& k, const CUtensorMap& m) {
        std::lock_guard<std::mutex> lock(mu);
        key[next] = k; map[next] = m; used[next] = true; next = (next + 1) % N;
    }
};
MapCache g_maps;

/* Diagnostics: rpb_trace_enable() makes every tcgen05 launch stamp its milestones (rpb_umma::trace_mark) into a
 * small mapped host buffer that rpb_trace_read() copies out. */
unsigned long long* g_trace_buffer = nullptr;

/* Bound of one mbarrier wait inside the tcgen05 kernels, in SM clock cycles: about 2 s by default,
 * rpb_set_wait_limit_ms() or RPB_WAIT_LIMIT_MS changes it (a caller with a watchdog of its own wants less). */
std::atomic<long long> g_wait_limit{0};
long long wait_limit_cycles() {
    long long v = g_wait_limit.load(std::memory_order_relaxed);
    if (v > 0) return v;
    v = rpb_umma::WAIT_LIMIT_CYCLES;
    if (const char* e = getenv("RPB_WAIT_LIMIT_MS")) { const long long ms = atoll(e); if (ms > 0) v = ms * 2000000ll; }
    g_wait_limit.store(v, std::memory_order_relaxed);
    return v;
}
uint32_t epilogue_sleep_ns() {
    const char* e = getenv("RPB_EPI_SLEEP_NS");          /* read per launch: lets one process compare settings */
    const int v = e ? atoi(e) : 0;
    return (uint32_t)(v < 0 ? 0 : v);
}

int forced_family() {
    int f = g_force.load();
    if (f >= 0) return f;
    const char* env = getenv("RPB_FORCE_KERNEL");
    f = 0;
    if (env) {
        if (!strcmp(env, "simt")) f = RPB_KERNEL_SIMT;
        else if (!strcmp(env, "umma")) f = RPB_KERNEL_UMMA;
    }
    g_force.store(f);
    return f;
}

int device_state(int device_id, DeviceState** out) {
    if (device_id < 0 || device_id >= MAX_DEVICES) {
        fprintf(stderr, "recpulse_b200: invalid device id %d\n", device_id);
        return -1;
    }
    DeviceState& d = g_dev[device_id];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!d.ready.load(std::memory_order_relaxed)) {
            RPB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device_id));
            RPB_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device_id));
            if (!g_status_words) {
                void* w = nullptr;
                RPB_CUDA(cudaHostAlloc(&w, sizeof(int) * MAX_DEVICES, cudaHostAllocPortable | cudaHostAllocMapped));
                memset(w, 0, sizeof(int) * MAX_DEVICES);
                g_status_words = reinterpret_cast<int*>(w);
            }
            d.status = g_status_words + device_id;
            RPB_CUDA(cudaMalloc(&d.bal_flags, sizeof(int) * 4 * BAL_MAX_UNITS));
            RPB_CUDA(cudaMemset(d.bal_flags, 0, sizeof(int) * 4 * BAL_MAX_UNITS));
            {
                void* w = nullptr;
                RPB_CUDA(cudaHostAlloc(&w, sizeof(int) * PLACE_MAX, cudaHostAllocPortable | cudaHostAllocMapped));
                d.place_smid = reinterpret_cast<int*>(w);
                for (int i = 0; i < PLACE_MAX; ++i) d.place_smid[i] = -1;
            }
            RPB_CUDA(cudaMalloc(&d.sync_ctrs, SYNC_CTRS * 128));
            RPB_CUDA(cudaMemset(d.sync_ctrs, 0, SYNC_CTRS * 128));
            RPB_CUDA(cudaEventCreateWithFlags(&d.scratch_free, cudaEventDisableTiming));
            {   /* temporaries for packed operands come from the stream-ordered pool: let it keep freed blocks */
                const char* e = getenv("RPB_POOL");
                cudaMemPool_t pool;
                unsigned long long keep = ~0ull;
                if (!(e && atoi(e) == 0) && cudaDeviceGetDefaultMemPool(&pool, device_id) == cudaSuccess)
                    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
                cudaGetLastError();
            }
            if (!g_encode) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult qres;
                RPB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
                if (!fn || qres != cudaDriverEntryPointSuccess) {
                    fprintf(stderr, "recpulse_b200: cuTensorMapEncodeTiled not available\n");
                    return -1;
                }
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            }
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return 0;
}

/* Scratch for K-split partial tiles: one buffer per device, grown on demand.  A launch on a
 * stream other than the previous user's first waits for that user's reduction to finish. */
bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone;
}

int get_scratch(DeviceState* d, size_t bytes, cudaStream_t stream, void** out) {
    std::lock_guard<std::mutex> lock(d->mu);
    const bool cap = capturing(stream);
    if (bytes > d->scratch_bytes) {
        if (cap) {
            fprintf(stderr, "recpulse_b200: the K-split scratch would have to grow during stream capture; run the same "
                            "shapes once before capturing (or size it with rpb_scratch_reserve)\n");
            return -1;
        }
        if (d->scratch_pinned) {
            /* a captured graph has this buffer's address in its kernel arguments and tensor maps: freeing it
             * would make the next replay write freed memory */
            fprintf(stderr, "recpulse_b200: the K-split scratch (%zu bytes) was used inside a stream capture and cannot "
                            "grow to %zu bytes any more; call rpb_scratch_reserve before capturing, or rpb_scratch_reset "
                            "once every graph that used it is destroyed\n", d->scratch_bytes, bytes);
            return -1;
        }
        if (d->scratch) RPB_CUDA(cudaFree(d->scratch));       /* synchronises the device */
        d->scratch = nullptr; d->scratch_bytes = 0; d->scratch_used = false;
        size_t want = bytes < (size_t(32) << 20) ? (size_t(32) << 20) : bytes + bytes / 4;
        RPB_CUDA(cudaMalloc(&d->scratch, want));
        d->scratch_bytes = want;
    }
    if (cap) d->scratch_pinned = true;
    /* inside a capture the graph's own edges order the users of the scratch; the guard event stays out of it */
    if (!cap && d->scratch_used && d->scratch_stream != stream)
        RPB_CUDA(cudaStreamWaitEvent(stream, d->scratch_free, 0));
    *out = d->scratch;
    return 0;
}
int release_scratch(DeviceState* d, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(d->mu);
    if (capturing(stream)) return 0;
    RPB_CUDA(cudaEventRecord(d->scratch_free, stream));
    d->scratch_stream = stream;
    d->scratch_used = true;
    return 0;
}

/* ------------------------------------------------------------------ SIMT launch */

template <typename T, typename Acc, int BM, int BN, int BK, int TM, int TN>
int launch_simt_cfg(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    rpb_simt::Args a;
    a.a = A; a.b = B; a.c = C;
    a.m = p.m; a.n = p.n; a.k = p.k; a.batch = p.batch; a.reduce = p.reduce;
    a.a_row = p.a_row; a.a_col = p.a_col; a.a_batch = p.a_batch; a.a_reduce = p.a_reduce;
    a.b_row = p.b_row; a.b_col = p.b_col; a.b_batch = p.b_batch; a.b_reduce = p.b_reduce;
    a.c_row = p.c_row; a.c_batch = p.c_batch; a.accumulate = p.accumulate; a.bias = p.bias;
    a.tiles_m = (p.m + BM - 1) / BM; a.tiles_n = (p.n + BN - 1) / BN;
    a.k_blocks = (p.k + BK - 1) / BK;
    a.k_iters = a.k_blocks * p.reduce;
    long long tiles = (long long)a.tiles_m * a.tiles_n * p.batch;
    int splits = 1;
    if (tiles < d->sm_count && a.k_iters >= 8) {
        long long want = (2LL * d->sm_count + tiles - 1) / tiles;
        long long cap = a.k_iters / 4;
        splits = (int)(want < cap ? want : cap);
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    a.iters_per_split = (a.k_iters + splits - 1) / splits;
    a.splits = (a.k_iters + a.iters_per_split - 1) / a.iters_per_split;
    a.partial = nullptr;
    long long blocks = tiles * a.splits;
    if (blocks > 0x7fffffffLL) { fprintf(stderr, "recpulse_b200: problem too large for one launch\n"); return -1; }
    if (a.splits > 1) {
        size_t bytes = sizeof(Acc) * (size_t)a.splits * p.batch * p.m * p.n;
        if (get_scratch(d, bytes, stream, &a.partial)) return -1;
    }
    constexpr int NT = (BM / TM) * (BN / TN);
    RPB_CUDA(rpb_launch(rpb_simt::gemm_kernel<T, Acc, BM, BN, BK, TM, TN>, dim3((unsigned)blocks), dim3(NT), 0, stream, 1, a));
    g_launches++;
    if (a.splits > 1) {
        rpb_simt::launch_splitk_reduce<T, Acc>(reinterpret_cast<const Acc*>(a.partial), reinterpret_cast<T*>(C), a.splits,
                                               p.batch, p.m, p.n, p.c_row, p.c_batch, p.accumulate, p.bias, d->sm_count, stream);
        g_launches++;
        if (release_scratch(d, stream)) return -1;
    }
    RPB_CUDA(cudaGetLastError());
    t_last_kernel = RPB_KERNEL_SIMT;
    return 0;
}

/* ------------------------------------------------------------------ float64 tensor-core launch */

template <bool A_MN, bool B_MN>
int launch_dmma_inst(const rpb_simt::Args& a, long long blocks, cudaStream_t stream) {
    auto kern = rpb_dmma::gemm_kernel<A_MN, B_MN>;
    static std::atomic<bool> attr_done[MAX_DEVICES];
    RPB_CUDA(smem_attr_once(kern, rpb_dmma::SMEM_BYTES, attr_done));
    RPB_CUDA(rpb_launch(kern, dim3((unsigned)blocks), dim3(rpb_dmma::THREADS), rpb_dmma::SMEM_BYTES, stream, 1, a));
    g_launches++;
    return 0;
}

/* returns 1 when the operands do not meet the kernel's layout requirements */
int launch_dmma(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    auto even = [](long long s) { return s > 0 && s % 2 == 0; };
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    bool a_mn, b_mn;
    if (p.a_col == 1 && (p.m == 1 || even(p.a_row))) a_mn = false;
    else if (p.a_row == 1 && (p.k == 1 || even(p.a_col))) a_mn = true;
    else return 1;
    if (p.b_col == 1 && (p.k == 1 || even(p.b_row))) b_mn = true;
    else if (p.b_row == 1 && (p.n == 1 || even(p.b_col))) b_mn = false;
    else return 1;
    if (!al16(A) || !al16(B)) return 1;
    if ((p.batch > 1 && (p.a_batch % 2 || p.b_batch % 2)) || (p.reduce > 1 && (p.a_reduce % 2 || p.b_reduce % 2))) return 1;
    if ((long long)p.m * p.n < 64 * 64) return 1;             /* tiny outputs: the small-tile kernel */

    rpb_simt::Args a;
    a.a = A; a.b = B; a.c = C;
    a.m = p.m; a.n = p.n; a.k = p.k; a.batch = p.batch; a.reduce = p.reduce;
    a.a_row = p.a_row; a.a_col = p.a_col; a.a_batch = p.a_batch; a.a_reduce = p.a_reduce;
    a.b_row = p.b_row; a.b_col = p.b_col; a.b_batch = p.b_batch; a.b_reduce = p.b_reduce;
    a.c_row = p.c_row; a.c_batch = p.c_batch; a.accumulate = p.accumulate; a.bias = p.bias;
    a.tiles_m = (p.m + rpb_dmma::BM - 1) / rpb_dmma::BM; a.tiles_n = (p.n + rpb_dmma::BN - 1) / rpb_dmma::BN;
    a.k_blocks = (p.k + rpb_dmma::BK - 1) / rpb_dmma::BK;
    a.k_iters = a.k_blocks * p.reduce;
    const long long tiles = (long long)a.tiles_m * a.tiles_n * p.batch;
    int splits = 1;
    if (tiles * 2 <= d->sm_count && a.k_iters >= 8) {
        long long want = d->sm_count / tiles, cap = a.k_iters / 4;
        splits = (int)(want < cap ? want : cap);
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    a.iters_per_split = (a.k_iters + splits - 1) / splits;
    a.splits = (a.k_iters + a.iters_per_split - 1) / a.iters_per_split;
    a.partial = nullptr;
    long long blocks = tiles * a.splits;
    if (blocks > 0x7fffffffLL) return 1;
    if (a.splits > 1 && get_scratch(d, sizeof(double) * (size_t)a.splits * p.batch * p.m * p.n, stream, &a.partial)) return -1;
    /* More tiles than SMs and a sparse last wave: deal (tile, K block) units evenly to one CTA per SM instead
     * (2048^3: 256 tiles = 1.73 waves of work ran as 2 waves) */
    {
        const char* e = getenv("RPB_DMMA_BALANCED");            /* 0: one CTA per tile always (A/B evidence) */
        const int env = e ? atoi(e) : 1;
        int sms = d->sm_count;
        if (p.max_sms > 0 && p.max_sms < sms) sms = p.max_sms;
        const long long waves = (tiles + sms - 1) / sms;
        if (env && a.splits == 1 && tiles > sms && a.k_iters >= 8 && tiles * 100 < waves * sms * 93) {
            void* ws = nullptr;
            if (get_scratch(d, sizeof(double) * (size_t)(sms - 1) * 2 * rpb_dmma::BM * rpb_dmma::BN, stream, &ws)) return -1;
            a.sk_ctas = sms; a.sk_units = tiles * a.k_iters; a.sk_scratch = reinterpret_cast<double*>(ws);
            blocks = sms;
        }
    }
    int rc;
    if (!a_mn && !b_mn) rc = launch_dmma_inst<false, false>(a, blocks, stream);
    else if (!a_mn && b_mn) rc = launch_dmma_inst<false, true>(a, blocks, stream);
    else if (a_mn && !b_mn) rc = launch_dmma_inst<true, false>(a, blocks, stream);
    else rc = launch_dmma_inst<true, true>(a, blocks, stream);
    if (rc) return -1;
    if (a.sk_ctas > 0) {
        RPB_CUDA(rpb_launch(rpb_dmma::balanced_fixup_kernel, dim3((unsigned)(a.sk_ctas - 1), 16), dim3(256), 0, stream, 1, a));
        g_launches++;
        if (release_scratch(d, stream)) return -1;
    }
    if (a.splits > 1) {
        rpb_simt::launch_splitk_reduce<double, double>(reinterpret_cast<const double*>(a.partial), reinterpret_cast<double*>(C),
                                                       a.splits, p.batch, p.m, p.n, p.c_row, p.c_batch, p.accumulate,
                                                       p.bias, d->sm_count, stream);
        g_launches++;
        if (release_scratch(d, stream)) return -1;
    }
    RPB_CUDA(cudaGetLastError());
    t_last_kernel = RPB_KERNEL_DMMA;
    return 0;
}

/* ------------------------------------------------------------------ float32 3xTF32 launch */

template <int BM, int BN, int WM, int WN, bool A_MN, bool B_MN>
int launch_tf32_inst(const rpb_simt::Args& a, long long blocks, cudaStream_t stream) {
    auto kern = rpb_tf32::gemm_kernel<BM, BN, WM, WN, A_MN, B_MN>;
    constexpr int smem = rpb_tf32::Cfg<BM, BN>::SMEM_BYTES;
    static std::atomic<bool> attr_done[MAX_DEVICES];
    RPB_CUDA(smem_attr_once(kern, smem, attr_done));
    RPB_CUDA(rpb_launch(kern, dim3((unsigned)blocks), dim3(WM * WN * 32), smem, stream, 1, a));
    g_launches++;
    return 0;
}

template <int BM, int BN, int WM, int WN>
int launch_tf32_cfg(const RpbProblem& p, void* C, const void* A, const void* B, bool a_mn, bool b_mn, DeviceState* d,
                    cudaStream_t stream) {
    rpb_simt::Args a;
    a.a = A; a.b = B; a.c = C;
    a.m = p.m; a.n = p.n; a.k = p.k; a.batch = p.batch; a.reduce = p.reduce;
    a.a_row = p.a_row; a.a_col = p.a_col; a.a_batch = p.a_batch; a.a_reduce = p.a_reduce;
    a.b_row = p.b_row; a.b_col = p.b_col; a.b_batch = p.b_batch; a.b_reduce = p.b_reduce;
    a.c_row = p.c_row; a.c_batch = p.c_batch; a.accumulate = p.accumulate; a.bias = p.bias;
    a.tiles_m = (p.m + BM - 1) / BM; a.tiles_n = (p.n + BN - 1) / BN;
    a.k_blocks = (p.k + rpb_tf32::BK - 1) / rpb_tf32::BK;
    a.k_iters = a.k_blocks * p.reduce;
    const long long tiles = (long long)a.tiles_m * a.tiles_n * p.batch;
    int splits = 1;
    if (tiles * 2 <= d->sm_count && a.k_iters >= 8) {
        long long want = d->sm_count / tiles, cap = a.k_iters / 4;
        splits = (int)(want < cap ? want : cap);
        if (splits > 64) splits = 64;
        if (splits < 1) splits = 1;
    }
    a.iters_per_split = (a.k_iters + splits - 1) / splits;
    a.splits = (a.k_iters + a.iters_per_split - 1) / a.iters_per_split;
    a.partial = nullptr;
    const long long blocks = tiles * a.splits;
    if (blocks > 0x7fffffffLL) return 1;
    if (a.splits > 1 && get_scratch(d, sizeof(float) * (size_t)a.splits * p.batch * p.m * p.n, stream, &a.partial)) return -1;
    int rc;
    if (!a_mn && !b_mn) rc = launch_tf32_inst<BM, BN, WM, WN, false, false>(a, blocks, stream);
    else if (!a_mn && b_mn) rc = launch_tf32_inst<BM, BN, WM, WN, false, true>(a, blocks, stream);
    else if (a_mn && !b_mn) rc = launch_tf32_inst<BM, BN, WM, WN, true, false>(a, blocks, stream);
    else rc = launch_tf32_inst<BM, BN, WM, WN, true, true>(a, blocks, stream);
    if (rc) return -1;
    if (a.splits > 1) {
        rpb_simt::launch_splitk_reduce<float, float>(reinterpret_cast<const float*>(a.partial), reinterpret_cast<float*>(C),
                                                     a.splits, p.batch, p.m, p.n, p.c_row, p.c_batch, p.accumulate,
                                                     p.bias, d->sm_count, stream);
        g_launches++;
        if (release_scratch(d, stream)) return -1;
    }
    RPB_CUDA(cudaGetLastError());
    t_last_kernel = RPB_KERNEL_TF32X3;
    return 0;
}

/* returns 1 when the operands do not meet the kernel's layout requirements */
int launch_tf32(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    auto mult4 = [](long long s) { return s > 0 && s % 4 == 0; };
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    bool a_mn, b_mn;
    if (p.a_col == 1 && (p.m == 1 || mult4(p.a_row))) a_mn = false;
    else if (p.a_row == 1 && (p.k == 1 || mult4(p.a_col))) a_mn = true;
    else return 1;
    if (p.b_col == 1 && (p.k == 1 || mult4(p.b_row))) b_mn = true;
    else if (p.b_row == 1 && (p.n == 1 || mult4(p.b_col))) b_mn = false;
    else return 1;
    if (!al16(A) || !al16(B)) return 1;
    if ((p.batch > 1 && (p.a_batch % 4 || p.b_batch % 4)) || (p.reduce > 1 && (p.a_reduce % 4 || p.b_reduce % 4))) return 1;
    if ((long long)p.m * p.n < 32 * 32) return 1;
    const long long big_tiles = (long long)((p.m + 127) / 128) * ((p.n + 127) / 128) * p.batch;
    if (big_tiles >= d->sm_count / 2) return launch_tf32_cfg<128, 128, 2, 4>(p, C, A, B, a_mn, b_mn, d, stream);
    return launch_tf32_cfg<64, 64, 2, 2>(p, C, A, B, a_mn, b_mn, d, stream);
}

template <typename T, typename Acc>
int launch_simt(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    if constexpr (sizeof(Acc) == 4) {
        if (p.m >= 512 && p.n >= 512) return launch_simt_cfg<T, Acc, 128, 128, 16, 8, 8>(p, C, A, B, d, stream);
    }
    return launch_simt_cfg<T, Acc, 64, 64, 16, 4, 4>(p, C, A, B, d, stream);
}

/* ------------------------------------------------------------------ tcgen05 launch */

struct OperandPlan {
    bool ok = false;
    bool mn_major = false;
    long long outer_stride = 0;     /* elements: stride of the non-contiguous matrix index */
    int batch_mul = 1, reduce_mul = 1;
    long long batch_stride = 0, reduce_stride = 0;
};

bool stride_ok(long long s, int es) { return s > 0 && (s * es) % 16 == 0 && (s * es) < (1LL << 40); }

/* mn/k: extents; mn_s/k_s: element strides of the output-side index and of the reduction index */
OperandPlan plan_operand(const void* base, int mn, int k, long long mn_s, long long k_s,
                         int batch, long long batch_s, int reduce, long long reduce_s, int es = 2) {
    OperandPlan o;
    if (reinterpret_cast<uintptr_t>(base) & 15u) return o;
    if (k_s == 1 && (mn == 1 || stride_ok(mn_s, es))) { o.mn_major = false; o.outer_stride = mn_s; }
    else if (mn_s == 1 && (k == 1 || stride_ok(k_s, es))) { o.mn_major = true; o.outer_stride = k_s; }
    else return o;
    if (batch > 1) {
        if (batch_s == 0) o.batch_mul = 0;
        else if (stride_ok(batch_s, es)) o.batch_stride = batch_s;
        else return o;
    }
    if (reduce > 1) {
        if (reduce_s == 0) o.reduce_mul = 0;
        else if (stride_ok(reduce_s, es)) o.reduce_stride = reduce_s;
        else return o;
    }
    o.ok = true;
    return o;
}

int encode_map(CUtensorMap* map, const void* base, const OperandPlan& o, int mn, int k, int batch, int reduce,
               int box_mn_rows, CUtensorMapDataType dt, int es = 2) {
    /* dims, innermost first: (contiguous index, other matrix index, summed problem, batch) */
    cuuint64_t dims[4]; cuuint64_t strides[3]; cuuint32_t box[4]; cuuint32_t estr[4] = {1, 1, 1, 1};
    const cuuint64_t inner = o.mn_major ? mn : k;
    const cuuint64_t outer = o.mn_major ? k : mn;
    dims[0] = inner; dims[1] = outer;
    dims[2] = (reduce > 1 && o.reduce_mul) ? reduce : 1;
    dims[3] = (batch > 1 && o.batch_mul) ? batch : 1;
    auto pad16 = [](unsigned long long b) { return (b + 15ull) & ~15ull; };
    unsigned long long s1 = (outer > 1 && o.outer_stride > 0) ? (unsigned long long)o.outer_stride * es : pad16(inner * es);
    if (s1 % 16) s1 = pad16(s1);
    unsigned long long s2 = dims[2] > 1 ? (unsigned long long)o.reduce_stride * es : pad16(s1 * outer);
    unsigned long long s3 = dims[3] > 1 ? (unsigned long long)o.batch_stride * es : pad16(s2 * dims[2]);
    const unsigned long long lim = (1ull << 40) - 16;
    if (s2 > lim) s2 = lim;
    if (s3 > lim) s3 = lim;
    strides[0] = s1; strides[1] = s2; strides[2] = s3;
    box[0] = 128 / es;                              /* the 128-byte swizzle span */
    box[1] = o.mn_major ? 128 / es : box_mn_rows;   /* MN-major: one K block of rows */
    box[2] = 1; box[3] = 1;
    /* 32-bit operands read MN-major by the tensor cores need the 128-byte swizzle with 32-byte atoms (the only
     * shared-memory layout tcgen05 accepts for transposed tf32); everything else uses the plain 128-byte swizzle */
    const CUtensorMapSwizzle swz = (es == 4 && o.mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    /* L2 promotion of the operand loads: 256 bytes measured best; RPB_L2_PROMO=0..3 (none, 64, 128, 256) for experiments */
    CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    if (const char* e = getenv("RPB_L2_PROMO")) {
        const int v = atoi(e);
        promo = v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : v == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
              : v == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    }
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base; key.dt = (int)dt; key.rank = 4; key.swz = 16 + (int)swz + 64 * (int)promo;
    for (int i = 0; i < 4; ++i) { key.d[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i < 3; ++i) key.s[i] = strides[i];
    if (g_maps.get(key, map)) return 0;
    CUresult r = g_encode(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swz, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) g_maps.put(key, *map);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "recpulse_b200: cuTensorMapEncodeTiled failed (%d) dims=[%llu,%llu,%llu,%llu] strides=[%llu,%llu,%llu]\n",
                (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
                (unsigned long long)dims[3], s1, s2, s3);
        return -1;
    }
    return 0;
}

/* tensor map for the epilogue's stores: [cols, rows, planes], boxes of box_cols x 32 rows (128 bytes wide) */
int encode_store_map(CUtensorMap* map, void* base, CUtensorMapDataType dt, int esize, long long cols, long long rows,
                     long long planes, long long row_stride, long long plane_stride, int box_cols) {
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(planes > 0 ? planes : 1)};
    unsigned long long s1 = (unsigned long long)row_stride * esize;
    unsigned long long s2 = dims[2] > 1 ? (unsigned long long)plane_stride * esize : ((s1 * rows + 15ull) & ~15ull);
    if (s1 % 16 || s2 % 16 || s1 >= (1ull << 40) || s2 >= (1ull << 40)) return -1;
    cuuint64_t strides[2] = {s1, s2};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base; key.dt = (int)dt; key.rank = 3; key.swz = 2;
    for (int i = 0; i < 3; ++i) { key.d[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i < 2; ++i) key.s[i] = strides[i];
    if (g_maps.get(key, map)) return 0;
    CUresult r = g_encode(map, dt, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) g_maps.put(key, *map);
    return r == CUDA_SUCCESS ? 0 : -1;
}

/* shared-memory matrix descriptor without the start address (128-byte swizzle, version 1) */
uint64_t smem_desc_base(bool mn_major, int es = 2) {
    if (es == 4 && mn_major) {
        /* transposed tf32: layout type 1 (128-byte swizzle, 32-byte atoms): atoms of 4 K rows x 128 bytes */
        const uint64_t sbo = 512 >> 4;                                /* next group of 4 K rows */
        const uint64_t lbo = (uint64_t)(32 * 128) >> 4;               /* next 32-element MN chunk (32 K rows further) */
        return (lbo << 16) | (sbo << 32) | (1ull << 46) | (1ull << 61);
    }
    const uint64_t sbo = 1024 >> 4;                                   /* next group of 8 rows */
    const uint64_t lbo = mn_major ? (uint64_t)((128 / es) * 128) >> 4 : 1;   /* next 128-byte-wide MN chunk */
    return (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

/* n-tiles per rasterisation group: the tiles in flight (one per CTA or per CTA pair) should cover a
 * block of C whose A row panels and B column panels hold about the same number of bytes:
 * mt * tile_m = nt * tile_n with mt * nt = tiles in flight */
int raster_group(int in_flight, int tile_m, int tile_n, int tiles_n) {
    int g = 1;
    while ((long long)(g + 1) * (g + 1) * tile_n <= (long long)in_flight * tile_m) ++g;
    if (g > tiles_n) g = tiles_n;
    return g < 1 ? 1 : g;
}

template <typename T, int BN, bool A_MN, bool B_MN, bool PAIR, int NH = 1>
int launch_umma_inst(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const CUtensorMap& mp,
                     const rpb_umma::Args& args, int grid, cudaStream_t stream) {
    using Cfg = rpb_umma::Config<BN, rpb_umma::Elem<T>::SPLIT, NH>;
    auto kern = rpb_umma::gemm_kernel<T, BN, A_MN, B_MN, PAIR, NH>;
    static std::atomic<bool> attr_done[MAX_DEVICES];
    RPB_CUDA(smem_attr_once(kern, Cfg::SMEM_BYTES, attr_done));
    RPB_CUDA(rpb_launch(kern, dim3((unsigned)grid), dim3(rpb_umma::Elem<T>::THREADS), Cfg::SMEM_BYTES, stream, PAIR ? 2 : 1,
                        ma, mb, mc, mp, args));
    g_launches++;
    RPB_CUDA(cudaGetLastError());
    return 0;
}

template <typename T, int BN, bool PAIR = false, int NH = 1>
int launch_umma_bn(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                   const CUtensorMap& mp, const rpb_umma::Args& args, int grid, cudaStream_t stream) {
    if (!a_mn && !b_mn) return launch_umma_inst<T, BN, false, false, PAIR, NH>(ma, mb, mc, mp, args, grid, stream);
    if (!a_mn && b_mn) return launch_umma_inst<T, BN, false, true, PAIR, NH>(ma, mb, mc, mp, args, grid, stream);
    if (a_mn && !b_mn) return launch_umma_inst<T, BN, true, false, PAIR, NH>(ma, mb, mc, mp, args, grid, stream);
    return launch_umma_inst<T, BN, true, true, PAIR, NH>(ma, mb, mc, mp, args, grid, stream);
}

/* Tile shape and K slices, chosen by a small cost model in microseconds fitted to measurements on B200
 * (cold operands).  A CTA's main loop advances one K block (128 bytes of K) per step.  The step time shrinks
 * far less than the arithmetic when the tile gets narrower: one tcgen05.mma took at least ~100-120 clocks to
 * issue and retire whatever its N (measured with the loads switched off: N = 256 runs at the tensor pipe's
 * rate, N = 128 at half of it, N = 64 at a quarter), so narrow tiles only pay when the wide ones leave most SMs
 * without work.  A CTA pair multiplies a 256 x 2BN tile with half the B traffic per SM and draws less power,
 * so it wins whenever it keeps about as many SMs busy.  Slicing K costs a second launch plus a round trip of
 * fp32 partial sums. */
struct TilePlan { int bn, splits, pair, wide; };   /* wide: the pair tile is two instructions wide (256 x 512) */
TilePlan plan_tiles(int m, int n, int batch, int k_iters, int sms, bool f32) {
    static int pair_env = -1;
    if (pair_env < 0) { const char* e = getenv("RPB_UMMA_PAIR"); pair_env = e ? (atoi(e) ? 2 : 1) : 0; }
    if (const char* e = getenv("RPB_UMMA_PLAN")) {                  /* "BN,splits,pair": pins the plan (experiments) */
        int b = 0, sp = 0, pr = 0;
        if (sscanf(e, "%d,%d,%d", &b, &sp, &pr) >= 2 && (b == 64 || b == 128 || (b == 256 && !pr)) && sp >= 1 &&
            (pr != 2 || (b == 128 && !f32 && m >= 256 && n >= 512))) {           /* pair = 2: the double-width tile */
            if (sp > k_iters) sp = k_iters;
            return TilePlan{b, sp > 128 ? 128 : sp, pr ? 1 : 0, pr == 2 ? 1 : 0};
        }
    }
    static const int cand_splits[] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128};
    /* microseconds per K block: one-CTA tiles 128 x {64, 128, 256}, pair tiles 256 x {128, 256} */
    static const double step16[5] = {0.26, 0.28, 0.41, 0.25, 0.38};
    static const double step32[5] = {0.70, 0.86, 1.50, 1.12, 1.33};
    const double* step = f32 ? step32 : step16;
    TilePlan best = {n <= 64 ? 64 : (n <= 128 ? 128 : 256), 1, 0, 0};
    double best_t = 1e30;
    for (int c = 0; c < 5; ++c) {
        const int pair = c >= 3;
        const int bn = pair ? (c == 3 ? 64 : 128) : 64 << c;
        const int tile_m = pair ? 256 : 128, tile_n = pair ? 2 * bn : bn;
        if (pair && (pair_env == 1 || m < 256 || n < tile_n)) continue;
        if (!pair && pair_env == 2 && m >= 256 && n >= 256) continue;
        if (tile_n > 64 && n <= tile_n / 2) continue;               /* never a tile twice as wide as C */
        const long long tiles = (long long)((m + tile_m - 1) / tile_m) * ((n + tile_n - 1) / tile_n) * batch;
        const int units = pair ? sms / 2 : sms;
        for (int sp : cand_splits) {
            if (sp > 1 && (k_iters / sp < 4 || tiles * sp > units)) break;
            const int ips = (k_iters + sp - 1) / sp;
            const long long waves = (tiles * sp + units - 1) / units;
            double t = (double)waves * (ips * step[c] + (pair ? 0.8 : 0.5));
            if (sp > 1) t += 3.5 + (double)sp * m * n * batch * 8.0 / 3.0e6;
            if (t < best_t) { best_t = t; best.bn = bn; best.splits = sp; best.pair = pair; best.wide = 0; }
        }
    }
    /* The double-width pair tile (256 x 512, two accumulators sharing the A tile) fetches a quarter fewer bytes per
     * FLOP than the 256 x 256 one.  Measured on 16-bit 8192-wide problems: 1.5-4% less time at the burst clock and
     * 4-8% more throughput under the power cap, where bytes moved are watts; but its tiles are twice as large, its
     * epilogue is only partly hidden and its last wave is not cut along K.  It replaces the 256 x 256 plan when the
     * model says so, with the 256 x 256 plan credited for its K-sliced last wave. */
    static int wide_env = -1;
    if (wide_env < 0) { const char* e = getenv("RPB_UMMA_WIDE"); wide_env = e ? (atoi(e) ? 2 : 1) : 0; }
    if (!f32 && wide_env != 1 && best.pair && best.bn == 128 && best.splits == 1 && n >= 512 && m >= 256) {
        const int units = sms / 2;
        const long long tiles_d = (long long)((m + 255) / 256) * ((n + 255) / 256) * batch;
        const long long tiles_w = (long long)((m + 255) / 256) * ((n + 511) / 512) * batch;
        double waves_d = (double)((tiles_d + units - 1) / units);
        const long long rem = tiles_d % units;
        if (batch == 1 && tiles_d > units && rem > 0 && rem * 2 <= units && k_iters >= 32) waves_d -= 0.5;
        const double waves_w = (double)((tiles_w + units - 1) / units);
        const double t_d = waves_d * (k_iters * step16[4] + 0.8);
        const double t_w = waves_w * (k_iters * 0.72 + 3.0);
        if (wide_env == 2 ? tiles_w >= 1 : t_w < t_d) { best.wide = 1; best_t = t_w; }
    }
    if (getenv("RPB_UMMA_PLAN_LOG"))
        fprintf(stderr, "rpb plan %dx%dx(%d blocks) batch %d: %s 128x%d%s, %d slices, model %.1f us\n", m, n, k_iters, batch,
                best.pair ? "pair" : "one-CTA", best.bn, best.wide ? " double-width" : "", best.splits, best_t);
    return best;
}

/* returns 1 when the problem cannot take the tcgen05 path (caller falls back to SIMT) */
template <typename T>
int launch_umma(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    if (d->cc_major != 10) return 1;
    constexpr int ES = (int)sizeof(T);
    constexpr int BK = rpb_umma::Elem<T>::BLOCK_K;
    constexpr bool F32 = rpb_umma::Elem<T>::SPLIT;
    OperandPlan pa = plan_operand(A, p.m, p.k, p.a_row, p.a_col, p.batch, p.a_batch, p.reduce, p.a_reduce, ES);
    OperandPlan pb = plan_operand(B, p.n, p.k, p.b_col, p.b_row, p.batch, p.b_batch, p.reduce, p.b_reduce, ES);
    if (!pa.ok || !pb.ok) return 1;

    const int k_iters_total = ((p.k + BK - 1) / BK) * p.reduce;
    int sms = d->sm_count;
    if (p.max_sms > 0 && p.max_sms < sms) sms = p.max_sms < 2 ? 2 : p.max_sms;
    /* BN = rows of B per CTA; a pair multiplies 256 x (2 BN) tiles */
    const TilePlan tp = plan_tiles(p.m, p.n, p.batch, k_iters_total, sms, F32);
    const bool pair = tp.pair != 0;
    const int BN = tp.bn;
    const int tile_m = pair ? 2 * rpb_umma::BLOCK_M : rpb_umma::BLOCK_M;
    const int inst_n = pair ? 2 * BN : BN;                          /* columns per tcgen05.mma and per accumulator */
    const int tile_n = tp.wide ? 2 * inst_n : inst_n;
    rpb_umma::Args a;
    memset(&a, 0, sizeof(a));
    a.m = p.m; a.n = p.n; a.k = p.k; a.batch = p.batch; a.reduce = p.reduce;
    a.k_blocks = (p.k + BK - 1) / BK;
    a.k_iters = a.k_blocks * p.reduce;
    a.tiles_m = (p.m + tile_m - 1) / tile_m;
    a.tiles_n = (p.n + tile_n - 1) / tile_n;
    long long tiles = (long long)a.tiles_m * a.tiles_n * p.batch;
    const int splits = tp.splits;
    a.iters_per_split = (a.k_iters + splits - 1) / splits;
    a.splits = (a.k_iters + a.iters_per_split - 1) / a.iters_per_split;
    a.total_work = tiles * a.splits;
    if (a.total_work + 4 * tiles > 0x7fffffffLL || (long long)a.tiles_m * a.tiles_n > 0x7fffffffLL) return 1;   /* the kernel decodes work items in 32 bits */
    a.group_n = raster_group(pair ? d->sm_count / 2 : d->sm_count, tile_m, tile_n, a.tiles_n);
    if (const char* e = getenv("RPB_GROUP_N")) {            /* experiments: n-tiles per rasterisation group */
        const int v = atoi(e);
        if (v >= 1) a.group_n = v < a.tiles_n ? v : a.tiles_n;
    }
    a.a_batch_mul = pa.batch_mul; a.a_reduce_mul = pa.reduce_mul;
    a.b_batch_mul = pb.batch_mul; a.b_reduce_mul = pb.reduce_mul;
    a.c = C; a.c_row = p.c_row; a.c_batch = p.c_batch; a.accumulate = p.accumulate;
    a.bias = p.bias;
    a.partial = nullptr;
    if (a.splits > 1) {
        void* ws = nullptr;
        size_t bytes = sizeof(float) * (size_t)a.splits * p.batch * p.m * p.n;
        if (get_scratch(d, bytes, stream, &ws)) return -1;
        a.partial = reinterpret_cast<float*>(ws);
    }
    const bool bf16 = p.dtype == DTYPE_BFLOAT16;
    const uint32_t fmt = F32 ? 2u : (bf16 ? 1u : 0u);             /* operand format: F16 = 0, BF16 = 1, TF32 = 2 */
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((pa.mn_major ? 1u : 0u) << 15) | ((pb.mn_major ? 1u : 0u) << 16) |
              ((uint32_t)(inst_n >> 3) << 17) | ((uint32_t)(tile_m >> 4) << 24);
    a.a_desc_base = smem_desc_base(pa.mn_major, ES);
    a.b_desc_base = smem_desc_base(pb.mn_major, ES);
    /* advance per instruction (32 bytes of K): K-major 32 bytes inside the swizzle row; MN-major the K rows it
     * covers (16 halves or 8 floats), 128 bytes each */
    const uint32_t mn_step = (uint32_t)(rpb_umma::Elem<T>::UMMA_K * 128) >> 4;
    a.a_kstep = pa.mn_major ? mn_step : 32 >> 4;
    a.b_kstep = pb.mn_major ? mn_step : 32 >> 4;
    a.status = d->status;
    a.wait_limit = wait_limit_cycles();
    a.epi_sleep_ns = epilogue_sleep_ns();
    a.trace = g_trace_buffer;
    /* double-width tiles: the second accumulator trails the first by this many K blocks at both ends of a tile
     * (at most stages - 1 = 3; measured on the row-sharded workload under the power cap: 0 -> 3 blocks = +1%) */
    a.wide_skew = 3;
    if (const char* e = getenv("RPB_WIDE_SKEW")) { const int v = atoi(e); a.wide_skew = v < 0 ? 0 : (v > 3 ? 3 : v); }

    CUtensorMap ma, mb;
    const CUtensorMapDataType dt = F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                       : (bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    if (encode_map(&ma, A, pa, p.m, p.k, p.batch, p.reduce, rpb_umma::BLOCK_M, dt, ES)) return -1;
    if (encode_map(&mb, B, pb, p.n, p.k, p.batch, p.reduce, BN, dt, ES)) return -1;

    /* output through shared memory + TMA store when the destination is TMA-addressable; the register
     * epilogue handles "C += AB" and odd alignments */
    CUtensorMap mc = ma;
    a.tma_store = 0;
    a.c_f32 = (p.c_f32 && a.splits == 1) ? 1 : 0;
    if (a.c_f32) {
        /* unrounded fp32 output of 16-bit operands: written like a K slice, straight into the caller's buffer */
        a.partial = reinterpret_cast<float*>(C);
        /* "C += AB" in float32 reads C back: the register epilogue */
        if (!p.accumulate && p.n % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0 &&
            encode_store_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.n, p.m, p.batch, p.n, (long long)p.m * p.n, 32) == 0)
            a.tma_store = 1;
    } else if (a.splits > 1) {
        if (p.n % 4 == 0 &&
            encode_store_map(&mc, a.partial, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.n, p.m, (long long)a.splits * p.batch,
                             p.n, (long long)p.m * p.n, 32) == 0)
            a.tma_store = 1;
    } else if (!p.accumulate && (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && p.c_row % (16 / ES) == 0 &&
               (p.batch == 1 || p.c_batch % (16 / ES) == 0)) {
        if (encode_store_map(&mc, C, dt, ES, p.n, p.m, p.batch, p.c_row, p.c_batch, 128 / ES) == 0) a.tma_store = 1;
    }

    {
        const char* e = getenv("RPB_EPI_PIPE");
        a.epi_pipe = e ? (atoi(e) ? 1 : 0) : 1;
    }
    /* the gate non-linearity lives in the register epilogue (it follows "C += AB" in its only user) */
    if (p.act && a.splits == 1) a.tma_store = 0;
    a.act = a.splits == 1 ? p.act : 0;
    /* Balanced schedule: with only a few waves of tiles, a last wave that is partly empty costs whole per cents
     * (4096^3 bf16: 256 tiles on 74 pairs = 3.46 waves run as 3.5 + a reduction launch).  Deal tiles x K-blocks evenly
     * instead; each CTA (pair) cuts at most two tiles, computes the piece at the end of its range first (fp32, to
     * scratch) and finishes the piece at the start of its range last, adding its neighbour's partial in the epilogue. */
    CUtensorMap mp = ma;
    a.bal = 0;
    {
        /* Off by default: measured on bf16 4096^3 it does not beat the K-sliced last wave (96.4 vs 94.6 us per GEMM;
         * the tiles in flight are spread over the whole output instead of sharing panels, and every CTA pays a
         * finishing epilogue at the very end).  RPB_BALANCED=1: where the last wave is sparse; 2: wherever it applies. */
        const char* be = getenv("RPB_BALANCED");
        const int env = be ? atoi(be) : 0;
        const long long units = pair ? sms / 2 : sms;
        if (env && !tp.wide && a.splits == 1 && p.batch == 1 && !p.c_f32 && a.tma_store == 1 && units >= 2 &&
            units <= BAL_MAX_UNITS && tiles > units && a.k_iters >= 16) {
            const long long waves = (tiles + units - 1) / units;
            const double idle = (double)(waves * units) / (double)tiles - 1.0;
            if (env > 1 || (idle >= 0.04 && waves <= 8)) {
                const size_t bytes = sizeof(float) * (size_t)units * tile_m * tile_n;      /* one fp32 tile per boundary */
                void* ws = nullptr;
                if (get_scratch(d, bytes, stream, &ws)) return -1;
                {
                    const long long total_units = tiles * a.k_iters;
                    a.bal = 1;
                    a.bal_per = total_units / units;
                    a.bal_extra = (int)(total_units % units);
                    a.bal_scratch = reinterpret_cast<float*>(ws);
                    a.bal_flags = d->bal_flags;
                    a.total_work = units;                    /* one CTA (pair) per range */
                    if (d->bal_dirty.exchange(false))
                        RPB_CUDA(cudaMemsetAsync(d->bal_flags, 0, sizeof(int) * 4 * BAL_MAX_UNITS, stream));
                }
            }
        }
    }
    /* Tail split: if the last wave of tiles would keep fewer than half of the CTAs (or CTA pairs) busy, cut
     * its tiles along K so that the wave is short instead of sparse (4096^3: 256 tiles on 74 pairs = 3 waves +
     * 34 tiles; with two K slices each the run takes 3.5 tile times instead of 4). */
    a.tail_begin = a.total_work; a.tail_splits = 1; a.tail_iters = a.k_iters;
    {
        const char* te = getenv("RPB_TAIL_SPLIT");        /* 0: off; 2: from 16 K blocks per tile on (tests) */
        const int env = te ? atoi(te) : 1;
        const long long units = pair ? sms / 2 : sms;
        const long long rem = units > 0 ? tiles % units : 0;
        const char* fe = getenv("RPB_TAIL_FUSE");
        const bool may_fuse = !(fe && atoi(fe) == 0) && rem * 64 <= 4 * BAL_MAX_UNITS;
        if (env && !tp.wide && !a.bal && a.splits == 1 && !p.c_f32 && p.batch == 1 && a.tma_store == 1 && tiles > units && rem > 0 && rem * 2 <= units) {
            long long ts = units / rem;
            if (ts > 4) ts = 4;
            if (ts > a.k_iters / 8) ts = a.k_iters / 8;
            /* Three or four slices need a reduction launch (~4 us): measured break-even at about 96 K blocks per tile.
             * Two slices are finished inside the kernel and pay from about 32 K blocks on (bf16 4096^3: 64). */
            const int min_iters = env > 1 ? 16 : ((ts == 2 && may_fuse) ? 32 : 96);
            if (a.k_iters < min_iters) ts = 1;
            if (ts >= 2) {
                const int per = (int)((a.k_iters + ts - 1) / ts);
                ts = (a.k_iters + per - 1) / per;
                const size_t bytes = sizeof(float) * (size_t)rem * ts * tile_m * tile_n;
                void* ws = nullptr;
                if (get_scratch(d, bytes, stream, &ws)) return -1;
                /* two slices: finished inside the kernel (whichever slice is second adds the first one's sums);
                 * more: fp32 tiles through map_p and a reduction launch */
                if (ts == 2 && may_fuse) {
                    a.tail_fuse = 1;
                    a.bal_scratch = reinterpret_cast<float*>(ws);
                    a.bal_flags = d->bal_flags;
                    a.tail_begin = tiles - rem; a.tail_splits = 2; a.tail_iters = per;
                    a.total_work = a.tail_begin + rem * 2;
                    if (d->bal_dirty.exchange(false))
                        RPB_CUDA(cudaMemsetAsync(d->bal_flags, 0, sizeof(int) * 4 * BAL_MAX_UNITS, stream));
                } else if (encode_store_map(&mp, ws, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, tile_n, tile_m, rem * ts, tile_n,
                                            (long long)tile_m * tile_n, 32) == 0) {
                    a.partial = reinterpret_cast<float*>(ws);
                    a.tail_begin = tiles - rem; a.tail_splits = (int)ts; a.tail_iters = per;
                    a.total_work = a.tail_begin + rem * ts;
                }
            }
        }
    }
    /* Rendezvous of the CTAs (pairs) at tile starts and every 32 K blocks, for launches of several waves of whole tiles
     * in round-robin order (Args.sync_ctr): without it the units drift apart by 2-3% per tile and every unit fetches
     * its operand panels from L2 by itself; in step, the L2 request coalescer serves units that share a panel with one
     * lookup (measured on 32768 x 8192 x 8192 bf16: sectors delivered per sector read 1.11 -> 1.2, DRAM reads -17%,
     * 3-5% less time at the burst clock, 2-4% more throughput under the power cap).  RPB_TILE_SYNC=0 switches it off,
     * 1 = tile starts only, n > 1 = every n K blocks, -n = the same for tiles of any length.
     * The units wait for one another, which presumes that all CTAs of the launch are resident: a persistent grid of at
     * most one CTA per SM is, unless another kernel holds SMs meanwhile.  The wait is therefore soft: a unit that has
     * waited ~30 us switches the rendezvous off for the rest of the launch (Args.sync_patience), so the worst case --
     * two such launches sharing the SMs, a replayed graph beside anything -- costs that once.  The two words are one of
     * SYNC_CTRS pairs, taken in turn and zeroed in stream order before the launch (a memset node in a capture). */
    {
        const char* e = getenv("RPB_TILE_SYNC");
        const int env_raw = e ? atoi(e) : 32;
        const int env = env_raw < 0 ? -env_raw : env_raw;                           /* negative: tiles of any length (tests) */
        const long long units = pair ? sms / 2 : sms;
        const long long whole = a.tail_splits > 1 ? a.tail_begin : a.total_work;     /* whole tiles in round-robin order */
        /* long tiles only: a rendezvous costs the producer about a microsecond, which its lead over the tensor pipe
         * (the stages in flight, ~2-3 us) hides a few times per 50+ us tile but not twice per 23 us tile (bf16 4096^3
         * with it: 100 -> 109 us) */
        if (env > 0 && !a.bal && a.splits == 1 && p.batch == 1 && whole >= 3 * units && (a.k_iters >= 128 || env_raw < 0)) {
            int* ctr = d->sync_ctrs + (size_t)(d->sync_serial.fetch_add(1) % SYNC_CTRS) * 32;
            RPB_CUDA(cudaMemsetAsync(ctr, 0, 2 * sizeof(int), stream));
            a.sync_ctr = ctr;
            a.sync_every = env > 1 ? env : 0;
            a.sync_items = whole;
            a.sync_patience = 60000;
            /* pause between polls of the counter: none (then four polls are kept in flight, a quarter of a round trip
             * apart).  The tighter the units leave a rendezvous, the more of their requests coalesce (32768 x 8192 x 8192
             * and 8192 x 32768 x 8192 under the power cap: pauses of 400 / 100 / 0 ns 1358 / 1366 / 1370 and 1378 / 1386 /
             * 1392 TFLOP/s; staggered polls another +0.2 / +0.5%); ~150 pollers for about a microsecond */
            a.sync_sleep = 0;
            if (const char* se = getenv("RPB_SYNC_SLEEP_NS")) { const int v = atoi(se); a.sync_sleep = (unsigned)(v < 0 ? 0 : v); }
        }
    }
    /* Placement-aware tile order (Args.wave_slot) for pair kernels on the full grid of a 148-SM part, column groups of
     * six tiles.  Measured: SM ids are dealt round-robin over the 8 GPCs at TPC granularity (TPC t sits in GPC t % 8; six
     * GPCs have 9 TPCs, two have 10), the SMs of a GPC share an L2 request coalescer, and the hardware places cluster c of
     * a full grid on the same TPC every time.  So eligible launches record the SM of every cluster in mapped host memory
     * until the table is complete; then the host deals each GPC's nine pairs a 3 x 3 block of the 12 x 6 tiles a wave
     * covers (the two left-over pairs take the two left-over tiles) and passes the permutation by value.  The permutation is indexed by cluster, so a launch that the hardware places
     * differently is still correct, it only shares less.  16384 x 8192 x 8192 bf16 (ncu): sectors delivered per
     * sector read 1.32 -> 1.49 (cuBLAS 1.47), L2 lookups 328 -> 290 M; +0.9% under the power cap.  RPB_PLACE=0: off. */
    if (pair && a.splits == 1 && p.batch == 1 && !a.bal && d->sm_count == 148 && sms == 148 && a.group_n == 6 &&
        a.tail_begin >= 74 && a.total_work >= 74) {
        const char* pe = getenv("RPB_PLACE");
        if (!(pe && atoi(pe) == 0)) {
            std::lock_guard<std::mutex> lock(d->place_mu);
            if (d->place_state == 0) {
                /* has an earlier launch filled in every cluster's SM?  (plain reads of mapped host memory: nothing here
                 * synchronises, queries or copies, so it is safe beside a stream capture) */
                const volatile int* rec = d->place_smid;
                bool all = true;
                for (int c = 0; c < 74; ++c) all = all && rec[c] >= 0;
                if (all) {
                    bool ok = true;
                    bool seen_tpc[74] = {}, seen_slot[74] = {};
                    for (int c = 0; c < 74 && ok; ++c) {
                        const int tpc = rec[c] >> 1;
                        if (tpc >= 74 || seen_tpc[tpc]) { ok = false; break; }
                        seen_tpc[tpc] = true;
                        const int g8 = tpc & 7, q = tpc >> 3;
                        const int sl = q >= 9 ? 72 + g8 : (3 * (g8 >> 1) + q / 3) * 6 + 3 * (g8 & 1) + q % 3;
                        if (sl >= 74 || seen_slot[sl]) { ok = false; break; }
                        seen_slot[sl] = true;
                        d->place_slot[c] = (unsigned char)sl;
                    }
                    d->place_state = ok ? 2 : 3;
                }
            }
            if (d->place_state == 2) {
                a.wave_slot_on = 1;
                memcpy(a.wave_slot, d->place_slot, 74);
            } else if (d->place_state == 0) {
                a.smid_out = d->place_smid;
            }
        }
    }
    if (a.act) t_act_fused = true;
    int grid = (int)(a.total_work < sms ? a.total_work : sms);
    int rc;
    if (pair) {
        const long long clusters = a.total_work < sms / 2 ? a.total_work : sms / 2;
        if (tp.wide) {
            if constexpr (!F32) rc = launch_umma_bn<T, 128, true, 2>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, (int)clusters * 2, stream);
            else rc = -1;
        }
        else if (BN == 64) rc = launch_umma_bn<T, 64, true>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, (int)clusters * 2, stream);
        else rc = launch_umma_bn<T, 128, true>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, (int)clusters * 2, stream);
    }
    else if (BN == 64) rc = launch_umma_bn<T, 64>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    else if (BN == 128) rc = launch_umma_bn<T, 128>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    else rc = launch_umma_bn<T, 256>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    if (rc) return -1;
    if ((a.bal || a.tail_fuse) && release_scratch(d, stream)) return -1;
    if (a.tail_splits > 1 && !a.tail_fuse) {
        const int rem = (int)(tiles - a.tail_begin);
        RPB_CUDA(rpb_launch(rpb_umma::tail_reduce_kernel<T>, dim3(rem, tile_m), dim3(tile_n / 4), 0, stream, 1,
                            (const float*)a.partial, reinterpret_cast<T*>(C), reinterpret_cast<const T*>(p.bias), p.m, p.n,
                            (long long)p.c_row, a.tiles_m, a.tiles_n, a.group_n, (int)a.tail_begin, a.tail_splits, tile_m, tile_n));
        g_launches++;
        RPB_CUDA(cudaGetLastError());
        if (release_scratch(d, stream)) return -1;
    }
    if (a.splits > 1 && p.c_f32) {
        rpb_simt::launch_splitk_reduce<float, float>(a.partial, reinterpret_cast<float*>(C), a.splits, p.batch, p.m, p.n, p.n,
                                                     (long long)p.m * p.n, p.accumulate, nullptr, d->sm_count, stream);
        g_launches++;
        RPB_CUDA(cudaGetLastError());
        if (release_scratch(d, stream)) return -1;
    } else if (a.splits > 1) {
        rpb_simt::launch_splitk_reduce<T, float>(a.partial, reinterpret_cast<T*>(C), a.splits, p.batch, p.m, p.n, p.c_row,
                                                 p.c_batch, p.accumulate, p.bias, d->sm_count, stream);
        g_launches++;
        RPB_CUDA(cudaGetLastError());
        if (release_scratch(d, stream)) return -1;
    }
    t_last_kernel = a.splits > 1 ? RPB_KERNEL_UMMA_SPLITK : RPB_KERNEL_UMMA;
    return 0;
}

/* ------------------------------------------------------------------ packing of layouts TMA cannot address */

/* dst[(z, o, i)] = src[z_b * batch_s + z_r * reduce_s + o * outer_s + i * inner_s] for o < outer, i < inner
 * (zero for inner <= i < inner_pad): the operand as packed rows of inner_pad elements. */
template <typename T>
__global__ void pack_operand_kernel(T* __restrict__ dst, const T* __restrict__ src, int outer, int inner, int inner_pad,
                                    long long outer_s, long long inner_s, int nbatch, long long batch_s, int nreduce,
                                    long long reduce_s)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long total = (long long)nbatch * nreduce * outer * inner_pad;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int i = (int)(e % inner_pad);
        long long t = e / inner_pad;
        const int o = (int)(t % outer); t /= outer;
        const int r = (int)(t % nreduce);
        const int b = (int)(t / nreduce);
        T v = T(0.f);
        if (i < inner) v = src[b * batch_s + r * reduce_s + o * outer_s + i * inner_s];
        dst[e] = v;
    }
}

/* dst[b][r][c] = src[b][r][c] for c < cols: takes the padding out of an output computed with an aligned
 * leading dimension */
template <typename T>
__global__ void unpack_rows_kernel(T* __restrict__ dst, const T* __restrict__ src, long long rows, int cols,
                                   long long dst_row_s, long long src_row_s, int nbatch, long long dst_batch_s,
                                   long long src_batch_s)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long total = (long long)nbatch * rows * cols;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int c = (int)(e % cols);
        long long t = e / cols;
        const long long r = t % rows;
        const int b = (int)(t / rows);
        dst[b * dst_batch_s + r * dst_row_s + c] = src[b * src_batch_s + r * src_row_s + c];
    }
}

template <typename T> int launch_umma(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream);

/* A large 16-bit (or fp32) problem whose operands are not TMA-addressable (odd leading dimension, unaligned
 * base, both strides != 1): copy the offending operands once, from the stream-ordered pool, into packed rows
 * padded to 16 bytes -- keeping the operand's orientation when one of its strides is 1, so that the copy reads
 * and writes contiguously -- and run the tcgen05 kernel on the copies.  RecPulse copies every non-contiguous
 * operand (ops/ops.c:21-25); here it only happens for layouts the TMA engine rejects.  1 = not applicable. */
template <typename T>
int launch_umma_packed(const RpbProblem& p, void* C, const void* A, const void* B, DeviceState* d, cudaStream_t stream) {
    if (d->cc_major != 10) return 1;
    constexpr int ES = (int)sizeof(T);
    constexpr int AL = 16 / ES;
    const double flops = 2.0 * p.m * p.n * (double)p.k * p.batch * p.reduce;
    if (flops < 5e8 || p.m < 64 || p.n < 64) return 1;
    OperandPlan pa = plan_operand(A, p.m, p.k, p.a_row, p.a_col, p.batch, p.a_batch, p.reduce, p.a_reduce, ES);
    OperandPlan pb = plan_operand(B, p.n, p.k, p.b_col, p.b_row, p.batch, p.b_batch, p.reduce, p.b_reduce, ES);
    const bool c_odd = !p.accumulate && ((reinterpret_cast<uintptr_t>(C) & 15u) != 0 || p.c_row % AL != 0 ||
                                          (p.batch > 1 && p.c_batch % AL != 0));
    if (pa.ok && pb.ok && !c_odd) return 1;             /* nothing to pack: the caller already tried the direct path */
    RpbProblem q = p;
    q.act = 0;                                          /* a padded C has other column quarters: the caller's pass applies it */
    void* tmp[3] = {nullptr, nullptr, nullptr};
    const void* A2 = A; const void* B2 = B;
    /* packs one operand; on return *mn_stride / *k_stride are its new element strides */
    auto pack = [&](int which, const void* src, int mn, long long mn_s, long long k_s, long long batch_s, long long reduce_s,
                    const void** out, long long* new_mn_s, long long* new_k_s, long long* new_reduce_s,
                    long long* new_batch_s) -> int {
        const bool keep_mn_major = mn_s == 1 && k_s != 1;
        const int outer = keep_mn_major ? p.k : mn, inner = keep_mn_major ? mn : p.k;
        const long long outer_s = keep_mn_major ? k_s : mn_s, inner_s = keep_mn_major ? mn_s : k_s;
        const int inner_pad = (inner + AL - 1) / AL * AL;
        const int nb = (p.batch > 1 && batch_s != 0) ? p.batch : 1;
        const int nr = (p.reduce > 1 && reduce_s != 0) ? p.reduce : 1;
        const size_t mat = (size_t)outer * inner_pad;
        const size_t elems = (size_t)nb * nr * mat;
        RPB_CUDA(cudaMallocAsync(&tmp[which], elems * ES, stream));     /* released by the caller on every exit */
        long long blocks = (long long)((elems + 255) / 256);
        if (blocks > d->sm_count * 16) blocks = d->sm_count * 16;
        RPB_CUDA(rpb_launch(pack_operand_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, 1, reinterpret_cast<T*>(tmp[which]),
                            reinterpret_cast<const T*>(src), outer, inner, inner_pad, outer_s, inner_s, nb, batch_s, nr, reduce_s));
        g_launches++;
        *out = tmp[which];
        *new_mn_s = keep_mn_major ? 1 : inner_pad;
        *new_k_s = keep_mn_major ? inner_pad : 1;
        *new_reduce_s = nr > 1 ? (long long)mat : 0;
        *new_batch_s = nb > 1 ? (long long)mat * nr : 0;
        return 0;
    };
    int rc = 0;
    if (!pa.ok) rc = pack(0, A, p.m, p.a_row, p.a_col, p.a_batch, p.a_reduce, &A2, &q.a_row, &q.a_col, &q.a_reduce, &q.a_batch);
    if (!rc && !pb.ok) rc = pack(1, B, p.n, p.b_col, p.b_row, p.b_batch, p.b_reduce, &B2, &q.b_col, &q.b_row, &q.b_reduce, &q.b_batch);
    /* an output with an odd leading dimension would fall to per-element stores: write it padded, then unpad */
    void* C2 = C;
    const int n_pad = (p.n + AL - 1) / AL * AL;
    if (!rc && c_odd) {
        if (cudaMallocAsync(&tmp[2], (size_t)p.batch * p.m * n_pad * ES, stream) != cudaSuccess) {
            fprintf(stderr, "recpulse_b200: no memory for the padded output: %s\n", cudaGetErrorString(cudaGetLastError()));
            rc = -1;
        } else {
            C2 = tmp[2];
            q.c_row = n_pad; q.c_batch = (long long)p.m * n_pad;
        }
    }
    if (!rc) rc = launch_umma<T>(q, C2, A2, B2, d, stream);
    if (!rc && c_odd) {
        const long long elems = (long long)p.batch * p.m * p.n;
        long long blocks = (elems + 255) / 256;
        if (blocks > d->sm_count * 16) blocks = d->sm_count * 16;
        if (rpb_launch(unpack_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, 1, reinterpret_cast<T*>(C),
                       reinterpret_cast<const T*>(C2), (long long)p.m, p.n, p.c_row, (long long)n_pad, p.batch, p.c_batch,
                       (long long)p.m * n_pad) != cudaSuccess) {
            fprintf(stderr, "recpulse_b200: unpad launch failed: %s\n", cudaGetErrorString(cudaGetLastError()));
            rc = -1;
        } else {
            g_launches++;
        }
    }
    /* every exit passes here: the temporaries go back to the pool in stream order */
    for (int i = 0; i < 3; ++i) if (tmp[i]) cudaFreeAsync(tmp[i], stream);
    return rc;
}

/* ------------------------------------------------------------------ dispatch */

int validate(const RpbProblem& p, const void* C, const void* A, const void* B) {
    if (!C || !A || !B) { fprintf(stderr, "recpulse_b200: NULL operand\n"); return -1; }
    if (p.m <= 0 || p.n <= 0 || p.k <= 0 || p.batch <= 0 || p.reduce <= 0) {
        fprintf(stderr, "recpulse_b200: non-positive dimension (m=%d k=%d n=%d batch=%d reduce=%d)\n",
                p.m, p.k, p.n, p.batch, p.reduce);
        return -1;
    }
    if (!rpb_dtype_size(p.dtype)) { fprintf(stderr, "recpulse_b200: unknown dtype %d\n", p.dtype); return -1; }
    if (p.c_row < p.n || (p.batch > 1 && p.c_batch == 0)) {
        fprintf(stderr, "recpulse_b200: output rows/batches must not overlap\n");
        return -1;
    }
    return 0;
}

int run_gemm_planned(const RpbProblem& in, void* C, const void* A, const void* B, int device_id, cudaStream_t stream) {
    if (validate(in, C, A, B)) return -1;
    RpbProblem p = in;
    /* a broadcast B with packed A / C batches is one tall GEMM; summed problems whose K ranges are
     * adjacent in memory are one long-K GEMM */
    if (p.batch > 1 && p.b_batch == 0 && p.a_batch == (long long)p.m * p.a_row &&
        p.c_batch == (long long)p.m * p.c_row && (long long)p.m * p.batch <= 0x7fffffffLL) {
        p.m *= p.batch; p.batch = 1;
    }
    if (p.reduce > 1 && p.a_reduce == (long long)p.k * p.a_col && p.b_reduce == (long long)p.k * p.b_row &&
        (long long)p.k * p.reduce <= 0x7fffffffLL) {
        p.k *= p.reduce; p.reduce = 1;
    }
    if (p.batch == 1) p.a_batch = p.b_batch = p.c_batch = 0;
    if (p.reduce == 1) p.a_reduce = p.b_reduce = 0;
    DeviceState* d = nullptr;
    if (device_state(device_id, &d)) return -1;
    const int forced = forced_family();
    const bool half_type = p.dtype == DTYPE_FLOAT16 || p.dtype == DTYPE_BFLOAT16;
    if (p.c_f32) {
        /* unrounded float32 output: a capability of the tcgen05 kernel only */
        if (!half_type || p.bias || p.act || p.c_row != p.n || (p.batch > 1 && p.c_batch != (long long)p.m * p.n)) {
            fprintf(stderr, "recpulse_b200: a float32 output needs float16 / bfloat16 operands, a packed C and no bias "
                            "or epilogue\n");
            return -1;
        }
        int rc = p.dtype == DTYPE_BFLOAT16 ? launch_umma<__nv_bfloat16>(p, C, A, B, d, stream)
                                           : launch_umma<__half>(p, C, A, B, d, stream);
        if (rc == 1) fprintf(stderr, "recpulse_b200: float32 output: the operand layout is not TMA-addressable\n");
        return rc ? -1 : 0;
    }
    if (half_type && forced != RPB_KERNEL_SIMT) {
        /* large problems with an operand or output the TMA engine cannot address are packed / padded first */
        int rc = p.dtype == DTYPE_BFLOAT16 ? launch_umma_packed<__nv_bfloat16>(p, C, A, B, d, stream)
                                           : launch_umma_packed<__half>(p, C, A, B, d, stream);
        if (rc <= 0) return rc;
        rc = p.dtype == DTYPE_BFLOAT16 ? launch_umma<__nv_bfloat16>(p, C, A, B, d, stream)
                                       : launch_umma<__half>(p, C, A, B, d, stream);
        if (rc <= 0) return rc;
        if (forced == RPB_KERNEL_UMMA) {
            fprintf(stderr, "recpulse_b200: tcgen05 path forced but the operand layout is not TMA-addressable\n");
            return -1;
        }
    }
    switch (p.dtype) {
        case DTYPE_FLOAT32: {
            if (forced != RPB_KERNEL_SIMT) {
                /* large outputs: 3xTF32 on tcgen05 (hi/lo split in shared memory); otherwise, and for layouts TMA
                 * cannot address, the mma.sync 3xTF32 kernel with its smaller tiles */
                static int env = -1;
                if (env < 0) { const char* e = getenv("RPB_FP32_UMMA"); env = e ? (atoi(e) ? 2 : 1) : 0; }
                const long long big_tiles = (long long)((p.m + 127) / 128) * ((p.n + 127) / 128) * p.batch;
                /* many output tiles, or few but with enough K to split over the SMs (a skinny dW = X^T.dY) */
                const bool heavy = p.m >= 128 && p.n >= 128 && (double)p.m * p.n * ((double)p.k * p.reduce) >= 1e9;
                if (env != 1 && (env == 2 || forced == RPB_KERNEL_UMMA || big_tiles >= d->sm_count / 2 || heavy)) {
                    int rc = launch_umma_packed<float>(p, C, A, B, d, stream);  /* odd strides: pack / pad once */
                    if (rc <= 0) return rc;
                    rc = launch_umma<float>(p, C, A, B, d, stream);
                    if (rc <= 0) return rc;
                }
                int rc = launch_tf32(p, C, A, B, d, stream);
                if (rc <= 0) return rc;
            }
            return launch_simt<float, float>(p, C, A, B, d, stream);
        }
        case DTYPE_FLOAT64: {
            if (forced != RPB_KERNEL_SIMT) {
                int rc = launch_dmma(p, C, A, B, d, stream);
                if (rc <= 0) return rc;
            }
            return launch_simt<double, double>(p, C, A, B, d, stream);
        }
        case DTYPE_FLOAT16: return launch_simt<__half, float>(p, C, A, B, d, stream);
        case DTYPE_BFLOAT16: return launch_simt<__nv_bfloat16, float>(p, C, A, B, d, stream);
    }
    return -1;
}

template <typename T, typename Acc>
int run_gates(void* y, long long rows, int n, long long ld, DeviceState* d, cudaStream_t s) {
    long long blocks = (rows * n + 255) / 256;
    const long long cap = (long long)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    RPB_CUDA(rpb_launch(rpb_gate::forward_kernel<T, Acc>, dim3((unsigned)blocks), dim3(256), 0, s, 1, reinterpret_cast<T*>(y), rows, n, ld));
    g_launches++;
    return 0;
}
template <typename T, typename Acc>
int run_gates_grad(void* dpre, const void* dy, const void* y, long long rows, int n, long long ld_dpre, long long ld_dy,
                   long long ld_y, DeviceState* d, cudaStream_t s) {
    long long blocks = (rows * n + 255) / 256;
    const long long cap = (long long)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    RPB_CUDA(rpb_launch(rpb_gate::backward_kernel<T, Acc>, dim3((unsigned)blocks), dim3(256), 0, s, 1, reinterpret_cast<T*>(dpre),
                        reinterpret_cast<const T*>(dy), reinterpret_cast<const T*>(y), rows, n, ld_dpre, ld_dy, ld_y));
    g_launches++;
    return 0;
}

/* The GEMM, then — when an epilogue non-linearity was asked for and the plan that ran did not apply it in its own
 * epilogue (only the tcgen05 kernel's register epilogue does; inlined into the mma.sync kernels it slowed the
 * launch-bound MLP / LSTM steps by a sixth) — one element-wise pass over C. */
int run_gemm(const RpbProblem& p, void* C, const void* A, const void* B, int device_id, cudaStream_t stream) {
    if (p.act && (p.act != 1 || p.n % 4 != 0)) {
        fprintf(stderr, "recpulse_b200: epilogue %d needs n to be a multiple of 4 (n=%d)\n", p.act, p.n);
        return -1;
    }
    t_act_fused = false;
    int rc = run_gemm_planned(p, C, A, B, device_id, stream);
    if (rc || !p.act || t_act_fused) return rc;
    DeviceState* d = nullptr;
    if (device_state(device_id, &d)) return -1;
    const size_t es = rpb_dtype_size(p.dtype);
    for (int b = 0; b < p.batch && !rc; ++b) {
        void* cb = reinterpret_cast<char*>(C) + (size_t)b * p.c_batch * es;
        switch (p.dtype) {
            case DTYPE_FLOAT32: rc = run_gates<float, float>(cb, p.m, p.n, p.c_row, d, stream); break;
            case DTYPE_FLOAT64: rc = run_gates<double, double>(cb, p.m, p.n, p.c_row, d, stream); break;
            case DTYPE_FLOAT16: rc = run_gates<__half, float>(cb, p.m, p.n, p.c_row, d, stream); break;
            case DTYPE_BFLOAT16: rc = run_gates<__nv_bfloat16, float>(cb, p.m, p.n, p.c_row, d, stream); break;
            default: rc = -1;
        }
    }
    return rc;
}

template <typename T, typename Acc>
int run_colsum(void* out, const void* in, long long rows, int cols, long long ld, int accumulate, DeviceState* d,
               cudaStream_t stream) {
    const int col_blocks = (cols + rpb_cols::COLS - 1) / rpb_cols::COLS;
    long long slabs = (4LL * d->sm_count + col_blocks - 1) / col_blocks;
    const long long max_slabs = (rows + 31) / 32;
    if (slabs > max_slabs) slabs = max_slabs;
    if (slabs > 4096) slabs = 4096;
    if (slabs < 1) slabs = 1;
    const long long rows_per_block = (rows + slabs - 1) / slabs;
    slabs = (rows + rows_per_block - 1) / rows_per_block;
    void* scratch = nullptr;
    if (get_scratch(d, sizeof(Acc) * (size_t)slabs * cols, stream, &scratch)) return -1;
    RPB_CUDA(rpb_launch(rpb_cols::partial_kernel<T, Acc>, dim3(col_blocks, (unsigned)slabs), dim3(rpb_cols::COLS * rpb_cols::LANES),
                        0, stream, 1, reinterpret_cast<const T*>(in), reinterpret_cast<Acc*>(scratch), rows, cols, ld,
                        rows_per_block));
    RPB_CUDA(rpb_launch(rpb_cols::final_kernel<T, Acc>, dim3((cols + 127) / 128), dim3(128), 0, stream, 1,
                        reinterpret_cast<const Acc*>(scratch), reinterpret_cast<T*>(out), (int)slabs, cols, accumulate));
    g_launches += 2;
    if (release_scratch(d, stream)) return -1;
    RPB_CUDA(cudaGetLastError());
    return 0;
}

/* The unmodified RecPulse extension, when one is loaded in this process (host tensors are its job). */
void* reference_symbol(const char* name) {
    static void* handle = nullptr;
    static bool searched = false;
    if (!searched) {
        searched = true;
        dl_iterate_phdr(
            [](struct dl_phdr_info* info, size_t, void* out) -> int {
                if (info->dlpi_name && strstr(info->dlpi_name, "recpulse_cuda")) {
                    *reinterpret_cast<void**>(out) = dlopen(info->dlpi_name, RTLD_NOLOAD | RTLD_NOW);
                    return 1;
                }
                return 0;
            },
            &handle);
    }
    return handle ? dlsym(handle, name) : nullptr;
}

}  // namespace

extern "C" {

void* rpb_reference_symbol(const char* name) { return reference_symbol(name); }
int rpb_take_status(int device_id);

void rpb_gemm_packed(RpbGemm* g, int m, int k, int n) {
    memset(g, 0, sizeof(*g));
    g->m = m; g->n = n; g->k = k; g->batch = 1; g->reduce = 1;
    g->a_row = k; g->a_col = 1; g->b_row = n; g->b_col = 1; g->c_row = n;
    g->a_batch = (long long)m * k; g->b_batch = (long long)k * n; g->c_batch = (long long)m * n;
}

int rp_matmul_ex(void* C, const void* A, const void* B, const RpbGemm* g, DType dtype, int device_id, void* stream) {
    if (!g) return -1;
    if (device_id < 0) {
        fprintf(stderr, "recpulse_b200: rp_matmul_ex needs a CUDA device (no CPU path in this library)\n");
        return -1;
    }
    RpbProblem p;
    p.m = g->m; p.n = g->n; p.k = g->k; p.batch = g->batch; p.reduce = g->reduce;
    p.a_row = g->a_row; p.a_col = g->a_col; p.a_batch = g->a_batch; p.a_reduce = g->a_reduce;
    p.b_row = g->b_row; p.b_col = g->b_col; p.b_batch = g->b_batch; p.b_reduce = g->b_reduce;
    p.c_row = g->c_row; p.c_batch = g->c_batch; p.accumulate = g->accumulate; p.dtype = (int)dtype;
    p.bias = g->bias; p.max_sms = g->max_sms; p.act = g->epilogue; p.c_f32 = g->c_float32;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    int rc = run_gemm(p, C, A, B, device_id, reinterpret_cast<cudaStream_t>(stream));
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rp_colsum_ex(void* out, const void* in, long long rows, int cols, long long row_stride, DType dtype,
                 int accumulate, int device_id, void* stream) {
    if (!out || !in || rows <= 0 || cols <= 0 || row_stride < cols || device_id < 0) return -1;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    DeviceState* d = nullptr;
    int rc = device_state(device_id, &d);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!rc) {
        switch ((int)dtype) {
            case DTYPE_FLOAT32: rc = run_colsum<float, float>(out, in, rows, cols, row_stride, accumulate, d, s); break;
            case DTYPE_FLOAT64: rc = run_colsum<double, double>(out, in, rows, cols, row_stride, accumulate, d, s); break;
            case DTYPE_FLOAT16: rc = run_colsum<__half, float>(out, in, rows, cols, row_stride, accumulate, d, s); break;
            case DTYPE_BFLOAT16: rc = run_colsum<__nv_bfloat16, float>(out, in, rows, cols, row_stride, accumulate, d, s); break;
            default: rc = -1;
        }
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rp_lstm_gates_ex(void* y, long long rows, int n, long long row_stride, DType dtype, int device_id, void* stream) {
    if (!y || rows <= 0 || n <= 0 || n % 4 != 0 || row_stride < n || device_id < 0) return -1;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    DeviceState* d = nullptr;
    int rc = device_state(device_id, &d);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!rc) {
        switch ((int)dtype) {
            case DTYPE_FLOAT32: rc = run_gates<float, float>(y, rows, n, row_stride, d, s); break;
            case DTYPE_FLOAT64: rc = run_gates<double, double>(y, rows, n, row_stride, d, s); break;
            case DTYPE_FLOAT16: rc = run_gates<__half, float>(y, rows, n, row_stride, d, s); break;
            case DTYPE_BFLOAT16: rc = run_gates<__nv_bfloat16, float>(y, rows, n, row_stride, d, s); break;
            default: rc = -1;
        }
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rp_lstm_gates_grad_ex(void* dpre, const void* dy, const void* y, long long rows, int n, long long dpre_stride,
                          long long dy_stride, long long y_stride, DType dtype, int device_id, void* stream) {
    if (!dpre || !dy || !y || rows <= 0 || n <= 0 || n % 4 != 0 || dpre_stride < n || dy_stride < n || y_stride < n ||
        device_id < 0)
        return -1;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    DeviceState* d = nullptr;
    int rc = device_state(device_id, &d);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!rc) {
        switch ((int)dtype) {
            case DTYPE_FLOAT32: rc = run_gates_grad<float, float>(dpre, dy, y, rows, n, dpre_stride, dy_stride, y_stride, d, s); break;
            case DTYPE_FLOAT64: rc = run_gates_grad<double, double>(dpre, dy, y, rows, n, dpre_stride, dy_stride, y_stride, d, s); break;
            case DTYPE_FLOAT16: rc = run_gates_grad<__half, float>(dpre, dy, y, rows, n, dpre_stride, dy_stride, y_stride, d, s); break;
            case DTYPE_BFLOAT16: rc = run_gates_grad<__nv_bfloat16, float>(dpre, dy, y, rows, n, dpre_stride, dy_stride, y_stride, d, s); break;
            default: rc = -1;
        }
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int matmul_kernel_device(void* C, const void* A, const void* B, int m, int k, int n, DType dtype) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    int dev = 0;
    RPB_CUDA(cudaGetDevice(&dev));
    RpbGemm g;
    rpb_gemm_packed(&g, m, k, n);
    RpbProblem p;
    p.m = m; p.n = n; p.k = k; p.batch = 1; p.reduce = 1;
    p.a_row = g.a_row; p.a_col = 1; p.a_batch = 0; p.a_reduce = 0;
    p.b_row = g.b_row; p.b_col = 1; p.b_batch = 0; p.b_reduce = 0;
    p.c_row = n; p.c_batch = 0; p.accumulate = 0; p.dtype = (int)dtype; p.bias = nullptr; p.max_sms = 0; p.act = 0;
    p.c_f32 = 0;
    if (run_gemm(p, C, A, B, dev, nullptr)) return -1;
    RPB_CUDA(cudaStreamSynchronize(nullptr));
    return rpb_take_status(dev) ? -1 : 0;
}

int rp_matmul(void* C, const void* A, const void* B, int m, int k, int n, DType dtype, int device_id) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    if (device_id == -1) {
        typedef int (*Fn)(void*, const void*, const void*, int, int, int, DType, int);
        Fn ref = reinterpret_cast<Fn>(reference_symbol("rp_matmul"));
        if (ref && ref != &rp_matmul) return ref(C, A, B, m, k, n, dtype, device_id);
        fprintf(stderr, "recpulse_b200: rp_matmul on host memory: this library has no CPU path\n");
        return -1;
    }
    RPB_CUDA(cudaSetDevice(device_id));
    return matmul_kernel_device(C, A, B, m, k, n, dtype);
}

int rp_matmul_host(void* C, const void* A, const void* B, int m, int k, int n, DType dtype, int device_id) {
    const size_t es = rpb_dtype_size((int)dtype);
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0 || !es || device_id < 0) return -1;
    RPB_CUDA(cudaSetDevice(device_id));
    const size_t ab = es * m * k, bb = es * k * n, cb = es * m * n;
    char* buf = nullptr;
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    RPB_CUDA(cudaMalloc(&buf, up(ab) + up(bb) + up(cb)));
    char* dA = buf; char* dB = buf + up(ab); char* dC = dB + up(bb);
    int rc = 0;
    if (cudaMemcpyAsync(dA, A, ab, cudaMemcpyHostToDevice, nullptr) != cudaSuccess ||
        cudaMemcpyAsync(dB, B, bb, cudaMemcpyHostToDevice, nullptr) != cudaSuccess) rc = -1;
    if (!rc) {
        RpbGemm g; rpb_gemm_packed(&g, m, k, n);
        rc = rp_matmul_ex(dC, dA, dB, &g, dtype, device_id, nullptr);
    }
    if (!rc && cudaMemcpyAsync(C, dC, cb, cudaMemcpyDeviceToHost, nullptr) != cudaSuccess) rc = -1;
    if (cudaStreamSynchronize(nullptr) != cudaSuccess) rc = -1;
    if (rpb_take_status(device_id)) rc = -1;
    cudaFree(buf);
    return rc;
}

int rpb_umma_plan(int m, int n, int k, int reduce, int batch, DType dtype, int sms, int* rows_of_b, int* k_slices,
                  int* cta_pair) {
    const size_t es = rpb_dtype_size((int)dtype);
    if (m <= 0 || n <= 0 || k <= 0 || reduce <= 0 || batch <= 0 || sms < 2 || (es != 2 && es != 4)) return -1;
    const int bk = 128 / (int)es;
    const long long k_iters = (long long)((k + bk - 1) / bk) * reduce;
    if (k_iters > 0x7fffffffLL) return -1;
    const TilePlan tp = plan_tiles(m, n, batch, (int)k_iters, sms, es == 4);
    if (rows_of_b) *rows_of_b = tp.bn;
    if (k_slices) *k_slices = tp.splits;
    if (cta_pair) *cta_pair = tp.wide ? 2 : tp.pair;
    return 0;
}
int rpb_last_kernel(void) { return t_last_kernel; }
unsigned long long rpb_launch_count(void) { return g_launches.load(); }
void rpb_force_kernel(int family) { g_force.store(family < 0 ? 0 : family); }
const char* rpb_version(void) { return RPB_VERSION; }

/* Reads and clears the status word of `device_id` WITHOUT synchronising: for entry points that have just
 * synchronised the stream their kernels ran on.  0 = ok (also when the device was never used). */
int rpb_take_status(int device_id) {
    if (device_id < 0 || device_id >= MAX_DEVICES || !g_status_words) return 0;
    volatile int* w = g_status_words + device_id;
    const int v = *w;
    if (v != 0) {
        *w = 0;
        g_dev[device_id].bal_dirty.store(true);
        fprintf(stderr, "recpulse_b200: a bounded wait inside the tcgen05 kernel ran out on device %d (code %d); the "
                        "result is invalid\n", device_id, v);
    }
    return v;
}

int rpb_device_status(int device_id) {
    DeviceState* d = nullptr;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return -1;
    if (prev != device_id && cudaSetDevice(device_id) != cudaSuccess) return -1;
    int v = -1;
    if (device_state(device_id, &d) == 0 && cudaDeviceSynchronize() == cudaSuccess) {
        volatile int* w = d->status;
        v = *w;
        if (v != 0) { *w = 0; d->bal_dirty.store(true); }
    }
    if (prev != device_id) cudaSetDevice(prev);
    return v;
}

void rpb_set_wait_limit_ms(int ms) { g_wait_limit.store(ms > 0 ? (long long)ms * 2000000ll : rpb_umma::WAIT_LIMIT_CYCLES); }

void rpb_count_launches(int n) { g_launches += (unsigned long long)n; }

int rpb_trace_enable(int on) {
    if (on && !g_trace_buffer) {
        void* w = nullptr;
        RPB_CUDA(cudaHostAlloc(&w, sizeof(unsigned long long) * 2 * rpb_umma::TRACE_SLOTS, cudaHostAllocPortable | cudaHostAllocMapped));
        memset(w, 0, sizeof(unsigned long long) * 2 * rpb_umma::TRACE_SLOTS);
        g_trace_buffer = reinterpret_cast<unsigned long long*>(w);
    } else if (!on && g_trace_buffer) {
        cudaDeviceSynchronize();
        cudaFreeHost(g_trace_buffer);
        g_trace_buffer = nullptr;
    }
    return 0;
}

int rpb_trace_read(unsigned long long* out, int count) {
    if (!out || !g_trace_buffer || count <= 0) return -1;
    const int n = count < 2 * rpb_umma::TRACE_SLOTS ? count : 2 * rpb_umma::TRACE_SLOTS;
    memcpy(out, g_trace_buffer, sizeof(unsigned long long) * n);
    memset(g_trace_buffer, 0, sizeof(unsigned long long) * 2 * rpb_umma::TRACE_SLOTS);
    return n;
}

/* Runs the kernels' bounded wait on a barrier that nobody will ever signal, with a short limit: the wait must
 * give up, leave its code in the device's status word and let the kernel return.  One CTA of one warp, no TMA, no
 * tensor memory.  Returns 0 when the kernel ran to completion (the status is then read with rpb_device_status). */
int rpb_selftest_bounded_wait(int device_id, long long limit_cycles) {
    if (limit_cycles <= 0 || limit_cycles > 200000000ll) return -1;       /* at most ~0.1 s */
    DeviceState* d = nullptr;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    int rc = device_state(device_id, &d);
    if (!rc) {
        rpb_umma::wait_selftest_kernel<<<1, 32>>>(d->status, limit_cycles);
        g_launches++;
        if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) rc = -1;
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rpb_scratch_reserve(int device_id, size_t bytes) {
    DeviceState* d = nullptr;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    int rc = device_state(device_id, &d);
    void* p = nullptr;
    if (!rc) rc = get_scratch(d, bytes, nullptr, &p);
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rpb_scratch_reset(int device_id) {
    DeviceState* d = nullptr;
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    int rc = device_state(device_id, &d);
    if (!rc) {
        std::lock_guard<std::mutex> lock(d->mu);
        if (d->scratch && cudaFree(d->scratch) != cudaSuccess) rc = -1;    /* synchronises the device */
        d->scratch = nullptr; d->scratch_bytes = 0; d->scratch_used = false; d->scratch_pinned = false;
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}

int rpb_mem_info(int device_id, size_t* free_bytes, size_t* total_bytes) {
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    size_t f = 0, t = 0;
    cudaError_t e = cudaMemGetInfo(&f, &t);
    if (prev != device_id) cudaSetDevice(prev);
    if (e != cudaSuccess) return -1;
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return 0;
}

}  // extern "C"

/* ====================================================================================
 * rp_matmul_noalloc: the K-split tcgen05 GEMM for callers that must not allocate.
 *
 * Some users of this library cannot let it call cudaMalloc: a training process that has
 * handed (nearly) all device memory to its own pool, so that an allocation made behind
 * its back fails or fragments the pool; and code in a latency-critical section, where
 * cudaMalloc / cudaFree stall the whole device.  The regular K-split path keeps its
 * partial tiles in a cudaMalloc'ed buffer that grows on demand.  This variant keeps them
 * in a fixed array that is part of the loaded library image instead, so nothing is ever
 * allocated -- at the price of a size limit and of RPB_NOALLOC_SCRATCH_BYTES of device
 * memory held by every GPU that loads the library, until the process exits.
 * ==================================================================================== */

#define RPB_NOALLOC_SCRATCH_BYTES (16u << 20)

/* Partial fp32 tiles [splits][m][n] of the call in flight.  In host code this name is only a
 * stand-in for the device object; the address a kernel can use comes from cudaGetSymbolAddress. */
static __device__ __align__(256) unsigned char g_noalloc_scratch[RPB_NOALLOC_SCRATCH_BYTES];
static __device__ int g_noalloc_status;

namespace {

struct NoAllocDevice {
    std::atomic<bool> ready{false};
    float* scratch = nullptr;       /* device address of g_noalloc_scratch on this device */
    int* status = nullptr;          /* device address of g_noalloc_status on this device */
    int sm_count = 0;
    int cc_major = 0;
};
NoAllocDevice g_noalloc_dev[MAX_DEVICES];

/* Once per device, with that device current: resolve the device addresses of the static
 * objects.  No allocation happens here or anywhere below. */
int noalloc_setup(int device_id, NoAllocDevice** out) {
    if (device_id < 0 || device_id >= MAX_DEVICES) {
        fprintf(stderr, "recpulse_b200: invalid device id %d\n", device_id);
        return -1;
    }
    NoAllocDevice& d = g_noalloc_dev[device_id];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!d.ready.load(std::memory_order_relaxed)) {
            void* p = nullptr;
            RPB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            d.scratch = reinterpret_cast<float*>(p);
            RPB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_status));
            d.status = reinterpret_cast<int*>(p);
            RPB_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device_id));
            RPB_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device_id));
            if (!g_encode) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult qres;
                RPB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
                if (!fn || qres != cudaDriverEntryPointSuccess) {
                    fprintf(stderr, "recpulse_b200: cuTensorMapEncodeTiled not available\n");
                    return -1;
                }
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            }
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return 0;
}

template <typename T>
int noalloc_launch(void* C, const void* A, const void* B, int m, int k, int n, int dtype, NoAllocDevice* d,
                   cudaStream_t stream) {
    OperandPlan pa = plan_operand(A, m, k, k, 1, 1, 0, 1, 0);
    OperandPlan pb = plan_operand(B, n, k, 1, n, 1, 0, 1, 0);
    if (!pa.ok || !pb.ok || (reinterpret_cast<uintptr_t>(C) & 15u)) {
        fprintf(stderr, "recpulse_b200: rp_matmul_noalloc needs 16-byte aligned pointers and k, n multiples of 8\n");
        return -1;
    }
    const int BN = n <= 64 ? 64 : (n <= 128 ? 128 : 256);
    rpb_umma::Args a;
    memset(&a, 0, sizeof(a));
    a.m = m; a.n = n; a.k = k; a.batch = 1; a.reduce = 1;
    a.k_blocks = (k + rpb_umma::Elem<T>::BLOCK_K - 1) / rpb_umma::Elem<T>::BLOCK_K;
    a.k_iters = a.k_blocks;
    a.tiles_m = (m + rpb_umma::BLOCK_M - 1) / rpb_umma::BLOCK_M;
    a.tiles_n = (n + BN - 1) / BN;
    const long long tiles = (long long)a.tiles_m * a.tiles_n;
    /* always split K when there is anything to split: this entry point is the scratch-using variant */
    long long splits = d->sm_count / tiles;
    if (splits > a.k_iters) splits = a.k_iters;
    if (splits > 128) splits = 128;
    if (splits < 2) splits = a.k_iters >= 2 ? 2 : 1;
    a.iters_per_split = (int)((a.k_iters + splits - 1) / splits);
    a.splits = (a.k_iters + a.iters_per_split - 1) / a.iters_per_split;
    const unsigned long long need = 4ull * a.splits * m * n;
    if (a.splits > 1 && need > RPB_NOALLOC_SCRATCH_BYTES) {
        fprintf(stderr,
                "recpulse_b200: rp_matmul_noalloc: %d x %d output split %d ways needs %llu bytes of scratch, the "
                "built-in buffer holds %u; use rp_matmul_ex for this size\n", m, n, a.splits, need,
                (unsigned)RPB_NOALLOC_SCRATCH_BYTES);
        return -1;
    }
    a.total_work = tiles * a.splits;
    a.group_n = raster_group(d->sm_count, rpb_umma::BLOCK_M, BN, a.tiles_n);
    a.a_batch_mul = a.a_reduce_mul = a.b_batch_mul = a.b_reduce_mul = 1;
    a.c = C; a.c_row = n; a.c_batch = 0; a.accumulate = 0;
    a.partial = a.splits > 1 ? d->scratch : nullptr;
    const bool bf16 = dtype == DTYPE_BFLOAT16;
    const uint32_t fmt = bf16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((pa.mn_major ? 1u : 0u) << 15) | ((pb.mn_major ? 1u : 0u) << 16) |
              ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(rpb_umma::BLOCK_M >> 4) << 24);
    a.a_desc_base = smem_desc_base(pa.mn_major);
    a.b_desc_base = smem_desc_base(pb.mn_major);
    a.a_kstep = pa.mn_major ? (2 * 1024) >> 4 : 32 >> 4;
    a.b_kstep = pb.mn_major ? (2 * 1024) >> 4 : 32 >> 4;
    a.status = d->status;
    a.wait_limit = wait_limit_cycles();
    a.epi_sleep_ns = 0;

    CUtensorMap ma, mb;
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    if (encode_map(&ma, A, pa, m, k, 1, 1, rpb_umma::BLOCK_M, dt)) return -1;
    if (encode_map(&mb, B, pb, n, k, 1, 1, BN, dt)) return -1;

    /* the array keeps the previous call's contents.  Every partial element that the reduction reads
     * is overwritten by this call's GEMM first, so only the status word has to start at zero. */
    RPB_CUDA(cudaMemsetAsync(d->status, 0, sizeof(int), stream));
    const CUtensorMap mc = ma;          /* register epilogue (tma_store = 0): the third map is not read */
    const CUtensorMap mp = ma;
    a.tail_begin = a.total_work; a.tail_splits = 1; a.tail_iters = a.k_iters;
    const int grid = (int)(a.total_work < d->sm_count ? a.total_work : d->sm_count);
    int rc;
    if (BN == 64) rc = launch_umma_bn<T, 64>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    else if (BN == 128) rc = launch_umma_bn<T, 128>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    else rc = launch_umma_bn<T, 256>(pa.mn_major, pb.mn_major, ma, mb, mc, mp, a, grid, stream);
    if (rc) return -1;
    if (a.splits > 1) {
        const long long elems = (long long)m * n;
        int rb = (int)((elems + 255) / 256); if (rb > d->sm_count * 8) rb = d->sm_count * 8;
        RPB_CUDA(rpb_launch(rpb_simt::splitk_reduce_kernel<T, float>, dim3(rb), dim3(256), 0, stream, 1, (const float*)a.partial,
                            reinterpret_cast<T*>(C), a.splits, 1, m, n, (long long)n, 0ll, 0, (const T*)nullptr));
        g_launches++;
        RPB_CUDA(cudaGetLastError());
    }
    t_last_kernel = a.splits > 1 ? RPB_KERNEL_UMMA_SPLITK : RPB_KERNEL_UMMA;
    return 0;
}

}  // namespace

extern "C" int rp_matmul_noalloc(void* C, const void* A, const void* B, int m, int k, int n, DType dtype,
                                 int device_id, void* stream, int* kernel_status) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    if (dtype != DTYPE_BFLOAT16 && dtype != DTYPE_FLOAT16) {
        fprintf(stderr, "recpulse_b200: rp_matmul_noalloc handles float16 and bfloat16 only\n");
        return -1;
    }
    int prev = -1;
    RPB_CUDA(cudaGetDevice(&prev));
    if (prev != device_id) RPB_CUDA(cudaSetDevice(device_id));
    NoAllocDevice* d = nullptr;
    int rc = noalloc_setup(device_id, &d);
    if (!rc && d->cc_major != 10) {
        fprintf(stderr, "recpulse_b200: rp_matmul_noalloc needs a compute capability 10.x device\n");
        rc = -1;
    }
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (!rc) {
        rc = dtype == DTYPE_BFLOAT16 ? noalloc_launch<__nv_bfloat16>(C, A, B, m, k, n, (int)dtype, d, s)
                                     : noalloc_launch<__half>(C, A, B, m, k, n, (int)dtype, d, s);
    }
    if (!rc && kernel_status) {
        /* optional: wait for the result and hand back the kernel's status word (stack destination,
         * nothing allocated) */
        int v = -1;
        if (cudaMemcpyAsync(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
            cudaStreamSynchronize(s) != cudaSuccess) rc = -1;
        *kernel_status = v;
        if (!rc && v != 0) rc = -1;
    }
    if (prev != device_id) cudaSetDevice(prev);
    return rc;
}
