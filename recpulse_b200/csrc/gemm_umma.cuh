/*
 * tcgen05 GEMM for float16 / bfloat16 and, as 3xTF32, float32 (fp32 accumulation in tensor memory).
 *
 * One persistent CTA per SM (or one cluster of two CTAs per pair of SMs, cta_group::2):
 *   warp 0        TMA producer: 128B-swizzled tiles of A and B into a shared-memory ring
 *   warp 1        owns tensor memory; one lane issues tcgen05.mma (M = 128 or 256, K = 32 bytes per instruction)
 *   warps 2..9    epilogue: tcgen05.ld of the fp32 accumulator, bias, rounding, staging in shared memory
 *                 and TMA stores (or register stores with optional "+= C"); fp32 partial tiles
 *                 when K is split across CTAs.  Two warps share each tensor-memory lane quarter
 *                 and take alternate column chunks.
 *   warps 10..13  float32 only: split each delivered tile into hi and lo TF32 parts in shared memory
 * Two accumulators in tensor memory let the epilogue of tile i overlap the main loop of tile i+1.
 * Large 16-bit problems take a double-width pair tile instead (256 x 512: the two accumulators belong to one
 * tile and share its A operand, a quarter fewer bytes fetched per FLOP); there the second accumulator trails
 * the first by a few K blocks at both ends of a tile and the epilogue hands each accumulator back as soon as
 * it is in registers, which hides the epilogue without a spare buffer.
 *
 * Operands are read where they lie: each one may be K-major (reduction index
 * contiguous) or MN-major (output index contiguous); the TMA descriptor is built from
 * the tensor's own strides and the MMA descriptors carry the matching major bit, so
 * the transposed operands of the backward GEMMs (dC.B^T, A^T.dC) need no copy.
 *
 * Every wait on an mbarrier is bounded.  When a bound runs out the kernel records a
 * code in *status, all roles leave their loops, tensor memory is released and the
 * kernel returns; the host reports the failure (rpb_device_status).
 */
#ifndef RPB_GEMM_UMMA_CUH
#define RPB_GEMM_UMMA_CUH

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rpb_common.h"

namespace rpb_umma {

constexpr int BLOCK_M = 128;
constexpr int EPI_WARPS = 8;           /* two per tensor-memory lane quarter: even / odd column chunks */
constexpr int SPLIT_WARPS = 4;         /* float32 only: warps that take operand tiles apart into hi + lo */

/* Per element type.  One K block is always 128 bytes wide (one swizzle row): 64 halves or 32 floats.
 * float32 runs as 3xTF32: the tile that TMA delivered is split in shared memory into hi (the value with
 * its low 13 mantissa bits cleared, exact in TF32) and lo = x - hi, and each K step issues
 * lo*hi + hi*lo + hi*hi on kind::tf32 (fp32 accumulate).  The dropped lo*lo is below 2^-22 of the product. */
template <typename T> struct Elem {
    static constexpr int BYTES = sizeof(T);
    static constexpr bool SPLIT = BYTES == 4;
    static constexpr int BLOCK_K = 128 / BYTES;          /* elements per K block                       */
    static constexpr int UMMA_K = 32 / BYTES;            /* elements per instruction along K (32 bytes) */
    static constexpr int CHUNK = 128 / BYTES;            /* MN-major operands: elements per 128-byte chunk */
    static constexpr int THREADS = (2 + EPI_WARPS + (SPLIT ? SPLIT_WARPS : 0)) * 32;
};
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;   /* default bound of one wait: about 2 s of SM clock */
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int TRACE_SLOTS = 64;        /* 0 entry, 1 set-up done, 2 first TMA issued, 3 first stage landed, 4 last MMA committed,
                                        * 5 kernel end; 8 + 4 i .. : item i  MMA start / MMA committed / epilogue start / epilogue end
                                        * (items 0..6); double-width tiles also 36 + i: second accumulator complete, 50 + i: the MMA
                                        * warp has the first accumulator back (items 0..13; overlapping the slots of items 7 and up) */

/* NH: accumulators per tile.  2 = the double-width pair tile 256 x 4BN, whose two instruction-wide halves share the
 * A tile: a stage then holds one A tile and two B sub-tiles of BN rows. */
template <int BN, bool SPLIT = false, int NH = 1> struct Config {
    static constexpr int A_BYTES = BLOCK_M * 128;
    static constexpr int B_SUB_BYTES = BN * 128;
    static constexpr int B_BYTES = NH * B_SUB_BYTES;
    static constexpr int LOAD_BYTES = A_BYTES + B_BYTES;                 /* what TMA delivers per stage */
    static constexpr int STAGE_BYTES = SPLIT ? 2 * LOAD_BYTES : LOAD_BYTES;   /* [A | B | A_lo | B_lo]   */
    /* epilogue staging for TMA stores: one buffer of 32 rows x 128 bytes per epilogue warp */
    static constexpr int STORE_BUF_BYTES = 32 * 128;
    static constexpr int STORE_BYTES = EPI_WARPS * STORE_BUF_BYTES;
    static constexpr int STAGES_RAW = (SMEM_LIMIT - 2048 - STORE_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct Args {
    int m, n, k;
    int batch, reduce;
    int k_blocks;          /* ceil(k / elements per K block) */
    int k_iters;           /* reduce * k_blocks */
    int splits;            /* CTAs sharing one output tile along K (1 = none) */
    int iters_per_split;
    int tiles_m, tiles_n;
    int group_n;           /* n-tiles per rasterisation group */
    long long total_work;  /* tiles_m * tiles_n * batch * splits (+ the extra K slices of tail tiles) */
    /* Tail split: when the last wave of tiles would leave most SMs idle, the tiles of that wave (work items
     * >= tail_begin) are cut along K into tail_splits slices of tail_iters K blocks each; the slices go to
     * fp32 tiles in scratch ([tail tile][slice][TILE_M x ACC_N], map_p) and tail_reduce_kernel adds them. */
    long long tail_begin;  /* == number of output tiles when there is no tail split */
    int tail_splits, tail_iters;
    int a_batch_mul, a_reduce_mul, b_batch_mul, b_reduce_mul;   /* 0 when that operand is broadcast */
    void* c;               /* output (T), or nullptr when splits > 1 */
    long long c_row, c_batch;
    int accumulate;
    int tma_store;         /* 1: the epilogue writes through shared memory + TMA store (map_c), 0: register stores */
    float* partial;        /* [splits][batch][m][n] fp32 when splits > 1 */
    const void* bias;      /* n values of T added to every row (by the reduction pass when K is split), or null */
    uint32_t idesc;        /* tcgen05 instruction descriptor */
    uint64_t a_desc_base, b_desc_base;   /* shared-memory descriptors without start address */
    uint32_t a_kstep, b_kstep;           /* descriptor advance per UMMA_K, in 16-byte units */
    int* status;
    int act;               /* 1: LSTM gate non-linearities on the finished sum (register epilogue, no K slices) */
    /* Balanced schedule (bal != 0; needs splits == batch == 1 and at least one tile per CTA or pair): the
     * tiles x K-block units are dealt evenly and contiguously, bal_per units to every CTA (pair) and one more to the
     * first bal_extra of them.  A range starts / ends inside at most one tile each.  Of the two pieces of a cut tile
     * the SHORTER one is computed first thing by its holder and goes as an fp32 tile to the scratch slot of that
     * boundary; the LONGER one is computed last by the neighbour, whose epilogue adds the slot before it writes C.
     * The two are handed over through bal_flags: per slot and CTA rank a `ready` count (the writer's epilogue warps)
     * and a `done` count (the reader's; the last one resets both). */
    /* tail_fuse != 0 (tail_splits == 2): the two K slices of a tail tile run side by side in the last wave; per
     * epilogue warp, whichever slice reaches its epilogue first leaves its fp32 sums in bal_scratch (slot = tail tile)
     * and the other adds them and writes C -- a + b in either order, so the result does not depend on who was first.
     * bal_flags holds [tail tile][rank][warp][ticket, ready]; the finishing warp clears both. */
    int tail_fuse;
    /* Diagnostics: when not null, CTA 0 and the last CTA stamp %globaltimer (ns) at the kernel's milestones into
     * trace[cta == 0 ? 0 : 1][TRACE_SLOTS] (see trace_mark): where a launch's fixed cost goes. */
    unsigned long long* trace;
    int bal;
    long long bal_per;
    int bal_extra;
    float* bal_scratch;         /* fp32 partial tiles, one per boundary between neighbours: [slot][CTA rank][lane
                                 * quarter][32-column chunk][8][32 lanes] float4, so that a warp's accesses are contiguous */
    int* bal_flags;             /* [slots][2 ranks][ready, done] */
    long long wait_limit;  /* bound of every mbarrier wait, in SM clock cycles */
    uint32_t epi_sleep_ns; /* back-off between polls of the epilogue warps' wait for a finished accumulator (0 = spin) */
    int epi_pipe;          /* 1: the 16-bit TMA-store epilogue runs software-pipelined (RPB_EPI_PIPE=0 for the plain loop) */
    /* Rendezvous of the units (sync_ctr != null; round-robin order, the whole tiles of the first sync_items work items):
     * before a CTA's (pair's) producers load their nth tile, and every sync_every K blocks inside it, every unit whose
     * nth item takes part must have got there -- the leader's producer counts itself in at sync_ctr[0], both producers
     * poll it until it reaches the number of arrivals due by then.  Units that share an operand panel then ask L2 for the
     * same lines at nearly the same time, which the L2 request coalescer turns into one lookup.  sync_ctr[1] is the
     * launch's `off` word: a unit that has waited sync_patience clocks sets it and nobody waits any more.  The host zeroes
     * both words in stream order before the launch. */
    int* sync_ctr;
    long long sync_items;
    long long sync_patience;
    int sync_every;        /* also every so many K blocks inside a tile (0: at tile starts only) */
    unsigned sync_sleep;   /* ns between polls of the counter */
    /* Placement-aware tile order (pairs on a full grid).  smid_out != null: the leader of unit u stores the SM it runs on
     * in smid_out[u] (mapped host memory; the host learns where the hardware puts the clusters).  wave_slot_on:
     * in every full wave of whole tiles unit u computes tile wave * units + wave_slot[u] instead of wave * units + u; the
     * host builds that permutation so that the units of one GPC -- which share an L2 request coalescer -- take a 3 x 3
     * block of the wave's tiles and ask for the same three A panels and three B panels. */
    int* smid_out;
    int wave_slot_on;
    unsigned char wave_slot[80];
    int wide_skew;         /* double-width tiles: K blocks by which the second accumulator trails the first at a tile's ends */
    int c_f32;             /* 1: the output is packed float32 [batch][m][n] (unrounded sums of 16-bit operands); the
                            * epilogue then writes it like a K slice: `partial` = the output when splits == 1 */
};

/* ------------------------------------------------------------------ PTX wrappers */

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
/* Bounded wait: gives up after `limit` cycles of the SM clock (Args.wait_limit; about 2 s by default).
 * false = gave up (or another role already did): the caller leaves its main loop and the kernel tears down. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, long long limit, uint32_t sleep_ns = 0) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        /* long waits (an epilogue warp waits a whole tile time for its accumulator) may back off between polls
         * instead of keeping 32 lanes on the barrier: fewer issue slots and less power for the same result */
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((i & 255u) == 255u || (sleep_ns && (i & 7u) == 7u)) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) break;
        }
    }
    *abort_flag = 1;
    /* the status word may live in mapped host memory (read by the host without a copy), where device atomics are
     * not defined: a plain store of the first code seen is enough, any non-zero value means "result invalid" */
    volatile int* st = status;
    if (*st == 0) *st = code;
    __threadfence_system();
    return false;
}
/* One lane of a converged warp.  The producer and MMA warps run their loops with all 32 lanes and elect the
 * issuing lane per iteration: loop counters, shared-memory addresses and descriptors then stay warp-uniform,
 * which lets the compiler keep them in uniform registers, where TMA and tcgen05.mma take their operands.  (With
 * the whole loop under "lane == 0" every issue paid for moving its operands there: ~100 clocks per
 * tcgen05.mma, measured, which capped every tile shape at ~420 clocks per K block.) */
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
/* all lanes of a converged warp wait; the outcome is uniform */
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int* status, int code, long long limit) {
    const bool ok = mbar_wait(bar, parity, abort_flag, status, code, limit);
    return __all_sync(0xffffffffu, ok);
}
/* PAIR: the copy may signal an mbarrier in the other CTA of the pair (cta_group::2); never multicast */
template <bool PAIR>
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
    if (PAIR) {
        asm volatile(
            "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    } else {
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5, %6}], [%2];"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
    }
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
/* at most `N` of this thread's bulk store groups may still be reading shared memory */
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
/* shared::cluster address of `addr` (a shared::cta address) in CTA `rank` of this cluster */
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
/* Descriptors travel as two 32-bit words: the low word (start address and leading-dimension offset) changes
 * per stage and per instruction, the high word never does, so the loop only does 32-bit adds. */
template <bool PAIR>
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
    if (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    }
}
template <bool PAIR>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                         uint32_t idesc, uint32_t accumulate) {
    if (PAIR) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "setp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    }
}
/* The mbarrier receives one arrival once every tcgen05.mma issued so far by this thread has
 * completed; for a pair the arrival is delivered to the same barrier in both CTAs. */
template <bool PAIR>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if (PAIR) {
        const uint16_t mask = 3;
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"(mask) : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(bar) : "memory");
    }
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_load_32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);          /* .x = lo in the low half */
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

/* v[j] += bias[col + j] for the 32 columns a thread holds; columns >= n are left alone */
template <typename T>
__device__ __forceinline__ void add_bias_32(uint32_t (&v)[32], const T* bias, int col, int n) {
    const T* bp = bias + col;
    constexpr int PER = 16 / (int)sizeof(T);             /* elements per 16-byte load */
    if (col + 32 <= n && (reinterpret_cast<uintptr_t>(bp) & 15u) == 0) {
#pragma unroll
        for (int q = 0; q < 32 / PER; ++q) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(bp) + q);
            const T* b8 = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int e = 0; e < PER; ++e) v[PER * q + e] = __float_as_uint(__uint_as_float(v[PER * q + e]) + to_f32<T>(b8[e]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < n) v[j] = __float_as_uint(__uint_as_float(v[j]) + to_f32<T>(bp[j]));
    }
}

/* Tile index -> (m-tile, n-tile): tiles are walked in column groups of `group_n` n-tiles, n fastest. */
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_n, int& mt, int& nt) {
    const int per_group = group_n * tiles_m;
    const int g = t / per_group;
    const int r = t - g * per_group;
    const int gn = min(group_n, tiles_n - g * group_n);
    mt = r / gn;
    nt = g * group_n + (r - mt * gn);
}

__device__ __forceinline__ void trace_mark(unsigned long long* trace, int slot) {
    if (trace && slot < TRACE_SLOTS && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        trace[(blockIdx.x == 0 ? 0 : TRACE_SLOTS) + slot] = t;
    }
}

/* ------------------------------------------------------------------ kernel */

/* PAIR = false: one CTA per output tile of 128 x BN  (tcgen05 cta_group::1).
 * PAIR = true : a cluster of two CTAs per output tile of 256 x 2BN (cta_group::2).  CTA r of the
 *               pair loads rows [128r, 128r+128) of the A tile and columns [BN r, BN r + BN) of the
 *               B tile, the leader CTA (rank 0) issues M=256, N=2BN instructions that read both
 *               CTAs' shared memory, and each CTA's tensor memory receives its own 128 rows of the
 *               accumulator.  Each operand byte is fetched from L2 by one SM only (no multicast), so
 *               L2 traffic per FLOP drops by a third against PAIR = false at the same MMA shape per SM. */
/* NH = 2 (pairs of 16-bit types only): the tile is two instructions wide, 256 x 4BN.  Every K block is multiplied into
 *               two accumulators that share the A tile, which takes another quarter off the bytes fetched per
 *               FLOP (and off the power they cost).  The two accumulators fill tensor memory, so there is no second
 *               buffer: instead the second accumulator runs SKEW K blocks behind the first at both ends of a
 *               tile, so that the epilogue drains the first one while the second is still being multiplied, and the
 *               next tile starts on the first accumulator while the second one is being drained. */
template <typename T, int BN, bool A_MN, bool B_MN, bool PAIR, int NH = 1>
__global__ void __launch_bounds__(Elem<T>::THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_p, const Args args)
{
    using E = Elem<T>;
    constexpr bool SPLIT = E::SPLIT;
    constexpr int BLOCK_K = E::BLOCK_K, UMMA_K = E::UMMA_K, CHUNK = E::CHUNK;
    using Cfg = Config<BN, SPLIT, NH>;
    static_assert(NH == 1 || (NH == 2 && PAIR && !SPLIT && BN == 128), "double-width tiles: 16-bit pairs of 256 x 512");
    constexpr int ACC_N = PAIR ? 2 * BN : BN;              /* accumulator columns = instruction N */
    constexpr int TILE_N = NH * ACC_N;                     /* columns of C per tile */
    constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;
    constexpr uint32_t TMEM_COLS = 2 * ACC_N;              /* NH = 1: two buffers; NH = 2: the tile's two accumulators */
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32, "tensor memory columns");
    extern __shared__ uint8_t smem_raw[];
    /* the swizzle pattern and the descriptors' base_offset = 0 need 1024-byte aligned tiles */
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t store_base = smem_base + Cfg::STAGES * Cfg::STAGE_BYTES;       /* 1024-aligned */
    const uint32_t bar_base = store_base + Cfg::STORE_BYTES;
    /* barrier words: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], ready[STAGES], then tmem ptr, abort flag */
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
    auto tfull_bar = [&](int i) { return bar_base + 8u * (2 * Cfg::STAGES + i); };
    auto tempty_bar = [&](int i) { return bar_base + 8u * (2 * Cfg::STAGES + 2 + i); };
    auto ready_bar = [&](int s) { return bar_base + 8u * (2 * Cfg::STAGES + 4 + s); };   /* float32: tile split into hi / lo */
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::STORE_BYTES +
                                                      8 * (3 * Cfg::STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) trace_mark(args.trace, 0);
    uint32_t cta_rank = 0;
    if (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1);
            if (SPLIT) mbar_init(ready_bar(s), (PAIR ? 2 : 1) * SPLIT_WARPS);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(tfull_bar(i), 1); mbar_init(tempty_bar(i), (PAIR ? 2 : 1) * EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        if (args.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
        if (args.tail_splits > 1 || args.bal) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                         ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) { __syncwarp(); cluster_sync(); }   /* the peer's barriers are initialised before anyone signals them */
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) trace_mark(args.trace, 1);
    rpb_pdl_trigger();          /* the next kernel in the stream may begin its own set-up */
    rpb_pdl_wait();             /* everything below touches memory the previous kernel may still be writing */

    /* one work item per CTA (PAIR = false) or per cluster (PAIR = true) */
    const long long work_begin = PAIR ? blockIdx.x / 2 : blockIdx.x;
    const long long work_step = PAIR ? gridDim.x / 2 : gridDim.x;

    /* Work items are dealt round-robin, so the items in flight are consecutive indices.  Within one
     * (batch, split) the output tiles are walked in column groups of `group_n` n-tiles, n fastest:
     * the tiles in flight then cover a near-square block of C and share their A row panels and B
     * column panels in L2 instead of streaming all of A once per wave.
     * kind 0: a whole tile (or K slice when splits > 1); kind 1: a piece whose fp32 partial goes to scratch slot
     * `slot` through map_p (a K slice of a tail tile, or the head piece of the balanced schedule); kind 2: the tail
     * piece of the balanced schedule, finished with the partial in `slot`. */
    struct Item { int mt, nt, split, bz, it0, it1, kind, slot; };
    const long long unit_id = PAIR ? blockIdx.x / 2 : blockIdx.x;     /* this CTA's (pair's) index */
    if (args.smid_out && leader && threadIdx.x == 0) {
        uint32_t sm;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
        args.smid_out[unit_id] = (int)sm;
    }
    const uint32_t my_slot = args.wave_slot_on ? (uint32_t)args.wave_slot[unit_id] : (uint32_t)unit_id;
    auto next_item = [&](long long& w, int& phase, Item& o) -> bool {
        if (args.bal) {
            /* This CTA's (pair's) range [s, e) of tile x K-block units starts inside tile ta (at K block ka) and ends
             * inside tile tb (at kb).  A cut tile is FINISHED by whoever holds its longer piece, as that one's last
             * work; the shorter piece is computed first thing by its holder and travels as fp32 through slot =
             * index of the boundary between the two neighbours.  Order: partial pieces, whole tiles, finishing pieces. */
            const long long s = unit_id * args.bal_per + min(unit_id, (long long)args.bal_extra);
            const long long e = s + args.bal_per + (unit_id < args.bal_extra ? 1 : 0);
            const long long ta = s / args.k_iters, tb = e / args.k_iters;
            const int ka = (int)(s - ta * args.k_iters), kb = (int)(e - tb * args.k_iters);
            const bool tail_fin = ka != 0 && 2 * ka <= args.k_iters;        /* my piece [ka, K) is the longer one */
            const bool head_fin = kb != 0 && 2 * kb > args.k_iters;         /* my piece [0, kb) is the longer one */
            o.split = 0; o.bz = 0;
            for (;;) {
                const int ph = phase++;
                if (ph == 0) { w = ta + (ka ? 1 : 0); }
                if ((ph == 0 && ka && !tail_fin) || (ph == 3 && ka && tail_fin)) {          /* piece [ka, K) of tile ta */
                    tile_coords((int)ta, args.tiles_m, args.tiles_n, args.group_n, o.mt, o.nt);
                    o.it0 = ka; o.it1 = args.k_iters; o.kind = ph == 0 ? 1 : 2; o.slot = (int)unit_id - 1;
                    return true;
                }
                if ((ph == 1 && kb && !head_fin) || (ph == 4 && kb && head_fin)) {          /* piece [0, kb) of tile tb */
                    tile_coords((int)tb, args.tiles_m, args.tiles_n, args.group_n, o.mt, o.nt);
                    o.it0 = 0; o.it1 = kb; o.kind = ph == 1 ? 1 : 2; o.slot = (int)unit_id;
                    return true;
                }
                if (ph == 2) {
                    if (w < tb) {
                        tile_coords((int)w, args.tiles_m, args.tiles_n, args.group_n, o.mt, o.nt);
                        o.it0 = 0; o.it1 = args.k_iters; o.kind = 0; o.slot = 0;
                        ++w;
                        phase = 2;                       /* stay in this phase until the whole tiles are done */
                        return true;
                    }
                }
                if (ph >= 5) return false;
            }
        }
        if (w >= args.total_work) return false;
        /* 32-bit arithmetic: the host keeps tiles x slices below 2^31, and 64-bit divisions cost hundreds of clocks
         * in code that sits between one tile's last MMA and the next tile's first */
        const uint32_t wi = (uint32_t)w, tb32 = (uint32_t)args.tail_begin;
        if (wi >= tb32) {                           /* K slice of a tail tile (only with splits == batch == 1) */
            const uint32_t j = wi - tb32;
            const uint32_t tile = j / (uint32_t)args.tail_splits;
            o.split = (int)(j - tile * (uint32_t)args.tail_splits);
            o.bz = 0;
            tile_coords((int)(tb32 + tile), args.tiles_m, args.tiles_n, args.group_n, o.mt, o.nt);
            o.it0 = o.split * args.tail_iters;
            o.it1 = min(o.it0 + args.tail_iters, args.k_iters);
            o.kind = 1; o.slot = (int)j;
        } else {
            const uint32_t tiles_mn = (uint32_t)(args.tiles_m * args.tiles_n);
            uint32_t q = wi / tiles_mn;
            int t = (int)(wi - q * tiles_mn);
            if (args.wave_slot_on) {                    /* splits == batch == 1: wi is the tile, wi % units this unit */
                const uint32_t units = (uint32_t)work_step, wave = wi / units;
                if ((wave + 1u) * units <= tb32) t = (int)(wave * units + my_slot);
            }
            const uint32_t bz = q / (uint32_t)args.splits;
            o.split = (int)(q - bz * (uint32_t)args.splits);
            o.bz = (int)bz;
            tile_coords(t, args.tiles_m, args.tiles_n, args.group_n, o.mt, o.nt);
            o.it0 = o.split * args.iters_per_split;
            o.it1 = min(o.it0 + args.iters_per_split, args.k_iters);
            o.kind = 0; o.slot = 0;
        }
        w += work_step;
        return true;
    };

    if (warp == 0) {
        {
            /* The loop below is one warp's serial code and bounds the K-block rate of narrow tiles, so it carries
             * running values (stage addresses, K coordinates) instead of recomputing them per block. */
            constexpr bool REMOTE_BAR = PAIR && !SPLIT;
            int stage = 0; uint32_t parity = 1u;                      /* empty barriers: first pass falls through */
            uint32_t sa = smem_base, eb = empty_bar(0), fb = full_bar(0);
            bool alive = true, traced = false;
            long long w = work_begin; int phase_w = 0; Item item;
            /* rendezvous of all units that are at the same point of their nth whole tile (Args.sync_ctr).  Soft: a unit
             * that has waited `sync_patience` clocks sets the launch's `off` word and from then on nobody waits -- so CTAs
             * that are not resident (another kernel holds their SMs) cost one patience, not a hang or an error. */
            long long tile_no = 0; int sync_target = 0;
            bool sync_on = args.sync_ctr != nullptr;
            auto rendezvous = [&]() {
                long long part = args.sync_items - tile_no * work_step;                  /* units whose nth item takes part */
                part = part < 0 ? 0 : (part < work_step ? part : work_step);
                sync_target += (int)part;
                int off = 0;
                if (lane == 0) {
                    if (leader) atomicAdd(args.sync_ctr, 1);
                    const volatile int* c = args.sync_ctr;
                    const long long t0 = clock64();
                    if (args.sync_sleep) {
                        for (uint32_t i = 0; c[0] < sync_target; ++i) {
                            if (c[1]) break;
                            __nanosleep(args.sync_sleep);
                            if ((i & 15u) == 15u && clock64() - t0 > args.sync_patience) { atomicExch(args.sync_ctr + 1, 1); break; }
                        }
                    } else {
                        /* Four polls in flight, issued a quarter of an L2 round trip apart and each re-issued when it
                         * returns: the counter is sampled every ~150 ns instead of once per round trip, so the units leave
                         * the rendezvous closer together. */
                        int v0 = c[0]; __nanosleep(120);
                        int v1 = c[0]; __nanosleep(120);
                        int v2 = c[0]; __nanosleep(120);
                        int v3 = c[0];
                        for (uint32_t i = 0;; ++i) {
                            if (v0 >= sync_target) break;
                            v0 = c[0];
                            if (v1 >= sync_target) break;
                            v1 = c[0];
                            if (v2 >= sync_target) break;
                            v2 = c[0];
                            if (v3 >= sync_target) break;
                            v3 = c[0];
                            if ((i & 3u) == 3u && (c[1] || clock64() - t0 > args.sync_patience)) {
                                if (!c[1]) atomicExch(args.sync_ctr + 1, 1);
                                break;
                            }
                        }
                    }
                    off = c[1];
                }
                if (__shfl_sync(0xffffffffu, off, 0)) sync_on = false;
            };
            while (alive && next_item(w, phase_w, item)) {
                const int mt = item.mt, nt = item.nt, bz = item.bz, it0 = item.it0, it1 = item.it1;
                int since_sync = 0;
                /* whole tiles of the full waves take part (not the K slices of a cut last wave) */
                const bool sync_item = sync_on && tile_no * work_step + unit_id < args.sync_items;
                if (sync_item) rendezvous();
                const int row0 = mt * TILE_M + (int)cta_rank * BLOCK_M;     /* this CTA's rows of A */
                const int col0 = nt * TILE_N + (int)cta_rank * BN;          /* this CTA's columns of B (first accumulator) */
                const int r0 = it0 / args.k_blocks;
                int kb = it0 - r0 * args.k_blocks, k0 = kb * BLOCK_K;
                int a_r = r0 * args.a_reduce_mul, b_r = r0 * args.b_reduce_mul;
                const int a_b = bz * args.a_batch_mul, b_b = bz * args.b_batch_mul;
                for (int left = it1 - it0; left > 0; --left) {
                    if (sync_item && sync_on && args.sync_every > 0 && ++since_sync > args.sync_every) {
                        since_sync = 1;
                        rendezvous();
                    }
                    if (!mbar_wait_warp(eb, parity, abort_flag, args.status, 1, args.wait_limit)) { alive = false; break; }
                    if (args.trace && !traced && lane == 0) { trace_mark(args.trace, 2); }
                    traced = true;
                    if (elect_one()) {
                        const uint32_t sb = sa + Cfg::A_BYTES;
                        uint32_t tb = fb;
                        if (REMOTE_BAR) {
                            /* both CTAs of a pair report their bytes to the leader's barrier */
                            if (leader) mbar_expect_tx(fb, 2 * Cfg::LOAD_BYTES);
                            tb = cluster_addr(fb, 0);
                        } else {
                            /* float32 pairs: each CTA first splits its own tiles, so its loads report locally */
                            mbar_expect_tx(fb, Cfg::LOAD_BYTES);
                        }
                        if (!A_MN) {
                            tma_load_4d<REMOTE_BAR>(sa, &map_a, tb, k0, row0, a_r, a_b);
                        } else {
#pragma unroll
                            for (int c = 0; c < BLOCK_M / CHUNK; ++c)
                                tma_load_4d<REMOTE_BAR>(sa + c * (BLOCK_K * 128), &map_a, tb, row0 + c * CHUNK, k0, a_r, a_b);
                        }
#pragma unroll
                        for (int h = 0; h < NH; ++h) {
                            const uint32_t sbh = sb + h * Cfg::B_SUB_BYTES;
                            const int colh = col0 + h * ACC_N;
                            if (!B_MN) {
                                tma_load_4d<REMOTE_BAR>(sbh, &map_b, tb, k0, colh, b_r, b_b);
                            } else {
#pragma unroll
                                for (int c = 0; c < BN / CHUNK; ++c)
                                    tma_load_4d<REMOTE_BAR>(sbh + c * (BLOCK_K * 128), &map_b, tb, colh + c * CHUNK, k0, b_r, b_b);
                            }
                        }
                    }
                    __syncwarp();
                    k0 += BLOCK_K;
                    if (++kb == args.k_blocks) { kb = 0; k0 = 0; a_r += args.a_reduce_mul; b_r += args.b_reduce_mul; }
                    sa += Cfg::STAGE_BYTES; eb += 8u; fb += 8u;
                    if (++stage == Cfg::STAGES) { stage = 0; parity ^= 1u; sa = smem_base; eb = empty_bar(0); fb = full_bar(0); }
                }
                ++tile_no;
            }
        }
    } else if (warp == 1) {
        if (leader) {
            int stage = 0; uint32_t phase = 0;
            uint32_t local_tile = 0;
            /* descriptor words: the start address (16-byte units, 14 bits) sits in the low word, whose other bits and
             * the high word are fixed per operand; shared memory ends below 2^18 bytes, so adding stage and K offsets
             * to the low word never carries out of the address field */
            const uint32_t a_hi = (uint32_t)(args.a_desc_base >> 32), b_hi = (uint32_t)(args.b_desc_base >> 32);
            const uint32_t a_lo0 = (uint32_t)args.a_desc_base + (smem_base >> 4);
            const uint32_t b_lo0 = (uint32_t)args.b_desc_base + ((smem_base + Cfg::A_BYTES) >> 4);
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            uint32_t wb = SPLIT ? ready_bar(0) : full_bar(0), eb = empty_bar(0);
            const uint32_t a_kstep = args.a_kstep, b_kstep = args.b_kstep, idesc = args.idesc;
            bool alive = true;
            long long w = work_begin; int phase_w = 0; Item item;
            for (; alive && next_item(w, phase_w, item); ++local_tile) {
                const int it0 = item.it0, it1 = item.it1;
                if constexpr (NH == 2) {
                    /* Two accumulators per tile (tensor-memory columns [0, ACC_N) and [ACC_N, 2 ACC_N)), one A tile and two
                     * B sub-tiles per stage.  The second accumulator runs `head` K blocks behind the first at the start of a
                     * tile and `tail` blocks behind at its end (the stages concerned stay in shared memory meanwhile), so the
                     * first accumulator is handed to the epilogue early and taken back early.  In between, every stage is
                     * multiplied into both accumulators and freed. */
                    static_assert(NH == 1 || Cfg::STAGES >= 4, "the lead of the first accumulator holds up to three stages");
                    const int SKEW = args.wide_skew;
                    constexpr uint32_t BH = (uint32_t)(Cfg::B_SUB_BYTES >> 4);
                    const uint32_t acc_phase = local_tile & 1u;
                    const int iters = it1 - it0;
                    const int head = iters < SKEW ? iters : SKEW;
                    const int tail = iters >= 2 * SKEW ? SKEW : 0;
                    uint32_t acc[2] = {0u, 0u};
                    /* `count` K blocks from the ring position: multiply into the accumulators of `hmask`, after waiting
                     * for the data (wait) and/or freeing the stage afterwards (free_stage) */
                    auto run = [&](int count, int hmask, bool wait, bool free_stage) -> bool {
                        for (int j = 0; j < count; ++j) {
                            if (wait && !mbar_wait_warp(wb, phase, abort_flag, args.status, 3, args.wait_limit)) return false;
                            tc_fence_after();
                            if (elect_one()) {
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    if (!(hmask & (1 << h))) continue;
                                    uint32_t ac = acc[h];
#pragma unroll
                                    for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
                                        umma_f16<PAIR>(tmem_base + h * ACC_N, a_lo + kk * a_kstep, a_hi, b_lo + h * BH + kk * b_kstep, b_hi,
                                                       idesc, ac);
                                        ac = 1u;
                                    }
                                }
                                if (free_stage) umma_commit<PAIR>(eb);
                            }
                            __syncwarp();
                            if (hmask & 1) acc[0] = 1u;
                            if (hmask & 2) acc[1] = 1u;
                            a_lo += Cfg::STAGE_BYTES >> 4; b_lo += Cfg::STAGE_BYTES >> 4; wb += 8u; eb += 8u;
                            if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0; wb = full_bar(0); eb = empty_bar(0); }
                        }
                        return true;
                    };
                    if (args.trace && lane == 0) trace_mark(args.trace, 8 + 4 * (int)local_tile);
                    bool ok = mbar_wait_warp(tempty_bar(0), acc_phase ^ 1u, abort_flag, args.status, 2, args.wait_limit);
                    if (args.trace && lane == 0 && local_tile < 6) trace_mark(args.trace, 50 + (int)local_tile);   /* first accumulator taken back */
                    int s_stage = stage; uint32_t s_phase = phase, s_a = a_lo, s_b = b_lo, s_wb = wb, s_eb = eb;
                    ok = ok && run(head, 1, true, false);
                    ok = ok && mbar_wait_warp(tempty_bar(1), acc_phase ^ 1u, abort_flag, args.status, 2, args.wait_limit);
                    if (ok) {
                        stage = s_stage; phase = s_phase; a_lo = s_a; b_lo = s_b; wb = s_wb; eb = s_eb;
                        run(head, 2, false, true);
                        if (args.trace && lane == 0 && local_tile == 0) trace_mark(args.trace, 3);
                        ok = run(iters - head - tail, 3, true, true);
                    }
                    if (ok && tail) {
                        s_stage = stage; s_phase = phase; s_a = a_lo; s_b = b_lo; s_wb = wb; s_eb = eb;
                        ok = run(tail, 1, true, false);
                        if (ok) {
                            if (elect_one()) umma_commit<PAIR>(tfull_bar(0));       /* first accumulator complete */
                            __syncwarp();
                            stage = s_stage; phase = s_phase; a_lo = s_a; b_lo = s_b; wb = s_wb; eb = s_eb;
                            run(tail, 2, false, true);
                            if (elect_one()) umma_commit<PAIR>(tfull_bar(1));
                            __syncwarp();
                        }
                    } else if (ok) {
                        if (elect_one()) { umma_commit<PAIR>(tfull_bar(0)); umma_commit<PAIR>(tfull_bar(1)); }
                        __syncwarp();
                    }
                    if (!ok) { alive = false; break; }
                    if (args.trace && lane == 0) { trace_mark(args.trace, 9 + 4 * (int)local_tile); trace_mark(args.trace, 4); }
                    continue;
                }
                const uint32_t ab = local_tile & 1u;
                const uint32_t acc_phase = (local_tile >> 1) & 1u;
                if (!mbar_wait_warp(tempty_bar(ab), acc_phase ^ 1u, abort_flag, args.status, 2, args.wait_limit)) { alive = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * ACC_N;
                uint32_t acc = 0u;                                  /* the first instruction of a tile overwrites */
                if (args.trace && lane == 0) trace_mark(args.trace, 8 + 4 * (int)local_tile);
                for (int left = it1 - it0; left > 0; --left) {
                    /* float32: the stage is usable once the split warps (of both CTAs of a pair) are done with it */
                    if (!mbar_wait_warp(wb, phase, abort_flag, args.status, 3, args.wait_limit)) { alive = false; break; }
                    if (args.trace && lane == 0 && local_tile == 0 && left == it1 - it0) trace_mark(args.trace, 3);
                    tc_fence_after();
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
                            const uint32_t ak = a_lo + kk * a_kstep, bk = b_lo + kk * b_kstep;
                            if (SPLIT) {
                                constexpr uint32_t LO = (uint32_t)(Cfg::LOAD_BYTES >> 4);  /* lo tiles sit LOAD_BYTES further */
                                umma_tf32<PAIR>(d_tmem, ak + LO, a_hi, bk, b_hi, idesc, acc);   /* small terms first */
                                umma_tf32<PAIR>(d_tmem, ak, a_hi, bk + LO, b_hi, idesc, 1u);
                                umma_tf32<PAIR>(d_tmem, ak, a_hi, bk, b_hi, idesc, 1u);
                            } else {
                                umma_f16<PAIR>(d_tmem, ak, a_hi, bk, b_hi, idesc, acc);
                            }
                            acc = 1u;
                        }
                        umma_commit<PAIR>(eb);                      /* frees the stage (in both CTAs of a pair) */
                    }
                    __syncwarp();
                    acc = 1u;
                    a_lo += Cfg::STAGE_BYTES >> 4; b_lo += Cfg::STAGE_BYTES >> 4; wb += 8u; eb += 8u;
                    if (++stage == Cfg::STAGES) {
                        stage = 0; phase ^= 1u; a_lo = a_lo0; b_lo = b_lo0;
                        wb = SPLIT ? ready_bar(0) : full_bar(0); eb = empty_bar(0);
                    }
                }
                if (alive && elect_one()) umma_commit<PAIR>(tfull_bar(ab));  /* accumulator complete */
                __syncwarp();
                if (args.trace && lane == 0) { trace_mark(args.trace, 9 + 4 * (int)local_tile); trace_mark(args.trace, 4); }
            }
        }
    } else if (SPLIT && warp >= 2 + EPI_WARPS) {
        /* float32 only: take the stage's A and B tiles apart into hi (in place) and lo (a second copy of
         * the tile, LOAD_BYTES further).  Element-wise on the swizzled bytes, so the layout is untouched. */
        const int st = (int)threadIdx.x - (2 + EPI_WARPS) * 32;
        int stage = 0; uint32_t phase = 0;
        bool alive = true;
        long long w = work_begin; int phase_w = 0; Item item;
        while (alive && next_item(w, phase_w, item)) {
            const int it0 = item.it0, it1 = item.it1;
            for (int it = it0; it < it1; ++it) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 5, args.wait_limit)) { alive = false; break; }
                const uint32_t base = smem_base + stage * Cfg::STAGE_BYTES;
#pragma unroll 4
                for (int i = st; i < Cfg::LOAD_BYTES / 16; i += SPLIT_WARPS * 32) {
                    const uint32_t addr = base + (uint32_t)i * 16u;
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr) : "memory");
                    const uint32_t h0 = x0 & 0xFFFFE000u, h1 = x1 & 0xFFFFE000u, h2 = x2 & 0xFFFFE000u, h3 = x3 & 0xFFFFE000u;
                    st_shared_v4(addr, h0, h1, h2, h3);
                    st_shared_v4(addr + Cfg::LOAD_BYTES,
                                 __float_as_uint(__uint_as_float(x0) - __uint_as_float(h0)),
                                 __float_as_uint(__uint_as_float(x1) - __uint_as_float(h1)),
                                 __float_as_uint(__uint_as_float(x2) - __uint_as_float(h2)),
                                 __float_as_uint(__uint_as_float(x3) - __uint_as_float(h3)));
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   /* generic writes -> tensor-core reads */
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(ready_bar(stage), 0));
                    else mbar_arrive(ready_bar(stage));
                }
                if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        /* epilogue: warp w may touch tensor-memory lanes 32*(w%4) .. +31 */
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;                 /* 0: even column chunks, 1: odd ones */
        const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
        uint32_t local_tile = 0;
        bool alive = true;
        T* cT = reinterpret_cast<T*>(args.c);
        long long w = work_begin; int phase_w = 0; Item item;
        for (; alive && next_item(w, phase_w, item); ++local_tile) {
            const int mt = item.mt, nt = item.nt, split = item.split, bz = item.bz;
            if (args.trace && warp == 2 && lane == 0 && local_tile > 0) trace_mark(args.trace, 11 + 4 * (int)(local_tile - 1));
            /* NH = 1: one pass over the tile's accumulator (two buffers, taken in turn).  NH = 2: the tile's two
             * accumulators one after the other.  The two warps of a lane quarter take alternate column chunks.
             * `continue` below means "this accumulator is done". */
#pragma unroll 1
            for (int h = 0; h < NH && alive; ++h) {
            const uint32_t ab = NH == 2 ? (uint32_t)h : (local_tile & 1u);
            const uint32_t acc_phase = NH == 2 ? (local_tile & 1u) : ((local_tile >> 1) & 1u);
            const int ncol0 = nt * TILE_N + h * ACC_N;              /* first column of C behind this accumulator */
            if (!mbar_wait(tfull_bar(ab), acc_phase, abort_flag, args.status, 4, args.wait_limit, args.epi_sleep_ns)) { alive = false; break; }
            __syncwarp();
            tc_fence_after();
            if (args.trace && warp == 2 && lane == 0) {
                if (h == 0) trace_mark(args.trace, 10 + 4 * (int)local_tile);
                else if (local_tile < 6) trace_mark(args.trace, 36 + (int)local_tile);     /* second accumulator complete */
            }
            const int row = mt * TILE_M + (int)cta_rank * BLOCK_M + quarter * 32 + lane;
            const bool row_ok = row < args.m;
            /* How this warp treats the item.  0: output tile.  1: fp32 piece through map_p (K slice of a tail tile,
             * reduced by a second kernel).  2: finish a cut tile with the neighbour's partial (balanced schedule).
             * 3: leave an fp32 partial in bal_scratch (balanced: the shorter piece; fused tail: the first slice to get
             * here).  4: fused tail, second slice to get here: finish with the first one's partial. */
            int mode = item.kind;
            int* tk = nullptr;
            if (args.bal && item.kind == 1) mode = 3;
            if (args.tail_fuse && item.kind == 1) {
                tk = args.bal_flags + ((((long long)(item.slot >> 1) * 2 + (int)cta_rank) * EPI_WARPS) + (warp - 2)) * 2;
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(tk, 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                mode = ticket == 0 ? 3 : 4;
            }
            const long long pslot = args.tail_fuse ? (item.slot >> 1) : item.slot;
            if (mode == 3) {
                /* fp32 sums to the slot, in the layout the finishing warp reads them in (same lane quarter, 32-column
                 * chunk, lane: contiguous 512 bytes per warp access).  The fused tail uses the finishing warp's own
                 * column assignment, so that the hand-over is warp to warp. */
                float4* dst = reinterpret_cast<float4*>(args.bal_scratch) +
                              ((pslot * 2 + (int)cta_rank) * 4 + quarter) * (ACC_N / 32) * 256 + lane;
                const int row_warp = mt * TILE_M + (int)cta_rank * BLOCK_M + quarter * 32;
                const int span = (args.tail_fuse && !SPLIT) ? 64 : 32;          /* columns per loop step */
#pragma unroll 1
                for (int c0 = half * span; c0 < ACC_N; c0 += 2 * span) {
#pragma unroll 1
                    for (int cc = c0; cc < c0 + span; cc += 32) {
                        uint32_t v[32];
                        __syncwarp();
                        tmem_load_32(tmem_base + ab * ACC_N + cc + lane_field, v);
                        if (ncol0 + cc >= args.n || row_warp >= args.m) continue;      /* warp-uniform */
                        float4* d4 = dst + (cc / 32) * 256;
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            __stcg(d4 + q * 32, make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                            __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(tempty_bar(ab), 0));
                    else mbar_arrive(tempty_bar(ab));
                    __threadfence();                      /* the warp's stores (ordered before by the warp barrier) are published */
                    if (tk) {
                        asm volatile("st.release.gpu.global.s32 [%0], 1;" ::"l"(tk + 1) : "memory");
                    } else {
                        int* f = args.bal_flags + ((long long)item.slot * 2 + (int)cta_rank) * 2;
                        asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(f) : "memory");
                    }
                }
                continue;
            }
            if (args.tma_store) {
                /* Each warp stages 32 rows x 128 bytes in the 128-byte swizzle the store's tensor map
                 * expects (16-byte chunk c of row r at position c ^ (r & 7)) and one lane hands the box to
                 * the TMA engine, which writes whole lines and clips rows >= M / columns >= N itself.
                 * One 4 KB buffer per warp; the two warps of a lane quarter take alternate chunks. */
                const int row_warp = mt * TILE_M + (int)cta_rank * BLOCK_M + quarter * 32;
                const uint32_t buf = store_base + (uint32_t)(warp - 2) * Cfg::STORE_BUF_BYTES;
                const uint32_t my_row = (uint32_t)lane * 128u;
                const uint32_t sw = (uint32_t)lane & 7u;
                const bool tail_item = mode == 1;
                const bool partial_out = args.splits > 1 || tail_item || args.c_f32;
                const bool wide = partial_out || SPLIT;                     /* rows of fp32: 32 columns per 128 bytes */
                const int cols_per_box = wide ? 32 : 64;                    /* 128 bytes of fp32 or of 16-bit T */
                const int zc = partial_out ? split * args.batch + bz : bz;
                /* balanced schedule, finishing piece: the other piece of this tile was computed by the previous CTA
                 * (pair) at the very start of its run; its rows of the partial tile are complete once its eight
                 * epilogue warps have counted themselves in */
                const float4* part = nullptr;
                int* flag = nullptr;
                if (mode == 2 || mode == 4) {
                    /* balanced: all eight warps of the neighbour's CTA have counted in; fused tail: this warp's partner */
                    const int* watch = mode == 2 ? args.bal_flags + ((long long)item.slot * 2 + (int)cta_rank) * 2 : tk + 1;
                    const int need = mode == 2 ? EPI_WARPS : 1;
                    if (mode == 2) flag = const_cast<int*>(watch);
                    bool ok = true;
                    if (lane == 0) {
                        const long long t0 = clock64();
                        int seen = 0;
                        for (uint32_t i = 0;; ++i) {
                            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(watch) : "memory");
                            if (seen >= need) break;
                            __nanosleep(100);
                            if ((i & 63u) == 63u && (*abort_flag || clock64() - t0 > args.wait_limit)) { ok = false; break; }
                        }
                        if (!ok) {
                            *abort_flag = 1;
                            volatile int* st = args.status;
                            if (*st == 0) *st = 6;
                            __threadfence_system();
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) { alive = false; break; }
                    part = reinterpret_cast<const float4*>(args.bal_scratch) +
                           ((pslot * 2 + (int)cta_rank) * 4 + quarter) * (ACC_N / 32) * 256 + lane;
                }
                if constexpr (!SPLIT) {
                    if (!wide && !part && args.epi_pipe) {
                        /* 16-bit rows of C, the common case.  Measured in SM clocks per 64-column chunk of a warp: the
                         * tcgen05.ld pair ~45, rounding and packing ~200, and the hand-over to the TMA engine (wait for the
                         * previous store to have read the buffer, st.shared, proxy fence, issue) 500-900.  So the warp first
                         * pulls BOTH of its chunks of the accumulator into registers (the first one packed to 16 bits), gives
                         * the accumulator back to the MMA warp -- a few hundred clocks after it was completed -- and only
                         * then stages and stores. */
                        const bool rows_in = row_warp < args.m;             /* warp-uniform */
                        const int ca = half * 64, cb = ca + 128;            /* this warp's chunks of the accumulator */
                        const bool two = cb < ACC_N;
                        uint32_t v[32], v2[32], pk[32];
                        if (ca < ACC_N) {
                            __syncwarp();
                            tmem_load_32_nowait(tmem_base + ab * ACC_N + ca + lane_field, v);
                            tmem_load_32_nowait(tmem_base + ab * ACC_N + ca + 32 + lane_field, v2);
                            tmem_load_wait();
                            if (args.bias) {
                                add_bias_32<T>(v, reinterpret_cast<const T*>(args.bias), ncol0 + ca, args.n);
                                add_bias_32<T>(v2, reinterpret_cast<const T*>(args.bias), ncol0 + ca + 32, args.n);
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                pk[i] = pack2<T>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                pk[16 + i] = pack2<T>(__uint_as_float(v2[2 * i]), __uint_as_float(v2[2 * i + 1]));
                            }
                            if (two) {
                                __syncwarp();
                                tmem_load_32_nowait(tmem_base + ab * ACC_N + cb + lane_field, v);
                                tmem_load_32_nowait(tmem_base + ab * ACC_N + cb + 32 + lane_field, v2);
                                tmem_load_wait();
                            }
                        }
                        tc_fence_before();                                  /* every lane's reads are complete */
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR) mbar_arrive_cluster(cluster_addr(tempty_bar(ab), 0));
                            else mbar_arrive(tempty_bar(ab));
                        }
                        /* one chunk: registers -> staging buffer (128-byte swizzle) -> TMA store */
                        auto put = [&](int c0) {
                            if (ncol0 + c0 < args.n && rows_in) {
                                if (lane == 0) tma_store_wait_read<0>();    /* the previous store has read `buf` */
                                __syncwarp();
#pragma unroll
                                for (uint32_t c = 0; c < 8; ++c)
                                    st_shared_v4(buf + my_row + ((c ^ sw) << 4), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                                __syncwarp();
                                if (lane == 0) tma_store_3d(&map_c, buf, ncol0 + c0, row_warp, zc);
                            }
                        };
                        if (ca < ACC_N) put(ca);
                        if (ca < ACC_N && two) {
                            if (args.bias) {
                                add_bias_32<T>(v, reinterpret_cast<const T*>(args.bias), ncol0 + cb, args.n);
                                add_bias_32<T>(v2, reinterpret_cast<const T*>(args.bias), ncol0 + cb + 32, args.n);
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                pk[i] = pack2<T>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                pk[16 + i] = pack2<T>(__uint_as_float(v2[2 * i]), __uint_as_float(v2[2 * i + 1]));
                            }
                            put(cb);
                        }
                        continue;
                    }
                }
#pragma unroll 1
                for (int c0 = half * cols_per_box; c0 < ACC_N; c0 += 2 * cols_per_box) {
                    const int col = ncol0 + c0;
                    uint32_t v[32], v2[32];
                    __syncwarp();
                    /* the accumulator reads of this chunk overlap the TMA engine draining the previous one */
                    tmem_load_32_nowait(tmem_base + ab * ACC_N + c0 + lane_field, v);
                    if (!wide) tmem_load_32_nowait(tmem_base + ab * ACC_N + c0 + 32 + lane_field, v2);
                    tmem_load_wait();
                    if (col >= args.n || row_warp >= args.m) continue;      /* warp-uniform */
                    if (part) {                                             /* the other piece's sums for the same elements */
                        if constexpr (!SPLIT) {
                            const float4* p4 = part + (c0 / 32) * 256;
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float4 x = __ldcg(p4 + q * 32), y = __ldcg(p4 + 256 + q * 32);
                                v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + x.x);
                                v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + x.y);
                                v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + x.z);
                                v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + x.w);
                                v2[4 * q] = __float_as_uint(__uint_as_float(v2[4 * q]) + y.x);
                                v2[4 * q + 1] = __float_as_uint(__uint_as_float(v2[4 * q + 1]) + y.y);
                                v2[4 * q + 2] = __float_as_uint(__uint_as_float(v2[4 * q + 2]) + y.z);
                                v2[4 * q + 3] = __float_as_uint(__uint_as_float(v2[4 * q + 3]) + y.w);
                            }
                        } else {
                            const float4* p4 = part + (c0 / 32) * 256;
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float4 x = __ldcg(p4 + q * 32);
                                v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + x.x);
                                v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + x.y);
                                v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + x.z);
                                v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + x.w);
                            }
                        }
                    }
                    if (args.bias && !partial_out) {
                        add_bias_32<T>(v, reinterpret_cast<const T*>(args.bias), col, args.n);
                        if (!wide) add_bias_32<T>(v2, reinterpret_cast<const T*>(args.bias), col + 32, args.n);
                    }
                    if (lane == 0) tma_store_wait_read<0>();                /* the previous store has read `buf` */
                    __syncwarp();
                    if (wide) {
#pragma unroll
                        for (uint32_t c = 0; c < 8; ++c)
                            st_shared_v4(buf + my_row + ((c ^ sw) << 4), v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                    } else if constexpr (!SPLIT) {
#pragma unroll
                        for (uint32_t c = 0; c < 4; ++c) {
                            st_shared_v4(buf + my_row + ((c ^ sw) << 4),
                                         pack2<T>(__uint_as_float(v[8 * c]), __uint_as_float(v[8 * c + 1])),
                                         pack2<T>(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3])),
                                         pack2<T>(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5])),
                                         pack2<T>(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7])));
                            st_shared_v4(buf + my_row + (((c + 4) ^ sw) << 4),
                                         pack2<T>(__uint_as_float(v2[8 * c]), __uint_as_float(v2[8 * c + 1])),
                                         pack2<T>(__uint_as_float(v2[8 * c + 2]), __uint_as_float(v2[8 * c + 3])),
                                         pack2<T>(__uint_as_float(v2[8 * c + 4]), __uint_as_float(v2[8 * c + 5])),
                                         pack2<T>(__uint_as_float(v2[8 * c + 6]), __uint_as_float(v2[8 * c + 7])));
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   /* generic writes -> async proxy */
                    __syncwarp();
                    if (lane == 0) {
                        if (tail_item)   /* compact scratch: [slot][row inside the tile][column inside the tile] */
                            tma_store_3d(&map_p, buf, c0, (int)cta_rank * BLOCK_M + quarter * 32, item.slot);
                        else
                            tma_store_3d(&map_c, buf, col, row_warp, zc);
                    }
                }
                tc_fence_before();
                __syncwarp();                 /* every lane's accumulator reads are done: one arrival per warp */
                if (lane == 0) {
                    if (PAIR) mbar_arrive_cluster(cluster_addr(tempty_bar(ab), 0));
                    else mbar_arrive(tempty_bar(ab));
                }
                if (flag) {
                    /* this warp has read its rows of the partial; the last of the eight readers clears both counts
                     * for the next launch (no memset between launches, and a replayed CUDA graph stays correct) */
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence();
                        if (atomicAdd(flag + 1, 1) == EPI_WARPS - 1) { flag[1] = 0; __threadfence(); atomicExch(flag, 0); }
                    }
                }
                if (mode == 4) {                  /* both slices of this warp's part are done: ticket and flag back to zero */
                    __syncwarp();
                    if (lane == 0) { __threadfence(); atomicExch(tk + 1, 0); atomicExch(tk, 0); }
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = half * 32; c0 < ACC_N; c0 += 64) {
                uint32_t v[32];
                __syncwarp();                 /* tcgen05.ld is warp-collective */
                tmem_load_32(tmem_base + ab * ACC_N + c0 + lane_field, v);
                const int col = ncol0 + c0;
                if (!row_ok || col >= args.n) {
                    /* nothing to store for this lane */
                } else if (args.splits > 1 || args.c_f32) {
                    float* dst = args.partial + (((long long)split * args.batch + bz) * args.m + row) * (long long)args.n + col;
                    const bool add = args.c_f32 && args.accumulate;      /* float32 output that keeps a running sum */
                    if (col + 32 <= args.n && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 f = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                                   __uint_as_float(v[j + 3]));
                            if (add) {
                                const float4 o = *reinterpret_cast<const float4*>(dst + j);
                                f.x += o.x; f.y += o.y; f.z += o.z; f.w += o.w;
                            }
                            *reinterpret_cast<float4*>(dst + j) = f;
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < args.n; ++j) dst[j] = __uint_as_float(v[j]) + (add ? dst[j] : 0.f);
                    }
                } else {
                    T* dst = cT + bz * args.c_batch + (long long)row * args.c_row + col;
                    if (args.bias) add_bias_32<T>(v, reinterpret_cast<const T*>(args.bias), col, args.n);
                    if constexpr (SPLIT) {
                        if (col + 32 <= args.n && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 f = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                                       __uint_as_float(v[j + 3]));
                                if (args.accumulate) {
                                    const float4 o = *reinterpret_cast<const float4*>(dst + j);
                                    f.x += o.x; f.y += o.y; f.z += o.z; f.w += o.w;
                                }
                                if (args.act) {
                                    const int q = args.n >> 2;
                                    f.x = rpb_gate_act(f.x, col + j, q); f.y = rpb_gate_act(f.y, col + j + 1, q);
                                    f.z = rpb_gate_act(f.z, col + j + 2, q); f.w = rpb_gate_act(f.w, col + j + 3, q);
                                }
                                *reinterpret_cast<float4*>(dst + j) = f;
                            }
                        } else {
                            for (int j = 0; j < 32 && col + j < args.n; ++j) {
                                float f = __uint_as_float(v[j]);
                                if (args.accumulate) f += to_f32<T>(dst[j]);
                                if (args.act) f = rpb_gate_act(f, col + j, args.n >> 2);
                                dst[j] = from_f32<T>(f);
                            }
                        }
                    } else if (col + 32 <= args.n && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            float f[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[j + e]);
                            if (args.accumulate) {
                                uint4 old = *reinterpret_cast<const uint4*>(dst + j);
                                const T* o = reinterpret_cast<const T*>(&old);
#pragma unroll
                                for (int e = 0; e < 8; ++e) f[e] += to_f32<T>(o[e]);
                            }
                            if (args.act) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) f[e] = rpb_gate_act(f[e], col + j + e, args.n >> 2);
                            }
                            uint4 out = make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]),
                                                   pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
                            *reinterpret_cast<uint4*>(dst + j) = out;
                        }
                    } else {
                        for (int j = 0; j < 32 && col + j < args.n; ++j) {
                            float f = __uint_as_float(v[j]);
                            if (args.accumulate) f += to_f32<T>(dst[j]);
                            if (args.act) f = rpb_gate_act(f, col + j, args.n >> 2);
                            dst[j] = from_f32<T>(f);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(cluster_addr(tempty_bar(ab), 0));   /* the leader owns the accumulator hand-off */
                else mbar_arrive(tempty_bar(ab));
            }
            }
        }
    }

    if (warp >= 2 && lane == 0 && args.tma_store) tma_store_wait_all();   /* staged rows have left shared memory */
    if (args.trace && warp == 2 && lane == 0) trace_mark(args.trace, 6);

    if (threadIdx.x == 0) trace_mark(args.trace, 5);
    /* teardown: if a wait gave up, let copies that are still in flight land first */
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) { __syncwarp(); cluster_sync(); }   /* neither CTA's shared or tensor memory goes away under the other */
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

/* Adds the K slices of the tail tiles in slice order and writes them into C (with the bias, rounding once).
 * grid = (tail tiles, rows of a tile), block = tile columns / 4. */
template <typename T>
__global__ void tail_reduce_kernel(const float* __restrict__ scratch, T* c, const T* bias, int m, int n, long long c_row,
                                   int tiles_m, int tiles_n, int group_n, int first_tail_tile, int slices,
                                   int tile_m, int tile_n)
{
    int mt, nt;
    tile_coords(first_tail_tile + (int)blockIdx.x, tiles_m, tiles_n, group_n, mt, nt);
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int lr = blockIdx.y, lc = threadIdx.x * 4;
    const int row = mt * tile_m + lr, col = nt * tile_n + lc;
    if (row >= m || col >= n) return;
    const size_t tile_elems = (size_t)tile_m * tile_n;
    const float* src = scratch + (size_t)blockIdx.x * slices * tile_elems + (size_t)lr * tile_n + lc;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sl = 0; sl < slices; ++sl) {
        const float4 x = *reinterpret_cast<const float4*>(src + sl * tile_elems);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    const float v[4] = {acc.x, acc.y, acc.z, acc.w};
    T* dst = c + (long long)row * c_row + col;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (col + e >= n) break;
        float x = v[e];
        if (bias) x += to_f32<T>(bias[col + e]);
        dst[e] = from_f32<T>(x);
    }
}

/* The bounded wait on its own: a barrier that expects one arrival and never gets it.  Every lane polls with the
 * given limit, the wait gives up, code 9 goes to *status and the kernel returns. */
__global__ void wait_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 9, limit_cycles);
    if (ok && threadIdx.x == 0) { volatile int* st = status; *st = -9; }     /* cannot happen: nobody arrives */
}

}  // namespace rpb_umma
#endif
