/*
 * float64 GEMM on the double-precision tensor-core path (mma.sync m16n8k8, f64 accumulate).
 *
 * CTA tile 128 x 128, K staged 32 at a time through a 3-stage cp.async ring (216 KB), 8 warps of 64 x 32.
 * Each operand is kept in shared memory in the orientation it has in global memory, so both
 * row-major and transposed views are copied with 16-byte cp.async along their contiguous index:
 *   K-contiguous  X[mn][k], leading dimension 36 doubles
 *   MN-contiguous X[k][mn], leading dimension 136 doubles
 * Both leading dimensions make the 8 x 4 (or 4 x 8) fragment reads of a warp hit every bank pair
 * exactly twice, the minimum for 32 lanes x 8 bytes.
 *
 * Schedules.  Plain: one CTA per output tile (times K slices for skinny outputs, partial sums reduced by a
 * second kernel).  Balanced (sk_ctas > 0): for outputs of more tiles than SMs whose last wave would be sparse
 * (2048^3: 256 tiles on 148 SMs = two waves for 1.73 waves of work), the (tile, K block) units are dealt
 * evenly and contiguously to one CTA per SM.  A CTA finishes the tile cut by its range start, runs its whole
 * tiles, and starts the tile cut by its range end; every CTA gets at least one tile's worth of units, so a tile
 * is cut at most once.  The two pieces of a cut tile go to scratch and `balanced_fixup_kernel` adds them in a
 * fixed order (deterministic; no atomics, no CTA waits for another).
 *
 * Requirements (checked by the dispatcher, which otherwise uses the general-stride kernel): the
 * contiguous index has stride 1, every other stride is even (16-byte multiples) and the base
 * pointers are 16-byte aligned.  Ragged M, N, K are zero-filled by cp.async's src-size operand.
 */
#ifndef RPB_GEMM_DMMA_CUH
#define RPB_GEMM_DMMA_CUH

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_simt.cuh"

namespace rpb_dmma {

constexpr int BM = 128, BN = 128, BK = 32, STAGES = 3, THREADS = 256;
constexpr int LD_K = BK + 4;    /* K-contiguous tile: [128][36]  */
constexpr int LD_MN = 136;      /* MN-contiguous tile: [32][136] */
constexpr int TILE_DOUBLES = 128 * LD_K;             /* 4608 >= 32 * 136 = 4352 */
constexpr int STAGE_DOUBLES = 2 * TILE_DOUBLES;
constexpr int SMEM_BYTES = STAGES * STAGE_DOUBLES * 8;

__device__ __forceinline__ void cp_async_16(double* dst, const double* src, int src_bytes) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void dmma_16x8x8(double (&c)[4], const double (&a)[4], const double (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
        : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

/* Copies one operand tile (128 along mn, 16 along k) into shared memory.  `mn_contig` selects the
 * orientation; `ext_mn`/`ext_k` are the operand's extents for zero fill. */
template <bool MN_CONTIG>
__device__ __forceinline__ void load_tile(double* smem, const double* g, long long stride_other, int mn0, int k0,
                                          int ext_mn, int ext_k, int tid) {
    if (!MN_CONTIG) {
        /* rows = mn (128), BK doubles of k per row = BK/2 vectors */
        constexpr int VPR = BK / 2;
#pragma unroll
        for (int i = 0; i < 128 * VPR / THREADS; ++i) {
            const int v = tid + i * THREADS;
            const int r = v / VPR, c = (v % VPR) * 2;
            const int gm = mn0 + r, gk = k0 + c;
            int bytes = 0;
            if (gm < ext_mn && gk < ext_k) bytes = (ext_k - gk >= 2) ? 16 : 8;
            const double* src = bytes ? g + (long long)gm * stride_other + gk : g;
            cp_async_16(smem + r * LD_K + c, src, bytes);
        }
    } else {
        /* rows = k (BK), 128 doubles of mn per row = 64 vectors */
#pragma unroll
        for (int i = 0; i < BK * 64 / THREADS; ++i) {
            const int v = tid + i * THREADS;
            const int r = v >> 6, c = (v & 63) * 2;
            const int gk = k0 + r, gm = mn0 + c;
            int bytes = 0;
            if (gk < ext_k && gm < ext_mn) bytes = (ext_mn - gm >= 2) ? 16 : 8;
            const double* src = bytes ? g + (long long)gk * stride_other + gm : g;
            cp_async_16(smem + r * LD_MN + c, src, bytes);
        }
    }
}

/* A_MN: A is stored m-contiguous (a_row == 1); B_MN: B is stored n-contiguous (b_col == 1). */
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const rpb_simt::Args p)
{
    extern __shared__ __align__(16) double smem[];
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;       /* warp tile origin inside the CTA tile */
    const int g = lane >> 2, t = lane & 3;
    /* balanced schedule: this CTA's range of (tile, K block) units */
    long long cursor = 0, range_end = 0;
    if (p.sk_ctas > 0) {
        const long long base = p.sk_units / p.sk_ctas, extra = p.sk_units % p.sk_ctas, b = blockIdx.x;
        cursor = b * base + (b < extra ? b : extra);
        range_end = cursor + base + (b < extra ? 1 : 0);
    }
  for (;;) {
    long long w = blockIdx.x;
    int split = 0, it0, it1;
    int cut = -1;                              /* balanced: 0 = head piece of a cut tile, 1 = tail piece, -1 = whole */
    if (p.sk_ctas > 0) {
        if (cursor >= range_end) break;
        w = cursor / p.k_iters;
        it0 = (int)(cursor - w * p.k_iters);
        const long long room = range_end - cursor;
        it1 = (p.k_iters - it0 <= room) ? p.k_iters : it0 + (int)room;
        cursor += it1 - it0;
        if (it0 > 0) cut = 1; else if (it1 < p.k_iters) cut = 0;
    }
    const int mt = (int)(w % p.tiles_m); w /= p.tiles_m;
    const int nt = (int)(w % p.tiles_n); w /= p.tiles_n;
    int bz;
    if (p.sk_ctas > 0) bz = (int)w;
    else {
        split = (int)(w % p.splits);
        bz = (int)(w / p.splits);
        it0 = split * p.iters_per_split;
        it1 = min(it0 + p.iters_per_split, p.k_iters);
    }
    const int row0 = mt * BM, col0 = nt * BN;

    const double* A = reinterpret_cast<const double*>(p.a) + bz * p.a_batch;
    const double* B = reinterpret_cast<const double*>(p.b) + bz * p.b_batch;
    const long long a_other = A_MN ? p.a_col : p.a_row;          /* stride of the non-contiguous index */
    const long long b_other = B_MN ? p.b_row : p.b_col;

    double acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0;

    const int n_it = it1 - it0;

    auto issue = [&](int it, int stage) {
        const int r = it / p.k_blocks;
        const int k0 = (it - r * p.k_blocks) * BK;
        double* sa = smem + stage * STAGE_DOUBLES;
        double* sb = sa + TILE_DOUBLES;
        load_tile<A_MN>(sa, A + r * p.a_reduce, a_other, row0, k0, p.m, p.k, tid);
        load_tile<B_MN>(sb, B + r * p.b_reduce, b_other, col0, k0, p.n, p.k, tid);
    };

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_it) issue(it0 + s, s);
        cp_async_commit();
    }
    for (int i = 0; i < n_it; ++i) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (i + STAGES - 1 < n_it) issue(it0 + i + STAGES - 1, (i + STAGES - 1) % STAGES);
        cp_async_commit();
        const double* sa = smem + (i % STAGES) * STAGE_DOUBLES;
        const double* sb = sa + TILE_DOUBLES;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 8) {
            double af[4][4], bf[4][2];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int r = wm + mi * 16 + g;
                if (!A_MN) {
                    af[mi][0] = sa[r * LD_K + kk + t];           af[mi][1] = sa[(r + 8) * LD_K + kk + t];
                    af[mi][2] = sa[r * LD_K + kk + t + 4];       af[mi][3] = sa[(r + 8) * LD_K + kk + t + 4];
                } else {
                    af[mi][0] = sa[(kk + t) * LD_MN + r];        af[mi][1] = sa[(kk + t) * LD_MN + r + 8];
                    af[mi][2] = sa[(kk + t + 4) * LD_MN + r];    af[mi][3] = sa[(kk + t + 4) * LD_MN + r + 8];
                }
            }
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) {
                const int c = wn + ni * 8 + g;
                if (B_MN) { bf[ni][0] = sb[(kk + t) * LD_MN + c]; bf[ni][1] = sb[(kk + t + 4) * LD_MN + c]; }
                else      { bf[ni][0] = sb[c * LD_K + kk + t];    bf[ni][1] = sb[c * LD_K + kk + t + 4]; }
            }
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) dmma_16x8x8(acc[mi][ni], af[mi], bf[ni]);
        }
    }
    cp_async_wait<0>();

    /* accumulator fragment: (row g, cols 2t, 2t+1) and (row g+8, same cols) of each 16 x 8 block */
    if (cut >= 0) {
        /* piece of a cut tile: the tail piece belongs to the boundary before this CTA, the head piece to the one
         * after it; compact [128][128] tile, rows and columns beyond M, N hold zeros times nothing (never read) */
        double* S = p.sk_scratch + ((long long)(cut == 1 ? blockIdx.x - 1 : blockIdx.x) * 2 + cut) * (BM * BN);
#pragma unroll
        for (int mi = 0; mi < 4; ++mi)
#pragma unroll
            for (int ni = 0; ni < 4; ++ni)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = wm + mi * 16 + g + h * 8, c = wn + ni * 8 + 2 * t;
                    *reinterpret_cast<double2*>(S + r * BN + c) = make_double2(acc[mi][ni][2 * h], acc[mi][ni][2 * h + 1]);
                }
        __syncthreads();                       /* shared memory is reused by the next piece */
        continue;
    }
    const bool to_partial = p.splits > 1;
    double* P = to_partial ? reinterpret_cast<double*>(p.partial) + ((long long)split * p.batch + bz) * p.m * (long long)p.n
                           : nullptr;
    double* C = reinterpret_cast<double*>(p.c) + bz * p.c_batch;
#pragma unroll
    for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = row0 + wm + mi * 16 + g + h * 8;
                const int c = col0 + wn + ni * 8 + 2 * t;
                if (r >= p.m) continue;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (c + e >= p.n) continue;
                    double v = acc[mi][ni][2 * h + e];
                    if (to_partial) P[(long long)r * p.n + c + e] = v;
                    else {
                        double* dst = C + (long long)r * p.c_row + c + e;
                        if (p.bias) v += reinterpret_cast<const double*>(p.bias)[c + e];
                        if (p.accumulate) v += *dst;
                        *dst = v;
                    }
                }
            }
    if (p.sk_ctas == 0) break;
    __syncthreads();                           /* shared memory is reused by the next tile */
  }
}

/* Adds the two pieces of every tile that the balanced schedule cut between CTA i and CTA i + 1 (block i) and
 * writes the tile: head + tail (+ bias) (+ C when accumulating), always in that order. */
__global__ void __launch_bounds__(256)
balanced_fixup_kernel(const rpb_simt::Args p)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long base = p.sk_units / p.sk_ctas, extra = p.sk_units % p.sk_ctas, b = blockIdx.x + 1;
    const long long boundary = b * base + (b < extra ? b : extra);      /* first unit of CTA b */
    long long w = boundary / p.k_iters;
    if (boundary - w * p.k_iters == 0) return;                          /* CTA b starts on a tile boundary */
    const int mt = (int)(w % p.tiles_m); w /= p.tiles_m;
    const int nt = (int)(w % p.tiles_n);
    const int bz = (int)(w / p.tiles_n);
    const double* head = p.sk_scratch + (long long)blockIdx.x * 2 * (BM * BN);
    const double* tail = head + BM * BN;
    double* C = reinterpret_cast<double*>(p.c) + bz * p.c_batch;
    const double* bias = reinterpret_cast<const double*>(p.bias);
    /* gridDim.y blocks share a tile so that the pass is not bound by the latency of 147 blocks' loads */
    const int per = BM * BN / gridDim.y;
    for (int i = blockIdx.y * per + threadIdx.x; i < (blockIdx.y + 1) * per; i += blockDim.x) {
        const int r = mt * BM + i / BN, c = nt * BN + i % BN;
        if (r >= p.m || c >= p.n) continue;
        double v = head[i] + tail[i];
        if (bias) v += bias[c];
        double* dst = C + (long long)r * p.c_row + c;
        if (p.accumulate) v += *dst;
        *dst = v;
    }
}

}  // namespace rpb_dmma
#endif
