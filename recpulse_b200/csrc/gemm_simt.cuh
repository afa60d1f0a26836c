/*
 * CUDA-core GEMM (FFMA / DFMA) for float32 and float64, and the general-stride path
 * for float16 / bfloat16 operands whose layout the TMA engine cannot address
 * (a stride that is not a multiple of 16 bytes, a view with both strides != 1).
 *
 * C[b] (+)= sum_r A[b,r] . B[b,r]; every operand is read through its own element
 * strides, so transposed and broadcast views cost nothing extra.  Tiles of
 * BM x BN outputs per CTA, TM x TN per thread, K staged through shared memory in
 * the accumulation type.  When the output has too few tiles to fill the GPU the K
 * range (including the summed-problem index r) is split across CTAs; partial tiles go
 * to a scratch buffer and splitk_reduce_kernel adds them in a fixed order, so results
 * do not depend on scheduling.
 */
#ifndef RPB_GEMM_SIMT_CUH
#define RPB_GEMM_SIMT_CUH

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rpb_common.h"

namespace rpb_simt {

template <typename Acc, typename T> __device__ __forceinline__ Acc widen(T v) { return static_cast<Acc>(v); }
template <> __device__ __forceinline__ float widen<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T, typename Acc> __device__ __forceinline__ T narrow(Acc v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half narrow<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

struct Args {
    const void* a; const void* b; void* c;
    int m, n, k, batch, reduce;
    long long a_row, a_col, a_batch, a_reduce;
    long long b_row, b_col, b_batch, b_reduce;
    long long c_row, c_batch;
    int accumulate;
    int tiles_m, tiles_n;
    int k_blocks, k_iters, splits, iters_per_split;
    void* partial;          /* [splits][batch][m][n] in the accumulation type, when splits > 1 */
    const void* bias;       /* n values of T added to every output row (applied by the reduction when K is split) */
    /* float64 tensor-core kernel only: balanced schedule over (tile, K block) units, see gemm_dmma.cuh */
    int sk_ctas = 0;                /* 0 = one CTA per tile (and K slice) */
    long long sk_units = 0;         /* tiles * k_iters */
    double* sk_scratch = nullptr;   /* [sk_ctas - 1][2][128 x 128] partial tiles of the tiles cut between two CTAs */
};

template <typename T, typename Acc, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_kernel(const Args p)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    rpb_pdl_trigger();
    rpb_pdl_wait();
    __shared__ Acc As[BK][BM + 4];
    __shared__ Acc Bs[BK][BN + 4];

    long long w = blockIdx.x;
    const int mt = (int)(w % p.tiles_m); w /= p.tiles_m;
    const int nt = (int)(w % p.tiles_n); w /= p.tiles_n;
    const int split = (int)(w % p.splits);
    const int bz = (int)(w / p.splits);

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const int row0 = mt * BM, col0 = nt * BN;

    const T* A = reinterpret_cast<const T*>(p.a) + bz * p.a_batch;
    const T* B = reinterpret_cast<const T*>(p.b) + bz * p.b_batch;
    /* walk the contiguous direction of each operand with consecutive threads */
    const bool a_k_fast = (p.a_col == 1) || (p.a_row != 1 && p.a_col <= p.a_row);
    const bool b_n_fast = (p.b_col == 1) || (p.b_row != 1 && p.b_col <= p.b_row);

    Acc acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = Acc(0);

    const int it0 = split * p.iters_per_split;
    const int it1 = min(it0 + p.iters_per_split, p.k_iters);
    for (int it = it0; it < it1; ++it) {
        const int r = it / p.k_blocks;
        const int k0 = (it - r * p.k_blocks) * BK;
        const T* Ar = A + r * p.a_reduce;
        const T* Br = B + r * p.b_reduce;
#pragma unroll
        for (int e = tid; e < BM * BK; e += NT) {
            int i, l;
            if (a_k_fast) { i = e / BK; l = e % BK; } else { l = e / BM; i = e % BM; }
            const int gi = row0 + i, gl = k0 + l;
            Acc v = Acc(0);
            if (gi < p.m && gl < p.k) v = widen<Acc, T>(Ar[gi * p.a_row + gl * p.a_col]);
            As[l][i] = v;
        }
#pragma unroll
        for (int e = tid; e < BK * BN; e += NT) {
            int l, j;
            if (b_n_fast) { l = e / BN; j = e % BN; } else { j = e / BK; l = e % BK; }
            const int gl = k0 + l, gj = col0 + j;
            Acc v = Acc(0);
            if (gl < p.k && gj < p.n) v = widen<Acc, T>(Br[gl * p.b_row + gj * p.b_col]);
            Bs[l][j] = v;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < BK; ++l) {
            Acc av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[l][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) bv[j] = Bs[l][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

    if (p.splits > 1) {
        Acc* P = reinterpret_cast<Acc*>(p.partial) + ((long long)split * p.batch + bz) * p.m * (long long)p.n;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int gi = row0 + ty * TM + i;
            if (gi >= p.m) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int gj = col0 + tx * TN + j;
                if (gj < p.n) P[(long long)gi * p.n + gj] = acc[i][j];
            }
        }
    } else {
        T* C = reinterpret_cast<T*>(p.c) + bz * p.c_batch;
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int gi = row0 + ty * TM + i;
            if (gi >= p.m) continue;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int gj = col0 + tx * TN + j;
                if (gj >= p.n) continue;
                T* dst = C + (long long)gi * p.c_row + gj;
                Acc v = acc[i][j];
                if (p.bias) v += widen<Acc, T>(reinterpret_cast<const T*>(p.bias)[gj]);
                if (p.accumulate) v += widen<Acc, T>(*dst);
                *dst = narrow<T, Acc>(v);
            }
        }
    }
}

/* Adds the partial tiles of a K-split GEMM in split order and writes C (or C += sum). */
template <typename T, typename Acc>
__global__ void splitk_reduce_kernel(const Acc* __restrict__ partial, T* c, int splits, int batch,
                                     int m, int n, long long c_row, long long c_batch, int accumulate, const T* bias)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long per_split = (long long)batch * m * n;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_split; i += stride) {
        Acc s = Acc(0);
        for (int sp = 0; sp < splits; ++sp) s += partial[sp * per_split + i];
        const int col = (int)(i % n);
        const long long t = i / n;
        const int row = (int)(t % m);
        const int bz = (int)(t / m);
        T* dst = c + bz * c_batch + (long long)row * c_row + col;
        if (bias) s += widen<Acc, T>(bias[col]);
        if (accumulate) s += widen<Acc, T>(*dst);
        *dst = narrow<T, Acc>(s);
    }
}

/* Same reduction for n % 4 == 0: 4 consecutive outputs per thread (one 16/32-byte load per split)
 * and the splits dealt over 8 thread groups, so many loads are in flight even when the output is small
 * (a skinny dB with K in the tens of thousands).  Group g adds splits g, g+8, ... in order, then the
 * eight group sums are added in group order: a fixed association, independent of scheduling. */
template <typename T, typename Acc>
__global__ void __launch_bounds__(256)
splitk_reduce_vec_kernel(const Acc* __restrict__ partial, T* c, int splits, int batch, int m, int n,
                         long long c_row, long long c_batch, int accumulate, const T* bias)
{
    constexpr int GROUPS = 8, VECS = 32;
    rpb_pdl_trigger();
    rpb_pdl_wait();
    __shared__ Acc red[GROUPS][VECS][4];
    const long long per_split = (long long)batch * m * n;
    const long long nvec = per_split / 4;
    const int vec_in_block = threadIdx.x % VECS, grp = threadIdx.x / VECS;
    for (long long v0 = (long long)blockIdx.x * VECS; v0 < nvec; v0 += (long long)gridDim.x * VECS) {
        const long long v = v0 + vec_in_block;
        Acc s[4] = {Acc(0), Acc(0), Acc(0), Acc(0)};
        if (v < nvec) {
#pragma unroll 4
            for (int sp = grp; sp < splits; sp += GROUPS) {
                const Acc* src = partial + sp * per_split + v * 4;
                if (sizeof(Acc) == 4) {
                    const float4 x = *reinterpret_cast<const float4*>(src);
                    s[0] += x.x; s[1] += x.y; s[2] += x.z; s[3] += x.w;
                } else {
                    const double2 x = *reinterpret_cast<const double2*>(src);
                    const double2 y = *reinterpret_cast<const double2*>(src + 2);
                    s[0] += x.x; s[1] += x.y; s[2] += y.x; s[3] += y.y;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) red[grp][vec_in_block][e] = s[e];
        __syncthreads();
        if (grp == 0 && v < nvec) {
#pragma unroll
            for (int g = 1; g < GROUPS; ++g)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[e] += red[g][vec_in_block][e];
            const long long i = v * 4;
            const int col = (int)(i % n);
            const long long t = i / n;
            const int row = (int)(t % m);
            const int bz = (int)(t / m);
            T* dst = c + bz * c_batch + (long long)row * c_row + col;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                Acc x = s[e];
                if (bias) x += widen<Acc, T>(bias[col + e]);
                if (accumulate) x += widen<Acc, T>(dst[e]);
                dst[e] = narrow<T, Acc>(x);
            }
        }
        __syncthreads();
    }
}

template <typename T, typename Acc>
inline void launch_splitk_reduce(const Acc* partial, T* c, int splits, int batch, int m, int n, long long c_row,
                                 long long c_batch, int accumulate, const void* bias_v, int sm_count, cudaStream_t stream) {
    const T* bias = reinterpret_cast<const T*>(bias_v);
    const long long elems = (long long)batch * m * n;
    if (n % 4 == 0 && splits >= 4) {
        long long blocks = (elems / 4 + 31) / 32;
        if (blocks > sm_count * 8) blocks = sm_count * 8;
        rpb_launch(splitk_reduce_vec_kernel<T, Acc>, dim3((unsigned)blocks), dim3(256), 0, stream, 1, partial, c, splits, batch, m, n, c_row,
                   c_batch, accumulate, bias);
    } else {
        long long blocks = (elems + 255) / 256;
        if (blocks > sm_count * 8) blocks = sm_count * 8;
        rpb_launch(splitk_reduce_kernel<T, Acc>, dim3((unsigned)blocks), dim3(256), 0, stream, 1, partial, c, splits, batch, m, n, c_row,
                   c_batch, accumulate, bias);
    }
}

}  // namespace rpb_simt
#endif
