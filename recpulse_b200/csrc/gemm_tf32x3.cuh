/*
 * float32 GEMM on tensor cores with the 3xTF32 split: every fp32 operand value x is taken apart in
 * registers as x = hi + lo (hi = tf32(x), lo = tf32(x - hi)) and each product is formed as
 * lo*hi + hi*lo + hi*hi with fp32 accumulation (mma.sync m16n8k8 tf32).  The dropped lo*lo term is
 * below 2^-22 of the product, so results stay within fp32 rounding of a strict-fp32 GEMM.
 *
 * Same structure as the float64 kernel: BM x BN CTA tile, K staged 32 at a time through a 3-stage
 * cp.async ring, operands kept in shared memory in their global orientation (K-contiguous rows of
 * 36 floats, or MN-contiguous rows of BM+8 / BN+8 floats; both give conflict-free fragment reads).
 * Requirements (else the general-stride FFMA kernel runs): contiguous index with stride 1, other
 * strides multiples of 4 elements, 16-byte aligned bases.
 */
#ifndef RPB_GEMM_TF32X3_CUH
#define RPB_GEMM_TF32X3_CUH

#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_dmma.cuh"
#include "gemm_simt.cuh"

namespace rpb_tf32 {

constexpr int BK = 32, STAGES = 3, LD_K = BK + 4;

template <int BM, int BN> struct Cfg {
    static constexpr int A_FLOATS = (BM * LD_K > BK * (BM + 8)) ? BM * LD_K : BK * (BM + 8);
    static constexpr int B_FLOATS = (BN * LD_K > BK * (BN + 8)) ? BN * LD_K : BK * (BN + 8);
    static constexpr int STAGE_FLOATS = A_FLOATS + B_FLOATS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_FLOATS * 4;
};

__device__ __forceinline__ void cp_async_16f(float* dst, const float* src, int src_bytes) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    const float rest = x - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

/* copies an (EXT x 32) operand tile; MN_CONTIG selects [k][EXT+8] or [EXT][36] */
template <int EXT, int THREADS, bool MN_CONTIG>
__device__ __forceinline__ void load_tile(float* smem, const float* g, long long stride_other, int mn0, int k0,
                                          int ext_mn, int ext_k, int tid) {
    constexpr int VECS = EXT * BK / 4;
    if (!MN_CONTIG) {
#pragma unroll
        for (int i = 0; i < VECS / THREADS; ++i) {
            const int v = tid + i * THREADS;
            const int r = v >> 3, c = (v & 7) * 4;
            const int gm = mn0 + r, gk = k0 + c;
            int bytes = 0;
            if (gm < ext_mn && gk < ext_k) bytes = min(4, ext_k - gk) * 4;
            cp_async_16f(smem + r * LD_K + c, bytes ? g + (long long)gm * stride_other + gk : g, bytes);
        }
    } else {
        constexpr int VPR = EXT / 4;           /* vectors per k row */
#pragma unroll
        for (int i = 0; i < VECS / THREADS; ++i) {
            const int v = tid + i * THREADS;
            const int r = v / VPR, c = (v % VPR) * 4;
            const int gk = k0 + r, gm = mn0 + c;
            int bytes = 0;
            if (gk < ext_k && gm < ext_mn) bytes = min(4, ext_mn - gm) * 4;
            cp_async_16f(smem + r * (EXT + 8) + c, bytes ? g + (long long)gk * stride_other + gm : g, bytes);
        }
    }
}

template <int BM, int BN, int WM, int WN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(WM * WN * 32)
gemm_kernel(const rpb_simt::Args p)
{
    constexpr int THREADS = WM * WN * 32;
    constexpr int MI = BM / WM / 16, NI = BN / WN / 8;
    using C = Cfg<BM, BN>;
    extern __shared__ __align__(16) float smem_f[];
    rpb_pdl_trigger();
    rpb_pdl_wait();
    long long w = blockIdx.x;
    const int mt = (int)(w % p.tiles_m); w /= p.tiles_m;
    const int nt = (int)(w % p.tiles_n); w /= p.tiles_n;
    const int split = (int)(w % p.splits);
    const int bz = (int)(w / p.splits);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp / WN) * (BM / WM), wn = (warp % WN) * (BN / WN);
    const int g = lane >> 2, t = lane & 3;
    const int row0 = mt * BM, col0 = nt * BN;

    const float* A = reinterpret_cast<const float*>(p.a) + bz * p.a_batch;
    const float* B = reinterpret_cast<const float*>(p.b) + bz * p.b_batch;
    const long long a_other = A_MN ? p.a_col : p.a_row;
    const long long b_other = B_MN ? p.b_row : p.b_col;

    float acc[MI][NI][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    const int it0 = split * p.iters_per_split;
    const int it1 = min(it0 + p.iters_per_split, p.k_iters);
    const int n_it = it1 - it0;

    auto issue = [&](int it, int stage) {
        const int r = it / p.k_blocks;
        const int k0 = (it - r * p.k_blocks) * BK;
        float* sa = smem_f + stage * C::STAGE_FLOATS;
        float* sb = sa + C::A_FLOATS;
        load_tile<BM, THREADS, A_MN>(sa, A + r * p.a_reduce, a_other, row0, k0, p.m, p.k, tid);
        load_tile<BN, THREADS, B_MN>(sb, B + r * p.b_reduce, b_other, col0, k0, p.n, p.k, tid);
    };

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_it) issue(it0 + s, s);
        rpb_dmma::cp_async_commit();
    }
    for (int i = 0; i < n_it; ++i) {
        rpb_dmma::cp_async_wait<STAGES - 2>();
        __syncthreads();
        if (i + STAGES - 1 < n_it) issue(it0 + i + STAGES - 1, (i + STAGES - 1) % STAGES);
        rpb_dmma::cp_async_commit();
        const float* sa = smem_f + (i % STAGES) * C::STAGE_FLOATS;
        const float* sb = sa + C::A_FLOATS;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 8) {
            uint32_t ah[MI][4], al[MI][4], bh[NI][2], bl[NI][2];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const int r = wm + mi * 16 + g;
                float x[4];
                if (!A_MN) {
                    x[0] = sa[r * LD_K + kk + t];           x[1] = sa[(r + 8) * LD_K + kk + t];
                    x[2] = sa[r * LD_K + kk + t + 4];       x[3] = sa[(r + 8) * LD_K + kk + t + 4];
                } else {
                    x[0] = sa[(kk + t) * (BM + 8) + r];     x[1] = sa[(kk + t) * (BM + 8) + r + 8];
                    x[2] = sa[(kk + t + 4) * (BM + 8) + r]; x[3] = sa[(kk + t + 4) * (BM + 8) + r + 8];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) split_tf32(x[e], ah[mi][e], al[mi][e]);
            }
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) {
                const int c = wn + ni * 8 + g;
                float x[2];
                if (B_MN) { x[0] = sb[(kk + t) * (BN + 8) + c]; x[1] = sb[(kk + t + 4) * (BN + 8) + c]; }
                else      { x[0] = sb[c * LD_K + kk + t];       x[1] = sb[c * LD_K + kk + t + 4]; }
                split_tf32(x[0], bh[ni][0], bl[ni][0]);
                split_tf32(x[1], bh[ni][1], bl[ni][1]);
            }
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < NI; ++ni) {
                    mma_tf32(acc[mi][ni], al[mi], bh[ni]);      /* small terms first */
                    mma_tf32(acc[mi][ni], ah[mi], bl[ni]);
                    mma_tf32(acc[mi][ni], ah[mi], bh[ni]);
                }
        }
    }
    rpb_dmma::cp_async_wait<0>();

    const bool to_partial = p.splits > 1;
    float* P = to_partial ? reinterpret_cast<float*>(p.partial) + ((long long)split * p.batch + bz) * p.m * (long long)p.n
                          : nullptr;
    float* Cout = reinterpret_cast<float*>(p.c) + bz * p.c_batch;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = row0 + wm + mi * 16 + g + h * 8;
                const int c = col0 + wn + ni * 8 + 2 * t;
                if (r >= p.m) continue;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (c + e >= p.n) continue;
                    float v = acc[mi][ni][2 * h + e];
                    if (to_partial) P[(long long)r * p.n + c + e] = v;
                    else {
                        float* dst = Cout + (long long)r * p.c_row + c + e;
                        if (p.bias) v += reinterpret_cast<const float*>(p.bias)[c + e];
                        if (p.accumulate) v += *dst;
                        *dst = v;
                    }
                }
            }
}

}  // namespace rpb_tf32
#endif
