/*
 * Column sums of a row-major matrix: out[j] (+)= sum_i in[i][j].  Used for the bias gradient of a
 * Linear layer (the sum of dY over all rows), which RecPulse computes on the host after copying dY
 * back (reduce_grad_to_shape, ops/ops.c:6970-7101).
 *
 * Two passes with a fixed association, so results do not depend on scheduling: row slabs are summed
 * per block (8 row lanes per column, combined in lane order), then the slab sums are added in slab
 * order, optionally added to the existing output, and rounded once.
 */
#ifndef RPB_REDUCE_COLS_CUH
#define RPB_REDUCE_COLS_CUH

#include "gemm_simt.cuh"

namespace rpb_cols {

constexpr int COLS = 64, LANES = 4;      /* block = 64 columns x 4 row lanes */

template <typename T, typename Acc>
__global__ void __launch_bounds__(COLS * LANES)
partial_kernel(const T* __restrict__ in, Acc* __restrict__ partial, long long rows, int cols, long long ld,
               long long rows_per_block)
{
    __shared__ Acc red[LANES][COLS];
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int cx = threadIdx.x % COLS, ly = threadIdx.x / COLS;
    const int col = blockIdx.x * COLS + cx;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(rows, r0 + rows_per_block);
    Acc s = Acc(0);
    if (col < cols) {
#pragma unroll 4
        for (long long r = r0 + ly; r < r1; r += LANES) s += rpb_simt::widen<Acc, T>(in[r * ld + col]);
    }
    red[ly][cx] = s;
    __syncthreads();
    if (ly == 0 && col < cols) {
#pragma unroll
        for (int l = 1; l < LANES; ++l) s += red[l][cx];
        partial[(long long)blockIdx.y * cols + col] = s;
    }
}

template <typename T, typename Acc>
__global__ void final_kernel(const Acc* __restrict__ partial, T* out, int slabs, int cols, int accumulate)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= cols) return;
    Acc s = Acc(0);
    for (int b = 0; b < slabs; ++b) s += partial[(long long)b * cols + col];
    if (accumulate) s += rpb_simt::widen<Acc, T>(out[col]);
    out[col] = rpb_simt::narrow<T, Acc>(s);
}

}  // namespace rpb_cols
#endif
