/*
 * LSTM gate non-linearities on a [rows, 4H] matrix of gate pre-activations, in place, and their
 * derivative.  Column quarters are the i, f, g, o gates in that order (recpulse/module.py:296-300):
 * sigmoid on i, f, o and tanh on g, as sigmoid_kernel / tanh_kernel compute them
 * (functional/functional_device.cu:524-550: 1 / (1 + exp(-x)) in float for the 16-bit types).
 * One thread per element: the matrices of one cell step are a few hundred KB and the pass is launch-bound.
 */
#ifndef RPB_GATE_ACT_CUH
#define RPB_GATE_ACT_CUH

#include "gemm_simt.cuh"

namespace rpb_gate {

template <typename Acc> __device__ __forceinline__ Acc sigmoid(Acc x);
template <> __device__ __forceinline__ float sigmoid<float>(float x) { return 1.0f / (1.0f + expf(-x)); }
template <> __device__ __forceinline__ double sigmoid<double>(double x) { return 1.0 / (1.0 + exp(-x)); }
template <typename Acc> __device__ __forceinline__ Acc tanh_(Acc x);
template <> __device__ __forceinline__ float tanh_<float>(float x) { return tanhf(x); }
template <> __device__ __forceinline__ double tanh_<double>(double x) { return tanh(x); }

/* y[r, c] = act_c(y[r, c]), act = tanh for c in [2H, 3H), sigmoid elsewhere; n = 4H */
template <typename T, typename Acc>
__global__ void __launch_bounds__(256)
forward_kernel(T* y, long long rows, int n, long long ld)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int quarter = n / 4;
    const long long total = rows * n, stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        T* p = y + r * ld + c;
        const Acc v = rpb_simt::widen<Acc, T>(*p);
        const bool g = c >= 2 * quarter && c < 3 * quarter;
        *p = rpb_simt::narrow<T, Acc>(g ? tanh_<Acc>(v) : sigmoid<Acc>(v));
    }
}

/* dpre[r, c] = dy[r, c] * act_c'(pre) expressed through the activated value y:
 * g * (1 - y * y) for tanh, g * y * (1 - y) for sigmoid (backwards_tanh_host / backwards_sigmoid_host,
 * ops/grad_host.c:365-385, 622-640) */
template <typename T, typename Acc>
__global__ void __launch_bounds__(256)
backward_kernel(T* dpre, const T* dy, const T* y, long long rows, int n, long long ld_dpre, long long ld_dy, long long ld_y)
{
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const int quarter = n / 4;
    const long long total = rows * n, stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / n;
        const int c = (int)(i - r * n);
        const Acc g = rpb_simt::widen<Acc, T>(dy[r * ld_dy + c]);
        const Acc v = rpb_simt::widen<Acc, T>(y[r * ld_y + c]);
        const bool th = c >= 2 * quarter && c < 3 * quarter;
        const Acc d = th ? g * (Acc(1) - v * v) : (g * v) * (Acc(1) - v);
        dpre[r * ld_dpre + c] = rpb_simt::narrow<T, Acc>(d);
    }
}

}  // namespace rpb_gate
#endif
