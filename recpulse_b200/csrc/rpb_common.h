/* Internal definitions shared by the CUDA translation units of librecpulse_b200. */
#ifndef RPB_COMMON_H
#define RPB_COMMON_H

#include <stdint.h>
#include "../../include/recpulse_b200.h"

#define RPB_VERSION "recpulse_b200 0.1 (sm_100a)"

/* Fully resolved GEMM problem handed to a kernel launcher.  Strides in elements. */
struct RpbProblem {
    int m, n, k;
    int batch, reduce;
    long long a_row, a_col, a_batch, a_reduce;
    long long b_row, b_col, b_batch, b_reduce;
    long long c_row, c_batch;
    int accumulate;
    int dtype;                 /* DType code */
    const void* bias;          /* n values of dtype, or NULL */
    int max_sms;               /* 0 = all */
    int act;                   /* RpbGemm.epilogue: 0 none, 1 LSTM gate non-linearities by column quarter */
    int c_f32;                 /* RpbGemm.c_float32: C is packed float32 although the operands are 16-bit */
};

#ifdef __CUDACC__
/* Programmatic dependent launch: a kernel launched with the programmatic-serialisation attribute may start
 * while its predecessor in the stream is still running.  Every kernel of this library calls rpb_pdl_wait()
 * before its first access to global memory (it returns once the predecessor has completed and its writes
 * are visible) and rpb_pdl_trigger() as early as possible, so that the successor's launch latency and
 * prologue overlap this kernel's tail.  Both are no-ops for kernels launched the ordinary way. */
__device__ __forceinline__ void rpb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rpb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

/* Epilogue non-linearity of the LSTM gate block: columns [2q, 3q) of the n = 4q outputs go through tanh, the
 * others through the logistic function, as sigmoid_kernel / tanh_kernel of the reference compute them
 * (functional/functional_device.cu:524-550).  Applied to the finished sum (bias and C included) before rounding. */
__device__ __forceinline__ float rpb_gate_act(float v, int col, int quarter) {
    return (col >= 2 * quarter && col < 3 * quarter) ? tanhf(v) : 1.0f / (1.0f + expf(-v));
}
__device__ __forceinline__ double rpb_gate_act(double v, int col, int quarter) {
    return (col >= 2 * quarter && col < 3 * quarter) ? tanh(v) : 1.0 / (1.0 + exp(-v));
}

#include <cstdlib>
#include <utility>
#include <cuda_runtime.h>
/* Every kernel launch of the library goes through here: optional programmatic dependent launch (RPB_PDL=1)
 * and, for the two-CTA kernels, a cluster dimension.  Programmatic launch is off by default: measured on the
 * launch-bound workloads it did not shorten a step replayed from a CUDA graph (128x784x256 fp32 fwd+bwd:
 * 35 us without, 45 us with; fp16 broadcast-batched: 47 vs 48 us), because the persistent GEMM kernels leave
 * no SM for a successor to set up on until their CTAs exit. */
inline bool rpb_pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("RPB_PDL"); v = e ? (atoi(e) != 0) : 0; }
    return v != 0;
}
template <typename... KArgs, typename... Args>
inline cudaError_t rpb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (rpb_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr; cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
#endif

static inline size_t rpb_dtype_size(int dtype) {
    switch (dtype) {
        case DTYPE_FLOAT32: return 4;
        case DTYPE_FLOAT64: return 8;
        case DTYPE_FLOAT16: return 2;
        case DTYPE_BFLOAT16: return 2;
        default: return 0;
    }
}

#endif
