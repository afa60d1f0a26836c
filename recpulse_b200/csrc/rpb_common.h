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
};

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
