/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of RecPulse's matmul forward and
 * autograd backward, used as the parity checker by tests/, by the smoke test
 * and as the timed CPU baseline of bench.py.  Nothing in the shipped library
 * links, loads or calls this file.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this restatement against
 * (1) the known-answer vectors of the reference's own tests, (2) fixtures in
 * tests/golden/ that were produced by the unmodified reference
 * (tests/golden/make_golden.py) and (3) the reference compiled from its own
 * sources (oracle/_ref/recpulse_cuda.so) when that file is present.
 *
 * dtype codes follow core/tensor.h:7-13 of the reference.
 */
#ifndef RECPULSE_MATMUL_ORACLE_H
#define RECPULSE_MATMUL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_F32 = 0, ORC_F64 = 1, ORC_F16 = 2, ORC_BF16 = 3 };

/* core/half_precision.h:20-48, 50-83, 85-90, 92-97 */
float    orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16(float f);
float    orc_bf16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_bf16(float f);
void     orc_widen(const void* src, float* dst, size_t n, int dtype);
void     orc_narrow(const float* src, void* dst, size_t n, int dtype);

/* functional/functional_host.c:780-806 */
int orc_matmul_f32(float* C, const float* A, const float* B, int m, int k, int n);
int orc_matmul_f64(double* C, const double* A, const double* B, int m, int k, int n);

/* functional/functional.c:978-1002, host branch */
int orc_rp_matmul(void* C, const void* A, const void* B, int m, int k, int n, int dtype);

/* functional/functional.c:1130-1220 (host gather of a strided view, rank <= 8) */
int orc_contiguous(void* dst, const void* src, int ndim, const int* shape,
                   const int* strides, int dtype);

/* ops/ops.c:6816-6884 forward on (possibly strided) 2-D operands */
int orc_op_matmul(void* C, const void* A, const int* a_strides, const void* B,
                  const int* b_strides, int m, int k, int n, int dtype);

/* ops/ops.c:6759-6814; dA and/or dB may be NULL (that input does not require grad).
 * accumulate!=0 restates the rp_add branch (:6781-6789): grad += new, rounded in
 * the storage dtype as functional_host.c's add does (fp16/bf16: widen, add, narrow). */
int orc_matmul_backward(void* dA, void* dB, const void* A, const int* a_strides,
                        const void* B, const int* b_strides, const void* dC,
                        int m, int k, int n, int dtype, int accumulate);

/* Batched / broadcast-batched matmul: not in the reference.  Defined as a loop of
 * reference 2-D matmuls over the broadcast batch index; a_bstride / b_bstride are
 * batch strides in elements (0 = broadcast operand).  Operand matrices are packed
 * row-major. */
int orc_bmm(void* C, const void* A, const void* B, int batch, size_t a_bstride,
            size_t b_bstride, int m, int k, int n, int dtype);
/* Backward of the above.  A gradient of a broadcast operand is the sum over the
 * batch of the per-batch products, accumulated without intermediate rounding
 * (fp32 for f32/f16/bf16, fp64 for f64) and rounded to the storage dtype once. */
int orc_bmm_backward(void* dA, void* dB, const void* A, const void* B, const void* dC,
                     int batch, size_t a_bstride, size_t b_bstride,
                     int m, int k, int n, int dtype);

/* Linear layer as RecPulse composes it (recpulse/module.py:110-114): Y = op_add(op_matmul(X, W), bias),
 * i.e. the product is rounded to the storage dtype, then the broadcast add (ops/ops.c:129-210; f16/bf16:
 * widen, add in fp32, narrow) rounds again.  bias has n elements. */
int orc_linear_forward(void* Y, const void* X, const void* W, const void* bias, int m, int k, int n, int dtype);
/* Bias gradient, reduce_grad_to_shape (ops/ops.c:6970-7101): dY summed over rows in row order in fp32
 * (fp64 for float64), one narrowing at the end. */
int orc_bias_grad(void* dbias, const void* dY, long long rows, int n, int dtype);

/* Activated gates of an LSTM cell as RecPulse composes them (recpulse/module.py:289-300):
 * gates = op_add(op_matmul(X, W), op_matmul(H, U)), then op_add(bias) when bias != NULL, every node's output
 * rounded to the storage dtype; columns split in four (i, f, g, o); sigmoid 1 / (1 + expf(-x)) on i, f, o and
 * tanhf on g (functional/functional_host.c:498-545; f16/bf16 widen, compute in float, narrow).
 * X: m x kx, W: kx x n, H: m x kh, U: kh x n, n a multiple of 4. */
int orc_lstm_gates_forward(void* Y, const void* X, const void* W, const void* H, const void* U, const void* bias,
                           int m, int kx, int kh, int n, int dtype);
/* Gradient of the pre-activations from the activated output: g * y * (1 - y) for the sigmoid columns,
 * g * (1 - y * y) for the tanh columns (ops/grad_host.c:365-385, 622-640), in float (double for float64). */
int orc_lstm_gates_grad(void* dpre, const void* dY, const void* Y, long long rows, int n, int dtype);

/* One GRU cell step as RecPulse's GRUCell.forward composes it (recpulse/module.py:329-348), node by node with
 * every node's output rounded to the storage dtype: gi = X.Wih (+ bih), gh = H.Whh (+ bhh), chunks (r, z, n),
 * r = sigmoid(i_r + h_r), z = sigmoid(i_z + h_z), n = tanh(i_n + r * h_n), h' = (1 - z) * n + z * h.
 * X: m x kx, Wih: kx x 3hd, H: m x hd, Whh: hd x 3hd, biases 3hd elements or NULL. */
int orc_gru_cell_forward(void* Hn, const void* X, const void* Wih, const void* H, const void* Whh, const void* bih,
                         const void* bhh, int m, int kx, int hd, int dtype);
/* Gradients of all six leaves for the upstream gradient G of h' (any output pointer may be NULL except dX / dWih /
 * dWhh, which orc_matmul_backward fills). */
int orc_gru_cell_backward(void* dX, void* dWih, void* dH, void* dWhh, void* dbih, void* dbhh, const void* G, const void* X,
                          const void* Wih, const void* H, const void* Whh, const void* bih, const void* bhh,
                          int m, int kx, int hd, int dtype);

#ifdef __cplusplus
}
#endif
#endif
