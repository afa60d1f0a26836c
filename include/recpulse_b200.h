/*
 * recpulse_b200 -- Blackwell (sm_100a) dense-matmul path for RecPulse.
 *
 * C ABI of librecpulse_b200.so.  The first four entry points carry the exact
 * names and signatures of the RecPulse symbols they replace, so the library can
 * be linked in place of those functions or loaded in front of an unmodified
 * recpulse_cuda.so (symbol interposition).  Everything else is additive.
 *
 * Conventions kept from RecPulse: row-major, strides in ELEMENTS, `data`
 * already offset for views, int 0 / -1 and NULL for errors with a diagnostic
 * on stderr, results complete (stream synchronised) when an entry point that
 * has no stream argument returns.
 *
 * Device tensors only.  There is no CPU implementation in this library: a call
 * with device_id == -1 is forwarded to a loaded recpulse_cuda.so when there is
 * one (its own host code, untouched) and fails with -1 / NULL otherwise.
 */
#ifndef RECPULSE_B200_H
#define RECPULSE_B200_H

#include <stdbool.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- types shared with RecPulse (layout-identical) ------------------------
 * A translation unit that also needs RecPulse's own headers includes them FIRST
 * (their include guards are TENSOR_H and OPS_H); their definitions are then used
 * instead of the copies below. */
#ifndef TENSOR_H
typedef enum {                      /* core/tensor.h:7-13 */
    DTYPE_FLOAT32 = 0,
    DTYPE_FLOAT64 = 1,
    DTYPE_FLOAT16 = 2,
    DTYPE_BFLOAT16 = 3,
    DTYPE_PRESERVE = -1,
} DType;

typedef struct Tensor Tensor;
typedef struct GradFn GradFn;

typedef struct {                    /* core/tensor.h:18-24 */
    bool is_leaf;
    bool requires_grad;
    bool is_frozen;
    GradFn* grad_fn;
    Tensor* grad;
} Meta;

struct Tensor {                     /* core/tensor.h:27-42 */
    DType dtype;
    void* data;
    int ndim;
    size_t size;
    int* shape;
    int* strides;                   /* in elements */
    int device_id;                  /* -1 = host */
    bool owns_data;
    int refcount;
    Tensor* base_tensor;
    size_t data_offset;
    Meta* metadata;
};
#endif /* TENSOR_H */

#ifndef OPS_H
typedef void (*BackwardFunction)(GradFn* self, Tensor* grad_output);   /* ops/ops.h:12 */
struct GradFn {                     /* ops/ops.h:14-20 */
    BackwardFunction backward;
    Tensor** inputs;
    int num_inputs;
    void* saved_data;
    Tensor* owner;
};
#endif /* OPS_H */

/* ---- drop-in entry points --------------------------------------------------*/

/* Replaces matmul_kernel_device (functional/functional.h:426,
 * functional/functional_device.cu:991-1071): C[m,n] = A[m,k] . B[k,n], packed
 * row-major device pointers on the CURRENT device, legacy default stream,
 * synchronised before return.  0 on success, -1 on error. */
int matmul_kernel_device(void* C, const void* A, const void* B, int m, int k, int n, DType dtype);

/* Replaces rp_matmul (functional/functional.h:220, functional/functional.c:978-1006):
 * argument checks, cudaSetDevice(device_id) (not restored, as in RecPulse), then
 * matmul_kernel_device. */
int rp_matmul(void* C, const void* A, const void* B, int m, int k, int n, DType dtype, int device_id);

/* Replaces op_matmul (ops/ops.h:85, ops/ops.c:6816-6884).  Same checks (NULL,
 * inner dimension, dtype, device) and same autograd bookkeeping (Meta/GradFn
 * allocated with calloc/malloc, inputs retained, owner set).  Differences, all
 * additive: strided / transposed 2-D views are read in place (no contiguous
 * copy), and operands with ndim > 2 are accepted as batched matrices whose
 * leading dimensions broadcast NumPy-style.  The result is a new contiguous
 * tensor, refcount 1, owns_data.  Its data comes from the device's default stream-ordered memory
 * pool (cudaMallocAsync), which RecPulse's free_tensor may release with plain cudaFree; the
 * library raises that pool's release threshold so that freed blocks are reused instead of returned
 * to the driver -- a process-wide setting.  RPB_POOL=0 in the environment keeps the pool untouched
 * and allocates with cudaMalloc exactly like zeros_device_tensor (core/tensor_device.cu:44-46). */
Tensor* op_matmul(Tensor* a, Tensor* b);

/* Replaces backward_matmul_fn (ops/ops.c:6759-6814): dA = dC . B^T and
 * dB = A^T . dC for the inputs that require grad, reading A and B through their
 * strides.  A missing grad is assigned; an existing one is accumulated inside
 * the GEMM epilogue (no temporary, no separate add).  Gradients of broadcast
 * batch dimensions are summed over those dimensions.  On failure grads are left
 * untouched (the function is void, as in RecPulse). */
void backward_matmul_fn(GradFn* self, Tensor* grad_output);

/* ---- additive: Linear as one node ------------------------------------------*/

/* y = x . w + bias with the bias added in the GEMM epilogue (one rounding), as ONE autograd node.
 * RecPulse's Linear.forward (recpulse/module.py:110-114) is op_matmul followed by a broadcast op_add
 * (ops/ops.c:129-210) whose backward reduces dY on the host (reduce_grad_to_shape,
 * ops/ops.c:6970-7101).  Here the backward computes dX and dW as op_matmul's does and
 * dbias = column sums of dY on the device.  x: [..., k]; w: [k, n] (or batched like op_matmul);
 * bias: n elements (shape [n] or [1, ..., n]), same dtype and device.  bias may be NULL (= op_matmul). */
Tensor* op_linear(Tensor* x, Tensor* w, Tensor* bias);
void backward_linear_fn(GradFn* self, Tensor* grad_output);

/* y = x . w + h . u (+ bias) as ONE node: the gate pre-activations of an LSTM cell, which RecPulse
 * builds from two op_matmul nodes and an op_add (recpulse/module.py:289).  (A GRU cell keeps the two products
 * apart -- its candidate gate needs h . u on its own -- and has its own node, op_gru_cell.)  The second
 * product is accumulated into the output inside the GEMM epilogue.  Shapes as for op_linear, both products must have
 * the same result shape; bias may be NULL.  Backward gives all four matmul gradients and the bias gradient. */
Tensor* op_linear2(Tensor* x, Tensor* w, Tensor* h, Tensor* u, Tensor* bias);
void backward_linear2_fn(GradFn* self, Tensor* grad_output);

/* The activated gates of an LSTM cell as ONE node: y = act(x . w + h . u (+ bias)) with n = 4 * hidden
 * columns in the order i, f, g, o; sigmoid on i, f, o and tanh on g.  RecPulse builds this from two op_matmul,
 * up to three op_add, a chunk and four activation nodes (recpulse/module.py:289-300).  Backward turns dY into
 * the gradient of the pre-activations through the saved output (g y (1 - y), g (1 - y^2): ops/grad_host.c:365-385,
 * 622-640) and continues as backward_linear2_fn.  Operands as for op_linear2; n must be a multiple of 4. */
Tensor* op_lstm_gates(Tensor* x, Tensor* w, Tensor* h, Tensor* u, Tensor* bias);
void backward_lstm_gates_fn(GradFn* self, Tensor* grad_output);

/* The two element-wise passes of op_lstm_gates on raw device pointers, on `stream`, without synchronising:
 * in place y[r, c] = c in [n/2, 3n/4) ? tanh(y[r, c]) : 1 / (1 + exp(-y[r, c])), and
 * dpre[r, c] = dy[r, c] * act'(.) from the activated y.  Strides in elements between rows.  0 / -1. */
int rp_lstm_gates_ex(void* y, long long rows, int n, long long row_stride, DType dtype, int device_id, void* stream);
int rp_lstm_gates_grad_ex(void* dpre, const void* dy, const void* y, long long rows, int n, long long dpre_stride,
                          long long dy_stride, long long y_stride, DType dtype, int device_id, void* stream);

/* out[j] (+)= sum over i < rows of in[i * row_stride + j], j < cols; fp32 (fp64 for float64) sums in a
 * fixed order, one rounding.  Runs on `stream` without synchronising. */
int rp_colsum_ex(void* out, const void* in, long long rows, int cols, long long row_stride, DType dtype,
                 int accumulate, int device_id, void* stream);

/* A whole GRU cell step as ONE node: h' = (1 - z) n + z h with r = sigmoid(gi_r + gh_r), z = sigmoid(gi_z + gh_z),
 * n = tanh(gi_n + r gh_n), gi = x . w_ih (+ b_ih), gh = h . w_hh (+ b_hh); 3 * hidden columns in the order r, z, n.
 * RecPulse's GRUCell.forward (recpulse/module.py:329-348) keeps gi and gh apart (the candidate gate needs gh_n on its
 * own) and builds the step from two op_matmul, two op_add, two chunk and eleven element-wise nodes.  Here: two GEMMs
 * with the bias in their epilogues and one element-wise pass forward; one element-wise pass, four GEMMs and two
 * column sums backward, to all six leaves.  x: [m, k], w_ih: [k, 3 hidden], h: [m, hidden], w_hh: [hidden, 3 hidden],
 * b_ih / b_hh: 3 hidden elements or NULL.  The node keeps the activated gates and gh as two extra inputs without
 * gradient, which RecPulse's free_grad_fn releases like any retained input. */
Tensor* op_gru_cell(Tensor* x, Tensor* w_ih, Tensor* h, Tensor* w_hh, Tensor* b_ih, Tensor* b_hh);
void backward_gru_cell_fn(GradFn* self, Tensor* grad_output);

/* The two element-wise passes of op_gru_cell on raw device pointers, on `stream`, without synchronising.
 * gi, gh, dgi, dgh: packed [rows, 3 hidden]; h_next, g, dh: packed [rows, hidden]; h: row stride h_stride.
 * rp_gru_gates_ex overwrites gi with the activated (r, z, n).  rp_gru_gates_grad_ex writes the gradients of gi and
 * gh and, when dh is not NULL, the direct part g z of dL/dh (added to dh when dh_accumulate).  0 / -1. */
int rp_gru_gates_ex(void* h_next, void* gi, const void* gh, const void* h, long long rows, int hidden, long long h_stride,
                    DType dtype, int device_id, void* stream);
int rp_gru_gates_grad_ex(void* dgi, void* dgh, void* dh, int dh_accumulate, const void* g, const void* gi_act, const void* gh,
                         const void* h, long long rows, int hidden, long long h_stride, DType dtype, int device_id, void* stream);

/* ---- additive: conv2d on the GEMM path ---------------------------------------
 * RecPulse's conv2d loops over the images: im2col + rp_matmul per image forward (ops/ops.c:4761-4770), and in the
 * backward a materialised W^T, a materialised col^T per image and an rp_add per image (ops/ops.c:4536-4550,
 * 4575-4617), each step followed by a device synchronisation.  These entry points do the same arithmetic for ALL
 * images at once: one im2col pass into a resident [N, C_in kH kW, out_H out_W] buffer, then single GEMM launches --
 * the weight as a broadcast batch operand, transposes as stride swaps, the weight gradient as one summed problem
 * over the images (fp32 sums, one rounding, optionally added to an existing gradient in the same epilogue) -- and
 * one col2im pass that gathers in a fixed order (the reference scatters with atomicAdd).  Layouts are RecPulse's:
 * input [N, C_in, H, W], weight [C_out, C_in, kH, kW], output [N, C_out, out_H, out_W], all packed; bias is the
 * caller's.  Asynchronous on `stream`. */
typedef struct {
    int N, C_in, H, W, C_out, kH, kW;
    int stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w;
} RpbConv2d;
/* out_H / out_W of the convolution (ops/ops.c:4739-4740); -1 for an invalid geometry. */
int rp_conv2d_out_shape(const RpbConv2d* c, int* out_h, int* out_w);
/* Elements of the im2col buffer of all images (N * C_in kH kW * out_H out_W); -1 for an invalid geometry. */
long long rp_conv2d_col_elems(const RpbConv2d* c);
/* col_all = im2col(input) for every image (kept by the caller for the backward), out[img] = weight . col_all[img]. */
int rp_conv2d_forward_ex(void* out, const void* input, const void* weight, void* col_all, const RpbConv2d* c, DType dtype,
                         int device_id, void* stream);
/* grad_weight (+)= sum over images of grad_out[img] . col_all[img]^T (when grad_weight is not NULL), and
 * grad_input (+)= col2im(weight^T . grad_out[img]) (when grad_input is not NULL; dcol_ws is a workspace of
 * rp_conv2d_col_elems elements). */
int rp_conv2d_backward_ex(void* grad_input, int accumulate_input, void* grad_weight, int accumulate_weight, const void* grad_out,
                          const void* weight, const void* col_all, void* dcol_ws, const RpbConv2d* c, DType dtype, int device_id,
                          void* stream);

/* ---- additive: strided / batched GEMM on raw pointers ----------------------*/

typedef struct {
    int m, n, k;                    /* C[m,n] (+)= sum over k of A[m,k] * B[k,n]              */
    int batch;                      /* independent problems (>= 1)                           */
    int reduce;                     /* problems SUMMED into one C (>= 1); used for grads of  */
                                    /* broadcast operands: C = sum_r A_r . B_r               */
    long long a_row, a_col;         /* element strides of A[i,l]                             */
    long long a_batch, a_reduce;    /* element strides between batches / summed problems     */
    long long b_row, b_col;         /* element strides of B[l,j]                             */
    long long b_batch, b_reduce;
    long long c_row;                /* row stride of C; its column stride is 1               */
    long long c_batch;
    int accumulate;                 /* 0: C = AB ; 1: C = C + AB (one rounding of the sum)   */
    const void* bias;               /* NULL, or n values of the GEMM's dtype added to every  */
                                    /* row of every batch before the rounding (device memory)*/
    int max_sms;                    /* 0 = use every SM; otherwise the persistent tensor-core */
                                    /* kernels occupy at most this many SMs, leaving the rest */
                                    /* to work that runs beside the GEMM (a collective)       */
    int epilogue;                   /* 0: none; 1 (RPB_EPILOGUE_LSTM_GATES): after bias and "+= C", columns   */
                                    /* [n/2, 3n/4) go through tanh and the others through 1 / (1 + exp(-x))    */
                                    /* before the one rounding; n must be a multiple of 4                      */
    int c_float32;                  /* 1: float16 / bfloat16 operands, but C receives the UNROUNDED float32 sums */
                                    /* (packed [batch][m][n], c_row == n; no bias or epilogue; `accumulate`      */
                                    /* keeps a float32 running sum): partial gradients that are summed over row  */
                                    /* chunks or across GPUs before their one rounding                          */
} RpbGemm;
#define RPB_EPILOGUE_LSTM_GATES 1

/* Fills `g` for a packed row-major m x k times k x n product (batch = reduce = 1). */
void rpb_gemm_packed(RpbGemm* g, int m, int k, int n);

/* No RecPulse counterpart (RecPulse can only multiply packed matrices,
 * functional/functional.h:220).  Runs on `stream` (a cudaStream_t; NULL = legacy
 * default stream) of device `device_id` WITHOUT synchronising.  Any stride may be
 * zero (broadcast) except C's.  0 on success, -1 on error. */
int rp_matmul_ex(void* C, const void* A, const void* B, const RpbGemm* g, DType dtype,
                 int device_id, void* stream);

/* Same through HOST buffers: allocates device memory, copies A and B up,
 * multiplies, copies C down (packed operands).  Exists so a host-only caller and the
 * end-to-end benchmark can exercise the full path; -1 on error. */
int rp_matmul_host(void* C, const void* A, const void* B, int m, int k, int n, DType dtype,
                   int device_id);

/* Forward + backward of one matmul whose six matrices live in HOST memory (packed row-major):
 * C = A.B, dA = dC.B^T, dB = A^T.dC.  Any of C, dA, dB may be NULL (not wanted); dC is needed for dA / dB.
 * RecPulse copies whole tensors synchronously before it multiplies (tensor_copy_device,
 * core/tensor_device.cu:295-372); this call streams row chunks of A and dC so that the host-to-device
 * copies, the GEMMs and the device-to-host copies of the results overlap on three streams.  Pinned host
 * memory is needed for the overlap (pageable memory works, slower).  chunk_rows = 0 picks a chunk size.
 * Synchronous: results are in the host buffers on return.  Device buffers are cached per device;
 * rpb_release_host_pipeline frees them.  0 on success, -1 on error. */
int rp_matmul_fwdbwd_host(void* C, void* dA, void* dB, const void* A, const void* B, const void* dC,
                          int m, int k, int n, DType dtype, int device_id, int chunk_rows);
int rpb_release_host_pipeline(int device_id);

/* No counterpart in RecPulse.  C[m,n] = A[m,k] . B[k,n] for packed row-major float16 / bfloat16
 * operands, for callers that cannot let a library allocate: processes that have given all device
 * memory to their own pool (a hidden cudaMalloc would fail or fragment it) and latency-critical
 * sections where cudaMalloc / cudaFree, which stall the device, are off limits.  It is the K-split
 * tcgen05 GEMM with its partial tiles kept in a fixed 16 MiB array inside the library image instead
 * of an allocated buffer; it calls no cudaMalloc, cudaFree or other allocating routine.
 *   - Limit: (number of K splits) x m x n x 4 bytes must fit in 16 MiB, else -1 with a message
 *     (roughly m x n <= 2M elements for short K, less for long K).  Pointers 16-byte aligned, k and n
 *     multiples of 8.  Every GPU that loads the library holds the 16 MiB until the process exits.
 *   - The first call on a device looks up the device addresses of the built-in buffers; make that
 *     first call before starting any stream capture on that device.  Under CUDA's lazy module loading
 *     that first call (per device, and the first use of each dtype / tile width) is also what loads
 *     the kernel image and reserves the 16 MiB array, so it can itself fail for lack of memory if the
 *     caller's pool already holds the whole device: make it BEFORE handing memory to the pool.  Later
 *     calls leave the device's free memory untouched.
 *   - All calls on a device share the one array: two calls that overlap on the GPU (different
 *     streams, or different threads) race on it.  Serialise them.
 *   - Runs on `stream` (NULL = legacy default stream).  With kernel_status == NULL it returns once the
 *     work is queued.  With a pointer it waits for the result and stores the kernel's status word
 *     (0 = ok; non-zero = a bounded wait inside the kernel ran out, result invalid, return -1).  The
 *     word is cleared at the start of every call, so kernel_status is the only way to learn of such
 *     a failure: a caller that passes NULL and queues another call loses it. */
int rp_matmul_noalloc(void* C, const void* A, const void* B, int m, int k, int n, DType dtype,
                      int device_id, void* stream, int* kernel_status);

/* ---- additive: the path sharded over the GPUs of one box ---------------------
 * RecPulse's multi-GPU primitive is the whole-tensor peer copy tensor_copy_device
 * (core/tensor_device.cu:295-372, cudaDeviceEnablePeerAccess + cudaMemcpyPeer, reached from
 * tensor_to, core/tensor.c:82-144).  These entry points are what that layer needs for the matmul
 * path: rows of A (the batch of a batched product, folded into the rows) are split over the ranks,
 * B is replicated once into every GPU's own memory, forward and dA need no communication and the
 * dB partials are reduced over NVLink (NCCL) while the dA GEMM runs.  One RpbShard per rank; a rank
 * is a process or a thread that owns one GPU.  NCCL is located at run time (the process's own
 * libnccl.so.2, else the system's; RPB_NCCL_LIB overrides).  All calls are asynchronous on `stream`
 * unless stated otherwise; collectives must be issued by every rank in the same order. */
typedef struct RpbShard RpbShard;
#define RPB_SHARD_ID_BYTES 128
#define RPB_SHARD_SLICE_ONLY 1      /* backward flag: leave dB reduce-scattered (no all-gather) */

/* Rank 0 makes the 128-byte rendezvous id and hands it to the other ranks by any means (a file, a
 * pipe, MPI, a torch.distributed store ...). */
int rpb_shard_unique_id(void* id_out);
/* Joins the communicator of `world` ranks (collective: returns once every rank has called it).
 * world == 1 needs no id and no NCCL.  NULL on error. */
RpbShard* rpb_shard_create(const void* unique_id, int rank, int world, int device_id);
void rpb_shard_destroy(RpbShard* shard);
int rpb_shard_rank(const RpbShard* shard);
int rpb_shard_world(const RpbShard* shard);
/* comm_sms: SMs the dA GEMM leaves free while the dB reduction is in flight (the GEMM kernels are
 * persistent and would otherwise keep the collective's thread blocks waiting).  -1 (default): 16, or 32
 * when the exchange is expected to outlast the GEMM (few rows per rank); 0: none.
 * db_wire: 0 (default) = the float16 / bfloat16 dB partials cross NVLink as float32 sums and are
 * rounded once after the reduction; 1 = all-reduce in the operand type (half the bytes, one extra
 * rounding per reduction step). */
int rpb_shard_configure(RpbShard* shard, int comm_sms, int db_wire);
/* [begin, end) of the rows rank `rank` owns: an even split, the remainder to the first ranks. */
void rpb_shard_rows(long long rows, int world, int rank, long long* begin, long long* end);
/* Which elements [begin, end) of the k x n gradient dB rank `rank` holds after
 * rp_matmul_rowsharded_backward(..., flags, ...): its slice when RPB_SHARD_SLICE_ONLY applies (see there),
 * else everything.  Pure arithmetic.  0 / -1. */
int rpb_shard_db_slice_of(int k, int n, DType dtype, int world, int rank, int db_wire, int flags, long long* begin,
                          long long* end);
/* Collectives issued by this library since load (all shards of the process). */
unsigned long long rpb_shard_collective_count(void);

/* Replicates `bytes` bytes at `buf` from rank `root` into every rank's own buffer (ncclBroadcast):
 * the once-per-weight copy of B that tensor_copy_device does with cudaMemcpyPeer. */
int rp_shard_replicate(RpbShard* shard, void* buf, size_t bytes, int root, void* stream);
/* C_rows[rows, n] = A_rows[rows, k] . B[k, n] on this rank's rows; no communication. */
int rp_matmul_rowsharded_forward(RpbShard* shard, void* C_rows, const void* A_rows, const void* B, long long rows,
                                 int k, int n, DType dtype, void* stream);
/* dB[k, n] = sum over ranks of A_rows^T . dC_rows, then dA_rows[rows, k] = dC_rows . B^T.  The
 * partial dB GEMM is issued first and its reduction overlaps the dA GEMM; both are complete in
 * `stream` order when the call's work is.  Either of dA_rows / dB may be NULL (all ranks alike).
 * float16 / bfloat16: partial sums are reduced in float32 and rounded once, so dB has the same
 * single rounding as on one GPU.  With RPB_SHARD_SLICE_ONLY, and k * n divisible by the ranks
 * (in 16-byte units, dB of at least 1 MiB in float32), only this rank's k * n / world elements of
 * dB are written. */
int rp_matmul_rowsharded_backward(RpbShard* shard, void* dA_rows, void* dB, const void* A_rows, const void* B,
                                  const void* dC_rows, long long rows, int k, int n, DType dtype, int flags, void* stream);
/* All-gathers C for callers that need the whole output on every GPU: C_full[world * rows, n] from
 * every rank's C_rows[rows, n] (the same `rows` on every rank). */
int rp_matmul_gather_rows(RpbShard* shard, void* C_full, const void* C_rows, long long rows, int n, DType dtype,
                          void* stream);
/* rp_matmul_fwdbwd_host for this rank's rows of a sharded product, from HOST buffers, synchronous.
 * B is read from rank 0's host buffer only (one upload per box, then NVLink; other ranks may pass
 * NULL), A_rows / dC_rows stream in chunks as in rp_matmul_fwdbwd_host, dB is reduced on the devices
 * and each rank copies back only its slice: elements [*db_begin, *db_end) of the k x n matrix, at
 * that offset of `dB` (the whole matrix when it cannot be sliced evenly). */
int rp_matmul_rowsharded_fwdbwd_host(RpbShard* shard, void* C_rows, void* dA_rows, void* dB, const void* A_rows,
                                     const void* B, const void* dC_rows, long long rows, int k, int n, DType dtype,
                                     int chunk_rows, long long* db_begin, long long* db_end);

/* ---- additive: stream-ordered execution of the nodes -------------------------
 * RecPulse ends every device op with a device synchronisation (core/cuda_helpers.cu:14-26).  By
 * default the node entry points above (op_matmul ... backward_*_fn) keep that contract on the legacy
 * default stream.  rpb_node_stream changes it for the CALLING THREAD: the nodes then run on `stream`,
 * take outputs and gradients from the memory pool in that stream's order, release temporaries in
 * stream order, and with synchronise == 0 return as soon as their work is queued.  With stream == NULL
 * and synchronise == 0 everything stays ordered with RecPulse's own (legacy-stream) kernels and the
 * host simply stops waiting after every matmul.  rpb_node_synchronize waits for the thread's node
 * stream and reports a kernel that gave up (0 / -1).  rpb_node_stream(NULL, 1) restores the default. */
void rpb_node_stream(void* stream, int synchronise);
int rpb_node_synchronize(int device_id);

/* ---- additive: diagnostics and tuning --------------------------------------*/

enum {                              /* values of rpb_last_kernel()                           */
    RPB_KERNEL_NONE = 0,
    RPB_KERNEL_SIMT = 1,            /* FFMA / DFMA tiled kernel                              */
    RPB_KERNEL_UMMA = 2,            /* tcgen05 + TMEM + TMA kernel (f16 / bf16)              */
    RPB_KERNEL_UMMA_SPLITK = 3,     /* the same with K split over CTAs + reduction pass      */
    RPB_KERNEL_DMMA = 4,            /* float64 tensor-core kernel (mma.sync m16n8k8 f64)     */
    RPB_KERNEL_TF32X3 = 5           /* float32 on tensor cores, 3xTF32 split (mma.sync tf32) */
};
/* Which kernel family the last GEMM issued by the calling thread used. */
int rpb_last_kernel(void);
/* The tile plan the tcgen05 kernel would use for an m x n output over k (per summed problem; `reduce` of them)
 * on `sms` SMs: rows of B per CTA (64 / 128 / 256), K slices (1 = none) and whether two CTAs share a tile
 * (*cta_pair: 0 one CTA per 128-row tile, 1 a pair per 256 x 2*rows_of_b tile, 2 a pair per double-width tile of
 * 256 x 512 with two accumulators).
 * Pure host arithmetic (a cost model in microseconds per K block fitted to measurements): needs no GPU.
 * dtype: DTYPE_FLOAT32 plans the 3xTF32 kernel, the 16-bit types the f16 / bf16 one.  0 / -1. */
int rpb_umma_plan(int m, int n, int k, int reduce, int batch, DType dtype, int sms, int* rows_of_b, int* k_slices,
                  int* cta_pair);
/* Number of kernel launches issued by this library since load (all threads). */
unsigned long long rpb_launch_count(void);
/* 0 = choose automatically, RPB_KERNEL_SIMT / RPB_KERNEL_UMMA = force that family where it
 * applies.  Also settable with the environment variable RPB_FORCE_KERNEL=simt|umma. */
void rpb_force_kernel(int family);
/* Device-side status word of the last tcgen05 launch on `device_id`: 0 = ok, otherwise a
 * bounded wait inside the kernel ran out (the kernel returned early; results invalid).
 * Synchronises the device. */
int rpb_device_status(int device_id);
/* Bound of each wait on a barrier inside the tcgen05 kernels (default about 2 s of SM clock; also
 * RPB_WAIT_LIMIT_MS).  ms <= 0 restores the default. */
void rpb_set_wait_limit_ms(int ms);
/* Exercises that bound by itself: one small kernel waits, with `limit_cycles` (at most 2e8), on a barrier
 * nobody signals; the wait gives up, status code 9 is recorded and the kernel returns normally.  0 when the
 * kernel completed; rpb_device_status() then reports 9 once and 0 afterwards. */
int rpb_selftest_bounded_wait(int device_id, long long limit_cycles);
/* Where a tcgen05 launch's time goes: with tracing on, the first and the last CTA of every such launch stamp the GPU's
 * nanosecond timer at their milestones -- [0] entry, [1] set-up done, [2] first TMA copy issued, [3] first stage
 * landed, [4] last MMA committed, [6] last store drained, [5] teardown, and from [8] four stamps per work item (MMA
 * start, MMA committed, epilogue start, epilogue end) -- into two rows of 64 slots.  rpb_trace_read copies up to
 * `count` stamps out (synchronise first) and clears them; it returns how many, or -1 when tracing is off. */
int rpb_trace_enable(int on);
int rpb_trace_read(unsigned long long* out, int count);
/* Library version string. */
const char* rpb_version(void);
/* The per-device scratch buffer (K-slice partial sums, column-sum partials) grows on demand, which frees
 * and reallocates it.  A CUDA graph captured while the buffer was in use holds its address, so after such
 * a capture the buffer can no longer grow: a call that needs more fails with -1.  rpb_scratch_reserve sizes
 * it up front (call before capturing); rpb_scratch_reset frees it and lifts the pin once every graph that
 * used it has been destroyed.  Eager calls and graph replays that use the scratch on one device must not
 * overlap in time.  Both synchronise the device. */
int rpb_scratch_reserve(int device_id, size_t bytes);
int rpb_scratch_reset(int device_id);
/* cudaMemGetInfo of `device_id` (diagnostics: lets a caller check that a call allocated nothing). */
int rpb_mem_info(int device_id, size_t* free_bytes, size_t* total_bytes);

/* ---- additive: minimal tensor helpers for C callers without RecPulse --------
 * They follow RecPulse's allocation conventions (struct, shape, strides and Meta from
 * malloc/calloc, device data releasable with cudaFree: from the stream-ordered pool, or from
 * cudaMalloc with RPB_POOL=0), so tensors made here can be released by RecPulse's free_tensor
 * and vice versa. */
Tensor* rpb_tensor_from_host(const void* host_data, DType dtype, int ndim, const int* shape,
                             int device_id, bool requires_grad);
Tensor* rpb_tensor_empty(DType dtype, int ndim, const int* shape, int device_id);
/* A view sharing `base`'s data: explicit shape/strides (elements) and element offset.  When
 * `base` requires grad the view gets its own Meta and collects its own gradient. */
Tensor* rpb_tensor_view(Tensor* base, int ndim, const int* shape, const int* strides,
                        size_t offset_elems);
/* Copies a (possibly strided) tensor to a packed host buffer of t->size elements. */
int rpb_tensor_to_host(const Tensor* t, void* host_out);
/* Overwrites a packed device tensor's values from a packed host buffer, keeping its device buffer. */
int rpb_tensor_write_host(Tensor* t, const void* host_data);
/* Releases t's accumulated gradient and clears the pointer. */
void rpb_tensor_zero_grad(Tensor* t);
/* Drops one reference; frees at zero (data, grad, grad_fn with its retained inputs, base). */
void rpb_tensor_release(Tensor* t);
/* Runs the backward function recorded on `out` with upstream gradient `grad_output`
 * and frees the node (single-use graph, as tensor_backward does, core/tensor.c:219-347).
 * Only a single matmul node is walked; RecPulse's tensor_backward remains the real driver. */
int rpb_backward_node(Tensor* out, Tensor* grad_output);

#ifdef __cplusplus
}
#endif
#endif /* RECPULSE_B200_H */
