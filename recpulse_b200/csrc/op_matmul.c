/*
 * Host side of the matmul path in C: the autograd node (op_matmul), its backward
 * (backward_matmul_fn) and the few tensor helpers a C caller needs when RecPulse
 * itself is not linked.  Works on RecPulse's Tensor / Meta / GradFn structs in place
 * and keeps RecPulse's allocation conventions (malloc/calloc for host structs,
 * cudaMalloc for device data) so either side can free what the other made.
 *
 * Unlike ops/ops.c:6816-6884 of RecPulse nothing is copied: strided and transposed
 * views go to the GEMM as strides, batched operands as batch strides, and gradient
 * accumulation happens in the GEMM epilogue.
 */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "rpb_common.h"

#define RPB_MAX_BATCH_DIMS 8

void* rpb_reference_symbol(const char* name);   /* gemm_dispatch.cu */
int rpb_take_status(int device_id);             /* gemm_dispatch.cu: kernel status word, read without a copy */
static void bias_grad_into(Tensor* bias, Tensor* grad_output);

/* ------------------------------------------------------------------ where and how the nodes run
 * RecPulse ends every device op with a device synchronisation (core/cuda_helpers.cu:14-26) and its callers
 * rely on results being complete on return; that is the default here too (legacy default stream, stream
 * synchronised before an entry point returns).  rpb_node_stream() changes it for the calling thread: the
 * nodes then launch on the given stream, take their outputs from the pool in that stream's order, give
 * temporaries back in stream order and -- with synchronise == 0 -- return as soon as the work is queued. */
static __thread cudaStream_t t_stream = NULL;
static __thread int t_sync = 1;

void rpb_node_stream(void* stream, int synchronise) {
    t_stream = (cudaStream_t)stream;
    t_sync = synchronise != 0;
}

/* end of an entry point: wait (unless told not to) and report a kernel that gave up */
static int node_finish(int device_id) {
    if (!t_sync) return 0;
    cudaError_t e = cudaStreamSynchronize(t_stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "recpulse_b200: synchronising after a node failed: %s\n", cudaGetErrorString(e));
        return -1;
    }
    return rpb_take_status(device_id) ? -1 : 0;
}

int rpb_node_synchronize(int device_id) {
    if (cudaStreamSynchronize(t_stream) != cudaSuccess) return -1;
    return rpb_take_status(device_id) ? -1 : 0;
}

/* ------------------------------------------------------------------ tensor helpers */

static void free_dims(Tensor* t) {
    free(t->shape);
    free(t->strides);
}

static Tensor* alloc_struct(DType dtype, int ndim, const int* shape, int device_id) {
    if (ndim <= 0 || !shape || !rpb_dtype_size(dtype)) return NULL;
    size_t total = 1;
    for (int d = 0; d < ndim; d++) {
        if (shape[d] <= 0) return NULL;
        if (total > ((size_t)-1) / (size_t)shape[d]) return NULL;
        total *= (size_t)shape[d];
    }
    Tensor* t = (Tensor*)calloc(1, sizeof(Tensor));
    if (!t) return NULL;
    t->shape = (int*)malloc(sizeof(int) * ndim);
    t->strides = (int*)malloc(sizeof(int) * ndim);
    if (!t->shape || !t->strides) { free_dims(t); free(t); return NULL; }
    long long s = 1;
    for (int d = ndim - 1; d >= 0; d--) { t->shape[d] = shape[d]; t->strides[d] = (int)s; s *= shape[d]; }
    t->dtype = dtype; t->ndim = ndim; t->size = total; t->device_id = device_id;
    t->owns_data = true; t->refcount = 1;
    return t;
}

/* Output and gradient buffers come from the device's stream-ordered memory pool, with the pool told to keep
 * freed memory instead of returning it to the driver: after the first training step an allocation costs a
 * microsecond or two instead of a cudaMalloc.  Whoever releases the tensor (this library or RecPulse's
 * free_tensor_device, core/tensor_device.cu:269-293) may use plain cudaFree on such memory.  Falls back to
 * cudaMalloc when the pool is unavailable.  RPB_POOL=0 forces cudaMalloc. */
static int device_alloc(void** out, size_t bytes, int device_id) {
    static int pool_state[64];          /* 0 = not set up, 1 = in use, -1 = unavailable */
    if (device_id >= 0 && device_id < 64 && pool_state[device_id] == 0) {
        const char* e = getenv("RPB_POOL");
        cudaMemPool_t pool;
        unsigned long long keep = ~0ull;
        if ((e && atoi(e) == 0) || cudaDeviceGetDefaultMemPool(&pool, device_id) != cudaSuccess ||
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) {
            cudaGetLastError();
            pool_state[device_id] = -1;
        } else {
            pool_state[device_id] = 1;
        }
    }
    if (device_id >= 0 && device_id < 64 && pool_state[device_id] == 1) {
        if (cudaMallocAsync(out, bytes, t_stream) == cudaSuccess) return 0;
        cudaGetLastError();
    }
    return cudaMalloc(out, bytes) == cudaSuccess ? 0 : -1;
}

/* Uninitialised contiguous device tensor.  RecPulse's zeros_device_tensor
 * (core/tensor_device.cu:12-63) also memsets; the GEMM overwrites every element, so no memset here. */
Tensor* rpb_tensor_empty(DType dtype, int ndim, const int* shape, int device_id) {
    if (device_id < 0) { fprintf(stderr, "recpulse_b200: device tensors only\n"); return NULL; }
    Tensor* t = alloc_struct(dtype, ndim, shape, device_id);
    if (!t) return NULL;
    if (cudaSetDevice(device_id) != cudaSuccess || device_alloc(&t->data, t->size * rpb_dtype_size(dtype), device_id) != 0) {
        fprintf(stderr, "recpulse_b200: cudaMalloc of %zu bytes failed: %s\n", t->size * rpb_dtype_size(dtype),
                cudaGetErrorString(cudaGetLastError()));
        free_dims(t); free(t);
        return NULL;
    }
    return t;
}

Tensor* rpb_tensor_from_host(const void* host_data, DType dtype, int ndim, const int* shape, int device_id,
                             bool requires_grad) {
    if (!host_data) return NULL;
    Tensor* t = rpb_tensor_empty(dtype, ndim, shape, device_id);
    if (!t) return NULL;
    if (cudaMemcpy(t->data, host_data, t->size * rpb_dtype_size(dtype), cudaMemcpyHostToDevice) != cudaSuccess) {
        rpb_tensor_release(t);
        return NULL;
    }
    if (requires_grad) {
        t->metadata = (Meta*)calloc(1, sizeof(Meta));
        if (!t->metadata) { rpb_tensor_release(t); return NULL; }
        t->metadata->is_leaf = true;
        t->metadata->requires_grad = true;
    }
    return t;
}

Tensor* rpb_tensor_view(Tensor* base, int ndim, const int* shape, const int* strides, size_t offset_elems) {
    if (!base || ndim <= 0 || !shape || !strides) return NULL;
    Tensor* t = alloc_struct(base->dtype, ndim, shape, base->device_id);
    if (!t) return NULL;
    memcpy(t->strides, strides, sizeof(int) * ndim);
    t->data = (char*)base->data + offset_elems * rpb_dtype_size(base->dtype);
    t->owns_data = false;
    t->data_offset = base->data_offset + offset_elems;
    t->base_tensor = base;
    base->refcount++;
    if (base->metadata && base->metadata->requires_grad) {
        /* the view collects its own gradient (in the view's shape); RecPulse's view ops route it
         * back to the leaf through their own autograd nodes, which are outside this library */
        t->metadata = (Meta*)calloc(1, sizeof(Meta));
        if (!t->metadata) { rpb_tensor_release(t); return NULL; }
        t->metadata->requires_grad = true;
    }
    return t;
}

/* Overwrites the values of a packed device tensor in place (same buffer: what a captured graph reads). */
int rpb_tensor_write_host(Tensor* t, const void* host_data) {
    if (!t || !host_data || t->device_id < 0 || !t->data) return -1;
    long long s = 1;
    for (int d = t->ndim - 1; d >= 0; d--) { if (t->strides[d] != s) return -1; s *= t->shape[d]; }
    if (cudaSetDevice(t->device_id) != cudaSuccess) return -1;
    if (t_stream && cudaStreamSynchronize(t_stream) != cudaSuccess) return -1;
    return cudaMemcpy(t->data, host_data, t->size * rpb_dtype_size(t->dtype), cudaMemcpyHostToDevice) == cudaSuccess ? 0 : -1;
}

/* Drops the accumulated gradient (the next backward assigns a fresh one). */
void rpb_tensor_zero_grad(Tensor* t) {
    if (!t || !t->metadata || !t->metadata->grad) return;
    rpb_tensor_release(t->metadata->grad);
    t->metadata->grad = NULL;
}

static bool is_contiguous(const Tensor* t) {      /* functional/functional.c:1117-1128 */
    long long s = 1;
    for (int d = t->ndim - 1; d >= 0; d--) {
        if (t->strides[d] != s) return false;
        s *= t->shape[d];
    }
    return true;
}

int rpb_tensor_to_host(const Tensor* t, void* host_out) {
    if (!t || !host_out || t->device_id < 0 || t->ndim > RPB_MAX_BATCH_DIMS + 2) return -1;
    const size_t es = rpb_dtype_size(t->dtype);
    if (cudaSetDevice(t->device_id) != cudaSuccess) return -1;
    if (t_stream && cudaStreamSynchronize(t_stream) != cudaSuccess) return -1;   /* work queued by asynchronous nodes */
    if (is_contiguous(t))
        return cudaMemcpy(host_out, t->data, t->size * es, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
    /* strided view: one 2-D copy per innermost row pair (diagnostic path, not a hot path) */
    int idx[RPB_MAX_BATCH_DIMS + 2] = {0};
    const int nd = t->ndim;
    size_t rows = t->size / (size_t)t->shape[nd - 1];
    for (size_t r = 0; r < rows; r++) {
        long long off = 0;
        for (int d = 0; d < nd - 1; d++) off += (long long)idx[d] * t->strides[d];
        char* dst = (char*)host_out + r * (size_t)t->shape[nd - 1] * es;
        const char* src = (const char*)t->data + off * (long long)es;
        if (cudaMemcpy2D(dst, es, src, (size_t)t->strides[nd - 1] * es, es, (size_t)t->shape[nd - 1],
                         cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
        for (int d = nd - 2; d >= 0; d--) { if (++idx[d] < t->shape[d]) break; idx[d] = 0; }
    }
    return 0;
}

static void free_node(GradFn* fn) {               /* ops/ops.c:7227-7322, generic branch */
    if (!fn) return;
    free(fn->saved_data);
    for (int i = 0; i < fn->num_inputs; i++)
        if (fn->inputs && fn->inputs[i] && fn->inputs[i] != fn->owner) rpb_tensor_release(fn->inputs[i]);
    free(fn->inputs);
    free(fn);
}

void rpb_tensor_release(Tensor* t) {              /* core/tensor.c:360-379, core/tensor_device.cu:269-293 */
    if (!t) return;
    if (t->refcount > 1) { t->refcount--; return; }
    Tensor* base = t->base_tensor;
    if (t->metadata) {
        if (t->metadata->grad_fn) { free_node(t->metadata->grad_fn); t->metadata->grad_fn = NULL; }
        if (t->metadata->grad) rpb_tensor_release(t->metadata->grad);
    }
    if (t->owns_data && t->data) {
        if (t->device_id >= 0) {
            cudaSetDevice(t->device_id);
            /* a thread that runs its nodes asynchronously frees in stream order too (cudaFree would wait for
             * the device, and is not allowed while the stream is being captured) */
            if (t_sync || cudaFreeAsync(t->data, t_stream) != cudaSuccess) cudaFree(t->data);
        }
        else free(t->data);
    }
    free_dims(t);
    free(t->metadata);
    free(t);
    rpb_tensor_release(base);
}

/* ------------------------------------------------------------------ batch geometry */

typedef struct { long long extent, a, b, c; } BatchDim;      /* strides in elements */

/* Merge dimensions that form one arithmetic progression in all three operands. */
static int collapse(BatchDim* d, int n) {
    int changed = 1;
    while (changed) {
        changed = 0;
        for (int i = 0; i < n && !changed; i++) {
            for (int j = 0; j < n && !changed; j++) {
                if (i == j) continue;
                /* j becomes the outer part of i */
                if (d[j].a == d[i].a * d[i].extent && d[j].b == d[i].b * d[i].extent &&
                    d[j].c == d[i].c * d[i].extent) {
                    d[i].extent *= d[j].extent;
                    d[j] = d[n - 1];
                    n--;
                    changed = 1;
                }
            }
        }
    }
    return n;
}

/* Runs C (+)= A.B for one matmul whose leading dimensions are split into independent ("batch") and
 * summed ("reduce") lists.  One list entry of each kind goes into the kernel; the rest is looped here. */
static int run_batched(void* C, const void* A, const void* B, RpbGemm g, BatchDim* bd, int nb, BatchDim* rd, int nr,
                       DType dtype, int device_id) {
    nb = collapse(bd, nb);
    nr = collapse(rd, nr);
    const size_t es = rpb_dtype_size(dtype);
    /* pick the largest entry of each kind for the kernel */
    int kb = -1, kr = -1;
    for (int i = 0; i < nb; i++) if (kb < 0 || bd[i].extent > bd[kb].extent) kb = i;
    for (int i = 0; i < nr; i++) if (kr < 0 || rd[i].extent > rd[kr].extent) kr = i;
    if (kb >= 0) {
        if (bd[kb].extent > 0x7fffffffLL) return -1;
        g.batch = (int)bd[kb].extent; g.a_batch = bd[kb].a; g.b_batch = bd[kb].b; g.c_batch = bd[kb].c;
        bd[kb] = bd[--nb];
    }
    if (kr >= 0) {
        if (rd[kr].extent > 0x7fffffffLL) return -1;
        g.reduce = (int)rd[kr].extent; g.a_reduce = rd[kr].a; g.b_reduce = rd[kr].b;
        rd[kr] = rd[--nr];
    }
    /* odometer over what is left: batch entries first (outer), reduce entries inner */
    BatchDim loop[2 * RPB_MAX_BATCH_DIMS];
    int kind[2 * RPB_MAX_BATCH_DIMS];
    int nl = 0;
    for (int i = 0; i < nb; i++) { loop[nl] = bd[i]; kind[nl++] = 0; }
    for (int i = 0; i < nr; i++) { loop[nl] = rd[i]; kind[nl++] = 1; }
    long long idx[2 * RPB_MAX_BATCH_DIMS] = {0};
    const int base_acc = g.accumulate;
    for (;;) {
        long long oa = 0, ob = 0, oc = 0;
        int later_reduce = 0;
        for (int i = 0; i < nl; i++) {
            oa += idx[i] * loop[i].a; ob += idx[i] * loop[i].b; oc += idx[i] * loop[i].c;
            if (kind[i] == 1 && idx[i] > 0) later_reduce = 1;
        }
        g.accumulate = base_acc || later_reduce;
        if (rp_matmul_ex((char*)C + oc * (long long)es, (const char*)A + oa * (long long)es,
                         (const char*)B + ob * (long long)es, &g, dtype, device_id, t_stream) != 0) return -1;
        int d = nl - 1;
        for (; d >= 0; d--) { if (++idx[d] < loop[d].extent) break; idx[d] = 0; }
        if (d < 0) break;
    }
    return 0;
}

static int broadcast_batch(const Tensor* a, const Tensor* b, int* out_nd, int* out_shape) {
    const int na = a->ndim - 2, nbd = b->ndim - 2;
    const int nd = na > nbd ? na : nbd;
    if (nd > RPB_MAX_BATCH_DIMS) return -1;
    for (int i = 0; i < nd; i++) {
        const int ia = i - (nd - na), ib = i - (nd - nbd);
        const int ea = ia >= 0 ? a->shape[ia] : 1, eb = ib >= 0 ? b->shape[ib] : 1;
        if (ea != eb && ea != 1 && eb != 1) return -1;
        out_shape[i] = ea > eb ? ea : eb;
    }
    *out_nd = nd;
    return 0;
}

/* stride of tensor t along broadcast batch dimension i (of nd), 0 where t is broadcast */
static long long batch_stride(const Tensor* t, int nd, int i) {
    const int it = i - (nd - (t->ndim - 2));
    if (it < 0 || t->shape[it] == 1) return 0;
    return t->strides[it];
}

/* ------------------------------------------------------------------ autograd node */

static bool bias_ok(const Tensor* bias, const Tensor* a, int n) {
    if (bias->dtype != a->dtype || bias->device_id != a->device_id) return false;
    if ((int)bias->size != n || bias->shape[bias->ndim - 1] != n || bias->strides[bias->ndim - 1] != 1) return false;
    return true;
}

/* out (+)= a . b (+ bias) for operands that already passed the shape checks; out is packed with the
 * broadcast batch shape of a and b */
static int product_into(Tensor* out, const Tensor* a, const Tensor* b, const Tensor* bias, int accumulate, int epilogue,
                        int nd, const int* oshape) {
    const int m = a->shape[a->ndim - 2], k = a->shape[a->ndim - 1], n = b->shape[b->ndim - 1];
    RpbGemm g;
    rpb_gemm_packed(&g, m, k, n);
    g.a_row = a->strides[a->ndim - 2]; g.a_col = a->strides[a->ndim - 1];
    g.b_row = b->strides[b->ndim - 2]; g.b_col = b->strides[b->ndim - 1];
    g.a_batch = g.b_batch = g.c_batch = 0;
    g.bias = bias ? bias->data : NULL;
    g.accumulate = accumulate;
    g.epilogue = epilogue;
    BatchDim bd[RPB_MAX_BATCH_DIMS];
    int nbd = 0;
    for (int i = 0; i < nd; i++) {
        if (oshape[i] == 1) continue;
        bd[nbd].extent = oshape[i];
        bd[nbd].a = batch_stride(a, nd, i); bd[nbd].b = batch_stride(b, nd, i); bd[nbd].c = out->strides[i];
        nbd++;
    }
    return run_batched(out->data, a->data, b->data, g, bd, nbd, NULL, 0, a->dtype, a->device_id);
}

static bool operands_ok(const Tensor* a, const Tensor* b) {      /* ops/ops.c:6817-6820, with ndim >= 2 */
    if (!a || !b) return false;
    if (a->ndim < 2 || b->ndim < 2) return false;
    if (a->shape[a->ndim - 1] != b->shape[b->ndim - 2]) return false;
    return a->dtype == b->dtype && a->device_id == b->device_id;
}

/* Meta + GradFn for a fresh output, with RecPulse's grad_fn_attach bookkeeping (ops/ops.c:11-19) */
static int attach_node(Tensor* out, BackwardFunction backward, Tensor** in, int n_in) {
    out->metadata = (Meta*)calloc(1, sizeof(Meta));
    GradFn* fn = (GradFn*)calloc(1, sizeof(GradFn));
    Tensor** inputs = (Tensor**)malloc(n_in * sizeof(Tensor*));
    if (!out->metadata || !fn || !inputs) { free(fn); free(inputs); return -1; }
    out->metadata->requires_grad = true;
    out->metadata->is_leaf = false;
    fn->backward = backward;
    fn->num_inputs = n_in;
    fn->inputs = inputs;
    fn->saved_data = NULL;
    fn->owner = out;
    for (int i = 0; i < n_in; i++) { inputs[i] = in[i]; if (in[i] != out) in[i]->refcount++; }
    out->metadata->grad_fn = fn;
    return 0;
}

static bool wants_grad(const Tensor* t) { return t && t->metadata && t->metadata->requires_grad; }

/* shared by op_matmul (bias == NULL) and op_linear */
static Tensor* matmul_node(Tensor* a, Tensor* b, Tensor* bias) {
    if (!a || !b) return NULL;
    if (a->ndim < 2 || b->ndim < 2) return NULL;
    if (a->shape[a->ndim - 1] != b->shape[b->ndim - 2]) return NULL;
    if (a->dtype != b->dtype || a->device_id != b->device_id) return NULL;
    if (a->device_id < 0) {
        /* host tensors stay with RecPulse's own implementation when it is loaded */
        typedef Tensor* (*Fn)(Tensor*, Tensor*);
        Fn ref = (Fn)rpb_reference_symbol("op_matmul");
        if (!bias && ref && ref != &op_matmul) return ref(a, b);
        fprintf(stderr, "recpulse_b200: matmul on host tensors: this library has no CPU path\n");
        return NULL;
    }
    if (bias && !bias_ok(bias, a, b->shape[b->ndim - 1])) return NULL;

    const int m = a->shape[a->ndim - 2], n = b->shape[b->ndim - 1];
    int nd = 0, oshape[RPB_MAX_BATCH_DIMS + 2];
    if (broadcast_batch(a, b, &nd, oshape)) return NULL;
    oshape[nd] = m; oshape[nd + 1] = n;

    Tensor* out = rpb_tensor_empty(a->dtype, nd + 2, oshape, a->device_id);
    if (!out) return NULL;

    int rc = product_into(out, a, b, bias, 0, 0, nd, oshape);
    /* callers assume the result is complete on return (every RecPulse device op synchronises) */
    if (rc == 0) rc = node_finish(a->device_id);
    if (rc != 0) {
        fprintf(stderr, "recpulse_b200: matmul node: the product could not be computed\n");
        rpb_tensor_release(out);
        return NULL;
    }

    if (wants_grad(a) || wants_grad(b) || wants_grad(bias)) {
        Tensor* in[3] = {a, b, bias};
        if (attach_node(out, bias ? backward_linear_fn : backward_matmul_fn, in, bias ? 3 : 2)) {
            rpb_tensor_release(out);
            return NULL;
        }
    }
    return out;
}

/* grad of `x` (one of the two inputs): target = x's grad tensor, new or existing */
static int grad_into(Tensor* x, const Tensor* other, const Tensor* grad_output, int side, int nd, const int* oshape) {
    const Tensor* a = side == 0 ? x : other;
    const Tensor* b = side == 0 ? other : x;
    const int m = a->shape[a->ndim - 2], k = a->shape[a->ndim - 1], n = b->shape[b->ndim - 1];

    Tensor* grad = x->metadata->grad;
    const bool fresh = grad == NULL;
    if (fresh) {
        grad = rpb_tensor_empty(x->dtype, x->ndim, x->shape, x->device_id);
        if (!grad) return -1;
    } else if (!is_contiguous(grad) || grad->size != x->size || grad->dtype != x->dtype) {
        fprintf(stderr, "recpulse_b200: existing grad is not a packed tensor of the input's shape\n");
        return -1;
    }

    RpbGemm g;
    memset(&g, 0, sizeof(g));
    g.batch = g.reduce = 1;
    g.accumulate = fresh ? 0 : 1;
    const long long go_row = grad_output->strides[grad_output->ndim - 2];
    const long long go_col = grad_output->strides[grad_output->ndim - 1];
    const void *A, *B;
    if (side == 0) {            /* dA[m,k] = dC[m,n] . B^T[n,k] */
        g.m = m; g.n = k; g.k = n;
        g.a_row = go_row; g.a_col = go_col;
        g.b_row = b->strides[b->ndim - 1]; g.b_col = b->strides[b->ndim - 2];
        A = grad_output->data; B = b->data;
    } else {                    /* dB[k,n] = A^T[k,m] . dC[m,n] */
        g.m = k; g.n = n; g.k = m;
        g.a_row = a->strides[a->ndim - 1]; g.a_col = a->strides[a->ndim - 2];
        g.b_row = go_row; g.b_col = go_col;
        A = a->data; B = grad_output->data;
    }
    g.c_row = grad->strides[grad->ndim - 2];

    BatchDim bd[RPB_MAX_BATCH_DIMS], rd[RPB_MAX_BATCH_DIMS];
    int nb = 0, nr = 0;
    for (int i = 0; i < nd; i++) {
        if (oshape[i] == 1) continue;
        const long long sx = batch_stride(x, nd, i);          /* 0: x is broadcast here -> sum */
        const long long so = batch_stride(other, nd, i);
        const long long sg = grad_output->strides[i + (grad_output->ndim - 2 - nd)];
        BatchDim e;
        e.extent = oshape[i];
        e.a = side == 0 ? sg : so;                            /* side 1: A operand is `other` = a */
        e.b = side == 0 ? so : sg;
        if (sx == 0) { e.c = 0; rd[nr++] = e; }
        else {
            const int ix = i - (nd - (x->ndim - 2));
            e.c = grad->strides[ix];
            bd[nb++] = e;
        }
    }
    int rc = run_batched(grad->data, A, B, g, bd, nb, rd, nr, x->dtype, x->device_id);
    if (rc == 0) rc = node_finish(x->device_id);
    if (rc != 0) {
        if (fresh) rpb_tensor_release(grad);
        return -1;
    }
    if (fresh) x->metadata->grad = grad;
    return 0;
}

Tensor* op_matmul(Tensor* a, Tensor* b) { return matmul_node(a, b, NULL); }

Tensor* op_linear(Tensor* x, Tensor* w, Tensor* bias) { return matmul_node(x, w, bias); }

/* dA and dB of a device matmul node; 0 when grad_output matches the node */
static int matmul_grads(Tensor* a, Tensor* b, Tensor* grad_output) {
    int nd = 0, oshape[RPB_MAX_BATCH_DIMS + 2];
    if (broadcast_batch(a, b, &nd, oshape)) return -1;
    if (grad_output->ndim != nd + 2 || grad_output->dtype != a->dtype || grad_output->device_id != a->device_id) {
        fprintf(stderr, "recpulse_b200: matmul backward: upstream gradient does not match the output\n");
        return -1;
    }
    if (a->metadata && a->metadata->requires_grad) grad_into(a, b, grad_output, 0, nd, oshape);
    if (b->metadata && b->metadata->requires_grad) grad_into(b, a, grad_output, 1, nd, oshape);
    return 0;
}

void backward_matmul_fn(GradFn* self, Tensor* grad_output) {
    if (!self || !grad_output || self->num_inputs != 2 || !self->inputs) return;
    Tensor* a = self->inputs[0];
    Tensor* b = self->inputs[1];
    if (!a || !b) return;
    if (a->device_id < 0) {
        typedef void (*Fn)(GradFn*, Tensor*);
        Fn ref = (Fn)rpb_reference_symbol("backward_matmul_fn");
        if (ref && ref != &backward_matmul_fn) ref(self, grad_output);
        return;
    }
    matmul_grads(a, b, grad_output);
}

/* dX and dW as for op_matmul; dbias = sum of dY over every leading index (assigned, or accumulated
 * into an existing grad with one rounding) */
void backward_linear_fn(GradFn* self, Tensor* grad_output) {
    if (!self || !grad_output || self->num_inputs != 3 || !self->inputs) return;
    Tensor* x = self->inputs[0];
    Tensor* w = self->inputs[1];
    Tensor* bias = self->inputs[2];
    if (!x || !w || !bias || x->device_id < 0) return;
    if (matmul_grads(x, w, grad_output)) return;
    bias_grad_into(bias, grad_output);
}

/* bias gradient shared by the Linear nodes */
static void bias_grad_into(Tensor* bias, Tensor* grad_output) {
    if (!wants_grad(bias)) return;
    if (!is_contiguous(grad_output)) {
        fprintf(stderr, "recpulse_b200: upstream gradient must be packed for the bias gradient\n");
        return;
    }
    const int n = grad_output->shape[grad_output->ndim - 1];
    const long long rows = (long long)(grad_output->size / (size_t)n);
    Tensor* grad = bias->metadata->grad;
    const bool fresh = grad == NULL;
    if (fresh) {
        grad = rpb_tensor_empty(bias->dtype, bias->ndim, bias->shape, bias->device_id);
        if (!grad) return;
    } else if (!is_contiguous(grad) || grad->size != bias->size) {
        return;
    }
    int rc = rp_colsum_ex(grad->data, grad_output->data, rows, n, n, bias->dtype, fresh ? 0 : 1, bias->device_id, t_stream);
    if (rc == 0) rc = node_finish(bias->device_id);
    if (rc != 0) { if (fresh) rpb_tensor_release(grad); return; }
    if (fresh) bias->metadata->grad = grad;
}

/* shared by op_linear2 (gates = 0) and op_lstm_gates (gates = 1: the activation pass runs on the result) */
static Tensor* linear2_node(Tensor* x, Tensor* w, Tensor* h, Tensor* u, Tensor* bias, int gates) {
    if (!operands_ok(x, w) || !operands_ok(h, u)) return NULL;
    if (x->dtype != h->dtype || x->device_id != h->device_id) return NULL;
    if (x->device_id < 0) {
        fprintf(stderr, "recpulse_b200: op_linear2 / op_lstm_gates on host tensors: this library has no CPU path\n");
        return NULL;
    }
    const int n = w->shape[w->ndim - 1];
    if (u->shape[u->ndim - 1] != n) return NULL;
    if (gates && n % 4 != 0) return NULL;
    if (bias && !bias_ok(bias, x, n)) return NULL;
    int nd = 0, oshape[RPB_MAX_BATCH_DIMS + 2], nd2 = 0, oshape2[RPB_MAX_BATCH_DIMS + 2];
    if (broadcast_batch(x, w, &nd, oshape) || broadcast_batch(h, u, &nd2, oshape2)) return NULL;
    oshape[nd] = x->shape[x->ndim - 2]; oshape[nd + 1] = n;
    oshape2[nd2] = h->shape[h->ndim - 2]; oshape2[nd2 + 1] = n;
    if (nd != nd2 || memcmp(oshape, oshape2, sizeof(int) * (nd + 2)) != 0) return NULL;   /* both products, same shape */

    Tensor* out = rpb_tensor_empty(x->dtype, nd + 2, oshape, x->device_id);
    if (!out) return NULL;
    int rc = product_into(out, x, w, bias, 0, 0, nd, oshape);
    /* the second product lands in the epilogue's "+= C"; for the gate block the same epilogue then applies the
     * non-linearities to the finished sum (or, for plans that cannot, one pass over the output does) */
    if (rc == 0) rc = product_into(out, h, u, NULL, 1, gates ? RPB_EPILOGUE_LSTM_GATES : 0, nd, oshape);
    if (rc == 0) rc = node_finish(x->device_id);
    if (rc != 0) { rpb_tensor_release(out); return NULL; }
    if (wants_grad(x) || wants_grad(w) || wants_grad(h) || wants_grad(u) || wants_grad(bias)) {
        Tensor* in[5] = {x, w, h, u, bias};
        if (attach_node(out, gates ? backward_lstm_gates_fn : backward_linear2_fn, in, bias ? 5 : 4)) {
            rpb_tensor_release(out);
            return NULL;
        }
    }
    return out;
}

Tensor* op_linear2(Tensor* x, Tensor* w, Tensor* h, Tensor* u, Tensor* bias) { return linear2_node(x, w, h, u, bias, 0); }

Tensor* op_lstm_gates(Tensor* x, Tensor* w, Tensor* h, Tensor* u, Tensor* bias) { return linear2_node(x, w, h, u, bias, 1); }

void backward_linear2_fn(GradFn* self, Tensor* grad_output) {
    if (!self || !grad_output || (self->num_inputs != 4 && self->num_inputs != 5) || !self->inputs) return;
    Tensor** in = self->inputs;
    if (!in[0] || !in[1] || !in[2] || !in[3] || in[0]->device_id < 0) return;
    if (matmul_grads(in[0], in[1], grad_output)) return;
    if (matmul_grads(in[2], in[3], grad_output)) return;
    if (self->num_inputs == 5 && in[4]) bias_grad_into(in[4], grad_output);
}

void backward_lstm_gates_fn(GradFn* self, Tensor* grad_output) {
    if (!self || !grad_output || !self->owner || (self->num_inputs != 4 && self->num_inputs != 5) || !self->inputs) return;
    Tensor* y = self->owner;                    /* the activated gates */
    if (y->device_id < 0 || grad_output->dtype != y->dtype || grad_output->size != y->size) return;
    if (!is_contiguous(grad_output) || !is_contiguous(y)) {
        fprintf(stderr, "recpulse_b200: op_lstm_gates backward needs packed output and upstream gradient\n");
        return;
    }
    const int n = y->shape[y->ndim - 1];
    Tensor* dpre = rpb_tensor_empty(y->dtype, y->ndim, y->shape, y->device_id);
    if (!dpre) return;
    int rc = rp_lstm_gates_grad_ex(dpre->data, grad_output->data, y->data, (long long)(y->size / (size_t)n), n, n, n, n,
                                   y->dtype, y->device_id, t_stream);
    if (rc == 0) backward_linear2_fn(self, dpre);
    rpb_tensor_release(dpre);
}

/* ------------------------------------------------------------------ GRU cell (recpulse/module.py:329-348) */

typedef struct { int has_b_ih, has_b_hh; } GruSaved;     /* flat: RecPulse's free_grad_fn releases it with free() */

static bool packed_2d(const Tensor* t) { return t && t->ndim == 2 && is_contiguous(t); }

Tensor* op_gru_cell(Tensor* x, Tensor* w_ih, Tensor* h, Tensor* w_hh, Tensor* b_ih, Tensor* b_hh) {
    if (!operands_ok(x, w_ih) || !operands_ok(h, w_hh)) return NULL;
    if (x->ndim != 2 || h->ndim != 2 || w_ih->ndim != 2 || w_hh->ndim != 2) return NULL;
    if (x->dtype != h->dtype || x->device_id != h->device_id || x->shape[0] != h->shape[0]) return NULL;
    if (x->device_id < 0) {
        fprintf(stderr, "recpulse_b200: op_gru_cell on host tensors: this library has no CPU path\n");
        return NULL;
    }
    const int m = x->shape[0], hidden = h->shape[1], n3 = 3 * hidden;
    if (w_ih->shape[1] != n3 || w_hh->shape[1] != n3 || w_hh->shape[0] != hidden) return NULL;
    if (h->strides[1] != 1) return NULL;
    if ((b_ih && !bias_ok(b_ih, x, n3)) || (b_hh && !bias_ok(b_hh, x, n3))) return NULL;
    int gshape[2] = {m, n3}, oshape[2] = {m, hidden};
    Tensor* gi = rpb_tensor_empty(x->dtype, 2, gshape, x->device_id);
    Tensor* gh = rpb_tensor_empty(x->dtype, 2, gshape, x->device_id);
    Tensor* out = rpb_tensor_empty(x->dtype, 2, oshape, x->device_id);
    int rc = (gi && gh && out) ? 0 : -1;
    /* the two products stay apart (the candidate gate multiplies gh_n by r before the sum); biases ride in the epilogues */
    if (rc == 0) rc = product_into(gi, x, w_ih, b_ih, 0, 0, 0, gshape);
    if (rc == 0) rc = product_into(gh, h, w_hh, b_hh, 0, 0, 0, gshape);
    if (rc == 0) rc = rp_gru_gates_ex(out->data, gi->data, gh->data, h->data, m, hidden, h->strides[0], x->dtype, x->device_id, t_stream);
    if (rc == 0) rc = node_finish(x->device_id);
    if (rc != 0) { rpb_tensor_release(gi); rpb_tensor_release(gh); rpb_tensor_release(out); return NULL; }
    if (wants_grad(x) || wants_grad(w_ih) || wants_grad(h) || wants_grad(w_hh) || wants_grad(b_ih) || wants_grad(b_hh)) {
        /* inputs: x, w_ih, h, w_hh, [b_ih], [b_hh], activated gates, gh.  The last two carry no Meta: RecPulse's
         * tensor_backward skips them (core/tensor.c:251, 296) and free_grad_fn releases them (ops/ops.c:7227-7322). */
        Tensor* in[8];
        int n_in = 0;
        in[n_in++] = x; in[n_in++] = w_ih; in[n_in++] = h; in[n_in++] = w_hh;
        if (b_ih) in[n_in++] = b_ih;
        if (b_hh) in[n_in++] = b_hh;
        in[n_in++] = gi; in[n_in++] = gh;
        GruSaved* saved = (GruSaved*)malloc(sizeof(GruSaved));
        if (!saved || attach_node(out, backward_gru_cell_fn, in, n_in)) {
            free(saved); rpb_tensor_release(gi); rpb_tensor_release(gh); rpb_tensor_release(out);
            return NULL;
        }
        saved->has_b_ih = b_ih != NULL; saved->has_b_hh = b_hh != NULL;
        out->metadata->grad_fn->saved_data = saved;
    }
    rpb_tensor_release(gi);             /* the node (if any) holds its own references */
    rpb_tensor_release(gh);
    return out;
}

void backward_gru_cell_fn(GradFn* self, Tensor* grad_output) {
    if (!self || !grad_output || !self->inputs || !self->saved_data || !self->owner) return;
    const GruSaved* saved = (const GruSaved*)self->saved_data;
    const int n_in = 6 + saved->has_b_ih + saved->has_b_hh;
    if (self->num_inputs != n_in) return;
    Tensor** in = self->inputs;
    Tensor *x = in[0], *w_ih = in[1], *h = in[2], *w_hh = in[3];
    Tensor* b_ih = saved->has_b_ih ? in[4] : NULL;
    Tensor* b_hh = saved->has_b_hh ? in[4 + saved->has_b_ih] : NULL;
    Tensor *gi = in[n_in - 2], *gh = in[n_in - 1];
    if (!x || !w_ih || !h || !w_hh || !gi || !gh || x->device_id < 0) return;
    const int m = x->shape[0], hidden = h->shape[1];
    if (grad_output->dtype != x->dtype || grad_output->device_id != x->device_id || !packed_2d(grad_output) ||
        grad_output->shape[0] != m || grad_output->shape[1] != hidden) {
        fprintf(stderr, "recpulse_b200: op_gru_cell backward: upstream gradient must be a packed [m, hidden] tensor\n");
        return;
    }
    Tensor* dgi = rpb_tensor_empty(x->dtype, 2, gi->shape, x->device_id);
    Tensor* dgh = rpb_tensor_empty(x->dtype, 2, gi->shape, x->device_id);
    if (!dgi || !dgh) { rpb_tensor_release(dgi); rpb_tensor_release(dgh); return; }
    /* the direct part of dL/dh (g z) opens h's gradient; the GEMM below then adds dgh . w_hh^T in its epilogue */
    void* dh = NULL;
    int dh_acc = 0;
    Tensor* fresh_dh = NULL;
    if (wants_grad(h)) {
        if (h->metadata->grad) {
            if (is_contiguous(h->metadata->grad) && h->metadata->grad->size == h->size) { dh = h->metadata->grad->data; dh_acc = 1; }
        } else {
            fresh_dh = rpb_tensor_empty(h->dtype, h->ndim, h->shape, h->device_id);
            if (fresh_dh) dh = fresh_dh->data;
        }
    }
    int rc = rp_gru_gates_grad_ex(dgi->data, dgh->data, dh, dh_acc, grad_output->data, gi->data, gh->data, h->data, m, hidden,
                                  h->strides[0], x->dtype, x->device_id, t_stream);
    if (rc == 0 && fresh_dh) { h->metadata->grad = fresh_dh; fresh_dh = NULL; }
    if (rc == 0) rc = matmul_grads(x, w_ih, dgi);
    if (rc == 0) rc = matmul_grads(h, w_hh, dgh);
    if (rc == 0 && b_ih) bias_grad_into(b_ih, dgi);
    if (rc == 0 && b_hh) bias_grad_into(b_hh, dgh);
    rpb_tensor_release(fresh_dh);
    rpb_tensor_release(dgi);
    rpb_tensor_release(dgh);
}

int rpb_backward_node(Tensor* out, Tensor* grad_output) {
    if (!out || !grad_output || !out->metadata || !out->metadata->grad_fn) return -1;
    GradFn* fn = out->metadata->grad_fn;
    fn->backward(fn, grad_output);
    free_node(fn);
    out->metadata->grad_fn = NULL;
    return 0;
}
