/*
 * Element-wise companions of the GEMMs for the callers next to the matmul path:
 *   - the GRU cell's gate arithmetic (recpulse/module.py:334-348) and its gradient, one pass each,
 *   - conv2d as im2col of ALL images + single batched GEMM launches (ops/ops.c:4761-4770 forward,
 *     :4536-4550 input gradient, :4575-4617 weight gradient, which loop per image and copy transposes).
 * All run on the caller's stream without synchronising.
 */
#include <cstdio>
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "rpb_common.h"

extern "C" void rpb_count_launches(int n);      /* gemm_dispatch.cu */

namespace {

#define CL_CUDA(call)                                                                           \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess) {                                                                \
            fprintf(stderr, "recpulse_b200: %s failed: %s\n", #call, cudaGetErrorString(e_));   \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

template <typename T> struct AccOf { typedef float type; };
template <> struct AccOf<double> { typedef double type; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type ld(const T* p) { return (typename AccOf<T>::type)(*p); }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(*p); }
template <typename T, typename A> __device__ __forceinline__ void st(T* p, A v) { *p = (T)v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16, float>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void st<__half, float>(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float sigm(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ double sigm(double v) { return 1.0 / (1.0 + exp(-v)); }
__device__ __forceinline__ float tnh(float v) { return tanhf(v); }
__device__ __forceinline__ double tnh(double v) { return tanh(v); }

/* gi = x.W_ih (+ b_ih), gh = h.W_hh (+ b_hh), both [rows, 3 hidden] with column blocks (r, z, n):
 *   r = sigmoid(gi_r + gh_r), z = sigmoid(gi_z + gh_z), n = tanh(gi_n + r * gh_n), h' = (1 - z) n + z h.
 * r, z, n overwrite gi (the backward needs them); gh is left as it is (its n block is needed again). */
template <typename T>
__global__ void gru_forward_kernel(T* __restrict__ h_next, T* __restrict__ gi, const T* __restrict__ gh,
                                   const T* __restrict__ h, long long rows, int hidden, long long h_stride) {
    typedef typename AccOf<T>::type A;
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long total = rows * hidden;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += step) {
        const long long i = e / hidden;
        const int j = (int)(e - i * hidden);
        T* gir = gi + i * 3 * hidden + j;
        const T* ghr = gh + i * 3 * hidden + j;
        const A r = sigm(ld(gir) + ld(ghr));
        const A z = sigm(ld(gir + hidden) + ld(ghr + hidden));
        const A n = tnh(ld(gir + 2 * hidden) + r * ld(ghr + 2 * hidden));
        const A hv = ld(h + i * h_stride + j);
        st(gir, r); st(gir + hidden, z); st(gir + 2 * hidden, n);
        st(h_next + e, (A(1) - z) * n + z * hv);
    }
}

/* From g = dL/dh' and the saved r, z, n (in gi) and gh_n:
 *   dn = g (1 - z), dz = g (h - n), da_n = dn (1 - n^2), da_z = dz z (1 - z), dr = da_n gh_n, da_r = dr r (1 - r)
 *   dgi = (da_r, da_z, da_n), dgh = (da_r, da_z, da_n r), and the direct part of dL/dh = g z (assigned or added). */
template <typename T>
__global__ void gru_backward_kernel(T* __restrict__ dgi, T* __restrict__ dgh, T* __restrict__ dh, int dh_accumulate,
                                    const T* __restrict__ g, const T* __restrict__ gi, const T* __restrict__ gh,
                                    const T* __restrict__ h, long long rows, int hidden, long long h_stride) {
    typedef typename AccOf<T>::type A;
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long total = rows * hidden;
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += step) {
        const long long i = e / hidden;
        const int j = (int)(e - i * hidden);
        const long long o = i * 3 * hidden + j;
        const A r = ld(gi + o), z = ld(gi + o + hidden), n = ld(gi + o + 2 * hidden), hn = ld(gh + o + 2 * hidden);
        const A gv = ld(g + e), hv = ld(h + i * h_stride + j);
        const A dan = gv * (A(1) - z) * (A(1) - n * n);
        const A daz = gv * (hv - n) * z * (A(1) - z);
        const A dar = dan * hn * r * (A(1) - r);
        st(dgi + o, dar); st(dgi + o + hidden, daz); st(dgi + o + 2 * hidden, dan);
        st(dgh + o, dar); st(dgh + o + hidden, daz); st(dgh + o + 2 * hidden, dan * r);
        if (dh) {
            A d = gv * z;
            if (dh_accumulate) d += ld(dh + e);
            st(dh + e, d);
        }
    }
}

/* col[img][(c kH + kh) kW + kw][oh out_W + ow] = im[img][c][oh sh + kh dh - ph][ow sw + kw dw - pw] (0 outside):
 * the layout of im2col_2d_kernel (functional/functional_device.cu:1665-1693) for every image at once. */
template <typename T>
__global__ void im2col_all_kernel(T* __restrict__ col, const T* __restrict__ im, RpbConv2d c, int out_h, int out_w,
                                  long long total) {
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
        const int ow = (int)(idx % out_w);
        long long t = idx / out_w;
        const int oh = (int)(t % out_h); t /= out_h;
        const int kw = (int)(t % c.kW); t /= c.kW;
        const int kh = (int)(t % c.kH); t /= c.kH;
        const int ch = (int)(t % c.C_in);
        const long long img = t / c.C_in;
        const int hi = oh * c.stride_h + kh * c.dilation_h - c.pad_h;
        const int wi = ow * c.stride_w + kw * c.dilation_w - c.pad_w;
        T v = T(0.f);
        if (hi >= 0 && hi < c.H && wi >= 0 && wi < c.W) v = im[((img * c.C_in + ch) * c.H + hi) * (long long)c.W + wi];
        col[idx] = v;
    }
}

/* grad_im[img][c][hi][wi] (+)= sum over the (kh, kw, oh, ow) windows that cover the pixel, in a fixed order (one
 * thread per pixel gathers; the reference scatters with atomicAdd, functional_device.cu:1695-1725). */
template <typename T>
__global__ void col2im_all_kernel(T* __restrict__ grad_im, const T* __restrict__ col, RpbConv2d c, int out_h, int out_w,
                                  long long total, int accumulate) {
    typedef typename AccOf<T>::type A;
    rpb_pdl_trigger();
    rpb_pdl_wait();
    const long long step = (long long)gridDim.x * blockDim.x;
    const long long col_cols = (long long)out_h * out_w;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
        const int wi = (int)(idx % c.W);
        long long t = idx / c.W;
        const int hi = (int)(t % c.H); t /= c.H;
        const int ch = (int)(t % c.C_in);
        const long long img = t / c.C_in;
        A acc = accumulate ? ld(grad_im + idx) : A(0);
        for (int kh = 0; kh < c.kH; ++kh) {
            const int hn = hi + c.pad_h - kh * c.dilation_h;
            if (hn < 0 || hn % c.stride_h) continue;
            const int oh = hn / c.stride_h;
            if (oh >= out_h) continue;
            for (int kw = 0; kw < c.kW; ++kw) {
                const int wn = wi + c.pad_w - kw * c.dilation_w;
                if (wn < 0 || wn % c.stride_w) continue;
                const int ow = wn / c.stride_w;
                if (ow >= out_w) continue;
                const long long row = ((long long)ch * c.kH + kh) * c.kW + kw;
                acc += ld(col + (img * ((long long)c.C_in * c.kH * c.kW) + row) * col_cols + (long long)oh * out_w + ow);
            }
        }
        st(grad_im + idx, acc);
    }
}

int grid_for(long long total, int device_id) {
    static int sms[64];
    int n = 148;
    if (device_id >= 0 && device_id < 64) {
        if (!sms[device_id]) cudaDeviceGetAttribute(&sms[device_id], cudaDevAttrMultiProcessorCount, device_id);
        if (sms[device_id] > 0) n = sms[device_id];
    }
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)n * 16;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

struct DeviceScope {
    int prev = -1; bool moved = false;
    int enter(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) return -1;
        if (prev != device) { if (cudaSetDevice(device) != cudaSuccess) return -1; moved = true; }
        return 0;
    }
    ~DeviceScope() { if (moved) cudaSetDevice(prev); }
};

int conv_dims(const RpbConv2d* c, int* out_h, int* out_w, long long* col_rows, long long* col_cols) {
    if (!c || c->N <= 0 || c->C_in <= 0 || c->H <= 0 || c->W <= 0 || c->C_out <= 0 || c->kH <= 0 || c->kW <= 0 ||
        c->stride_h <= 0 || c->stride_w <= 0 || c->pad_h < 0 || c->pad_w < 0 || c->dilation_h <= 0 || c->dilation_w <= 0)
        return -1;
    const int oh = (c->H + 2 * c->pad_h - c->dilation_h * (c->kH - 1) - 1) / c->stride_h + 1;     /* ops/ops.c:4739-4740 */
    const int ow = (c->W + 2 * c->pad_w - c->dilation_w * (c->kW - 1) - 1) / c->stride_w + 1;
    if (oh <= 0 || ow <= 0) return -1;
    *out_h = oh; *out_w = ow;
    *col_rows = (long long)c->C_in * c->kH * c->kW;
    *col_cols = (long long)oh * ow;
    if (*col_rows > 0x7fffffffLL || *col_cols > 0x7fffffffLL) return -1;
    return 0;
}

template <typename T>
int launch_gru_fwd(void* h_next, void* gi, const void* gh, const void* h, long long rows, int hidden, long long h_stride,
                   int device_id, cudaStream_t s) {
    CL_CUDA(rpb_launch(gru_forward_kernel<T>, dim3(grid_for(rows * hidden, device_id)), dim3(256), 0, s, 1, reinterpret_cast<T*>(h_next),
                       reinterpret_cast<T*>(gi), reinterpret_cast<const T*>(gh), reinterpret_cast<const T*>(h), rows, hidden, h_stride));
    rpb_count_launches(1);
    return 0;
}
template <typename T>
int launch_gru_bwd(void* dgi, void* dgh, void* dh, int acc, const void* g, const void* gi, const void* gh, const void* h,
                   long long rows, int hidden, long long h_stride, int device_id, cudaStream_t s) {
    CL_CUDA(rpb_launch(gru_backward_kernel<T>, dim3(grid_for(rows * hidden, device_id)), dim3(256), 0, s, 1, reinterpret_cast<T*>(dgi),
                       reinterpret_cast<T*>(dgh), reinterpret_cast<T*>(dh), acc, reinterpret_cast<const T*>(g),
                       reinterpret_cast<const T*>(gi), reinterpret_cast<const T*>(gh), reinterpret_cast<const T*>(h), rows, hidden,
                       h_stride));
    rpb_count_launches(1);
    return 0;
}
template <typename T>
int launch_im2col(void* col, const void* im, const RpbConv2d& c, int oh, int ow, long long total, int device_id, cudaStream_t s) {
    CL_CUDA(rpb_launch(im2col_all_kernel<T>, dim3(grid_for(total, device_id)), dim3(256), 0, s, 1, reinterpret_cast<T*>(col),
                       reinterpret_cast<const T*>(im), c, oh, ow, total));
    rpb_count_launches(1);
    return 0;
}
template <typename T>
int launch_col2im(void* gim, const void* col, const RpbConv2d& c, int oh, int ow, long long total, int acc, int device_id,
                  cudaStream_t s) {
    CL_CUDA(rpb_launch(col2im_all_kernel<T>, dim3(grid_for(total, device_id)), dim3(256), 0, s, 1, reinterpret_cast<T*>(gim),
                       reinterpret_cast<const T*>(col), c, oh, ow, total, acc));
    rpb_count_launches(1);
    return 0;
}

#define BY_DTYPE(dtype, call)                                                     \
    switch ((int)(dtype)) {                                                       \
        case DTYPE_FLOAT32: rc = call<float>; break;                              \
        case DTYPE_FLOAT64: rc = call<double>; break;                             \
        case DTYPE_FLOAT16: rc = call<__half>; break;                             \
        case DTYPE_BFLOAT16: rc = call<__nv_bfloat16>; break;                     \
        default: rc = -1;                                                         \
    }

}  // namespace

extern "C" {

int rp_gru_gates_ex(void* h_next, void* gi, const void* gh, const void* h, long long rows, int hidden, long long h_stride,
                    DType dtype, int device_id, void* stream) {
    if (!h_next || !gi || !gh || !h || rows <= 0 || hidden <= 0 || h_stride < hidden || device_id < 0) return -1;
    DeviceScope scope;
    if (scope.enter(device_id)) return -1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int rc;
    switch ((int)dtype) {
        case DTYPE_FLOAT32: rc = launch_gru_fwd<float>(h_next, gi, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_FLOAT64: rc = launch_gru_fwd<double>(h_next, gi, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_FLOAT16: rc = launch_gru_fwd<__half>(h_next, gi, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_BFLOAT16: rc = launch_gru_fwd<__nv_bfloat16>(h_next, gi, gh, h, rows, hidden, h_stride, device_id, s); break;
        default: rc = -1;
    }
    return rc;
}

int rp_gru_gates_grad_ex(void* dgi, void* dgh, void* dh, int dh_accumulate, const void* g, const void* gi_act, const void* gh,
                         const void* h, long long rows, int hidden, long long h_stride, DType dtype, int device_id, void* stream) {
    if (!dgi || !dgh || !g || !gi_act || !gh || !h || rows <= 0 || hidden <= 0 || h_stride < hidden || device_id < 0) return -1;
    DeviceScope scope;
    if (scope.enter(device_id)) return -1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int rc;
    switch ((int)dtype) {
        case DTYPE_FLOAT32: rc = launch_gru_bwd<float>(dgi, dgh, dh, dh_accumulate, g, gi_act, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_FLOAT64: rc = launch_gru_bwd<double>(dgi, dgh, dh, dh_accumulate, g, gi_act, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_FLOAT16: rc = launch_gru_bwd<__half>(dgi, dgh, dh, dh_accumulate, g, gi_act, gh, h, rows, hidden, h_stride, device_id, s); break;
        case DTYPE_BFLOAT16: rc = launch_gru_bwd<__nv_bfloat16>(dgi, dgh, dh, dh_accumulate, g, gi_act, gh, h, rows, hidden, h_stride, device_id, s); break;
        default: rc = -1;
    }
    return rc;
}

long long rp_conv2d_col_elems(const RpbConv2d* c) {
    int oh, ow; long long cr, cc;
    if (conv_dims(c, &oh, &ow, &cr, &cc)) return -1;
    return (long long)c->N * cr * cc;
}

int rp_conv2d_out_shape(const RpbConv2d* c, int* out_h, int* out_w) {
    int oh, ow; long long cr, cc;
    if (conv_dims(c, &oh, &ow, &cr, &cc)) return -1;
    if (out_h) *out_h = oh;
    if (out_w) *out_w = ow;
    return 0;
}

int rp_conv2d_forward_ex(void* out, const void* input, const void* weight, void* col_all, const RpbConv2d* c, DType dtype,
                         int device_id, void* stream) {
    int oh, ow; long long cr, cc;
    if (!out || !input || !weight || !col_all || device_id < 0 || !rpb_dtype_size((int)dtype) || conv_dims(c, &oh, &ow, &cr, &cc)) return -1;
    DeviceScope scope;
    if (scope.enter(device_id)) return -1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long total = (long long)c->N * cr * cc;
    int rc;
    switch ((int)dtype) {
        case DTYPE_FLOAT32: rc = launch_im2col<float>(col_all, input, *c, oh, ow, total, device_id, s); break;
        case DTYPE_FLOAT64: rc = launch_im2col<double>(col_all, input, *c, oh, ow, total, device_id, s); break;
        case DTYPE_FLOAT16: rc = launch_im2col<__half>(col_all, input, *c, oh, ow, total, device_id, s); break;
        case DTYPE_BFLOAT16: rc = launch_im2col<__nv_bfloat16>(col_all, input, *c, oh, ow, total, device_id, s); break;
        default: rc = -1;
    }
    if (rc) return -1;
    /* out[img] = W[C_out, col_rows] . col[img][col_rows, col_cols]: the weight is a broadcast batch operand, one launch */
    RpbGemm g;
    rpb_gemm_packed(&g, c->C_out, (int)cr, (int)cc);
    g.batch = c->N; g.a_batch = 0; g.b_batch = cr * cc; g.c_batch = (long long)c->C_out * cc;
    return rp_matmul_ex(out, weight, col_all, &g, dtype, device_id, stream);
}

int rp_conv2d_backward_ex(void* grad_input, int accumulate_input, void* grad_weight, int accumulate_weight, const void* grad_out,
                          const void* weight, const void* col_all, void* dcol_ws, const RpbConv2d* c, DType dtype, int device_id,
                          void* stream) {
    int oh, ow; long long cr, cc;
    if (!grad_out || device_id < 0 || !rpb_dtype_size((int)dtype) || conv_dims(c, &oh, &ow, &cr, &cc)) return -1;
    if ((!grad_input && !grad_weight) || (grad_input && (!weight || !dcol_ws)) || (grad_weight && !col_all)) return -1;
    DeviceScope scope;
    if (scope.enter(device_id)) return -1;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (grad_weight) {
        /* dW[C_out, col_rows] (+)= sum over images of dout[img][C_out, col_cols] . col[img]^T: the images are summed
         * problems of ONE launch (fp32 sums, one rounding), col read transposed through its strides */
        RpbGemm g;
        memset(&g, 0, sizeof(g));
        g.m = c->C_out; g.n = (int)cr; g.k = (int)cc; g.batch = 1; g.reduce = c->N;
        g.a_row = cc; g.a_col = 1; g.a_reduce = (long long)c->C_out * cc;
        g.b_row = 1; g.b_col = cc; g.b_reduce = cr * cc;
        g.c_row = cr; g.accumulate = accumulate_weight ? 1 : 0;
        if (rp_matmul_ex(grad_weight, grad_out, col_all, &g, dtype, device_id, stream)) return -1;
    }
    if (grad_input) {
        /* dcol[img][col_rows, col_cols] = W^T . dout[img]: W read transposed through its strides, one launch */
        RpbGemm g;
        memset(&g, 0, sizeof(g));
        g.m = (int)cr; g.n = (int)cc; g.k = c->C_out; g.batch = c->N; g.reduce = 1;
        g.a_row = 1; g.a_col = cr; g.a_batch = 0;
        g.b_row = cc; g.b_col = 1; g.b_batch = (long long)c->C_out * cc;
        g.c_row = cc; g.c_batch = cr * cc;
        if (rp_matmul_ex(dcol_ws, weight, grad_out, &g, dtype, device_id, stream)) return -1;
        const long long total = (long long)c->N * c->C_in * c->H * c->W;
        int rc;
        switch ((int)dtype) {
            case DTYPE_FLOAT32: rc = launch_col2im<float>(grad_input, dcol_ws, *c, oh, ow, total, accumulate_input, device_id, s); break;
            case DTYPE_FLOAT64: rc = launch_col2im<double>(grad_input, dcol_ws, *c, oh, ow, total, accumulate_input, device_id, s); break;
            case DTYPE_FLOAT16: rc = launch_col2im<__half>(grad_input, dcol_ws, *c, oh, ow, total, accumulate_input, device_id, s); break;
            case DTYPE_BFLOAT16: rc = launch_col2im<__nv_bfloat16>(grad_input, dcol_ws, *c, oh, ow, total, accumulate_input, device_id, s); break;
            default: rc = -1;
        }
        if (rc) return -1;
    }
    return 0;
}

}  // extern "C"
