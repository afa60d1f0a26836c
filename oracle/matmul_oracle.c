/*
 * TEST INFRASTRUCTURE ONLY -- see matmul_oracle.h.  Every function cites the
 * reference lines it restates.  Build with -ffp-contract=off (oracle/Makefile):
 * the reference's loops round the multiply and the add separately.
 */
#include "matmul_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>

static size_t esize(int dtype) {
    switch (dtype) {
        case ORC_F32: return 4;
        case ORC_F64: return 8;
        case ORC_F16: case ORC_BF16: return 2;
        default: return 0;
    }
}

static float bits_to_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t float_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* core/half_precision.h:20-48 */
float orc_fp16_to_fp32(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, frac = h & 0x3FFu;
    if (e == 0) {
        if (!frac) return bits_to_float(s);
        /* subnormal: frac/1024 * 2^-14, both steps exact in fp32 */
        float v = ((float)frac / 1024.0f) * (1.0f / 16384.0f);
        return s ? -v : v;
    }
    if (e == 0x1Fu) return bits_to_float(s | 0x7F800000u | (frac << 13));
    return bits_to_float(s | ((e + 112u) << 23) | (frac << 13));
}

/* core/half_precision.h:50-83: round-half-UP on the dropped bits (not RNE); the
 * carry of the +1 is allowed to ripple into the exponent field. */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t u = float_to_bits(f);
    uint32_t s = (u >> 16) & 0x8000u;
    uint32_t be = (u >> 23) & 0xFFu;
    uint32_t frac = u & 0x7FFFFFu;
    int32_t e = (int32_t)be - 112;              /* -127 + 15 */
    if (be == 0xFFu)
        return (uint16_t)(frac ? (s | 0x7C00u | (frac >> 13) | 1u) : (s | 0x7C00u));
    if (e <= 0) {
        if (e < -10) return (uint16_t)s;
        frac |= 0x800000u;
        int sh = 14 - e;
        uint16_t r = (uint16_t)(s | (frac >> sh));
        return (uint16_t)(r + ((frac >> (sh - 1)) & 1u));
    }
    if (e >= 0x1F) return (uint16_t)(s | 0x7C00u);
    uint16_t r = (uint16_t)(s | ((uint32_t)e << 10) | (frac >> 13));
    return (uint16_t)(r + ((frac >> 12) & 1u));
}

/* core/half_precision.h:85-90 */
float orc_bf16_to_fp32(uint16_t h) { return bits_to_float((uint32_t)h << 16); }

/* core/half_precision.h:92-97: add bit 15 to the upper half, no NaN special case */
uint16_t orc_fp32_to_bf16(float f) {
    uint32_t u = float_to_bits(f);
    return (uint16_t)((u >> 16) + ((u >> 15) & 1u));
}

/* core/half_precision.h:115-127 */
void orc_widen(const void* src, float* dst, size_t n, int dtype) {
    const uint16_t* s = (const uint16_t*)src;
    if (dtype == ORC_F16) for (size_t i = 0; i < n; i++) dst[i] = orc_fp16_to_fp32(s[i]);
    else                  for (size_t i = 0; i < n; i++) dst[i] = orc_bf16_to_fp32(s[i]);
}
void orc_narrow(const float* src, void* dst, size_t n, int dtype) {
    uint16_t* d = (uint16_t*)dst;
    if (dtype == ORC_F16) for (size_t i = 0; i < n; i++) d[i] = orc_fp32_to_fp16(src[i]);
    else                  for (size_t i = 0; i < n; i++) d[i] = orc_fp32_to_bf16(src[i]);
}

/* functional/functional_host.c:780-792.  The running sum lives in C itself, in
 * the storage precision, in (i, j, l) order. */
int orc_matmul_f32(float* C, const float* A, const float* B, int m, int k, int n) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    for (int i = 0; i < m; i++) {
        const float* arow = A + (size_t)i * k;
        for (int j = 0; j < n; j++) {
            volatile float acc = 0.0f;          /* forces a rounding per step */
            for (int l = 0; l < k; l++) {
                float p = arow[l] * B[(size_t)l * n + j];
                acc = acc + p;
            }
            C[(size_t)i * n + j] = acc;
        }
    }
    return 0;
}

/* functional/functional_host.c:794-806 */
int orc_matmul_f64(double* C, const double* A, const double* B, int m, int k, int n) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    for (int i = 0; i < m; i++) {
        const double* arow = A + (size_t)i * k;
        for (int j = 0; j < n; j++) {
            volatile double acc = 0.0;
            for (int l = 0; l < k; l++) {
                double p = arow[l] * B[(size_t)l * n + j];
                acc = acc + p;
            }
            C[(size_t)i * n + j] = acc;
        }
    }
    return 0;
}

/* functional/functional.c:978-1002: f16/bf16 are widened to fp32, multiplied by
 * the fp32 loop and narrowed once at the end. */
int orc_rp_matmul(void* C, const void* A, const void* B, int m, int k, int n, int dtype) {
    if (!C || !A || !B || m <= 0 || k <= 0 || n <= 0) return -1;
    if (dtype == ORC_F32) return orc_matmul_f32((float*)C, (const float*)A, (const float*)B, m, k, n);
    if (dtype == ORC_F64) return orc_matmul_f64((double*)C, (const double*)A, (const double*)B, m, k, n);
    if (dtype != ORC_F16 && dtype != ORC_BF16) return -1;
    size_t na = (size_t)m * k, nb = (size_t)k * n, nc = (size_t)m * n;
    float* wa = (float*)malloc(na * 4);
    float* wb = (float*)malloc(nb * 4);
    float* wc = (float*)malloc(nc * 4);
    int rc = -1;
    if (wa && wb && wc) {
        orc_widen(A, wa, na, dtype);
        orc_widen(B, wb, nb, dtype);
        rc = orc_matmul_f32(wc, wa, wb, m, k, n);
        if (rc == 0) orc_narrow(wc, C, nc, dtype);
    }
    free(wa); free(wb); free(wc);
    return rc;
}

/* functional/functional.c:1130-1220: element gather in row-major index order. */
int orc_contiguous(void* dst, const void* src, int ndim, const int* shape,
                   const int* strides, int dtype) {
    size_t es = esize(dtype);
    if (!dst || !src || ndim <= 0 || ndim > 8 || !es) return -1;
    size_t total = 1;
    for (int d = 0; d < ndim; d++) { if (shape[d] <= 0) return -1; total *= (size_t)shape[d]; }
    int idx[8] = {0};
    for (size_t o = 0; o < total; o++) {
        long off = 0;
        for (int d = 0; d < ndim; d++) off += (long)idx[d] * strides[d];
        memcpy((char*)dst + o * es, (const char*)src + off * (long)es, es);
        for (int d = ndim - 1; d >= 0; d--) { if (++idx[d] < shape[d]) break; idx[d] = 0; }
    }
    return 0;
}

static void* packed_copy(const void* src, const int* strides, int rows, int cols, int dtype) {
    int shape[2] = {rows, cols};
    int packed[2] = {cols, 1};
    void* p = malloc((size_t)rows * cols * esize(dtype));
    if (!p) return NULL;
    if (orc_contiguous(p, src, 2, shape, strides ? strides : packed, dtype) != 0) { free(p); return NULL; }
    return p;
}

/* ops/ops.c:6816-6847: both inputs are made contiguous (ensure_contiguous,
 * ops.c:21-25), then rp_matmul. */
int orc_op_matmul(void* C, const void* A, const int* a_strides, const void* B,
                  const int* b_strides, int m, int k, int n, int dtype) {
    if (m <= 0 || k <= 0 || n <= 0) return -1;
    void* ac = packed_copy(A, a_strides, m, k, dtype);
    void* bc = packed_copy(B, b_strides, k, n, dtype);
    int rc = (ac && bc) ? orc_rp_matmul(C, ac, bc, m, k, n, dtype) : -1;
    free(ac); free(bc);
    return rc;
}

/* functional_host.c add (element-wise a+b in the storage dtype); for f16/bf16 the
 * reference's rp_add widens each element, adds in fp32 and narrows. */
static void grad_add(void* acc, const void* inc, size_t cnt, int dtype) {
    if (dtype == ORC_F32) { float* a = (float*)acc; const float* b = (const float*)inc; for (size_t i = 0; i < cnt; i++) a[i] = a[i] + b[i]; }
    else if (dtype == ORC_F64) { double* a = (double*)acc; const double* b = (const double*)inc; for (size_t i = 0; i < cnt; i++) a[i] = a[i] + b[i]; }
    else {
        uint16_t* a = (uint16_t*)acc; const uint16_t* b = (const uint16_t*)inc;
        for (size_t i = 0; i < cnt; i++) {
            float x, y;
            orc_widen(&a[i], &x, 1, dtype); orc_widen(&b[i], &y, 1, dtype);
            float s = x + y;
            orc_narrow(&s, &a[i], 1, dtype);
        }
    }
}

/* ops/ops.c:6759-6814: dA[m,k] = dC[m,n] x contiguous(B^T)[n,k],
 * dB[k,n] = contiguous(A^T)[k,m] x dC[m,n]. */
int orc_matmul_backward(void* dA, void* dB, const void* A, const int* a_strides,
                        const void* B, const int* b_strides, const void* dC,
                        int m, int k, int n, int dtype, int accumulate) {
    size_t es = esize(dtype);
    if (!es || m <= 0 || k <= 0 || n <= 0 || !dC) return -1;
    int pa[2] = {k, 1}, pb[2] = {n, 1};
    if (!a_strides) a_strides = pa;
    if (!b_strides) b_strides = pb;
    if (dA) {
        int ts[2] = {b_strides[1], b_strides[0]};          /* rp_transpose view of B */
        void* bt = packed_copy(B, ts, n, k, dtype);
        void* g = malloc((size_t)m * k * es);
        int rc = (bt && g) ? orc_rp_matmul(g, dC, bt, m, n, k, dtype) : -1;
        if (rc == 0) { if (accumulate) grad_add(dA, g, (size_t)m * k, dtype); else memcpy(dA, g, (size_t)m * k * es); }
        free(bt); free(g);
        if (rc) return rc;
    }
    if (dB) {
        int ts[2] = {a_strides[1], a_strides[0]};
        void* at = packed_copy(A, ts, k, m, dtype);
        void* g = malloc((size_t)k * n * es);
        int rc = (at && g) ? orc_rp_matmul(g, at, dC, k, m, n, dtype) : -1;
        if (rc == 0) { if (accumulate) grad_add(dB, g, (size_t)k * n, dtype); else memcpy(dB, g, (size_t)k * n * es); }
        free(at); free(g);
        if (rc) return rc;
    }
    return 0;
}

int orc_bmm(void* C, const void* A, const void* B, int batch, size_t a_bstride,
            size_t b_bstride, int m, int k, int n, int dtype) {
    size_t es = esize(dtype);
    if (!es || batch <= 0) return -1;
    for (int b = 0; b < batch; b++) {
        int rc = orc_rp_matmul((char*)C + (size_t)b * m * n * es,
                               (const char*)A + b * a_bstride * es,
                               (const char*)B + b * b_bstride * es, m, k, n, dtype);
        if (rc) return rc;
    }
    return 0;
}

/* Unrounded per-batch product in the accumulation type (float, or double for f64). */
static int wide_product(void* out, const void* X, const void* Y, int m, int k, int n, int dtype) {
    if (dtype == ORC_F64) return orc_matmul_f64((double*)out, (const double*)X, (const double*)Y, m, k, n);
    if (dtype == ORC_F32) return orc_matmul_f32((float*)out, (const float*)X, (const float*)Y, m, k, n);
    float* wx = (float*)malloc((size_t)m * k * 4);
    float* wy = (float*)malloc((size_t)k * n * 4);
    int rc = -1;
    if (wx && wy) {
        orc_widen(X, wx, (size_t)m * k, dtype); orc_widen(Y, wy, (size_t)k * n, dtype);
        rc = orc_matmul_f32((float*)out, wx, wy, m, k, n);
    }
    free(wx); free(wy);
    return rc;
}

static void* transpose_packed(const void* X, int rows, int cols, int dtype) {
    int ts[2] = {1, cols};
    return packed_copy(X, ts, cols, rows, dtype);
}

int orc_bmm_backward(void* dA, void* dB, const void* A, const void* B, const void* dC,
                     int batch, size_t a_bstride, size_t b_bstride,
                     int m, int k, int n, int dtype) {
    size_t es = esize(dtype), ws = (dtype == ORC_F64) ? 8 : 4;
    if (!es || batch <= 0) return -1;
    int rc = 0;
    for (int side = 0; side < 2 && !rc; side++) {
        void* grad = side == 0 ? dA : dB;
        if (!grad) continue;
        size_t bstride = side == 0 ? a_bstride : b_bstride;
        int gr = side == 0 ? m : k, gc = side == 0 ? k : n;
        size_t gsz = (size_t)gr * gc;
        int reduce = (bstride == 0 && batch > 1);
        void* sum = reduce ? calloc(gsz, ws) : NULL;
        void* tmp = reduce ? malloc(gsz * ws) : NULL;
        if (reduce && (!sum || !tmp)) { free(sum); free(tmp); return -1; }
        for (int b = 0; b < batch && !rc; b++) {
            const char* Ab = (const char*)A + b * a_bstride * es;
            const char* Bb = (const char*)B + b * b_bstride * es;
            const char* Gb = (const char*)dC + (size_t)b * m * n * es;
            void* t = side == 0 ? transpose_packed(Bb, k, n, dtype) : transpose_packed(Ab, m, k, dtype);
            if (!t) { rc = -1; break; }
            if (!reduce) {
                char* out = (char*)grad + b * bstride * es;
                rc = side == 0 ? orc_rp_matmul(out, Gb, t, m, n, k, dtype)
                               : orc_rp_matmul(out, t, Gb, k, m, n, dtype);
            } else {
                rc = side == 0 ? wide_product(tmp, Gb, t, m, n, k, dtype)
                               : wide_product(tmp, t, Gb, k, m, n, dtype);
                if (!rc) {
                    if (ws == 8) for (size_t i = 0; i < gsz; i++) ((double*)sum)[i] += ((double*)tmp)[i];
                    else         for (size_t i = 0; i < gsz; i++) ((float*)sum)[i] = ((float*)sum)[i] + ((float*)tmp)[i];
                }
            }
            free(t);
        }
        if (reduce && !rc) {
            if (dtype == ORC_F64 || dtype == ORC_F32) memcpy(grad, sum, gsz * ws);
            else orc_narrow((const float*)sum, grad, gsz, dtype);
        }
        free(sum); free(tmp);
    }
    return rc;
}

/* recpulse/module.py:110-114 + ops/ops.c:129-210 */
int orc_linear_forward(void* Y, const void* X, const void* W, const void* bias, int m, int k, int n, int dtype) {
    int rc = orc_rp_matmul(Y, X, W, m, k, n, dtype);
    if (rc || !bias) return rc;
    for (int i = 0; i < m; i++) {
        if (dtype == ORC_F32) { float* y = (float*)Y + (size_t)i * n; const float* b = (const float*)bias; for (int j = 0; j < n; j++) y[j] = y[j] + b[j]; }
        else if (dtype == ORC_F64) { double* y = (double*)Y + (size_t)i * n; const double* b = (const double*)bias; for (int j = 0; j < n; j++) y[j] = y[j] + b[j]; }
        else grad_add((uint16_t*)Y + (size_t)i * n, bias, (size_t)n, dtype);   /* widen, add, narrow per element */
    }
    return 0;
}

/* ops/ops.c:6970-7101 */
int orc_bias_grad(void* dbias, const void* dY, long long rows, int n, int dtype) {
    if (!dbias || !dY || rows <= 0 || n <= 0) return -1;
    if (dtype == ORC_F64) {
        double* r = (double*)dbias; const double* g = (const double*)dY;
        for (int j = 0; j < n; j++) r[j] = 0.0;
        for (long long i = 0; i < rows; i++) for (int j = 0; j < n; j++) { volatile double t = r[j] + g[i * n + j]; r[j] = t; }
        return 0;
    }
    float* acc = (float*)calloc((size_t)n, sizeof(float));
    if (!acc) return -1;
    for (long long i = 0; i < rows; i++)
        for (int j = 0; j < n; j++) {
            float g;
            if (dtype == ORC_F32) g = ((const float*)dY)[i * n + j];
            else orc_widen((const uint16_t*)dY + i * n + j, &g, 1, dtype);
            volatile float t = acc[j] + g; acc[j] = t;
        }
    if (dtype == ORC_F32) memcpy(dbias, acc, (size_t)n * 4); else orc_narrow(acc, dbias, (size_t)n, dtype);
    free(acc);
    return 0;
}

/* recpulse/module.py:289-300 over functional/functional_host.c:498-545 */
int orc_lstm_gates_forward(void* Y, const void* X, const void* W, const void* H, const void* U, const void* bias,
                           int m, int kx, int kh, int n, int dtype) {
    if (!Y || !X || !W || !H || !U || m <= 0 || kx <= 0 || kh <= 0 || n <= 0 || n % 4 != 0) return -1;
    const size_t es = dtype == ORC_F64 ? 8 : (dtype == ORC_F32 ? 4 : 2);
    const size_t cnt = (size_t)m * n;
    void* t2 = malloc(cnt * es);
    if (!t2) return -1;
    int rc = orc_rp_matmul(Y, X, W, m, kx, n, dtype);
    if (rc == 0) rc = orc_rp_matmul(t2, H, U, m, kh, n, dtype);
    if (rc) { free(t2); return rc; }
    const int q = n / 4;
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            const size_t e = (size_t)i * n + j;
            const int is_tanh = j >= 2 * q && j < 3 * q;
            if (dtype == ORC_F64) {
                double* y = (double*)Y; const double* b = (const double*)bias;
                volatile double v = y[e] + ((const double*)t2)[e];
                if (b) { volatile double w2 = v + b[j]; v = w2; }
                y[e] = is_tanh ? tanh(v) : 1.0 / (1.0 + exp(-v));
            } else if (dtype == ORC_F32) {
                float* y = (float*)Y; const float* b = (const float*)bias;
                volatile float v = y[e] + ((const float*)t2)[e];
                if (b) { volatile float w2 = v + b[j]; v = w2; }
                y[e] = is_tanh ? tanhf(v) : 1.0f / (1.0f + expf(-v));
            } else {
                uint16_t* y = (uint16_t*)Y;
                float a, c, s;
                orc_widen(y + e, &a, 1, dtype); orc_widen((const uint16_t*)t2 + e, &c, 1, dtype);
                s = a + c; orc_narrow(&s, y + e, 1, dtype);                       /* op_add rounds */
                if (bias) {
                    orc_widen(y + e, &a, 1, dtype); orc_widen((const uint16_t*)bias + j, &c, 1, dtype);
                    s = a + c; orc_narrow(&s, y + e, 1, dtype);
                }
                orc_widen(y + e, &a, 1, dtype);
                s = is_tanh ? tanhf(a) : 1.0f / (1.0f + expf(-a));
                orc_narrow(&s, y + e, 1, dtype);
            }
        }
    free(t2);
    return 0;
}

/* ops/grad_host.c:365-385, 622-640 */
int orc_lstm_gates_grad(void* dpre, const void* dY, const void* Y, long long rows, int n, int dtype) {
    if (!dpre || !dY || !Y || rows <= 0 || n <= 0 || n % 4 != 0) return -1;
    const int q = n / 4;
    for (long long i = 0; i < rows; i++)
        for (int j = 0; j < n; j++) {
            const size_t e = (size_t)i * n + j;
            const int is_tanh = j >= 2 * q && j < 3 * q;
            if (dtype == ORC_F64) {
                const double g = ((const double*)dY)[e], y = ((const double*)Y)[e];
                ((double*)dpre)[e] = is_tanh ? g * (1 - y * y) : g * y * (1.0 - y);
            } else {
                float g, y, r;
                if (dtype == ORC_F32) { g = ((const float*)dY)[e]; y = ((const float*)Y)[e]; }
                else { orc_widen((const uint16_t*)dY + e, &g, 1, dtype); orc_widen((const uint16_t*)Y + e, &y, 1, dtype); }
                r = is_tanh ? g * (1.0f - y * y) : g * y * (1.0f - y);
                if (dtype == ORC_F32) ((float*)dpre)[e] = r; else orc_narrow(&r, (uint16_t*)dpre + e, 1, dtype);
            }
        }
    return 0;
}

/* ------------------------------------------------------------------ GRU cell, recpulse/module.py:329-348
 * The cell is restated node by node, each node's output rounded to the storage dtype exactly where the
 * reference rounds it (float16 / bfloat16: widen, compute in float, narrow -- functional/functional.c's HALF
 * branches and ops/grad_host.c:61-79; float32 / float64: native arithmetic). */

typedef double (*Ew2)(double, double);          /* only used to name the operation; arithmetic is per dtype below */
enum { EW_ADD, EW_MUL, EW_RSUB1, EW_SIGMOID, EW_TANH, EW_NEG, EW_DSIGMOID, EW_DTANH };

/* out[i] = op(a[i], b[i]) in the storage dtype.  EW_RSUB1: 1 - a (functional_host.c:226-240); EW_SIGMOID / EW_TANH
 * (functional_host.c:498-545); EW_NEG: -a (backwards_sub_x2, grad_host.c:149); EW_DSIGMOID: a * b * (1 - b) and
 * EW_DTANH: a * (1 - b * b) with a = upstream gradient, b = the node's output (grad_host.c:365-385, 622-640). */
static void ew(void* out, const void* a, const void* b, size_t n, int op, int dtype) {
    for (size_t i = 0; i < n; i++) {
        if (dtype == ORC_F64) {
            const double x = ((const double*)a)[i], y = b ? ((const double*)b)[i] : 0.0;
            double r;
            switch (op) {
                case EW_ADD: r = x + y; break;
                case EW_MUL: r = x * y; break;
                case EW_RSUB1: r = 1.0 - x; break;
                case EW_SIGMOID: r = 1.0 / (1.0 + exp(-x)); break;
                case EW_TANH: r = tanh(x); break;
                case EW_NEG: r = -x; break;
                case EW_DSIGMOID: r = x * y * (1.0 - y); break;
                default: r = x * (1.0 - y * y); break;
            }
            ((double*)out)[i] = r;
        } else {
            float x, y = 0.0f, r;
            if (dtype == ORC_F32) { x = ((const float*)a)[i]; if (b) y = ((const float*)b)[i]; }
            else { orc_widen((const uint16_t*)a + i, &x, 1, dtype); if (b) orc_widen((const uint16_t*)b + i, &y, 1, dtype); }
            switch (op) {
                case EW_ADD: r = x + y; break;
                case EW_MUL: r = x * y; break;
                case EW_RSUB1: r = 1.0f - x; break;
                case EW_SIGMOID: r = 1.0f / (1.0f + expf(-x)); break;
                case EW_TANH: r = tanhf(x); break;
                case EW_NEG: r = -x; break;
                case EW_DSIGMOID: r = x * y * (1.0f - y); break;
                default: r = x * (1.0f - y * y); break;
            }
            if (dtype == ORC_F32) ((float*)out)[i] = r; else orc_narrow(&r, (uint16_t*)out + i, 1, dtype);
        }
    }
}

/* columns [c0, c0 + w) of a packed [rows, cols] matrix as a packed [rows, w] copy (chunk + contiguous) */
static void take_cols(void* out, const void* in, int rows, int cols, int c0, int w, size_t es) {
    for (int i = 0; i < rows; i++)
        memcpy((char*)out + (size_t)i * w * es, (const char*)in + ((size_t)i * cols + c0) * es, (size_t)w * es);
}
static void put_cols(void* out, const void* in, int rows, int cols, int c0, int w, size_t es) {
    for (int i = 0; i < rows; i++)
        memcpy((char*)out + ((size_t)i * cols + c0) * es, (const char*)in + (size_t)i * w * es, (size_t)w * es);
}
/* out[i][j] = a[i][j] + bias[j]: the broadcast op_add (ops/ops.c:129-210) */
static void add_bias_rows(void* out, const void* a, const void* bias, int rows, int cols, int dtype) {
    const size_t es = esize(dtype);
    for (int i = 0; i < rows; i++)
        ew((char*)out + (size_t)i * cols * es, (const char*)a + (size_t)i * cols * es, bias, (size_t)cols, EW_ADD, dtype);
}

typedef struct { void *gi, *gh, *r, *z, *n, *hn, *t1, *h_next; } GruState;

static void gru_free(GruState* s) {
    free(s->gi); free(s->gh); free(s->r); free(s->z); free(s->n); free(s->hn); free(s->t1); free(s->h_next);
}

static int gru_forward_state(GruState* s, const void* X, const void* Wih, const void* H, const void* Whh, const void* bih,
                             const void* bhh, int m, int kx, int hd, int dtype) {
    const size_t es = esize(dtype), mh = (size_t)m * hd, m3 = 3 * mh;
    memset(s, 0, sizeof(*s));
    s->gi = malloc(m3 * es); s->gh = malloc(m3 * es);
    s->r = malloc(mh * es); s->z = malloc(mh * es); s->n = malloc(mh * es); s->hn = malloc(mh * es);
    s->t1 = malloc(mh * es); s->h_next = malloc(mh * es);
    void* a = malloc(mh * es); void* b = malloc(mh * es);
    int rc = (s->gi && s->gh && s->r && s->z && s->n && s->hn && s->t1 && s->h_next && a && b) ? 0 : -1;
    if (!rc) rc = orc_rp_matmul(s->gi, X, Wih, m, kx, 3 * hd, dtype);
    if (!rc) rc = orc_rp_matmul(s->gh, H, Whh, m, hd, 3 * hd, dtype);
    if (!rc) {
        if (bih) add_bias_rows(s->gi, s->gi, bih, m, 3 * hd, dtype);
        if (bhh) add_bias_rows(s->gh, s->gh, bhh, m, 3 * hd, dtype);
        take_cols(a, s->gi, m, 3 * hd, 0, hd, es); take_cols(b, s->gh, m, 3 * hd, 0, hd, es);
        ew(a, a, b, mh, EW_ADD, dtype); ew(s->r, a, NULL, mh, EW_SIGMOID, dtype);             /* r = sigmoid(i_r + h_r) */
        take_cols(a, s->gi, m, 3 * hd, hd, hd, es); take_cols(b, s->gh, m, 3 * hd, hd, hd, es);
        ew(a, a, b, mh, EW_ADD, dtype); ew(s->z, a, NULL, mh, EW_SIGMOID, dtype);             /* z = sigmoid(i_z + h_z) */
        take_cols(a, s->gi, m, 3 * hd, 2 * hd, hd, es); take_cols(s->hn, s->gh, m, 3 * hd, 2 * hd, hd, es);
        ew(b, s->r, s->hn, mh, EW_MUL, dtype);                                                /* r * h_n */
        ew(a, a, b, mh, EW_ADD, dtype); ew(s->n, a, NULL, mh, EW_TANH, dtype);                /* n = tanh(i_n + r h_n) */
        ew(s->t1, s->z, NULL, mh, EW_RSUB1, dtype);                                           /* 1 - z */
        ew(a, s->t1, s->n, mh, EW_MUL, dtype);                                                /* (1 - z) n */
        ew(b, s->z, H, mh, EW_MUL, dtype);                                                    /* z h */
        ew(s->h_next, a, b, mh, EW_ADD, dtype);
    }
    free(a); free(b);
    return rc;
}

int orc_gru_cell_forward(void* Hn, const void* X, const void* Wih, const void* H, const void* Whh, const void* bih,
                         const void* bhh, int m, int kx, int hd, int dtype) {
    if (!Hn || !X || !Wih || !H || !Whh || m <= 0 || kx <= 0 || hd <= 0 || !esize(dtype)) return -1;
    GruState s;
    int rc = gru_forward_state(&s, X, Wih, H, Whh, bih, bhh, m, kx, hd, dtype);
    if (!rc) memcpy(Hn, s.h_next, (size_t)m * hd * esize(dtype));
    gru_free(&s);
    return rc;
}

/* The backward chain of the same nodes (ops/ops.c:77-127 add, :322-420 mul, :1564-1660 tanh / sigmoid, :6260-6283
 * rsub_scalar, chunk / slice scatter, matmul :6759-6814, bias through reduce_grad_to_shape) for the upstream
 * gradient G of h'.  Gradients that collect two contributions (z, h) add them with one rounding, as rp_add does. */
int orc_gru_cell_backward(void* dX, void* dWih, void* dH, void* dWhh, void* dbih, void* dbhh, const void* G, const void* X,
                          const void* Wih, const void* H, const void* Whh, const void* bih, const void* bhh,
                          int m, int kx, int hd, int dtype) {
    if (!G || !X || !Wih || !H || !Whh || m <= 0 || kx <= 0 || hd <= 0 || !esize(dtype)) return -1;
    const size_t es = esize(dtype), mh = (size_t)m * hd, m3 = 3 * mh;
    GruState s;
    int rc = gru_forward_state(&s, X, Wih, H, Whh, bih, bhh, m, kx, hd, dtype);
    void *dn = malloc(mh * es), *dz = malloc(mh * es), *t = malloc(mh * es), *dan = malloc(mh * es), *daz = malloc(mh * es),
         *dar = malloc(mh * es), *dhn = malloc(mh * es), *dh1 = malloc(mh * es), *dgi = malloc(m3 * es), *dgh = malloc(m3 * es),
         *dh2 = malloc(mh * es);
    if (!dn || !dz || !t || !dan || !daz || !dar || !dhn || !dh1 || !dgi || !dgh || !dh2) rc = -1;
    if (!rc) {
        ew(t, G, s.n, mh, EW_MUL, dtype);                /* d(1 - z) = G n                      */
        ew(dn, G, s.t1, mh, EW_MUL, dtype);              /* dn = G (1 - z)                      */
        ew(dz, G, H, mh, EW_MUL, dtype);                 /* dz (from z h) = G h                 */
        ew(dh1, G, s.z, mh, EW_MUL, dtype);              /* dh (from z h) = G z                 */
        ew(t, t, NULL, mh, EW_NEG, dtype);               /* through 1 - z: -G n                 */
        ew(dz, dz, t, mh, EW_ADD, dtype);                /* both uses of z                      */
        ew(dan, dn, s.n, mh, EW_DTANH, dtype);           /* through tanh                        */
        ew(dar, dan, s.hn, mh, EW_MUL, dtype);           /* dr = da_n h_n                       */
        ew(dhn, dan, s.r, mh, EW_MUL, dtype);            /* dh_n = da_n r                       */
        ew(dar, dar, s.r, mh, EW_DSIGMOID, dtype);       /* through sigmoid                     */
        ew(daz, dz, s.z, mh, EW_DSIGMOID, dtype);
        put_cols(dgi, dar, m, 3 * hd, 0, hd, es); put_cols(dgi, daz, m, 3 * hd, hd, hd, es); put_cols(dgi, dan, m, 3 * hd, 2 * hd, hd, es);
        put_cols(dgh, dar, m, 3 * hd, 0, hd, es); put_cols(dgh, daz, m, 3 * hd, hd, hd, es); put_cols(dgh, dhn, m, 3 * hd, 2 * hd, hd, es);
        int sx[2] = {kx, 1}, swi[2] = {3 * hd, 1}, sh[2] = {hd, 1};
        rc = orc_matmul_backward(dX, dWih, X, sx, Wih, swi, dgi, m, kx, 3 * hd, dtype, 0);
        if (!rc) rc = orc_matmul_backward(dh2, dWhh, H, sh, Whh, swi, dgh, m, hd, 3 * hd, dtype, 0);
        if (!rc && dH) ew(dH, dh1, dh2, mh, EW_ADD, dtype);
        if (!rc && dbih) rc = orc_bias_grad(dbih, dgi, m, 3 * hd, dtype);
        if (!rc && dbhh) rc = orc_bias_grad(dbhh, dgh, m, 3 * hd, dtype);
    }
    free(dn); free(dz); free(t); free(dan); free(daz); free(dar); free(dhn); free(dh1); free(dgi); free(dgh); free(dh2);
    gru_free(&s);
    return rc;
}
