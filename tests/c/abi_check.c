/* Plain-C user of librecpulse_b200.so: includes the public header as C11, and (when run with "run" on
 * a machine with a GPU) multiplies a small bf16 problem through rp_matmul_host and through the autograd
 * node, checking the results against a scalar loop.  Exit code 0 = ok. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "recpulse_b200.h"

static uint16_t to_bf16(float f) { uint32_t u; memcpy(&u, &f, 4); return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16); }
static float from_bf16(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }

int main(int argc, char** argv) {
    printf("%s\n", rpb_version());
    if (argc < 2 || strcmp(argv[1], "run") != 0) return 0;      /* link check only */

    enum { M = 96, K = 160, N = 64 };
    static uint16_t a[M * K], b[K * N], c[M * N], g[M * N], da[M * K], db[K * N];
    static float ref[M * N];
    srand(1);
    for (int i = 0; i < M * K; i++) a[i] = to_bf16((float)rand() / RAND_MAX - 0.5f);
    for (int i = 0; i < K * N; i++) b[i] = to_bf16((float)rand() / RAND_MAX - 0.5f);
    for (int i = 0; i < M * N; i++) g[i] = to_bf16(1.0f);
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float s = 0.f;
            for (int l = 0; l < K; l++) s += from_bf16(a[i * K + l]) * from_bf16(b[l * N + j]);
            ref[i * N + j] = s;
        }
    if (rp_matmul_host(c, a, b, M, K, N, DTYPE_BFLOAT16, 0) != 0) { fprintf(stderr, "rp_matmul_host failed\n"); return 1; }
    double num = 0, den = 0;
    for (int i = 0; i < M * N; i++) { double d = from_bf16(c[i]) - ref[i]; num += d * d; den += (double)ref[i] * ref[i]; }
    if (sqrt(num / den) > 1e-2) { fprintf(stderr, "rp_matmul_host: relative error %g\n", sqrt(num / den)); return 1; }

    /* the autograd node on RecPulse's own structs */
    int sa[2] = {M, K}, sb[2] = {K, N}, sg[2] = {M, N};
    Tensor* A = rpb_tensor_from_host(a, DTYPE_BFLOAT16, 2, sa, 0, true);
    Tensor* B = rpb_tensor_from_host(b, DTYPE_BFLOAT16, 2, sb, 0, true);
    Tensor* G = rpb_tensor_from_host(g, DTYPE_BFLOAT16, 2, sg, 0, false);
    if (!A || !B || !G) return 1;
    Tensor* Y = op_matmul(A, B);
    if (!Y || !Y->metadata || !Y->metadata->grad_fn || A->refcount != 2) { fprintf(stderr, "op_matmul node wrong\n"); return 1; }
    if (rpb_backward_node(Y, G) != 0 || !A->metadata->grad || !B->metadata->grad || A->refcount != 1) return 1;
    if (rpb_tensor_to_host(A->metadata->grad, da) != 0 || rpb_tensor_to_host(B->metadata->grad, db) != 0) return 1;
    /* dA = 1 . B^T: every row is the row sums of B */
    for (int l = 0; l < K; l++) {
        float s = 0.f;
        for (int j = 0; j < N; j++) s += from_bf16(b[l * N + j]);
        if (fabsf(from_bf16(da[l]) - s) > 0.02f * (fabsf(s) + 1.f)) { fprintf(stderr, "dA[%d] = %g, expected %g\n", l, from_bf16(da[l]), s); return 1; }
    }
    if (op_matmul(A, G) != NULL) { fprintf(stderr, "inner-dimension mismatch accepted\n"); return 1; }
    rpb_tensor_release(Y); rpb_tensor_release(G); rpb_tensor_release(A); rpb_tensor_release(B);
    if (rpb_device_status(0) != 0) return 1;
    printf("C ABI OK\n");
    return 0;
}
