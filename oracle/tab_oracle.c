/*
 * CPU oracle for TAB's quantise + popcount-convolution path, in plain C with OpenMP.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA path is compared with, and the "port"
 * CPU baseline the benchmark times.  Nothing in the product path links or calls it.
 *
 * It restates the reference's pipeline stage by stage, with the same loop structure as the
 * reference's CPU backend: quantise -> zero-bordered pad -> explicit im2row -> popcount GEMM
 * (OpenMP parallel-for over output rows, scalar 64-bit popcount) -> float32.
 *
 *   quantise   TAB_GEMM.cu:163-208 (ternary), :211-247 (binary), :150-160 (BTN_W); per-n threshold
 *              ths[n] as in TAB_CPU.cpp:67,72; NHWC input as in TAB_GEMM.cu:184,231
 *   pad        TAB_GEMM.cuh:73-89 with zero borders (TAB_CPU.cpp:39,155)
 *   im2row     TAB_GEMM.cuh:92-115 (== TAB_CPU.h:27-63 for 3x3)
 *   GEMMs      TAB_CPU.cpp:242-328 (== TAB_GEMM.cu:25-147)
 *   pipeline   TAB_GEMM.cu:325-527; output float32 [N][OH][OW][KN] (:349,:509,:526)
 *
 * Parity status: pinned, stage by stage, against the reference's own code run on the host - its CUDA
 * kernel bodies (TAB_GEMM.cu:25-247, TAB_GEMM.cuh:73-115) and its CPU GEMMs (TAB_CPU.cpp:242-328),
 * both compiled by build.py from the files where they lie into oracle/_ref - and against the
 * committed golden vectors that code produced; the reference itself ships no golden vectors.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define CNTBITS 64
#define popcnt64(a) __builtin_popcountll(a)

static int packed_channels(int C) { return (C + CNTBITS - 1) / CNTBITS; }
static int act_bits(int type) { return (type == 2 || type == 3) ? 1 : 2; }      /* TAB_GEMM.cu:367-372 */
static int weight_bits(int type) { return (type == 1 || type == 3) ? 1 : 2; }   /* TAB_GEMM.cu:374-379 */

/* fp32 NHWC -> packed planes [N][H][W][PC][bits]; btn[n] = popcount of the magnitude plane (bits 2). */
void oracle_quantize(const float* x, const float* ths, int64_t* qx, int32_t* btn,
                     int bitwidth, int N, int H, int W, int C) {
    const int PC = packed_channels(C);
    const int bits = (bitwidth == 1) ? 1 : 2;                     /* TAB_GEMM.cu:267,309 */
    const long HW = (long)H * W;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float t = ths[n];
        long cnt = 0;
        for (long hw = 0; hw < HW; hw++) {
            const float* row = x + ((long)n * HW + hw) * C;
            int64_t* out = qx + ((long)n * HW + hw) * PC * bits;
            for (int pc = 0; pc < PC; pc++) {
                uint64_t b1 = 0, b2 = 0;
                const int cend = (pc + 1) * CNTBITS < C ? (pc + 1) * CNTBITS : C;
                for (int c = pc * CNTBITS; c < cend; c++) {
                    const uint64_t one = (uint64_t)1 << (c - pc * CNTBITS);
                    const float v = row[c];
                    if (bits == 2) {
                        if (v > t) b2 |= one;                              /* +1 */
                        else if (v < -t) { b1 |= one; b2 |= one; }         /* -1 */
                    } else {
                        if (v < t) b1 |= one;                              /* -1 */
                    }
                }
                if (bits == 2) {
                    out[pc * 2 + 0] = (int64_t)b1;
                    out[pc * 2 + 1] = (int64_t)b2;
                    cnt += popcnt64(b2);
                } else {
                    out[pc] = (int64_t)b1;
                }
            }
        }
        if (btn) btn[n] = (bits == 2) ? (int32_t)cnt : 0;
    }
}

/* [N][H][W][Cp] -> zero-bordered [N][PH][PW][Cp]. */
void oracle_pad(const int64_t* a, int64_t* y, int N, int H, int W, int Cp, int P1, int P2) {
    const int PH = H + 2 * P1, PW = W + 2 * P2;
    memset(y, 0, sizeof(int64_t) * (size_t)N * PH * PW * Cp);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
        for (int h = 0; h < H; h++)
            memcpy(y + (((size_t)n * PH + h + P1) * PW + P2) * Cp, a + ((size_t)n * H + h) * W * Cp,
                   sizeof(int64_t) * (size_t)W * Cp);
}

/* [N][H][W][Cp] (already padded) -> rows [N*OH*OW][KH*KW*Cp]. */
void oracle_im2row(const int64_t* a, int64_t* y, int N, int H, int W, int Cp, int KH, int KW, int S1, int S2) {
    const int OH = (H - KH + 1) / S1, OW = (W - KW + 1) / S2;
    if (OH <= 0 || OW <= 0) return;
    const size_t W1 = (size_t)KH * KW * Cp;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++)
        for (int oh = 0; oh < OH; oh++)
            for (int ow = 0; ow < OW; ow++) {
                int64_t* yb = y + (((size_t)n * OH + oh) * OW + ow) * W1;
                const int64_t* ab = a + (((size_t)n * H + (size_t)oh * S1) * W + (size_t)ow * S2) * Cp;
                for (int kh = 0; kh < KH; kh++)
                    memcpy(yb + (size_t)kh * KW * Cp, ab + (size_t)kh * W * Cp, sizeof(int64_t) * (size_t)KW * Cp);
            }
}

/* The four popcount GEMMs.  a: [M][K*ab], b: [KN][K*wb], planes interleaved per word; y int32 [M][KN]. */
void oracle_gemm(const int64_t* a, const int64_t* b, const int32_t* btn, int32_t* y,
                 int type, long M, int KN, int K, int NUM) {
#pragma omp parallel for schedule(static)
    for (long m = 0; m < M; m++) {
        for (int n = 0; n < KN; n++) {
            int c1 = 0, c2 = 0;
            switch (type) {
                case 0: {   /* TNN: TAB_CPU.cpp:252-259 */
                    const int64_t* ar = a + (size_t)m * K * 2;
                    const int64_t* br = b + (size_t)n * K * 2;
                    for (int k = 0; k < K; k++) {
                        const int64_t p1 = ar[2 * k] ^ br[2 * k];
                        const int64_t p2 = ar[2 * k + 1] & br[2 * k + 1];
                        c1 += popcnt64(p2);
                        c2 += popcnt64(p1 & p2);
                    }
                    y[(size_t)m * KN + n] = c1 - c2 - c2;
                    break;
                }
                case 1: {   /* TBN: TAB_CPU.cpp:276-283 */
                    const int64_t* ar = a + (size_t)m * K * 2;
                    const int64_t* br = b + (size_t)n * K;
                    for (int k = 0; k < K; k++) {
                        const int64_t p1 = ar[2 * k] ^ br[k];
                        const int64_t p2 = ar[2 * k + 1];
                        c1 += popcnt64(p2);
                        c2 += popcnt64(p1 & p2);
                    }
                    y[(size_t)m * KN + n] = c1 - c2 - c2;
                    break;
                }
                case 2: {   /* BTN: TAB_CPU.cpp:299-304 */
                    const int64_t* ar = a + (size_t)m * K;
                    const int64_t* br = b + (size_t)n * K * 2;
                    for (int k = 0; k < K; k++) c2 += popcnt64((ar[k] ^ br[2 * k]) & br[2 * k + 1]);
                    y[(size_t)m * KN + n] = btn[n] - c2 - c2;
                    break;
                }
                default: {  /* BNN: TAB_CPU.cpp:320-324 */
                    const int64_t* ar = a + (size_t)m * K;
                    const int64_t* br = b + (size_t)n * K;
                    for (int k = 0; k < K; k++) c1 += popcnt64(ar[k] ^ br[k]);
                    y[(size_t)m * KN + n] = NUM - c1 - c1;
                    break;
                }
            }
        }
    }
}

/*
 * Whole TAB_Conv2d on the CPU.  y: float32 [N][OH][OW][KN].  Returns 0, or -1 for bad arguments,
 * -2 when scratch memory cannot be allocated.  gemm_fn, when not NULL, replaces oracle_gemm for the
 * GEMM stage (used to run the reference's own compiled GEMMs inside the same pipeline).
 */
typedef void (*gemm_fn_t)(const int64_t*, const int64_t*, const int32_t*, int32_t*, int, long, int, int, int);

int oracle_conv2d_with(gemm_fn_t gemm_fn, const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                       float* y, int type, int p1, int p2, int s1, int s2,
                       int N, int H, int W, int C, int KN, int KH, int KW) {
    if (type < 0 || type > 3 || s1 < 1 || s2 < 1 || p1 < 0 || p2 < 0 || KH < 1 || KW < 1 || C < 1) return -1;
    const int PH = H + 2 * p1, PW = W + 2 * p2;
    const int OH = (PH - KH + 1) / s1, OW = (PW - KW + 1) / s2;      /* TAB_GEMM.cu:354-357 */
    if (N <= 0 || KN <= 0 || OH <= 0 || OW <= 0) return 0;
    const int PC = packed_channels(C), ab = act_bits(type);
    const int Cp = PC * ab;
    const long M = (long)N * OH * OW;
    const int K = KH * KW * PC;
    (void)weight_bits;
    int64_t* q = (int64_t*)malloc(sizeof(int64_t) * (size_t)N * H * W * Cp);
    int64_t* padded = (int64_t*)malloc(sizeof(int64_t) * (size_t)N * PH * PW * Cp);
    int64_t* rows = (int64_t*)malloc(sizeof(int64_t) * (size_t)M * K * ab);
    int32_t* yi = (int32_t*)malloc(sizeof(int32_t) * (size_t)M * KN);
    if (!q || !padded || !rows || !yi) { free(q); free(padded); free(rows); free(yi); return -2; }
    oracle_quantize(x, ths, q, NULL, ab == 1 ? 1 : 2, N, H, W, C);   /* TAB_GEMM.cu:419-426 */
    oracle_pad(q, padded, N, H, W, Cp, p1, p2);                       /* TAB_GEMM.cu:447-451 */
    oracle_im2row(padded, rows, N, PH, PW, Cp, KH, KW, s1, s2);       /* TAB_GEMM.cu:482-488 */
    (gemm_fn ? gemm_fn : oracle_gemm)(rows, qw, btn, yi, type, M, KN, K, KH * KW * C);   /* :509 */
#pragma omp parallel for schedule(static)
    for (long i = 0; i < M * KN; i++) y[i] = (float)yi[i];            /* TAB_GEMM.cu:53,349 */
    free(q); free(padded); free(rows); free(yi);
    return 0;
}

int oracle_conv2d(const float* x, const int64_t* qw, const float* ths, const int32_t* btn, float* y,
                  int type, int p1, int p2, int s1, int s2,
                  int N, int H, int W, int C, int KN, int KH, int KW) {
    return oracle_conv2d_with(NULL, x, qw, ths, btn, y, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
}


/* Threads the OpenMP loops above (and the reference's GEMMs, which share the runtime) will use; n > 0 sets it first.
 * A launcher may export OMP_NUM_THREADS=1 for its children: the CPU baseline sets the count it reports explicitly. */
int oracle_omp_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
