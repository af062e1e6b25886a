// Runs the reference's CUDA kernel bodies on the host, unmodified, for pinning the oracle stage by
// stage.  TEST INFRASTRUCTURE ONLY.
//
// This file holds no reference code.  build.py locates the kernel definitions (GetIdx, TerOnlyKernel,
// BinOnlyKernel, BTN_Weight, TNN/TBN/BTN/BNNGEMM in TAB_GEMM.cu; PadKernel, Img2RowKernel in
// TAB_GEMM.cuh) by signature in the files where they lie, writes them to a temporary include outside
// this repository (named by REF_CUDA_INC) and deletes it after the compile.  The kernels use nothing
// of CUDA but the execution-space qualifiers, the four index variables and __popcll, so they compile
// as plain C++ once those are supplied: the qualifiers are defined away, blockIdx / threadIdx /
// blockDim / gridDim are thread-local structs, and a "launch" is a loop over the reference's own
// launch shape (TAB_GEMM.cu:311-316, :419-426, :449, :484-486; TAB_GEMM.cuh:26-27).  No kernel of the
// reference synchronises its threads, so running them one after another is the same computation.
//
// What the host functions below add is the reference's host sequence restated (ConvWithCuda_TAB,
// TAB_GEMM.cu:325-527) with two documented repairs, both needed to run its kernels inside their
// own array bounds:
//   * the kernels read ths[blockIdx.x] with a grid of N*H blocks (TAB_GEMM.cu:166,184,231,311), i.e.
//     ths[n*H + h], while the interface passes one threshold per image (TAB_GPU.cpp:23,49): the
//     kernels are handed an array expanded to N*H entries, entry n*H + h holding ths[n];
//   * the padded buffer is cleared before PadKernel writes the interior (the reference leaves the
//     border to whatever cudaMalloc returned, TAB_GEMM.cu:391; its CPU backend zero-fills,
//     TAB_CPU.cpp:39,155).
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

struct RefDim3 { unsigned x = 1, y = 1, z = 1; };
static thread_local RefDim3 blockIdx, threadIdx, blockDim, gridDim;

#define __global__
#define __device__
#define BITS 2                                   /* TAB_GEMM.cuh:9 */
#define CNTBITS 64                               /* TAB_GEMM.cuh:10 */
#define popcnt64(a) __builtin_popcountll(a)      /* TAB_GEMM.cuh:11 maps it to __popcll */

#include REF_CUDA_INC

namespace {

// kernel<<<grid, block>>>(args...) as nested loops; blocks are spread over the host threads.
template <typename F>
void launch(unsigned gx, unsigned gy, unsigned bx, unsigned by, F body) {
    const long long nblocks = (long long)gx * gy;
#pragma omp parallel for schedule(static)
    for (long long b = 0; b < nblocks; b++) {
        gridDim.x = gx; gridDim.y = gy; blockDim.x = bx; blockDim.y = by;
        blockIdx.x = (unsigned)(b % gx); blockIdx.y = (unsigned)(b / gx);
        for (unsigned ty = 0; ty < by; ty++)
            for (unsigned tx = 0; tx < bx; tx++) {
                threadIdx.x = tx; threadIdx.y = ty;
                body();
            }
    }
}

std::vector<int64_t> one_bit_table() {           // TAB_GEMM.cu:252-258
    std::vector<int64_t> t(CNTBITS);
    for (int i = 0; i < CNTBITS; i++) t[i] = (int64_t)(1ULL << i);
    return t;
}

std::vector<float> expand_thresholds(const float* ths, int N, int H) {
    std::vector<float> e((size_t)N * H);
    for (int n = 0; n < N; n++)
        for (int h = 0; h < H; h++) e[(size_t)n * H + h] = ths[n];
    return e;
}

void quantize_stage(const float* x, const float* ths, int64_t* q, bool ternary, int N, int H, int W, int C) {
    if ((long long)N * H * W == 0) return;
    const std::vector<int64_t> onebit = one_bit_table();
    const std::vector<float> e = expand_thresholds(ths, N, H);
    if (ternary) launch((unsigned)(N * H), 1, (unsigned)W, 1, [&] { TerOnlyKernel(q, x, e.data(), onebit.data(), N, H, W, C); });
    else launch((unsigned)(N * H), 1, (unsigned)W, 1, [&] { BinOnlyKernel(q, x, e.data(), onebit.data(), N, H, W, C); });
}

void gemm_stage(const int64_t* a, const int64_t* b, const int32_t* btn, float* c, int type, int M, int KN, int K, int NUM) {
    const unsigned gx = (unsigned)(M / 16 + 1), gy = 16, bx = 16, by = (unsigned)(KN / 16 + 1);   // TAB_GEMM.cuh:26-27
    switch (type) {
        case 0: launch(gx, gy, bx, by, [&] { TNNGEMM(a, b, c, M, KN, K); }); break;
        case 1: launch(gx, gy, bx, by, [&] { TBNGEMM(a, b, c, M, KN, K); }); break;
        case 2: launch(gx, gy, bx, by, [&] { BTNGEMM(a, b, c, btn, M, KN, K); }); break;
        default: launch(gx, gy, bx, by, [&] { BNNGEMM(a, b, c, M, KN, K, NUM); }); break;
    }
}

}  // namespace

extern "C" {

// QuanWithCuda_TAB's device work (TAB_GEMM.cu:305-316): qx [N][H][W][PC][bits], btn [N] (pre-zeroed by the
// caller; like the reference, only the first 16*(N/16) entries are computed, and only for bitwidth > 1).
void ref_cuda_quantize(const float* x, const float* ths, int64_t* qx, int32_t* btn, int bitwidth, int N, int H, int W, int C) {
    quantize_stage(x, ths, qx, bitwidth > 1, N, H, W, C);
    if (bitwidth > 1 && N / 16 > 0) {
        const int PC = (C + CNTBITS - 1) / CNTBITS;
        launch(16, 1, (unsigned)(N / 16), 1, [&] { BTN_Weight(qx, btn, N, H * W * PC); });
    }
}

// PadKernel<<<N, H>>> into a cleared buffer y [N][H+2*P1][W+2*P2][Cw] (Cw = words per pixel).
void ref_cuda_pad(const int64_t* a, int64_t* y, int N, int H, int W, int Cw, int P1, int P2) {
    std::memset(y, 0, sizeof(int64_t) * (size_t)N * (H + 2 * P1) * (W + 2 * P2) * Cw);
    if ((long long)N * H == 0) return;
    launch((unsigned)N, 1, (unsigned)H, 1, [&] { PadKernel<int64_t>(y, a, N, H, W, Cw, P1, P2); });
}

// Img2RowKernel<<<(N, OH), OW>>> on an already padded input a [N][H][W][Cw]; y [N*OH*OW][KH*KW*Cw].
void ref_cuda_im2row(const int64_t* a, int64_t* y, int N, int H, int W, int Cw, int KH, int KW, int S1, int S2) {
    const int OH = (H - KH + 1) / S1, OW = (W - KW + 1) / S2;
    if (N <= 0 || OH <= 0 || OW <= 0) return;
    launch((unsigned)N, (unsigned)OH, (unsigned)OW, 1, [&] { Img2RowKernel<int64_t>(y, a, N, H, W, Cw, KH, KW, S1, S2); });
}

// GEMMWithCuda's launch (TAB_GEMM.cuh:22-46): c float [M][KN].
void ref_cuda_gemm(const int64_t* a, const int64_t* b, const int32_t* btn, float* c, int type, int M, int KN, int K, int NUM) {
    gemm_stage(a, b, btn, c, type, M, KN, K, NUM);
}

// ConvWithCuda_TAB (TAB_GEMM.cu:325-527): quantise, pad, im2row, GEMM.  y float [N*OH*OW][KN].  Returns 0, or -1
// when the output is empty.
int ref_cuda_conv2d(const float* x, const int64_t* qw, const float* ths, const int32_t* btn, float* y, int type,
                    int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW) {
    const int PH = H + 2 * p1, PW = W + 2 * p2;                          // :354-357
    const int OH = (PH - KH + 1) / s1, OW = (PW - KW + 1) / s2;
    if (N <= 0 || KN <= 0 || OH <= 0 || OW <= 0) return -1;
    const int PC = (C + CNTBITS - 1) / CNTBITS;
    const int MemC = (type == 2 || type == 3) ? PC : PC * BITS;          // :367-372
    std::vector<int64_t> pad_a((size_t)N * PH * PW * MemC, 0);           // :381 (cleared here, see the header)
    std::vector<int64_t> img_a((size_t)N * PH * PW * KH * KW * MemC, 0); // :382
    quantize_stage(x, ths, img_a.data(), type < 2, N, H, W, C);          // :419-426
    const int64_t* loc_a;
    const bool need_im2row = s1 > 1 || s2 > 1 || KH > 1 || KW > 1;       // :447
    if (p1 > 0 || p2 > 0) {
        launch((unsigned)N, 1, (unsigned)H, 1, [&] { PadKernel<int64_t>(pad_a.data(), img_a.data(), N, H, W, MemC, p1, p2); });
        loc_a = pad_a.data();
    } else if (need_im2row) {
        std::memcpy(pad_a.data(), img_a.data(), sizeof(int64_t) * pad_a.size());   // :453
        loc_a = pad_a.data();
    } else {
        loc_a = img_a.data();
    }
    if (need_im2row) {                                                   // :482-488
        launch((unsigned)N, (unsigned)OH, (unsigned)OW, 1,
               [&] { Img2RowKernel<int64_t>(img_a.data(), loc_a, N, PH, PW, MemC, KH, KW, s1, s2); });
        loc_a = img_a.data();
    }
    gemm_stage(loc_a, qw, btn, y, type, N * OH * OW, KN, KH * KW * PC, KH * KW * C);   // :509
    return 0;
}

}  // extern "C"
