// extern "C" entry points declared in include/tab_b200.h: argument validation, then kernel dispatch.
// No entry point in this file allocates or frees device memory, and none synchronises the host.
#include "tab_kernels.cuh"

namespace tab {

static thread_local int g_last_cuda_error = 0;

int record_cuda_error(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return TAB_E_CUDA;
}

void conv_set_csa(bool on);
void imma_set_variant(int v);
int umma_status_read_and_clear();
size_t imma_workspace_bytes(int N, int H, int W, int C, int KN, int KH, int KW, int p1, int p2, int s1, int s2);
int conv_imma_dispatch(const float* x, const int64_t* qw, const float* ths, float* y, void* workspace, int type,
                       int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW,
                       cudaStream_t stream, const float* residual, double* abs_sums, float* next_ths, float next_scale);
struct FusedTail;
int residual_abs_sum_dispatch(float* y, const float* residual, double* sums, int N, long long per_image, cudaStream_t s);
int quantize_int8_dispatch(const float* x, const float* ths, int8_t* qx8, int bits, int N, int H, int W, int C, cudaStream_t stream);
int quantize_int8_padded_dispatch(const float* x, const float* ths, int8_t* qx8, int bits, int N, int H, int W, int C,
                                  int KH, int KW, int p1, int p2, int s1, int s2, cudaStream_t stream);
int conv_int8_padded_dispatch(const int8_t* qx8p, const int8_t* w8, float* y, int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                              int KN, int KH, int KW, cudaStream_t stream, const float* residual, double* abs_sums);
int expand_weights_dispatch(const int64_t* qw, int8_t* w8, int wbits, int KN, int KH, int KW, int C, cudaStream_t stream);
int conv_int8_dispatch(const int8_t* qx8, const int8_t* w8, float* y, int binary_act, int p1, int p2, int s1, int s2,
                       int N, int H, int W, int C, int KN, int KH, int KW, cudaStream_t stream,
                       const float* residual, double* abs_sums, const FusedTail* tail);
static int g_conv_path = TAB_PATH_AUTO;

static bool dims_ok(int N, int H, int W, int C) { return N >= 0 && H >= 0 && W >= 0 && C >= 1; }

}  // namespace tab

using namespace tab;

extern "C" {

const char* tab_error_string(int code) {
    switch (code) {
        case TAB_OK: return "success";
        case TAB_E_BAD_ARGUMENT: return "bad argument (size, type or bitwidth out of range)";
        case TAB_E_NULL_POINTER: return "required pointer is NULL";
        case TAB_E_WORKSPACE: return "workspace too small or not 256-byte aligned";
        case TAB_E_CUDA: return "CUDA runtime error (see tab_last_cuda_error)";
        case TAB_E_TOO_LARGE: return "problem size exceeds the supported range";
        case TAB_E_ALIGNMENT: return "pointer not aligned to its element type";
        default: return "unknown error code";
    }
}

int tab_last_cuda_error(void) { return g_last_cuda_error; }

int tab_version(void) { return 100; }

int tab_quantize_launch(const float* x, const float* ths, int64_t* qx, int32_t* btn,
                        int bitwidth, int N, int H, int W, int C, tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (reinterpret_cast<uintptr_t>(btn) & 3) return TAB_E_ALIGNMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (btn) {
        cudaError_t e = cudaMemsetAsync(btn, 0, sizeof(int32_t) * (size_t)N, s);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    if ((long long)H * W == 0) return TAB_OK;
    if (!x || !ths || !qx) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(ths) & 3) ||
        (reinterpret_cast<uintptr_t>(qx) & 7))
        return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    const int bits = (bitwidth == 1) ? 1 : 2;                      // TAB_GEMM.cu:267,309
    return quantize_dispatch(x, ths, qx, bits == 2 ? btn : nullptr, bits, N, H, W, C, s);
}

static size_t popc_workspace_bytes(int type, int N, int H, int W, int C) {
    const size_t words = (size_t)N * H * W * packed_channels(C) * act_bits(type);
    return (words * 8 + 255) / 256 * 256;
}

size_t tab_conv2d_workspace_bytes(int type, int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW) {
    if (type < 0 || type > 3 || !dims_ok(N, H, W, C) || KN < 0 || KH < 1 || KW < 1 || p1 < 0 || p2 < 0 || s1 < 1 || s2 < 1) return 0;
    const size_t a = popc_workspace_bytes(type, N, H, W, C), b = imma_workspace_bytes(N, H, W, C, KN, KH, KW, p1, p2, s1, s2);
    return a > b ? a : b;
}

int tab_conv2d_set_path(int path) {
    if (path != TAB_PATH_AUTO && path != TAB_PATH_POPCOUNT) return TAB_E_BAD_ARGUMENT;
    const int prev = g_conv_path;
    g_conv_path = path;
    return prev;
}

static int conv_args_ok(int type, int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                        int KN, int KH, int KW) {
    if (type < 0 || type > 3) return TAB_E_BAD_ARGUMENT;
    if (!dims_ok(N, H, W, C) || KN < 0 || KH < 1 || KW < 1 || p1 < 0 || p2 < 0 || s1 < 1 || s2 < 1)
        return TAB_E_BAD_ARGUMENT;
    return TAB_OK;
}

int tab_conv2d_packed_launch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y,
                             int type, int p1, int p2, int s1, int s2,
                             int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) return TAB_OK;
    if (!qx || !qw || !y || (type == 2 && !btn)) return TAB_E_NULL_POINTER;
    const uintptr_t qx_mask = act_bits(type) == 2 ? 15 : 7;        // 16-byte (sign, magnitude) pairs
    if ((reinterpret_cast<uintptr_t>(qx) & qx_mask) || (reinterpret_cast<uintptr_t>(qw) & 7) ||
        (reinterpret_cast<uintptr_t>(y) & 3) || (reinterpret_cast<uintptr_t>(btn) & 3))
        return TAB_E_ALIGNMENT;
    return conv_packed_dispatch(qx, qw, btn, y, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                reinterpret_cast<cudaStream_t>(stream));
}

static int conv2d_impl(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                       float* y, void* workspace, size_t workspace_bytes, int type,
                       int p1, int p2, int s1, int s2,
                       int N, int H, int W, int C, int KN, int KH, int KW,
                       const float* residual, double* abs_sums, float* next_ths, float next_scale, tab_stream_t stream) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (next_ths && !abs_sums) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(abs_sums) & 7) || (reinterpret_cast<uintptr_t>(next_ths) & 3)) return TAB_E_ALIGNMENT;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    // empty output, or any path but the tensor-core one: the sums are cleared and the thresholds finished by
    // separate small launches (the tensor-core path folds both into its two kernels)
    auto clear_sums = [&]() -> int {
        if (!abs_sums || N <= 0) return TAB_OK;
        cudaError_t e = cudaMemsetAsync(abs_sums, 0, sizeof(double) * (size_t)N, s);
        return e == cudaSuccess ? TAB_OK : record_cuda_error(e);
    };
    auto finish_ths = [&]() -> int {
        if (!next_ths || N <= 0) return TAB_OK;
        return tab_threshold_from_sums_launch(abs_sums, next_ths, next_scale, N, (long long)KN * (oh > 0 ? oh : 0) * (ow > 0 ? ow : 0), stream);
    };
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) {
        rc = clear_sums();
        return rc != TAB_OK ? rc : finish_ths();
    }
    if (!x || !ths || !qw || !y || (type == 2 && !btn)) return TAB_E_NULL_POINTER;
    const size_t need = tab_conv2d_workspace_bytes(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return TAB_E_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(ths) & 3) ||
        (reinterpret_cast<uintptr_t>(residual) & 3))
        return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    if (g_conv_path == TAB_PATH_AUTO) {
        if ((reinterpret_cast<uintptr_t>(qw) & 7) || (reinterpret_cast<uintptr_t>(y) & 3)) return TAB_E_ALIGNMENT;
        const bool r8 = residual && ((reinterpret_cast<uintptr_t>(residual) & 7) == 0) && ((reinterpret_cast<uintptr_t>(y) & 7) == 0);
        if (!residual || r8) {
            rc = conv_imma_dispatch(x, qw, ths, y, workspace, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, s, residual, abs_sums,
                                    next_ths, next_scale);
            if (rc != TAB_E_TOO_LARGE) return rc;       // sizes beyond the tensor-core path: fall through
        }
    }
    rc = clear_sums();
    if (rc != TAB_OK) return rc;
    int64_t* qx = reinterpret_cast<int64_t*>(workspace);
    rc = quantize_dispatch(x, ths, qx, nullptr, act_bits(type), N, H, W, C, s);   // TAB_GEMM.cu:419-426
    if (rc != TAB_OK) return rc;
    rc = tab_conv2d_packed_launch(qx, qw, btn, y, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, stream);
    if (rc != TAB_OK || (!residual && !abs_sums)) return rc;
    // the popcount kernel has no fused epilogue: one extra pass adds the residual and sums |y|
    rc = residual_abs_sum_dispatch(y, residual, abs_sums, N, oh * ow * (long long)KN, s);
    return rc != TAB_OK ? rc : finish_ths();
}

int tab_conv2d_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                      float* y, void* workspace, size_t workspace_bytes, int type,
                      int p1, int p2, int s1, int s2,
                      int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    return conv2d_impl(x, qw, ths, btn, y, workspace, workspace_bytes, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                       nullptr, nullptr, nullptr, 0.f, stream);
}

int tab_conv2d_fused_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                            float* y, void* workspace, size_t workspace_bytes, int type,
                            int p1, int p2, int s1, int s2,
                            int N, int H, int W, int C, int KN, int KH, int KW,
                            const float* residual, double* abs_sums, tab_stream_t stream) {
    return conv2d_impl(x, qw, ths, btn, y, workspace, workspace_bytes, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                       residual, abs_sums, nullptr, 0.f, stream);
}

int tab_conv2d_chain_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                            float* y, void* workspace, size_t workspace_bytes, int type,
                            int p1, int p2, int s1, int s2,
                            int N, int H, int W, int C, int KN, int KH, int KW,
                            const float* residual, double* abs_sums, float* next_ths, float next_scale,
                            tab_stream_t stream) {
    return conv2d_impl(x, qw, ths, btn, y, workspace, workspace_bytes, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                       residual, abs_sums, next_ths, next_scale, stream);
}

int tab_quantize_int8_launch(const float* x, const float* ths, int8_t* qx8, int bitwidth,
                             int N, int H, int W, int C, tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if ((long long)N * H * W == 0) return TAB_OK;
    if (!x || !ths || !qx8) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(ths) & 3) || (reinterpret_cast<uintptr_t>(qx8) & 15))
        return TAB_E_ALIGNMENT;
    return quantize_int8_dispatch(x, ths, qx8, bitwidth == 1 ? 1 : 2, N, H, W, C, reinterpret_cast<cudaStream_t>(stream));
}

int tab_expand_weights_launch(const int64_t* qw, int8_t* w8, int bitwidth, int KN, int KH, int KW, int C, tab_stream_t stream) {
    if (KN < 0 || KH < 1 || KW < 1 || C < 1 || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if (KN == 0) return TAB_OK;
    if (!qw || !w8) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(qw) & 7) || (reinterpret_cast<uintptr_t>(w8) & 15)) return TAB_E_ALIGNMENT;
    return expand_weights_dispatch(qw, w8, bitwidth == 1 ? 1 : 2, KN, KH, KW, C, reinterpret_cast<cudaStream_t>(stream));
}

int tab_conv2d_int8_launch(const int8_t* qx8, const int8_t* w8, float* y, int type, int p1, int p2, int s1, int s2,
                           int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) return TAB_OK;
    if (!qx8 || !w8 || !y) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(qx8) & 15) || (reinterpret_cast<uintptr_t>(w8) & 15) || (reinterpret_cast<uintptr_t>(y) & 3))
        return TAB_E_ALIGNMENT;
    return conv_int8_dispatch(qx8, w8, y, act_bits(type) == 1, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                              reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr);
}

int tab_quantize_int8_padded_launch(const float* x, const float* ths, int8_t* qx8p, int bitwidth,
                                    int N, int H, int W, int C, int KH, int KW, int p1, int p2, int s1, int s2,
                                    tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1 || p1 < 0 || p2 < 0 || s1 < 1 || s2 < 1 || KH < 1 || KW < 1) return TAB_E_BAD_ARGUMENT;
    if ((long long)N * (H + 2LL * p1) * (W + 2LL * p2) == 0) return TAB_OK;
    if (!x || !ths || !qx8p) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(ths) & 3) || (reinterpret_cast<uintptr_t>(qx8p) & 15))
        return TAB_E_ALIGNMENT;
    return quantize_int8_padded_dispatch(x, ths, qx8p, bitwidth == 1 ? 1 : 2, N, H, W, C, KH, KW, p1, p2, s1, s2,
                                         reinterpret_cast<cudaStream_t>(stream));
}

int tab_conv2d_int8_padded_launch(const int8_t* qx8p, const int8_t* w8, float* y, int type, int p1, int p2, int s1, int s2,
                                  int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) return TAB_OK;
    if (!qx8p || !w8 || !y) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(qx8p) & 15) || (reinterpret_cast<uintptr_t>(w8) & 15) || (reinterpret_cast<uintptr_t>(y) & 3))
        return TAB_E_ALIGNMENT;
    return conv_int8_padded_dispatch(qx8p, w8, y, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, reinterpret_cast<cudaStream_t>(stream),
                                     nullptr, nullptr);
}

/* Test/benchmark hook: GEMM variant of the tensor-core path: 0 = default, 1 = mma.sync + im2col staging,
   2 = mma.sync (patch or im2col staging), 3 = tcgen05. */
void tab_debug_set_imma_variant(int v) { imma_set_variant(v); }
/* Test hook: code of the last expired wait in the tcgen05 kernel on this device (0 = none); clears it. */
int tab_debug_umma_status(void) { return umma_status_read_and_clear(); }

/* Test/benchmark hook: 1 = carry-save popcount tree (default), 0 = one POPC per word. */
void tab_debug_set_csa(int on) { conv_set_csa(on != 0); }

}  // extern "C"

#ifdef TAB_PERSIST_PROFILE
namespace tab { int persist_profile_read(unsigned long long* out16); void persist_set_debug(int v); }
extern "C" void tab_debug_persist_set(int v) { tab::persist_set_debug(v); }
extern "C" int tab_debug_persist_profile(unsigned long long* out16) { return tab::persist_profile_read(out16); }
#endif
