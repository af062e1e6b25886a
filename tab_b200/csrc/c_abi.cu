// extern "C" entry points declared in include/tab_b200.h: argument validation, then kernel dispatch.
// No entry point in this file allocates or frees device memory, and none synchronises the host (tab_device_status
// excepted, which exists to synchronise).
#include "tab_kernels.cuh"
#include "umma_common.cuh"

namespace tab {

static thread_local int g_last_cuda_error = 0;
static thread_local int g_conv_path = TAB_PATH_AUTO;

int record_cuda_error(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return TAB_E_CUDA;
}

int umma_status_read_and_clear();
const char* tc_last_kernel();
void tc_forget_last_kernel();
int tc_conv_dispatch(TcConvParams p, cudaStream_t stream);
bool tc_conv_covers(TcConvParams p);
int residual_abs_sum_dispatch(float* y, const float* residual, double* sums, int N, long long per_image, cudaStream_t s);

static bool dims_ok(int N, int H, int W, int C) { return N >= 0 && H >= 0 && W >= 0 && C >= 1; }
static size_t round256(size_t v) { return (v + 255) / 256 * 256; }
static bool misaligned(const void* p, uintptr_t mask) { return (reinterpret_cast<uintptr_t>(p) & mask) != 0; }

static size_t bits_bytes(int type, int N, int H, int W, int C) {
    return round256((size_t)N * H * W * packed_channels(C) * act_bits(type) * 8);
}
static size_t w8_bytes(int C, int KN, int KH, int KW) { return round256((size_t)KN * KH * KW * packed_channels(C) * 64); }

static int conv_args_ok(int type, int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW) {
    if (type < 0 || type > 3) return TAB_E_BAD_ARGUMENT;
    if (!dims_ok(N, H, W, C) || KN < 0 || KH < 1 || KW < 1 || p1 < 0 || p2 < 0 || s1 < 1 || s2 < 1) return TAB_E_BAD_ARGUMENT;
    return TAB_OK;
}

// Geometry part of the tensor-core parameter block (pointers and the tail are the caller's).
static TcConvParams tc_geometry(int type, int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW,
                                long long oh, long long ow) {
    TcConvParams p = {};
    p.N = N; p.H = H; p.W = W; p.C = C; p.PC = packed_channels(C); p.KN = KN; p.KH = KH; p.KW = KW;
    p.OH = (int)oh; p.OW = (int)ow; p.p1 = p1; p.p2 = p2; p.s1 = s1; p.s2 = s2;
    const long long M = (long long)N * oh * ow, Kw = (long long)KH * KW * p.PC;
    p.M = M < (1LL << 31) ? (int)M : 0x7FFFFFFF;
    p.Kw = Kw < (1LL << 31) ? (int)Kw : 0x7FFFFFFF;
    p.abits = act_bits(type);
    p.per_image = (double)KN * (double)oh * (double)ow;
    return p;
}

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
        case TAB_E_ALIGNMENT: return "pointer not aligned as the entry point requires";
        default: return "unknown error code";
    }
}

int tab_last_cuda_error(void) { return g_last_cuda_error; }

int tab_version(void) { return 200; }

int tab_device_status(void) { return umma_status_read_and_clear(); }

const char* tab_last_conv_kernel(void) { return tc_last_kernel(); }

int tab_quantize_launch(const float* x, const float* ths, int64_t* qx, int32_t* btn,
                        int bitwidth, int N, int H, int W, int C, tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (misaligned(btn, 3)) return TAB_E_ALIGNMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (btn) {
        cudaError_t e = cudaMemsetAsync(btn, 0, sizeof(int32_t) * (size_t)N, s);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    if ((long long)H * W == 0) return TAB_OK;
    if (!x || !ths || !qx) return TAB_E_NULL_POINTER;
    if (misaligned(x, 3) || misaligned(ths, 3) || misaligned(qx, 7)) return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    const int bits = (bitwidth == 1) ? 1 : 2;                      // TAB_GEMM.cu:267,309
    return quantize_dispatch(x, ths, qx, bits == 2 ? btn : nullptr, bits, N, H, W, C, s);
}

size_t tab_conv2d_workspace_bytes(int type, int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW) {
    if (conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW) != TAB_OK) return 0;
    return bits_bytes(type, N, H, W, C) + w8_bytes(C, KN, KH, KW) + 256;
}

int tab_conv2d_set_path(int path) {
    if (path != TAB_PATH_AUTO && path != TAB_PATH_POPCOUNT && path != TAB_PATH_POPCOUNT_PLAIN) return TAB_E_BAD_ARGUMENT;
    const int prev = g_conv_path;
    g_conv_path = path;
    return prev;
}

// Validation shared by the two entry points that run the popcount kernel on packed activations.
static int packed_checks(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y, int type) {
    if (!qx || !qw || !y || (type == 2 && !btn)) return TAB_E_NULL_POINTER;
    const uintptr_t qx_mask = act_bits(type) == 2 ? 15 : 7;        // 16-byte (sign, magnitude) pairs
    if (misaligned(qx, qx_mask) || misaligned(qw, 7) || misaligned(y, 3) || misaligned(btn, 3)) return TAB_E_ALIGNMENT;
    return TAB_OK;
}

int tab_conv2d_packed_launch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y,
                             int type, int p1, int p2, int s1, int s2,
                             int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) return TAB_OK;
    rc = packed_checks(qx, qw, btn, y, type);
    if (rc != TAB_OK) return rc;
    return conv_packed_dispatch(qx, qw, btn, y, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW,
                                reinterpret_cast<cudaStream_t>(stream), g_conv_path != TAB_PATH_POPCOUNT_PLAIN);
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
    if (misaligned(abs_sums, 7) || misaligned(next_ths, 3)) return TAB_E_ALIGNMENT;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    // empty output, or the popcount path: the sums are cleared and the thresholds finished by separate small launches
    // (the tensor-core path folds both into its two kernels)
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
    if (!workspace || workspace_bytes < need || misaligned(workspace, 255)) return TAB_E_WORKSPACE;
    if (misaligned(x, 3) || misaligned(ths, 3) || misaligned(residual, 3) || misaligned(qw, 7) || misaligned(y, 3) || misaligned(btn, 3))
        return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    int64_t* qx = reinterpret_cast<int64_t*>(workspace);
    int8_t* w8 = reinterpret_cast<int8_t*>(workspace) + bits_bytes(type, N, H, W, C);
    unsigned* counter = reinterpret_cast<unsigned*>(w8 + w8_bytes(C, KN, KH, KW));
    tc_forget_last_kernel();
    if (g_conv_path == TAB_PATH_AUTO && !misaligned(y, 15) && !misaligned(residual, 15)) {
        TcConvParams p = tc_geometry(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, oh, ow);
        p.qx = reinterpret_cast<const uint64_t*>(qx); p.w8 = w8; p.y = y; p.residual = residual; p.abs_sums = abs_sums;
        if (next_ths) { p.ths_out = next_ths; p.ths_scale = next_scale; p.done_counter = counter; }
        if (tc_conv_covers(p)) {
            // launch 1: quantise (TAB_GEMM.cu:419-426) + weight expansion + clears; launch 2: the GEMM
            QuantExtras ex;
            ex.zero_sums = abs_sums;
            ex.zero_counter = next_ths ? counter : nullptr;
            ex.qw = reinterpret_cast<const uint64_t*>(qw); ex.w8 = w8;
            ex.words = (long long)KN * KH * KW * p.PC; ex.wbits = weight_bits(type); ex.PC = p.PC; ex.C = C;
            rc = quantize_dispatch(x, ths, qx, nullptr, act_bits(type), N, H, W, C, s, &ex);
            if (rc != TAB_OK) return rc;
            return tc_conv_dispatch(p, s);
        }
    }
    rc = clear_sums();
    if (rc != TAB_OK) return rc;
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

int tab_expand_weights_launch(const int64_t* qw, int8_t* w8, int bitwidth, int KN, int KH, int KW, int C, tab_stream_t stream) {
    if (KN < 0 || KH < 1 || KW < 1 || C < 1 || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if (KN == 0) return TAB_OK;
    if (!qw || !w8) return TAB_E_NULL_POINTER;
    if (misaligned(qw, 7) || misaligned(w8, 15)) return TAB_E_ALIGNMENT;
    return expand_weights_dispatch(qw, w8, bitwidth == 1 ? 1 : 2, KN, KH, KW, C, reinterpret_cast<cudaStream_t>(stream));
}

size_t tab_conv2d_state_bytes(int N) { return N < 0 ? 0 : round256((size_t)N * 8 + 16); }   // sums, completion counter, two grid-barrier words

// Shared by the two GEMM-stage entry points: y (float) or y16 (int16) receives the result.
// next_qx (optional, with next_ths): the result quantised at next_bits against next_ths, as tab_quantize_launch would write it.
static int bits_impl(const int64_t* qx, const int8_t* w8, float* y, int16_t* y16, int type, int p1, int p2, int s1, int s2,
                     int N, int H, int W, int C, int KN, int KH, int KW,
                     const float* residual, void* state, float* next_ths, float next_scale, tab_stream_t stream,
                     int64_t* next_qx = nullptr, int next_bits = 0) {
    int rc = conv_args_ok(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW);
    if (rc != TAB_OK) return rc;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (next_ths && !state) return TAB_E_NULL_POINTER;
    if (next_qx && (!next_ths || next_bits < 1)) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (KN == 0 || oh <= 0 || ow <= 0) {                            // empty output: mean |y| of nothing is 0
        if (next_ths) {
            cudaError_t e = cudaMemsetAsync(next_ths, 0, sizeof(float) * (size_t)N, reinterpret_cast<cudaStream_t>(stream));
            if (e != cudaSuccess) return record_cuda_error(e);
        }
        return TAB_OK;
    }
    if (!qx || !w8 || (!y && !y16)) return TAB_E_NULL_POINTER;
    if (misaligned(qx, 15) || misaligned(w8, 15) || misaligned(y, 15) || misaligned(y16, 15) || misaligned(residual, 15) || misaligned(state, 7) ||
        misaligned(next_ths, 3) || misaligned(next_qx, 7))
        return TAB_E_ALIGNMENT;
    if (y16 && (long long)KH * KW * C > 32767) return TAB_E_TOO_LARGE;   // |y| <= KH*KW*C must fit 16 bits
    TcConvParams p = tc_geometry(type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, oh, ow);
    p.qx = reinterpret_cast<const uint64_t*>(qx); p.w8 = w8; p.y = y; p.y16 = y16; p.residual = residual;
    if (next_ths) {
        p.abs_sums = reinterpret_cast<double*>(state);
        p.done_counter = reinterpret_cast<unsigned*>(reinterpret_cast<double*>(state) + N);
        p.ths_out = next_ths; p.ths_scale = next_scale; p.self_clean = 1;
    }
    // The grid quantises its own result when the words line up with the filter count, the thresholds fit its shared memory
    // and the result is small (up to 8M values); otherwise the quantiser runs as a launch of its own behind it.  Same bits
    // either way.  Measured on B200 (GEMM stage + quantiser, us, in-kernel / separate launch): results of 0.1-0.8M values
    // 23-29 / 32-49; 6.4M values 46-57 / 45-57; 12.8M 54-87 / 52-83; 51M 124-189 / 116-161 - the quantiser's own grid has
    // twice the warps per SM of the GEMM kernel's 16 and streams large tensors faster than the launch it saves.
    const bool in_kernel = next_qx && (KN % 64) == 0 && N <= 8192 && (long long)N * oh * ow * KN <= (1LL << 23) && !misaligned(next_qx, 15) &&
                           !misaligned(y, 31);
    if (in_kernel) {
        p.next_qx = reinterpret_cast<uint64_t*>(next_qx); p.next_bits = next_bits == 1 ? 1 : 2;
        p.grid_bar = p.done_counter + 1;
    }
    tc_forget_last_kernel();
    rc = tc_conv_dispatch(p, reinterpret_cast<cudaStream_t>(stream));
    if (rc != TAB_OK || !next_qx || in_kernel) return rc;
    return quantize_dispatch(y16 ? static_cast<const void*>(y16) : static_cast<const void*>(y), next_ths, next_qx, nullptr, next_bits == 1 ? 1 : 2,
                             N, (int)oh, (int)ow, KN, reinterpret_cast<cudaStream_t>(stream), nullptr, y16 != nullptr);
}

int tab_conv2d_bits_launch(const int64_t* qx, const int8_t* w8, float* y, int type, int p1, int p2, int s1, int s2,
                           int N, int H, int W, int C, int KN, int KH, int KW,
                           const float* residual, void* state, float* next_ths, float next_scale, tab_stream_t stream) {
    return bits_impl(qx, w8, y, nullptr, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, residual, state, next_ths, next_scale, stream);
}

int tab_conv2d_bits_i16_launch(const int64_t* qx, const int8_t* w8, int16_t* y16, int type, int p1, int p2, int s1, int s2,
                               int N, int H, int W, int C, int KN, int KH, int KW,
                               void* state, float* next_ths, float next_scale, tab_stream_t stream) {
    return bits_impl(qx, w8, nullptr, y16, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, nullptr, state, next_ths, next_scale, stream);
}

int tab_conv2d_bits_next_launch(const int64_t* qx, const int8_t* w8, void* y, int y_is_int16, int type, int p1, int p2, int s1, int s2,
                                int N, int H, int W, int C, int KN, int KH, int KW,
                                const float* residual, void* state, float* next_ths, float next_scale,
                                int64_t* next_qx, int next_bitwidth, tab_stream_t stream) {
    if (!next_qx || !next_ths || !state) return TAB_E_NULL_POINTER;
    if (y_is_int16 && residual) return TAB_E_BAD_ARGUMENT;
    return bits_impl(qx, w8, y_is_int16 ? nullptr : static_cast<float*>(y), y_is_int16 ? static_cast<int16_t*>(y) : nullptr,
                     type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, residual, state, next_ths, next_scale, stream, next_qx, next_bitwidth);
}

int tab_quantize_auto_launch(const float* x, float scale, void* state, float* ths, int64_t* qx, int bitwidth, int N, int H, int W, int C,
                             tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (!ths || !state) return TAB_E_NULL_POINTER;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const long long per_image = (long long)H * W * C;
    if (per_image == 0) {
        cudaError_t e = cudaMemsetAsync(ths, 0, sizeof(float) * (size_t)N, s);
        return e == cudaSuccess ? TAB_OK : record_cuda_error(e);
    }
    if (!x || !qx) return TAB_E_NULL_POINTER;
    if (misaligned(x, 3) || misaligned(ths, 3) || misaligned(qx, 7) || misaligned(state, 7)) return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    double* sums = reinterpret_cast<double*>(state);
    unsigned* bar = reinterpret_cast<unsigned*>(sums + N) + 1;
    int rc = quantize_auto_dispatch(x, scale, sums, bar, ths, qx, bitwidth == 1 ? 1 : 2, N, H, W, C, device_status_word(), s);
    if (rc != TAB_E_TOO_LARGE) return rc;
    // shapes the one-launch form does not take: sums, thresholds, quantiser as launches of their own (x is not modified)
    rc = residual_abs_sum_dispatch(const_cast<float*>(x), nullptr, sums, N, per_image, s);
    if (rc != TAB_OK) return rc;
    rc = tab_threshold_from_sums_launch(sums, ths, scale, N, per_image, stream);
    if (rc != TAB_OK) return rc;
    cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(double) * (size_t)N, s);
    if (e != cudaSuccess) return record_cuda_error(e);
    return quantize_dispatch(x, ths, qx, nullptr, bitwidth == 1 ? 1 : 2, N, H, W, C, s, nullptr, false);
}

int tab_quantize_i16_launch(const int16_t* x, const float* ths, int64_t* qx, int bitwidth, int N, int H, int W, int C, tab_stream_t stream) {
    if (!dims_ok(N, H, W, C) || bitwidth < 1) return TAB_E_BAD_ARGUMENT;
    if ((long long)N * H * W == 0) return TAB_OK;
    if (!x || !ths || !qx) return TAB_E_NULL_POINTER;
    if (misaligned(x, 1) || misaligned(ths, 3) || misaligned(qx, 7)) return TAB_E_ALIGNMENT;
    if ((long long)H * W >= (1LL << 31)) return TAB_E_TOO_LARGE;
    return quantize_dispatch(x, ths, qx, nullptr, bitwidth == 1 ? 1 : 2, N, H, W, C, reinterpret_cast<cudaStream_t>(stream), nullptr, true);
}

}  // extern "C"
