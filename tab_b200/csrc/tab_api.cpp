// PyTorch extension module TAB_CUDA: the reference's binding surface (TAB_GPU.cpp:34-65) over the C ABI
// in include/tab_b200.h.  This is the only translation unit that includes torch headers; it holds no
// arithmetic.  Exports Quantize / Conv2d (TAB_GPU.cpp:63-64) and the aliases TAB_Quantize / TAB_Conv2d
// used by the reference's CPU module and README (TAB_CPU.cpp:637-638).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <vector>
#include "../../include/tab_b200.h"

// Same checks and messages as the reference (TAB_GPU.cpp:7-9).
#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) CHECK_CUDA(x); CHECK_CONTIGUOUS(x)

static void check_rc(int rc, const char* where) {
    TORCH_CHECK(rc == TAB_OK, where, ": ", tab_error_string(rc), " (code ", rc, ", cudaError ", tab_last_cuda_error(), ")");
}

static tab_stream_t current_stream() {
    return reinterpret_cast<tab_stream_t>(at::cuda::getCurrentCUDAStream().stream());
}

// Quantize the input to {+1,0,-1} (bitwidth != 1) or {+1,-1} (bitwidth == 1).  X: N,H,W,C float32;
// thresholds: float32[N].  Returns {QX int64 {N,H,W,PC,bits}, BTN_W int32 {N}}  (TAB_GPU.cpp:53-58).
std::vector<torch::Tensor> TAB_Quantize(torch::Tensor X, torch::Tensor thresholds, int bitwidth, int N, int H, int W, int C) {
    CHECK_INPUT(X);
    CHECK_INPUT(thresholds);
    // The reference converts dtypes and keeps a pointer into the temporary (TAB_GEMM.cu:279-280); here
    // the dtypes are required instead.
    TORCH_CHECK(X.scalar_type() == torch::kFloat32, "X must have dtype torch.float32");
    TORCH_CHECK(thresholds.scalar_type() == torch::kFloat32, "thresholds must have dtype torch.float32");
    TORCH_CHECK(N >= 0 && H >= 0 && W >= 0 && C >= 1 && bitwidth >= 1, "Quantize: sizes must be non-negative, C >= 1 and bitwidth >= 1");
    TORCH_CHECK(X.numel() == (int64_t)N * H * W * C, "X has ", X.numel(), " elements, expected N*H*W*C = ", (int64_t)N * H * W * C);
    TORCH_CHECK(thresholds.numel() == N, "thresholds has ", thresholds.numel(), " elements, expected N = ", N);
    const c10::cuda::CUDAGuard guard(X.device());
    const int bits = bitwidth == 1 ? 1 : 2;
    const int PC = (C + 63) / 64;
    auto QX = torch::empty({N, H, W, PC, bits}, torch::device(X.device()).dtype(torch::kInt64));
    auto BTN = torch::empty({N}, torch::device(X.device()).dtype(torch::kInt32));
    check_rc(tab_quantize_launch(X.data_ptr<float>(), thresholds.data_ptr<float>(), QX.data_ptr<int64_t>(),
                                 BTN.data_ptr<int32_t>(), bitwidth, N, H, W, C, current_stream()),
             "tab_quantize_launch");
    return {QX, BTN};
}

// Convolution of all TAB types: 0 TNN, 1 TBN, 2 BTN, 3 BNN (TAB_GPU.cpp:34-42).  Returns float32
// {N,KN,OH,OW} whose buffer is in [N][OH][OW][KN] order (TAB_GEMM.cu:509,526).
torch::Tensor TAB_Conv2d(torch::Tensor X, torch::Tensor QW, torch::Tensor thresholds, torch::Tensor btn, int type,
                         int padding1, int padding2, int stride1, int stride2,
                         int N, int H, int W, int C, int KN, int KH, int KW) {
    CHECK_INPUT(X);
    CHECK_INPUT(QW);
    CHECK_INPUT(thresholds);
    CHECK_INPUT(btn);
    TORCH_CHECK(X.scalar_type() == torch::kFloat32, "X must have dtype torch.float32");
    TORCH_CHECK(QW.scalar_type() == torch::kInt64, "QW must have dtype torch.int64");
    TORCH_CHECK(thresholds.scalar_type() == torch::kFloat32, "thresholds must have dtype torch.float32");
    TORCH_CHECK(btn.scalar_type() == torch::kInt32, "btn must have dtype torch.int32");
    TORCH_CHECK(type >= 0 && type <= 3, "type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)");
    TORCH_CHECK(N >= 0 && H >= 0 && W >= 0 && KN >= 0 && C >= 1 && KH >= 1 && KW >= 1 && padding1 >= 0 && padding2 >= 0 &&
                stride1 >= 1 && stride2 >= 1, "Conv2d: invalid size, padding or stride");
    const int PC = (C + 63) / 64;
    const int wb = (type == 1 || type == 3) ? 1 : 2;
    const int64_t need = (int64_t)KN * KH * KW * PC * wb;
    TORCH_CHECK(QW.numel() == need, "QW has ", QW.numel(), " words, type ", type, " needs KN*KH*KW*ceil(C/64)*", wb, " = ", need,
                " (quantise the weights at bitwidth ", wb, ")");
    TORCH_CHECK(type != 2 || btn.numel() == KN, "btn has ", btn.numel(), " elements, expected KN = ", KN);
    TORCH_CHECK(X.numel() == (int64_t)N * H * W * C, "X has ", X.numel(), " elements, expected N*H*W*C = ", (int64_t)N * H * W * C);
    TORCH_CHECK(thresholds.numel() == N, "thresholds has ", thresholds.numel(), " elements, expected N = ", N);
    const c10::cuda::CUDAGuard guard(X.device());
    const int64_t OH = std::max<int64_t>(((int64_t)H + 2 * padding1 - KH + 1) / stride1, 0);
    const int64_t OW = std::max<int64_t>(((int64_t)W + 2 * padding2 - KW + 1) / stride2, 0);
    auto Y = torch::empty({N, KN, OH, OW}, torch::device(X.device()).dtype(torch::kFloat32));
    const size_t ws_bytes = tab_conv2d_workspace_bytes(type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW);
    auto ws = torch::empty({(int64_t)std::max<size_t>(ws_bytes, 256)}, torch::device(X.device()).dtype(torch::kUInt8));
    check_rc(tab_conv2d_launch(X.data_ptr<float>(), QW.data_ptr<int64_t>(), thresholds.data_ptr<float>(),
                               btn.data_ptr<int32_t>(), Y.data_ptr<float>(), ws.data_ptr(), (size_t)ws.numel(), type,
                               padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW, current_stream()),
             "tab_conv2d_launch");
    return Y;
}

// Extension beyond the reference's surface: Conv2d with the residual addition and the statistics for the next
// layer's thresholds fused into the convolution.  residual may be an undefined tensor (None); threshold_scale
// <= 0 skips the thresholds.  Returns {Y, next_thresholds (empty when skipped)}.
std::vector<torch::Tensor> TAB_Conv2dFused(torch::Tensor X, torch::Tensor QW, torch::Tensor thresholds, torch::Tensor btn, int type,
                                           int padding1, int padding2, int stride1, int stride2,
                                           int N, int H, int W, int C, int KN, int KH, int KW,
                                           c10::optional<torch::Tensor> residual, double threshold_scale) {
    CHECK_INPUT(X);
    CHECK_INPUT(QW);
    CHECK_INPUT(thresholds);
    CHECK_INPUT(btn);
    TORCH_CHECK(X.scalar_type() == torch::kFloat32 && thresholds.scalar_type() == torch::kFloat32, "X and thresholds must be float32");
    TORCH_CHECK(QW.scalar_type() == torch::kInt64 && btn.scalar_type() == torch::kInt32, "QW must be int64 and btn int32");
    TORCH_CHECK(type >= 0 && type <= 3, "type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)");
    TORCH_CHECK(N >= 0 && H >= 0 && W >= 0 && KN >= 0 && C >= 1 && KH >= 1 && KW >= 1 && padding1 >= 0 && padding2 >= 0 &&
                stride1 >= 1 && stride2 >= 1, "Conv2d: invalid size, padding or stride");
    const int PC = (C + 63) / 64;
    const int wb = (type == 1 || type == 3) ? 1 : 2;
    TORCH_CHECK(QW.numel() == (int64_t)KN * KH * KW * PC * wb, "QW does not match KN*KH*KW*ceil(C/64)*", wb);
    TORCH_CHECK(X.numel() == (int64_t)N * H * W * C && thresholds.numel() == N, "X / thresholds do not match N*H*W*C / N");
    const c10::cuda::CUDAGuard guard(X.device());
    const int64_t OH = std::max<int64_t>(((int64_t)H + 2 * padding1 - KH + 1) / stride1, 0);
    const int64_t OW = std::max<int64_t>(((int64_t)W + 2 * padding2 - KW + 1) / stride2, 0);
    const float* rptr = nullptr;
    if (residual.has_value() && residual->defined()) {
        CHECK_INPUT((*residual));
        TORCH_CHECK(residual->scalar_type() == torch::kFloat32 && residual->numel() == (int64_t)N * KN * OH * OW, "residual must be float32 with N*KN*OH*OW elements");
        rptr = residual->data_ptr<float>();
    }
    auto Y = torch::empty({N, KN, OH, OW}, torch::device(X.device()).dtype(torch::kFloat32));
    const size_t ws_bytes = tab_conv2d_workspace_bytes(type, padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW);
    auto ws = torch::empty({(int64_t)std::max<size_t>(ws_bytes, 256)}, torch::device(X.device()).dtype(torch::kUInt8));
    torch::Tensor sums, next;
    const bool want = threshold_scale > 0;
    if (want) sums = torch::empty({std::max(N, 1)}, torch::device(X.device()).dtype(torch::kFloat64));
    next = torch::empty({want ? N : 0}, torch::device(X.device()).dtype(torch::kFloat32));
    check_rc(tab_conv2d_chain_launch(X.data_ptr<float>(), QW.data_ptr<int64_t>(), thresholds.data_ptr<float>(), btn.data_ptr<int32_t>(),
                                     Y.data_ptr<float>(), ws.data_ptr(), (size_t)ws.numel(), type, padding1, padding2, stride1, stride2,
                                     N, H, W, C, KN, KH, KW, rptr, want ? sums.data_ptr<double>() : nullptr,
                                     (want && N > 0) ? next.data_ptr<float>() : nullptr, (float)threshold_scale, current_stream()),
             "tab_conv2d_chain_launch");
    return {Y, next};
}

// Extensions for callers that keep prepared weights (tab_b200.nn.TABConv2d and the like): the stages of Conv2d on their own.
// ExpandWeights: packed weights -> int8 {KN,KH,KW,Cp}.
torch::Tensor TAB_ExpandWeights(torch::Tensor QW, int bitwidth, int KN, int KH, int KW, int C) {
    CHECK_INPUT(QW);
    TORCH_CHECK(QW.scalar_type() == torch::kInt64, "QW must have dtype torch.int64");
    TORCH_CHECK(KN >= 0 && KH >= 1 && KW >= 1 && C >= 1 && bitwidth >= 1, "ExpandWeights: invalid size or bitwidth");
    const int PC = (C + 63) / 64, bits = bitwidth == 1 ? 1 : 2;
    TORCH_CHECK(QW.numel() == (int64_t)KN * KH * KW * PC * bits, "QW has ", QW.numel(), " words, expected ", (int64_t)KN * KH * KW * PC * bits);
    const c10::cuda::CUDAGuard guard(QW.device());
    auto W8 = torch::empty({KN, KH, KW, PC * 64}, torch::device(QW.device()).dtype(torch::kInt8));
    check_rc(tab_expand_weights_launch(QW.data_ptr<int64_t>(), W8.data_ptr<int8_t>(), bits, KN, KH, KW, C, current_stream()),
             "tab_expand_weights_launch");
    return W8;
}

// QuantizeI16: Quantize on the int16 tensor Conv2dBits(..., out_int16 = true) returned; returns QX only.
torch::Tensor TAB_QuantizeI16(torch::Tensor X16, torch::Tensor thresholds, int bitwidth, int N, int H, int W, int C) {
    CHECK_INPUT(X16);
    CHECK_INPUT(thresholds);
    TORCH_CHECK(X16.scalar_type() == torch::kInt16, "X16 must have dtype torch.int16");
    TORCH_CHECK(thresholds.scalar_type() == torch::kFloat32, "thresholds must have dtype torch.float32");
    TORCH_CHECK(N >= 0 && H >= 0 && W >= 0 && C >= 1 && bitwidth >= 1, "Quantize: sizes must be non-negative, C >= 1 and bitwidth >= 1");
    TORCH_CHECK(X16.numel() == (int64_t)N * H * W * C && thresholds.numel() == N, "X16 / thresholds do not match N*H*W*C / N");
    const c10::cuda::CUDAGuard guard(X16.device());
    auto QX = torch::empty({N, H, W, (C + 63) / 64, bitwidth == 1 ? 1 : 2}, torch::device(X16.device()).dtype(torch::kInt64));
    check_rc(tab_quantize_i16_launch(X16.data_ptr<int16_t>(), thresholds.data_ptr<float>(), QX.data_ptr<int64_t>(), bitwidth, N, H, W, C, current_stream()),
             "tab_quantize_i16_launch");
    return QX;
}

// NewState: the zeroed block Conv2dBits needs when it is asked for thresholds.
torch::Tensor TAB_NewState(torch::Tensor like, int N) {
    CHECK_CUDA(like);
    return torch::zeros({(int64_t)std::max<size_t>(tab_conv2d_state_bytes(N), 8)}, torch::device(like.device()).dtype(torch::kUInt8));
}

// Conv2dBits: the GEMM stage of Conv2d on activations Quantize wrote (bitwidth 2 for types 0,1; 1 for types 2,3) and
// weights from ExpandWeights; residual / state may be None; threshold_scale <= 0 skips the thresholds; out_int16: Y as int16
// (no residual; the values are integers of magnitude at most KH*KW*C), for QuantizeI16.
// next_bitwidth 1 or 2 (needs threshold_scale > 0): the same call also quantises Y against the next thresholds, as
// Quantize(Y, next_thresholds, next_bitwidth, N, OH, OW, KN) would, and returns it as a third tensor.
// Returns {Y, next_thresholds (empty when skipped)[, next_QX]}.
std::vector<torch::Tensor> TAB_Conv2dBits(torch::Tensor QX, torch::Tensor W8, int type,
                                          int padding1, int padding2, int stride1, int stride2,
                                          int N, int H, int W, int C, int KN, int KH, int KW,
                                          c10::optional<torch::Tensor> residual, c10::optional<torch::Tensor> state, double threshold_scale,
                                          bool out_int16, int next_bitwidth) {
    CHECK_INPUT(QX);
    CHECK_INPUT(W8);
    TORCH_CHECK(QX.scalar_type() == torch::kInt64, "QX must have dtype torch.int64");
    TORCH_CHECK(W8.scalar_type() == torch::kInt8, "W8 must have dtype torch.int8");
    TORCH_CHECK(type >= 0 && type <= 3, "type must be 0 (TNN), 1 (TBN), 2 (BTN) or 3 (BNN)");
    TORCH_CHECK(N >= 0 && H >= 0 && W >= 0 && KN >= 0 && C >= 1 && KH >= 1 && KW >= 1 && padding1 >= 0 && padding2 >= 0 &&
                stride1 >= 1 && stride2 >= 1, "Conv2d: invalid size, padding or stride");
    const int PC = (C + 63) / 64, ab = (type == 2 || type == 3) ? 1 : 2;
    TORCH_CHECK(QX.numel() == (int64_t)N * H * W * PC * ab, "QX has ", QX.numel(), " words, type ", type, " needs ", (int64_t)N * H * W * PC * ab);
    TORCH_CHECK(W8.numel() == (int64_t)KN * KH * KW * PC * 64, "W8 has ", W8.numel(), " bytes, expected KN*KH*KW*Cp = ", (int64_t)KN * KH * KW * PC * 64);
    const c10::cuda::CUDAGuard guard(QX.device());
    const int64_t OH = std::max<int64_t>(((int64_t)H + 2 * padding1 - KH + 1) / stride1, 0);
    const int64_t OW = std::max<int64_t>(((int64_t)W + 2 * padding2 - KW + 1) / stride2, 0);
    const float* rptr = nullptr;
    if (residual.has_value() && residual->defined()) {
        CHECK_INPUT((*residual));
        TORCH_CHECK(residual->scalar_type() == torch::kFloat32 && residual->numel() == (int64_t)N * KN * OH * OW, "residual must be float32 with N*KN*OH*OW elements");
        rptr = residual->data_ptr<float>();
    }
    const bool want = threshold_scale > 0;
    void* sptr = nullptr;
    if (want) {
        TORCH_CHECK(state.has_value() && state->defined(), "threshold_scale needs a state block (NewState)");
        CHECK_INPUT((*state));
        TORCH_CHECK((size_t)state->numel() * state->element_size() >= tab_conv2d_state_bytes(N), "state block too small");
        sptr = state->data_ptr();
    }
    auto next = torch::empty({want ? N : 0}, torch::device(QX.device()).dtype(torch::kFloat32));
    if (next_bitwidth > 0) {
        TORCH_CHECK(want, "next_bitwidth needs threshold_scale > 0 (the thresholds the result is quantised against)");
        TORCH_CHECK(!(out_int16 && rptr), "out_int16 cannot be combined with a residual");
        auto Yn = torch::empty({N, KN, OH, OW}, torch::device(QX.device()).dtype(out_int16 ? torch::kInt16 : torch::kFloat32));
        auto QN = torch::empty({N, OH, OW, (KN + 63) / 64, next_bitwidth == 1 ? 1 : 2}, torch::device(QX.device()).dtype(torch::kInt64));
        if (N > 0)
            check_rc(tab_conv2d_bits_next_launch(QX.data_ptr<int64_t>(), W8.data_ptr<int8_t>(), Yn.data_ptr(), out_int16 ? 1 : 0, type,
                                                 padding1, padding2, stride1, stride2, N, H, W, C, KN, KH, KW, rptr, sptr, next.data_ptr<float>(),
                                                 (float)threshold_scale, QN.data_ptr<int64_t>(), next_bitwidth, current_stream()),
                     "tab_conv2d_bits_next_launch");
        return {Yn, next, QN};
    }
    if (out_int16) {
        TORCH_CHECK(rptr == nullptr, "out_int16 cannot be combined with a residual");
        auto Y16 = torch::empty({N, KN, OH, OW}, torch::device(QX.device()).dtype(torch::kInt16));
        check_rc(tab_conv2d_bits_i16_launch(QX.data_ptr<int64_t>(), W8.data_ptr<int8_t>(), Y16.data_ptr<int16_t>(), type, padding1, padding2, stride1, stride2,
                                            N, H, W, C, KN, KH, KW, sptr, (want && N > 0) ? next.data_ptr<float>() : nullptr, (float)threshold_scale,
                                            current_stream()),
                 "tab_conv2d_bits_i16_launch");
        return {Y16, next};
    }
    auto Y = torch::empty({N, KN, OH, OW}, torch::device(QX.device()).dtype(torch::kFloat32));
    check_rc(tab_conv2d_bits_launch(QX.data_ptr<int64_t>(), W8.data_ptr<int8_t>(), Y.data_ptr<float>(), type, padding1, padding2, stride1, stride2,
                                    N, H, W, C, KN, KH, KW, rptr, sptr, (want && N > 0) ? next.data_ptr<float>() : nullptr, (float)threshold_scale,
                                    current_stream()),
             "tab_conv2d_bits_launch");
    return {Y, next};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("Conv2dFused", &TAB_Conv2dFused, "Conv2d + residual + next-layer thresholds (extension)");
    m.def("ExpandWeights", &TAB_ExpandWeights, "Packed weights -> int8 for the tensor-core GEMM stage (extension)");
    m.def("QuantizeI16", &TAB_QuantizeI16, "Quantize on the int16 output of Conv2dBits(out_int16=True) (extension)");
    m.def("NewState", &TAB_NewState, "Zeroed state block for Conv2dBits thresholds (extension)");
    m.def("Conv2dBits", &TAB_Conv2dBits, "GEMM stage of Conv2d on Quantize's bit-planes and ExpandWeights' bytes (extension)",
          pybind11::arg("QX"), pybind11::arg("W8"), pybind11::arg("type"), pybind11::arg("padding1"), pybind11::arg("padding2"),
          pybind11::arg("stride1"), pybind11::arg("stride2"), pybind11::arg("N"), pybind11::arg("H"), pybind11::arg("W"), pybind11::arg("C"),
          pybind11::arg("KN"), pybind11::arg("KH"), pybind11::arg("KW"), pybind11::arg("residual"), pybind11::arg("state"),
          pybind11::arg("threshold_scale"), pybind11::arg("out_int16") = false, pybind11::arg("next_bitwidth") = 0);
    m.def("Quantize", &TAB_Quantize, "Ternarization or binarization of fp32 data in NHWC format");
    m.def("Conv2d", &TAB_Conv2d, "Conv2d of all TAB series CNNs (0 TNN, 1 TBN, 2 BTN, 3 BNN)");
    m.def("TAB_Quantize", &TAB_Quantize, "Alias of Quantize");
    m.def("TAB_Conv2d", &TAB_Conv2d, "Alias of Conv2d");
}
