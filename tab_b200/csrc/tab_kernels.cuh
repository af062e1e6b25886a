// Shared declarations for the sm_100a kernels behind the C ABI in include/tab_b200.h.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/tab_b200.h"

namespace tab {

// Records a CUDA failure for tab_last_cuda_error() and maps it to TAB_E_CUDA.
int record_cuda_error(cudaError_t e);

// cudaGetLastError() right after a launch -> TAB_OK or TAB_E_CUDA.
inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TAB_OK : record_cuda_error(e);
}

inline int packed_channels(int C) { return (C + 63) / 64; }
inline int act_bits(int type) { return (type == 2 || type == 3) ? 1 : 2; }      // TAB_GEMM.cu:367-372
inline int weight_bits(int type) { return (type == 1 || type == 3) ? 1 : 2; }   // TAB_GEMM.cu:374-379

// quantize_sm100.cu: bits is 1 or 2; btn may be null; btn must already be zero.
int quantize_dispatch(const float* x, const float* ths, int64_t* qx, int32_t* btn, int bits,
                      int N, int H, int W, int C, cudaStream_t stream);

// conv_sm100.cu: implicit-im2col popcount GEMM on packed activations.
int conv_packed_dispatch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y, int type,
                         int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                         int KN, int KH, int KW, cudaStream_t stream);

}  // namespace tab
