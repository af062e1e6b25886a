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

// Launch with programmatic stream serialisation: the kernel may be scheduled while its predecessor in the stream is
// still draining (the predecessor executed griddepcontrol.launch_dependents in every CTA); it must execute
// griddepcontrol.wait before it touches anything a predecessor wrote or may still read.  Works under stream capture
// (the dependency becomes a programmatic edge of the graph).
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e == cudaSuccess ? TAB_OK : record_cuda_error(e);
}

// The same for a kernel that runs as thread-block clusters of `cluster` CTAs along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
inline int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    return e == cudaSuccess ? TAB_OK : record_cuda_error(e);
}

#ifdef __CUDACC__
// Device side of the above.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

inline int packed_channels(int C) { return (C + 63) / 64; }
inline int act_bits(int type) { return (type == 2 || type == 3) ? 1 : 2; }      // TAB_GEMM.cu:367-372
inline int weight_bits(int type) { return (type == 1 || type == 3) ? 1 : 2; }   // TAB_GEMM.cu:374-379

// Small jobs a quantiser launch does on the side for the convolution that follows it (all optional).
struct QuantExtras {
    double* zero_sums = nullptr;         // [N]: cleared
    unsigned* zero_counter = nullptr;    // cleared
    const uint64_t* qw = nullptr;        // packed weights [KN][KH*KW*PC][wbits] to expand into w8 [KN][KH*KW*PC][64]
    int8_t* w8 = nullptr;
    long long words = 0;                 // KN*KH*KW*PC
    int wbits = 2, PC = 1, C = 64;       // of the weights
};

// quantize_sm100.cu: bits is 1 or 2; btn may be null; btn must already be zero.  in16: x holds int16 instead of float.
int quantize_dispatch(const void* x, const float* ths, int64_t* qx, int32_t* btn, int bits,
                      int N, int H, int W, int C, cudaStream_t stream, const QuantExtras* extras = nullptr, bool in16 = false);
int expand_weights_dispatch(const int64_t* qw, int8_t* w8, int wbits, int KN, int KH, int KW, int C, cudaStream_t stream);
// Thresholds scale * mean|x[n]| and the bit-planes against them in one launch (sums: N doubles, bar: two words, all zero
// before and after); TAB_E_TOO_LARGE when the shape needs the separate launches.
int quantize_auto_dispatch(const float* x, float scale, double* sums, unsigned* bar, float* ths_out, int64_t* qx, int bits,
                           int N, int H, int W, int C, int* status, cudaStream_t stream);
// Device word that records a bounded wait that ran out (shared with the tensor-core kernel); null if unavailable.
int* device_status_word();

// conv_sm100.cu: implicit-im2col popcount GEMM on packed activations.  csa: carry-save popcount tree (else one POPC per word).
int conv_packed_dispatch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y, int type,
                         int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                         int KN, int KH, int KW, cudaStream_t stream, bool csa = true);

}  // namespace tab
