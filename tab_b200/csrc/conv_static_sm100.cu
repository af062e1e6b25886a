// tab_conv2d_static_launch: TAB_Conv2d for callers that have no way to hand this library a device
// workspace and must not trigger a device allocation themselves.
//
// Who that is: a host program whose device memory is owned entirely by someone else's pool (an
// inference server that reserved the whole GPU at start-up, so a cudaMalloc made here would fail or
// fragment the pool), a binding from a language runtime that can pass input/output buffers it was given
// but cannot create new device buffers, and latency-critical loops where cudaMalloc/cudaFree are
// forbidden because they synchronise the device.  tab_conv2d_launch needs scratch for the bit-packed
// activations; this entry point keeps that scratch inside the library image instead, as a fixed
// array in device global memory that exists from the moment the library is loaded on a GPU until the
// process exits.  The price is a hard size limit, no concurrency (see below) and the slower of the two compute
// paths: this entry point always runs the bit-packed LOP3/POPC kernel, because the tensor-core path also needs the
// weights expanded to bytes, which a modest fixed array cannot hold.
#include <mutex>
#include "tab_kernels.cuh"

namespace tab {

// The scratch itself.  In HOST code the name g_static_scratch is only a handle for the runtime's
// symbol table, not a device address: it must never be passed to a kernel.  The device address is
// obtained once per device with cudaGetSymbolAddress (below) and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[TAB_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_setup_mutex;
static void* g_scratch_addr[kMaxDevices] = {};   // per-device address of g_static_scratch

// First call on a device: resolve the array's address in that device's copy of the module.
static int static_scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= kMaxDevices) return TAB_E_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);    // device `dev` is current here
        if (e != cudaSuccess) return record_cuda_error(e);
        if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255)) return TAB_E_ALIGNMENT;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return TAB_OK;
}

}  // namespace tab

using namespace tab;

extern "C" int tab_conv2d_static_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                                        float* y, int type, int p1, int p2, int s1, int s2,
                                        int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream) {
    if (type < 0 || type > 3 || N < 0 || H < 0 || W < 0 || C < 1 || KN < 0 || KH < 1 || KW < 1 ||
        p1 < 0 || p2 < 0 || s1 < 1 || s2 < 1)
        return TAB_E_BAD_ARGUMENT;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (N == 0 || KN == 0 || oh <= 0 || ow <= 0) return TAB_OK;
    // packed activations: N*H*W*ceil(C/64) words per plane, 2 planes for types 0,1 and 1 for types 2,3.  The size is
    // bounded factor by factor, so that no product of unchecked ints can wrap around before it is compared.
    const unsigned long long cap_words = (unsigned long long)TAB_STATIC_SCRATCH_BYTES / 8ULL;
    const unsigned long long pixels = (unsigned long long)H * (unsigned long long)W;      // both < 2^31: no overflow
    if (pixels >= (1ULL << 31) || pixels > cap_words) return TAB_E_TOO_LARGE;
    const unsigned long long per_image = pixels * (unsigned long long)packed_channels(C) * (unsigned long long)act_bits(type);   // < 2^59
    if (per_image > cap_words || (unsigned long long)N > cap_words / per_image) return TAB_E_TOO_LARGE;
    if (!x || !ths || !qw || !y || (type == 2 && !btn)) return TAB_E_NULL_POINTER;
    // same alignment rules as tab_conv2d_launch: nothing misaligned may reach a kernel
    if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(ths) & 3) || (reinterpret_cast<uintptr_t>(qw) & 7) ||
        (reinterpret_cast<uintptr_t>(y) & 3) || (reinterpret_cast<uintptr_t>(btn) & 3))
        return TAB_E_ALIGNMENT;
    void* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != TAB_OK) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int64_t* qx = reinterpret_cast<int64_t*>(scratch);
    // Every word of the packed tensor that the convolution reads is written by the quantiser first, so
    // nothing in the scratch has to start at zero and the previous call's contents are harmless.
    rc = quantize_dispatch(x, ths, qx, nullptr, act_bits(type), N, H, W, C, s);
    if (rc != TAB_OK) return rc;
    return conv_packed_dispatch(qx, qw, btn, y, type, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, s);
}
