// Register-only probes of the POPC and LOP3 issue rates, used by the benchmark as roofline
// denominators for the convolution (the reference has no counterpart).
#include "tab_kernels.cuh"

namespace tab {

constexpr int PROBE_THREADS = 256;
constexpr int PROBE_CHAINS = 8;

template <int KIND>
__global__ void __launch_bounds__(PROBE_THREADS) pipe_probe_kernel(uint32_t* sink, int iters, uint32_t seed) {
    uint32_t v[PROBE_CHAINS], a[PROBE_CHAINS];
#pragma unroll
    for (int i = 0; i < PROBE_CHAINS; i++) { v[i] = seed * (threadIdx.x + 1) + i * 7919u; a[i] = i; }
    const uint32_t c1 = seed * 3 + threadIdx.x, c2 = seed * 5 + 1;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < PROBE_CHAINS; i++) {
            if (KIND == 0) {
                uint32_t q;
                asm volatile("popc.b32 %0, %1;" : "=r"(q) : "r"(v[i]));
                v[i] = q ^ a[i];
                a[i] += q;
            } else {
                uint32_t r, r2;
                asm volatile("lop3.b32 %0, %1, %2, %3, 0x96;" : "=r"(r) : "r"(v[i]), "r"(v[(i + 1) & 7]), "r"(c1));
                asm volatile("lop3.b32 %0, %1, %2, %3, 0xE8;" : "=r"(r2) : "r"(r), "r"(v[(i + 3) & 7]), "r"(c2));
                v[i] = r2;
            }
        }
    }
    uint32_t s = 0;
#pragma unroll
    for (int i = 0; i < PROBE_CHAINS; i++) s += a[i] ^ v[i];
    sink[blockIdx.x * PROBE_THREADS + threadIdx.x] = s;
}

// s8 mma.sync from registers: 8 independent accumulator tiles per warp.
__global__ void __launch_bounds__(PROBE_THREADS) imma_probe_kernel(uint32_t* sink, int iters, uint32_t seed) {
    uint32_t a[4], b[2];
    int c[8][4];
#pragma unroll
    for (int i = 0; i < 4; i++) a[i] = seed * (threadIdx.x + 1) + i * 977u;
#pragma unroll
    for (int i = 0; i < 2; i++) b[i] = seed * 31u + threadIdx.x * 7u + i;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) c[j][i] = 0;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+r"(c[j][0]), "+r"(c[j][1]), "+r"(c[j][2]), "+r"(c[j][3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
    }
    int s = 0;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) s += c[j][i];
    sink[blockIdx.x * PROBE_THREADS + threadIdx.x] = (uint32_t)s;
}

// 1-bit mma.sync (m16n8k256, and.popc or xor.popc) from registers: shows whether a binary MMA is native.
template <int XOR>
__global__ void __launch_bounds__(PROBE_THREADS) b1mma_probe_kernel(uint32_t* sink, int iters, uint32_t seed) {
    uint32_t a[4], b[2];
    int c[8][4];
#pragma unroll
    for (int i = 0; i < 4; i++) a[i] = seed * (threadIdx.x + 1) + i * 977u;
#pragma unroll
    for (int i = 0; i < 2; i++) b[i] = seed * 31u + threadIdx.x * 7u + i;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) c[j][i] = 0;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (XOR)
                asm volatile("mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.xor.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+r"(c[j][0]), "+r"(c[j][1]), "+r"(c[j][2]), "+r"(c[j][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
            else
                asm volatile("mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+r"(c[j][0]), "+r"(c[j][1]), "+r"(c[j][2]), "+r"(c[j][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
        }
    }
    int s = 0;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) s += c[j][i];
    sink[blockIdx.x * PROBE_THREADS + threadIdx.x] = (uint32_t)s;
}

static int probe_blocks() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms * 8;
}

}  // namespace tab

namespace tab { int umma_probe_dispatch(int shape, int iters, uint32_t* sink, int blocks, double* ops_out, cudaStream_t stream); }

using namespace tab;

extern "C" size_t tab_pipe_probe_sink_bytes(void) { return (size_t)probe_blocks() * PROBE_THREADS * 4; }

extern "C" int tab_pipe_probe_launch(int kind, int iters, void* sink, double* ops_out, tab_stream_t stream) {
    if (kind < 0 || kind > 204 || iters < 1) return TAB_E_BAD_ARGUMENT;
    if (!sink) return TAB_E_NULL_POINTER;
    const int blocks = probe_blocks();
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (kind >= 5) return umma_probe_dispatch(kind - 5, iters, (uint32_t*)sink, blocks / 8, ops_out, s);   // one CTA per SM
    if (kind == 0) pipe_probe_kernel<0><<<blocks, PROBE_THREADS, 0, s>>>((uint32_t*)sink, iters, 12345u);
    else if (kind == 1) pipe_probe_kernel<1><<<blocks, PROBE_THREADS, 0, s>>>((uint32_t*)sink, iters, 12345u);
    else if (kind == 2) imma_probe_kernel<<<blocks, PROBE_THREADS, 0, s>>>((uint32_t*)sink, iters, 12345u);
    else if (kind == 3) b1mma_probe_kernel<0><<<blocks, PROBE_THREADS, 0, s>>>((uint32_t*)sink, iters, 12345u);
    else b1mma_probe_kernel<1><<<blocks, PROBE_THREADS, 0, s>>>((uint32_t*)sink, iters, 12345u);
    if (ops_out) {
        if (kind == 2) *ops_out = (double)blocks * (PROBE_THREADS / 32) * (double)iters * 8.0 * (16.0 * 8 * 32 * 2);
        else if (kind >= 3) *ops_out = (double)blocks * (PROBE_THREADS / 32) * (double)iters * 8.0 * (16.0 * 8 * 256 * 2);
        else *ops_out = (double)blocks * PROBE_THREADS * (double)iters * PROBE_CHAINS * (kind == 0 ? 1.0 : 2.0);
    }
    return check_launch();
}
