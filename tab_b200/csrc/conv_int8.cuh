// Definitions shared by the byte-operand (int8) convolution kernels: the mma.sync variants in
// conv_imma_sm100.cu and the tcgen05 variant in conv_umma_sm100.cu.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tab {

constexpr int IKW = 2;                       // 64-channel words per K chunk (128 bytes per smem row)
constexpr int IROW = IKW * 64;               // bytes per smem row

struct ImmaParams {
    const int8_t* qx;        // [N][H][W][Cp]
    const int8_t* w8;        // [KN][Kw][64]
    float* y;                // [M][KN]
    const float* residual;   // [M][KN] added to the result, or null
    double* abs_sums;        // [N]: += sum |y| per image, or null
    int N, H, W, PC, KN, KH, KW, OH, OW, p1, p2, s1, s2;
    int M, Kw;
    // Optional tail of a fused launch: the CTA that finishes last turns the sums into the next layer's thresholds,
    // ths_out[n] = ths_scale * abs_sums[n] / per_image (null = leave that to the caller).
    float* ths_out = nullptr;
    float ths_scale = 0.f;
    double per_image = 1.0;
    unsigned* done_counter = nullptr;   // zero before the launch
};

// Host-side description of that tail.
struct FusedTail { float* ths_out; float scale; unsigned* counter; };

// Called by every thread of every CTA at the end of a fused kernel, after the CTA's last atomic on abs_sums.
__device__ __forceinline__ void fused_finish(const ImmaParams& p) {
    if (p.ths_out == nullptr) return;
    __threadfence();
    int mine = 0;
    __syncthreads();                                                       // every thread's atomics are issued and fenced
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        mine = (atomicAdd(p.done_counter, 1u) == total - 1u);
    }
    const int last = __syncthreads_or(mine);                               // no shared memory: the kernels use all of it
    if (last) {
        __threadfence();
        for (int n = threadIdx.x; n < p.N; n += blockDim.x) {
            const double sum = __ldcg(p.abs_sums + n);                     // the other CTAs' atomics live in L2
            p.ths_out[n] = (float)((double)p.ths_scale * (sum / p.per_image));
        }
    }
}

__device__ __forceinline__ void cp16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void sts16(uint32_t dst, uint32_t v) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(v));
}
// smem byte offset of 16-byte unit `u` (0..7) of row `r`: XOR swizzle, conflict-free for 8 consecutive rows.
__device__ __forceinline__ uint32_t swz(int r, int u) { return (uint32_t)(r * IROW + ((u ^ (r & 7)) << 4)); }

}  // namespace tab
