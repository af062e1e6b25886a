// Issue-rate probe of the tensor pipe, used by the benchmark as the roofline denominator of the convolution's GEMM
// stage (the reference has no counterpart).
#include "tab_kernels.cuh"
#include "umma_common.cuh"

namespace tab {

// Issue-rate probe for the tensor pipe: every CTA (one per SM) issues `iters` x 4 int8 MMAs of 128 x TN x 32 on
// operands that already sit in shared memory (K-major, 128-byte swizzle, as the convolution kernels lay them out),
// with no copies and no epilogue - the rate the GEMM kernels can at best reach for that instruction shape.
// mode 0: back-to-back MMAs, one commit at the end.  mode 1: a commit after every group of 4 x NA MMAs (nobody
// waits on it).  mode 2: the groups go through a ring of four slots with the full/empty handshake the convolution
// kernels use (another thread plays the producer, without copying anything).
template <int TNI, int NA>
__global__ void __launch_bounds__(128, 1) umma_probe_kernel(uint32_t* __restrict__ sink, int iters, int* __restrict__ status,
                                                            int shift_rows, int mode) {
    constexpr int S = 4;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t sA = sbase + shift_rows * IROW, sB = sbase + (NA * UTM + 8) * IROW;
    const int tail = (NA * UTM + 8) * IROW + TNI * IROW;
    const uint32_t done = sbase + tail, dummy = done + 8, full = done + 16, empty = full + 8 * S, tslot = empty + 8 * S;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + tail + 16 + 16 * S);
    for (int i = threadIdx.x; i < tail / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x01ff0001u * (uint32_t)(i % 3);
    constexpr int TCOLS = NA * TNI < 32 ? 32 : NA * TNI;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 + 2 * S; i++) mbar_init(done + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(tslot), "r"((uint32_t)TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 32 && mode == 2) {
        for (unsigned g = 0; g < (unsigned)iters; g++) {
            const unsigned slot = g % S;
            if (g >= (unsigned)S && !mbar_wait(empty + 8 * slot, ((g / S) - 1) & 1u)) { if (status) atomicExch(status, 21); break; }
            mbar_arrive(full + 8 * slot);
        }
    }
    if (mode == 3) {
        // mode 2 with both roles run by whole warps and the issuing instructions under elect_one()
        const int warp = threadIdx.x >> 5;
        if (warp == 1) {
            for (unsigned g = 0; g < (unsigned)iters; g++) {
                const unsigned slot = g % S;
                if (g >= (unsigned)S && !mbar_wait(empty + 8 * slot, ((g / S) - 1) & 1u)) { if (status) atomicExch(status, 21); break; }
                if (elect_one()) mbar_arrive(full + 8 * slot);
                __syncwarp();
            }
        } else if (warp == 0) {
            constexpr uint32_t IDESC = umma_idesc(TNI);
            const uint64_t db = umma_desc(sB);
            const long long t0 = clock64();
            for (unsigned it = 0; it < (unsigned)iters; it++) {
                const unsigned slot = it % S;
                if (!mbar_wait(full + 8 * slot, (it / S) & 1u)) { if (status) atomicExch(status, 22); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < 4; k++) {
#pragma unroll
                        for (int a = 0; a < NA; a++)
                            umma_i8(tmem_base + a * TNI, umma_desc(sA + a * UTM * IROW) + 2 * k, db + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty + 8 * slot);
                }
                __syncwarp();
            }
            if (elect_one()) umma_commit(done);
            __syncwarp();
            const long long t1 = clock64();
            if (!mbar_wait(done, 0) && status) atomicExch(status, 20);
            const long long t2 = clock64();
            if (threadIdx.x == 0) { sink[2 * blockIdx.x] = (uint32_t)(t1 - t0); sink[2 * blockIdx.x + 1] = (uint32_t)(t2 - t0); }
        }
    } else if (threadIdx.x == 0) {
        constexpr uint32_t IDESC = umma_idesc(TNI);
        const uint64_t db = umma_desc(sB);
        const long long t0 = clock64();
        for (unsigned it = 0; it < (unsigned)iters; it++) {
            const unsigned slot = it % S;
            if (mode == 2) {
                if (!mbar_wait(full + 8 * slot, (it / S) & 1u)) { if (status) atomicExch(status, 22); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
#pragma unroll
                for (int a = 0; a < NA; a++)
                    umma_i8(tmem_base + a * TNI, umma_desc(sA + a * UTM * IROW) + 2 * k, db + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
            }
            if (mode == 1) umma_commit(dummy);
            if (mode == 2) umma_commit(empty + 8 * slot);
        }
        umma_commit(done);
        const long long t1 = clock64();
        if (!mbar_wait(done, 0) && status) atomicExch(status, 20);
        const long long t2 = clock64();
        sink[2 * blockIdx.x] = (uint32_t)(t1 - t0);                         // cycles spent issuing
        sink[2 * blockIdx.x + 1] = (uint32_t)(t2 - t0);                     // cycles until the last MMA retired
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TCOLS) : "memory");
    }
}

template <int TNI, int NA>
static int launch_umma_probe(uint32_t* sink, int iters, int blocks, int shift_rows, int mode, cudaStream_t stream) {
    const int smem_bytes = (NA * UTM + 8) * IROW + TNI * IROW + 128 + 1024;
    cudaError_t e = cudaFuncSetAttribute(umma_probe_kernel<TNI, NA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return record_cuda_error(e);
    umma_probe_kernel<TNI, NA><<<blocks, 128, smem_bytes, stream>>>(sink, iters, nullptr, shift_rows, mode);
    return check_launch();
}

// code = shape + 5 * shift + 40 * mode.  shape: 0 = N 64, 1 = N 128, 2 = N 256 (one A tile); 3 = N 64, 4 = N 128 with
// two A tiles sharing each B slice.  shift (0..7): rows by which A starts into its 1024-byte swizzle group.
// Returns the int8 operations of the whole launch through ops_out.
int umma_probe_dispatch(int code, int iters, uint32_t* sink, int blocks, double* ops_out, cudaStream_t stream) {
    const int mode = code / 40, shift_rows = (code % 40) / 5, shape = code % 5;
    if (mode > 3) return TAB_E_BAD_ARGUMENT;
    const int tn = (shape == 0 || shape == 3) ? 64 : ((shape == 1 || shape == 4) ? 128 : 256);
    const int na = shape >= 3 ? 2 : 1;
    if (ops_out) *ops_out = (double)blocks * iters * 4.0 * na * (128.0 * tn * 32 * 2);
    switch (shape) {
        case 0: return launch_umma_probe<64, 1>(sink, iters, blocks, shift_rows, mode, stream);
        case 1: return launch_umma_probe<128, 1>(sink, iters, blocks, shift_rows, mode, stream);
        case 2: return launch_umma_probe<256, 1>(sink, iters, blocks, shift_rows, mode, stream);
        case 3: return launch_umma_probe<64, 2>(sink, iters, blocks, shift_rows, mode, stream);
        case 4: return launch_umma_probe<128, 2>(sink, iters, blocks, shift_rows, mode, stream);
    }
    return TAB_E_BAD_ARGUMENT;
}

}  // namespace tab
