// TAB convolution GEMM stage on the 5th-generation tensor cores: tcgen05.mma kind::i8 with the s32
// accumulator in tensor memory (TMEM).  Same operands and the same results as conv_imma_sm100.cu (quantised
// values {-1,0,+1} as int8, exact int32 accumulation); replaces ldmatrix + mma.sync, whose issue rate capped
// that kernel at about half of the legacy instruction's own ceiling.
//
// One CTA = 256 threads = a 128 x TN output tile (TN = 64, 128 or 256 filters):
//   * all eight warps are loaders: the implicit-im2col gather of the activation rows and the weight rows go
//     to a ring of shared-memory stages with cp.async (16-byte units, zero fill / +1 fill for padding taps,
//     exactly as in the mma.sync kernel).  A stage holds 128 bytes of K per row in the K-major, 128-byte
//     swizzled layout the MMA's shared-memory descriptors expect: row r at r*128, 16-byte unit u at
//     ((u ^ (r & 7)) << 4), stage base 1024-byte aligned.
//   * once every thread's copies of a stage have landed (cp.async.wait_group, fence.proxy.async,
//     __syncthreads) thread 0 issues four tcgen05.mma (K = 32 bytes each) for the stage and one
//     tcgen05.commit that arrives on the stage's mbarrier when they have finished reading it;
//     the loaders wait on that mbarrier before they overwrite the stage, two iterations later.
//   * epilogue: tcgen05.ld brings the 128 x TN accumulator from TMEM to registers (warp w reads TMEM lanes
//     32*(w%4).., columns (w/4)*TN/2..), converts to float, optionally adds the residual and accumulates
//     per-image sums of |y|, and stores rows of [M][KN].
// Every wait on an mbarrier is bounded: on expiry the kernel records a code in *status, stops waiting,
// still frees its TMEM columns and returns.
#include <cuda.h>
#include "tab_kernels.cuh"
#include "conv_int8.cuh"
#include <mutex>

namespace tab {

constexpr int UTHREADS = 256;
constexpr int UTM = 128;                     // rows (output pixels) per CTA = M of one MMA
constexpr uint32_t UMMA_WAIT_LIMIT = 1u << 20;
constexpr int UMMA_SMEM_MAX = 227 * 1024;    // dynamic shared memory the tcgen05 kernels may ask for (one CTA per SM)

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count) : "memory");
}
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < UMMA_WAIT_LIMIT; i++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// One non-blocking probe of the phase with the given parity.
__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    return ok != 0;
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = (smem_addr & 0x3FFFFu) >> 4;                       // start address, LBO unused (0)
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);            // SBO, descriptor version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}
// Instruction descriptor: D s32, A/B signed 8-bit, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(UTM >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// MT blocks of 128 rows per CTA (one accumulator of TNI TMEM columns each, all sharing the weight tile);
// S ring stages; MMAs of a stage are issued D = S - 2 iterations after its copies were issued.
template <int MT, int TNI, int S, bool PADONE, bool FUSED>
__global__ void __launch_bounds__(UTHREADS, 1)
conv_umma_kernel(const ImmaParams p, int* __restrict__ status) {
    constexpr int TMI = UTM * MT;
    constexpr int STAGE = (TMI + TNI) * IROW;
    constexpr int D = (S >= 4) ? S - 2 : 1;
    constexpr int TCOLS = MT * TNI;                              // TMEM columns (a power of two >= 32)
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;                         // swizzle atoms need 1024-byte alignment
    unsigned char* smem = smem_raw + (sbase - raw);
    int4* rowinfo = reinterpret_cast<int4*>(smem + S * STAGE);             // {first-tap pixel, tap mask lo, hi, row valid}
    const uint32_t mbar0 = sbase + S * STAGE + TMI * 16;                   // S stage barriers (8 bytes each)
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + S * STAGE + TMI * 16 + S * 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * TMI;
    const int n0 = blockIdx.y * TNI;
    const int Cp = p.PC * 64;

    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(mbar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(sbase + S * STAGE + TMI * 16 + S * 8), "r"((uint32_t)TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int r = tid; r < TMI; r += UTHREADS) {
        const int m = m0 + r;
        const bool ok = m < p.M;
        const int mm = ok ? m : 0;
        const int ohw = p.OH * p.OW;
        const int n = mm / ohw;
        const int rr = mm - n * ohw;
        const int oh = rr / p.OW;
        const int ow = rr - oh * p.OW;
        const int ih0 = oh * p.s1 - p.p1, iw0 = ow * p.s2 - p.p2;
        unsigned long long mask = 0;
        if (ok) {
            for (int kh = 0; kh < p.KH; kh++)
                for (int kw = 0; kw < p.KW; kw++)
                    if ((unsigned)(ih0 + kh) < (unsigned)p.H && (unsigned)(iw0 + kw) < (unsigned)p.W)
                        mask |= 1ULL << (kh * p.KW + kw);
        }
        rowinfo[r] = make_int4(n * p.H * p.W + ih0 * p.W + iw0, (int)(unsigned)mask, (int)(unsigned)(mask >> 32), ok ? 1 : 0);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // ---- loader: this thread copies unit l_q of word l_wi of every chunk, rows l_row0 + 32 e ---------------
    const int l_unit = tid & 7, l_wi = l_unit >> 2, l_q = l_unit & 3, l_row0 = tid >> 3;
    int l_k = l_wi, l_kh, l_kw, l_pc;
    {
        const int tap = l_k / p.PC;
        l_pc = l_k - tap * p.PC;
        l_kh = tap / p.KW;
        l_kw = tap - l_kh * p.KW;
    }
    auto load_chunk = [&](int stage) {
        const uint32_t sA = sbase + stage * STAGE;
        const uint32_t sB = sA + TMI * IROW;
        const bool kvalid = l_k < p.Kw;
        const int tap = l_kh * p.KW + l_kw;
        const int tap_pix = l_kh * p.W + l_kw;
        const int8_t* abase = p.qx + (long long)l_pc * 64 + l_q * 16;
#pragma unroll
        for (int e = 0; e < TMI / 32; e++) {
            const int row = l_row0 + 32 * e;
            const int4 ri = rowinfo[row];
            const unsigned mword = tap < 32 ? (unsigned)ri.y : (unsigned)ri.z;
            const bool inside = (mword >> (tap & 31)) & 1u;
            const bool v = kvalid && inside;
            const int8_t* src = v ? abase + (long long)(ri.x + tap_pix) * Cp : p.qx;
            const uint32_t dst = sA + swz(row, l_unit);
            if (PADONE && kvalid && !inside && ri.w) sts16(dst, 0x01010101u);
            else cp16(dst, src, v);
        }
        const int8_t* bbase = p.w8 + ((long long)n0 * p.Kw + l_k) * 64 + l_q * 16;
#pragma unroll
        for (int e = 0; e < TNI / 32; e++) {
            const int row = l_row0 + 32 * e;
            const bool v = kvalid && (n0 + row) < p.KN;
            const int8_t* src = v ? bbase + (long long)row * p.Kw * 64 : p.w8;
            cp16(sB + swz(row, l_unit), src, v);
        }
        l_k += IKW;
        l_pc += IKW;
        while (l_pc >= p.PC) { l_pc -= p.PC; if (++l_kw == p.KW) { l_kw = 0; ++l_kh; } }
    };

    constexpr uint32_t IDESC = umma_idesc(TNI);
    const int nchunks = (p.Kw + IKW - 1) / IKW;
    bool dead = false;                                          // a bounded wait expired: stop waiting, finish the protocol
    for (int c = 0; c < nchunks + D; c++) {
        if (c < nchunks) {
            const int stage = c % S;
            if (c >= S && !dead) {
                // the MMAs that read this stage (chunk c - S) were committed two iterations ago
                if (!mbar_wait(mbar0 + 8 * stage, (uint32_t)((c / S) - 1) & 1u)) { dead = true; if (status) atomicExch(status, 1); }
            }
            load_chunk(stage);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int r = c - D;
        if (r >= 0) {
            asm volatile("cp.async.wait_group %0;" ::"n"(D) : "memory");     // chunk r's copies of this thread have landed
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // make them visible to the tensor core
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sA = sbase + (r % S) * STAGE;
                const uint64_t db = umma_desc(sA + TMI * IROW);
#pragma unroll
                for (int k = 0; k < IROW / 32; k++) {            // 32 bytes of K per MMA: advance the start address by 2 units
#pragma unroll
                    for (int mb = 0; mb < MT; mb++)
                        umma_i8(tmem_base + mb * TNI, umma_desc(sA + mb * UTM * IROW) + 2 * k, db + 2 * k, IDESC,
                                (r > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(mbar0 + 8 * (r % S));
            }
        }
    }
    // all MMAs are committed; the last commit covers every earlier one
    {
        const int last = nchunks - 1;
        if (!dead && !mbar_wait(mbar0 + 8 * (last % S), (uint32_t)(last / S) & 1u)) { dead = true; if (status) atomicExch(status, 2); }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- epilogue: TMEM -> registers -> float [M][KN] --------------------------------------------------------
    const int wq = warp & 3, wh = warp >> 2;                    // TMEM lane quarter, column half
    const int ohw = p.OH * p.OW;
    const bool few = ohw >= 16;                                 // 32 rows then touch at most three images
    const bool vec4 = (p.KN & 3) == 0;
#pragma unroll 1
    for (int mb = 0; mb < MT; mb++) {
        const int wrow0 = m0 + mb * UTM + wq * 32;
        const int m = wrow0 + lane;
        const bool row_ok = m < p.M;
        const int wimg0 = FUSED ? wrow0 / ohw : 0;
        const int wb1 = (wimg0 + 1) * ohw, wb2 = wb1 + ohw;
        float rsum = 0.f;
        float* __restrict__ yrow = p.y + (long long)(row_ok ? m : 0) * p.KN;
        const float* __restrict__ rrow = (FUSED && p.residual) ? p.residual + (long long)(row_ok ? m : 0) * p.KN : nullptr;
#pragma unroll 1
        for (int cb = 0; cb < TNI / 2; cb += 32) {
            const int col = wh * (TNI / 2) + cb;
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(mb * TNI + col), v);
            if (!row_ok) continue;
            const int nbase = n0 + col;
            if (vec4 && nbase + 32 <= p.KN) {
                float4 res[8];
#pragma unroll
                for (int q = 0; q < 8; q++)
                    res[q] = (FUSED && rrow) ? __ldg(reinterpret_cast<const float4*>(rrow + nbase) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    float4 o;
                    o.x = (float)(int)v[4 * q + 0] + res[q].x; o.y = (float)(int)v[4 * q + 1] + res[q].y;
                    o.z = (float)(int)v[4 * q + 2] + res[q].z; o.w = (float)(int)v[4 * q + 3] + res[q].w;
                    reinterpret_cast<float4*>(yrow + nbase)[q] = o;
                    if (FUSED) rsum += (fabsf(o.x) + fabsf(o.y)) + (fabsf(o.z) + fabsf(o.w));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (nbase + i < p.KN) {
                        float o = (float)(int)v[i];
                        if (FUSED && rrow) o += __ldg(rrow + nbase + i);
                        yrow[nbase + i] = o;
                        if (FUSED) rsum += fabsf(o);
                    }
                }
            }
        }
        if (FUSED && p.abs_sums) {
            if (few) {
                const int d = (m >= wb1) + (m >= wb2);
#pragma unroll
                for (int i = 0; i < 3; i++) {
                    double t = (row_ok && d == i) ? (double)rsum : 0.0;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
                    if (lane == 0 && t != 0.0 && wimg0 + i < p.N) atomicAdd(p.abs_sums + wimg0 + i, t);
                }
            } else if (row_ok) {
                atomicAdd(p.abs_sums + m / ohw, (double)rsum);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TCOLS) : "memory");
    }
    if (FUSED) fused_finish(p);
}

template <int MT, int TNI, int S, bool PADONE, bool FUSED>
static int launch_umma_f(const ImmaParams& p, int* status, cudaStream_t stream) {
    constexpr int TMI = UTM * MT;
    constexpr int smem_bytes = S * (TMI + TNI) * IROW + TMI * 16 + S * 8 + 16 + 1024;
    static_assert(smem_bytes <= 227 * 1024, "ring does not fit shared memory");
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(conv_umma_kernel<MT, TNI, S, PADONE, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid((unsigned)((p.M + TMI - 1) / TMI), (unsigned)((p.KN + TNI - 1) / TNI));
    conv_umma_kernel<MT, TNI, S, PADONE, FUSED><<<grid, UTHREADS, smem_bytes, stream>>>(p, status);
    return check_launch();
}

template <int MT, int TNI, int S>
static int launch_umma(const ImmaParams& p, bool padone, int* status, cudaStream_t stream) {
    const bool fused = p.residual || p.abs_sums;
    if (padone) return fused ? launch_umma_f<MT, TNI, S, true, true>(p, status, stream) : launch_umma_f<MT, TNI, S, true, false>(p, status, stream);
    return fused ? launch_umma_f<MT, TNI, S, false, true>(p, status, stream) : launch_umma_f<MT, TNI, S, false, false>(p, status, stream);
}

// Epilogue of the kernels that enumerate output positions on the zero-padded input grid: virtual row -> output
// pixel (rows outside the real output are dropped), TMEM -> registers -> float [M][KN], optional residual and
// per-image sums of |y|.
// NWH warp groups of four warps split the TN columns between them (warp = 4*group + TMEM lane quarter).
template <int MT, int TNI, bool FUSED, int NWH = 2>
__device__ __forceinline__ void grid_epilogue(const ImmaParams& p, uint32_t tmem_base, int R0, int n0, int PW, int PHW,
                                              int warp, int lane) {
    const int wq = warp & 3, wh = warp >> 2;
    const bool vec4 = (p.KN & 3) == 0;
#pragma unroll 1
    for (int mb = 0; mb < MT; mb++) {
        const int R = R0 + mb * UTM + wq * 32 + lane;
        const int n = R / PHW;
        const int rr = R - n * PHW;
        const int oh = rr / PW;
        const int ow = rr - oh * PW;
        const bool row_ok = n < p.N && oh < p.OH && ow < p.OW;
        const long long m = ((long long)n * p.OH + oh) * p.OW + ow;
        const int wimg0 = (R0 + mb * UTM + wq * 32) / PHW;                 // image of the warp's first row
        float rsum = 0.f;
        float* __restrict__ yrow = p.y + (row_ok ? m : 0) * p.KN;
        const float* __restrict__ rrow = (FUSED && p.residual) ? p.residual + (row_ok ? m : 0) * p.KN : nullptr;
#pragma unroll 1
        for (int cb = 0; cb < TNI / NWH; cb += 32) {
            const int col = wh * (TNI / NWH) + cb;
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(wq * 32) << 16) + (uint32_t)(mb * TNI + col), v);
            if (!row_ok) continue;
            const int nbase = n0 + col;
            if (vec4 && nbase + 32 <= p.KN) {
                float4 res[8];
#pragma unroll
                for (int q = 0; q < 8; q++)
                    res[q] = (FUSED && rrow) ? __ldg(reinterpret_cast<const float4*>(rrow + nbase) + q) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    float4 o;
                    o.x = (float)(int)v[4 * q + 0] + res[q].x; o.y = (float)(int)v[4 * q + 1] + res[q].y;
                    o.z = (float)(int)v[4 * q + 2] + res[q].z; o.w = (float)(int)v[4 * q + 3] + res[q].w;
                    reinterpret_cast<float4*>(yrow + nbase)[q] = o;
                    if (FUSED) rsum += (fabsf(o.x) + fabsf(o.y)) + (fabsf(o.z) + fabsf(o.w));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (nbase + i < p.KN) {
                        float o = (float)(int)v[i];
                        if (FUSED && rrow) o += __ldg(rrow + nbase + i);
                        yrow[nbase + i] = o;
                        if (FUSED) rsum += fabsf(o);
                    }
                }
            }
        }
        if (FUSED && p.abs_sums) {
            const int d = n - wimg0;                                       // 32 consecutive grid positions: usually one image, rarely more
#pragma unroll
            for (int i = 0; i < 3; i++) {
                double t = (row_ok && d == i) ? (double)rsum : 0.0;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
                if (lane == 0 && t != 0.0 && wimg0 + i < p.N) atomicAdd(p.abs_sums + wimg0 + i, t);
            }
            if (row_ok && d > 2) atomicAdd(p.abs_sums + n, (double)rsum);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Patch variant (stride 1): instead of an im2col tile per tap, the CTA stages the patch of input pixels
// once per pair of 64-channel words and points the MMA's A descriptor into it.
//
// Output positions are enumerated on the zero-padded input grid: virtual row R = (n*PH + oh)*PW + ow' with
// ow' in [0, PW).  For stride 1 the first tap of R is input pixel R itself and tap (kh, kw) is pixel
// R + kh*PW + kw, so the 128 rows of an MMA for any tap are 128 consecutive patch pixels: a K-major,
// 128-byte-swizzled operand that starts (kh*PW + kw) rows further into the same shared-memory patch.
// (The hardware applies the 128-byte swizzle to absolute shared-memory address bits, so a descriptor may
// start at any 128-byte row of a 1024-byte aligned buffer; measured: results stay exact with the
// descriptor's base-offset field left 0.)  Rows with ow' >= OW or oh >= OH are computed and dropped
// (7 % of the rows at 56x56, 13 % at 28x28).  A 3x3 layer copies each activation byte about 1.2 times
// instead of 9, which is what the copy-bound im2col kernel needed.
//
// Ring: one stage = the weights of one tap for the current word pair, [TN][128 B].  The patch of the next
// word pair goes into the second patch buffer while the current one is multiplied.
template <int MT, int TNI, int SB, bool PADONE, bool FUSED>
__global__ void __launch_bounds__(UTHREADS, (MT * TNI <= 256) ? 2 : 1)
conv_umma_patch_kernel(const ImmaParams p, int* __restrict__ status, const int prow, const int npb) {
    constexpr int TMI = UTM * MT;
    constexpr int BSTAGE = TNI * IROW;
    constexpr int DB = SB - 2;
    constexpr int TCOLS = MT * TNI;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t sPatch = sbase;                                         // [npb][prow][128 B], prow % 8 == 0
    const uint32_t sRing = sbase + npb * prow * IROW;                      // [SB][TNI][128 B]
    const int tail = npb * prow * IROW + SB * BSTAGE;
    int* patch_src = reinterpret_cast<int*>(smem + tail);                  // [prow]
    const uint32_t mbar0 = sbase + tail + prow * 4;                        // SB stage barriers, then 2 patch barriers
    const uint32_t mbarP = mbar0 + 8 * SB;
    const uint32_t tslot = mbarP + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + tail + prow * 4 + 8 * SB + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * TNI;
    const int Cp = p.PC * 64;
    const int PH = p.H + 2 * p.p1, PW = p.W + 2 * p.p2, PHW = PH * PW;
    const int T = p.KH * p.KW, ncp = (p.PC + 1) >> 1;
    const int R0 = blockIdx.x * TMI;                                       // first virtual row = first patch pixel
    const int P = TMI + (p.KH - 1) * PW + p.KW - 1;                        // patch pixels in use (<= prow)

    if (tid == 0) {
        for (int s = 0; s < SB + 2; s++) mbar_init(mbar0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(tslot), "r"((uint32_t)TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < P; i += UTHREADS) {                              // source pixel of every patch pixel, -1 = padding
        const int L = R0 + i;
        const int n = L / PHW;
        const int r = L - n * PHW;
        const int ph = r / PW;
        const int pw = r - ph * PW;
        const int ih = ph - p.p1, iw = pw - p.p2;
        const bool inside = n < p.N && ((unsigned)ih < (unsigned)p.H) && ((unsigned)iw < (unsigned)p.W);
        patch_src[i] = inside ? (n * p.H + ih) * p.W + iw : -1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // ---- loaders ------------------------------------------------------------------------------------------
    const int l_unit = tid & 7, l_word = l_unit >> 2, l_q = l_unit & 3, l_row0 = tid >> 3;
    auto load_patch = [&](int cp) {
        const int word = 2 * cp + l_word;
        if (word >= p.PC) return;                                          // odd word count: the upper half of the rows is never read
        const uint32_t buf = sPatch + (cp & (npb - 1)) * prow * IROW;
        const int8_t* abase = p.qx + (long long)word * 64 + l_q * 16;
        for (int pix = l_row0; pix < P; pix += UTHREADS / 8) {
            const int sp = patch_src[pix];
            const uint32_t dst = buf + swz(pix, l_unit);
            if (PADONE && sp < 0) sts16(dst, 0x01010101u);
            else cp16(dst, sp >= 0 ? abase + (long long)sp * Cp : p.qx, sp >= 0);
        }
    };
    auto load_b = [&](int c, int slot) {                                   // weights of tap (c % T), word pair (c / T)
        const int cp = c / T, tap = c - cp * T;
        const int word = 2 * cp + l_word;
        if (word >= p.PC) return;
        const uint32_t sB = sRing + slot * BSTAGE;
        const int8_t* bbase = p.w8 + ((long long)n0 * p.Kw + (long long)tap * p.PC + word) * 64 + l_q * 16;
#pragma unroll
        for (int e = 0; e < TNI / 32; e++) {
            const int row = l_row0 + 32 * e;
            const bool v = (n0 + row) < p.KN;
            cp16(sB + swz(row, l_unit), v ? bbase + (long long)row * p.Kw * 64 : p.w8, v);
        }
    };

    constexpr uint32_t IDESC = umma_idesc(TNI);
    const int nst = ncp * T;
    bool dead = false;
    for (int it = 0; it < nst + DB; it++) {
        if (it < nst) {
            const int slot = it % SB;
            const int cp = it / T, tap = it - cp * T;
            if (it >= SB && !dead) {
                if (!mbar_wait(mbar0 + 8 * slot, (uint32_t)((it / SB) - 1) & 1u)) { dead = true; if (status) atomicExch(status, 3); }
            }
            if (tap == 0) {
                if (cp >= npb && !dead) {                                  // the buffer's previous word pair must be fully multiplied
                    if (!mbar_wait(mbarP + 8 * (cp & 1), (uint32_t)((cp / 2) - 1) & 1u)) { dead = true; if (status) atomicExch(status, 4); }
                }
                load_patch(cp);
            }
            load_b(it, slot);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int r = it - DB;
        if (r >= 0) {
            asm volatile("cp.async.wait_group %0;" ::"n"(DB) : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int cp = r / T, tap = r - cp * T;
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                const uint32_t abuf = sPatch + (cp & (npb - 1)) * prow * IROW + (uint32_t)(kh * PW + kw) * IROW;
                const uint64_t db = umma_desc(sRing + (r % SB) * BSTAGE);
                const int ksteps = (2 * cp + 1 < p.PC) ? 4 : 2;            // one or two 64-channel words in this pair
                for (int k = 0; k < ksteps; k++) {
#pragma unroll
                    for (int mb = 0; mb < MT; mb++)
                        umma_i8(tmem_base + mb * TNI, umma_desc(abuf + mb * UTM * IROW) + 2 * k, db + 2 * k, IDESC,
                                (r > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(mbar0 + 8 * (r % SB));
                if (tap == T - 1) umma_commit(mbarP + 8 * (cp & 1));
            }
        }
    }
    {
        const int last = nst - 1;
        if (!dead && !mbar_wait(mbar0 + 8 * (last % SB), (uint32_t)(last / SB) & 1u)) { dead = true; if (status) atomicExch(status, 5); }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    grid_epilogue<MT, TNI, FUSED>(p, tmem_base, R0, n0, PW, PHW, warp, lane);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TCOLS) : "memory");
    }
    if (FUSED) fused_finish(p);
}

template <int MT, int TNI, int SB, bool PADONE, bool FUSED>
static int launch_umma_patch_f(const ImmaParams& p, int* status, int prow, int npb, cudaStream_t stream) {
    constexpr int TMI = UTM * MT;
    const int smem_bytes = npb * prow * IROW + SB * TNI * IROW + prow * 4 + 8 * (SB + 2) + 16 + 1024;
    static int configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || configured[dev] < smem_bytes) {
        e = cudaFuncSetAttribute(conv_umma_patch_kernel<MT, TNI, SB, PADONE, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = UMMA_SMEM_MAX;
    }
    const long long PH = p.H + 2LL * p.p1, PW = p.W + 2LL * p.p2;
    const long long Mv = (long long)(p.N - 1) * PH * PW + (long long)(p.OH - 1) * PW + p.OW;   // last useful virtual row + 1
    dim3 grid((unsigned)((Mv + TMI - 1) / TMI), (unsigned)((p.KN + TNI - 1) / TNI));
    conv_umma_patch_kernel<MT, TNI, SB, PADONE, FUSED><<<grid, UTHREADS, smem_bytes, stream>>>(p, status, prow, npb);
    return check_launch();
}

// Returns TAB_E_TOO_LARGE when this shape does not fit the patch variant (the caller then uses another kernel).
template <int MT, int TNI, int SB>
static int launch_umma_patch(const ImmaParams& p, bool padone, int* status, cudaStream_t stream) {
    const long long PH = p.H + 2LL * p.p1, PW = p.W + 2LL * p.p2;
    // at least SB taps: a patch buffer is only reused after commits that are issued SB - 2 iterations later
    if (p.s1 != 1 || p.s2 != 1 || p.KH * p.KW < SB || (long long)p.N * PH * PW >= (1LL << 31) - 4096) return TAB_E_TOO_LARGE;
    const int prow = (int)((UTM * MT + (p.KH - 1) * PW + p.KW - 1 + 7) / 8 * 8);
    const int npb = p.PC > 2 ? 2 : 1;
    const long long smem_bytes = (long long)npb * prow * IROW + (long long)SB * TNI * IROW + prow * 4LL + 8 * (SB + 2) + 16 + 1024;
    if (smem_bytes > UMMA_SMEM_MAX) return TAB_E_TOO_LARGE;
    const bool fused = p.residual || p.abs_sums;
    if (padone) return fused ? launch_umma_patch_f<MT, TNI, SB, true, true>(p, status, prow, npb, stream)
                             : launch_umma_patch_f<MT, TNI, SB, true, false>(p, status, prow, npb, stream);
    return fused ? launch_umma_patch_f<MT, TNI, SB, false, true>(p, status, prow, npb, stream)
                 : launch_umma_patch_f<MT, TNI, SB, false, false>(p, status, prow, npb, stream);
}

// ------------------------------------------------------------------------------------------------
// TMA variant of the patch kernel (stride 1): both operands arrive by tensor-map bulk copies, so the copy side
// costs one instruction per 16-32 KB instead of one cp.async per 16 bytes with per-row address arithmetic.
//
// The activations are quantised into a *padded* byte tensor [N*PH*PW][Cp] (border pixels hold the padding value:
// 0 for ternary, +1 for binary activations).  On that tensor the patch of a tile is simply rows
// [R0, R0 + prow) x 128 bytes - a plain 2-D box - and the weights of one tap for one pair of 64-channel words are
// the box rows [n0, n0 + TN) x 128 bytes of the [KN][Kw*64] byte matrix.  The copies use the 128-byte swizzle, which is
// the layout the MMA descriptors expect, and complete on "full" mbarriers (expect_tx); tcgen05.commit arrives on the
// "empty" barriers.  One thread runs the whole producer/MMA loop; the other threads only wait for the final commit
// and run the epilogue.  No multicast, one CTA per cluster.
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(tmap), "r"(mbar), "r"(x), "r"(y) : "memory");
}

constexpr int TMA_BOX_ROWS = 128;            // rows per activation box (16 KB)

template <int MT, int TNI, int SB, bool FUSED>
__global__ void __launch_bounds__(UTHREADS, (MT * TNI <= 256) ? 2 : 1)
conv_umma_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const ImmaParams p, int* __restrict__ status, const int prow, const int npb) {
    constexpr int BSTAGE = TNI * IROW;
    constexpr int DB = SB - 2;
    constexpr int TCOLS = MT * TNI;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t sPatch = sbase;                                         // [npb][prow][128 B], prow % 128 == 0
    const uint32_t sRing = sbase + npb * prow * IROW;                      // [SB][TNI][128 B]
    const int tail = npb * prow * IROW + SB * BSTAGE;
    const uint32_t fullB = sbase + tail, emptyB = fullB + 8 * SB;          // SB + SB stage barriers
    const uint32_t fullP = emptyB + 8 * SB, emptyP = fullP + 16, doneB = emptyP + 16;
    const uint32_t tslot = doneB + 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + tail + 16 * SB + 40);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.y * TNI;
    const int PH = p.H + 2 * p.p1, PW = p.W + 2 * p.p2, PHW = PH * PW;
    const int T = p.KH * p.KW, ncp = (p.PC + 1) >> 1;
    const int R0 = blockIdx.x * (UTM * MT);

    if (tid == 0) {
        for (int s = 0; s < 2 * SB + 5; s++) mbar_init(fullB + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(tslot), "r"((uint32_t)TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    bool dead = false;
    if (tid == 0) {
        constexpr uint32_t IDESC = umma_idesc(TNI);
        const int nst = ncp * T;
        const int nbox = prow / TMA_BOX_ROWS;
        for (int it = 0; it < nst + DB && !dead; it++) {
            if (it < nst) {
                const int slot = it % SB;
                const int cp = it / T, tap = it - cp * T;
                if (it >= SB && !mbar_wait(emptyB + 8 * slot, (uint32_t)((it / SB) - 1) & 1u)) { dead = true; if (status) atomicExch(status, 6); break; }
                if (tap == 0) {
                    const int pb = cp & (npb - 1);
                    if (cp >= npb && !mbar_wait(emptyP + 8 * pb, (uint32_t)((cp / npb) - 1) & 1u)) { dead = true; if (status) atomicExch(status, 7); break; }
                    mbar_expect_tx(fullP + 8 * pb, (uint32_t)(nbox * TMA_BOX_ROWS * IROW));
                    for (int b = 0; b < nbox; b++)
                        tma_load_2d(sPatch + (pb * prow + b * TMA_BOX_ROWS) * IROW, &tmA, 2 * cp * 64, R0 + b * TMA_BOX_ROWS, fullP + 8 * pb);
                }
                mbar_expect_tx(fullB + 8 * slot, (uint32_t)BSTAGE);
                tma_load_2d(sRing + slot * BSTAGE, &tmB, (tap * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
            }
            const int r = it - DB;
            if (r >= 0) {
                const int slot = r % SB;
                const int cp = r / T, tap = r - cp * T;
                const int pb = cp & (npb - 1);
                if (tap == 0 && !mbar_wait(fullP + 8 * pb, (uint32_t)(cp / npb) & 1u)) { dead = true; if (status) atomicExch(status, 8); break; }
                if (!mbar_wait(fullB + 8 * slot, (uint32_t)(r / SB) & 1u)) { dead = true; if (status) atomicExch(status, 9); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                const uint32_t abuf = sPatch + (uint32_t)(pb * prow + kh * PW + kw) * IROW;
                const uint64_t db = umma_desc(sRing + slot * BSTAGE);
                const int ksteps = (2 * cp + 1 < p.PC) ? 4 : 2;
                for (int k = 0; k < ksteps; k++) {
#pragma unroll
                    for (int mb = 0; mb < MT; mb++)
                        umma_i8(tmem_base + mb * TNI, umma_desc(abuf + mb * UTM * IROW) + 2 * k, db + 2 * k, IDESC,
                                (r > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(emptyB + 8 * slot);
                if (tap == T - 1) umma_commit(emptyP + 8 * pb);
            }
        }
        umma_commit(doneB);                                     // arrives when every MMA issued above has completed
    }
    __syncwarp();
    // everybody (the issuing thread included) waits for the accumulators; back off between polls
    {
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 16) && !ok; i++) {
            uint32_t t;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(t) : "r"(doneB), "r"(0u) : "memory");
            ok = t != 0;
            if (!ok) __nanosleep(200);
        }
        if (!ok && status) atomicExch(status, 10);
    }
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    grid_epilogue<MT, TNI, FUSED>(p, tmem_base, R0, n0, PW, PHW, warp, lane);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)TCOLS) : "memory");
    }
    if (FUSED) fused_finish(p);
}


// Epilogue with coalesced stores for a warp that owns TMEM lane quarter wq.  tcgen05.ld hands lane r the 32 columns
// of accumulator row r; written straight out, one store instruction would touch 32 different output rows.  The warp
// instead passes each 32x32 block through a private 4 KB shared-memory buffer (16-byte chunks XOR-swizzled by row, so
// both directions are conflict-free) and stores it transposed: eight lanes cover 128 contiguous bytes of one row,
// one instruction writes four full lines.  The residual is read the same way, and |y| is summed in double.
__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ int4 lds_v4(uint32_t a) {
    int4 r;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(a) : "memory");
    return r;
}

// The warp handles row blocks mb0, mb0 + mbstep, ... and columns [c0, c1) of the tile.
// |y| sums a warp has computed but not yet added to abs_sums: the global atomic is issued by the caller AFTER it has
// released the accumulator buffer (an mbarrier arrive has release semantics and would otherwise wait for the atomic's
// round trip to L2 on every tile).
struct PendingSums {
    int img0 = -1;
    double tot0 = 0.0, tot1 = 0.0;                                         // for images img0 and img0 + 1
};
__device__ __forceinline__ void flush_pending(const ImmaParams& p, PendingSums& ps, int lane) {
    if (ps.img0 >= 0 && lane == 0) {
        if (ps.tot0 != 0.0 && ps.img0 < p.N) atomicAdd(p.abs_sums + ps.img0, ps.tot0);
        if (ps.tot1 != 0.0 && ps.img0 + 1 < p.N) atomicAdd(p.abs_sums + ps.img0 + 1, ps.tot1);
    }
    ps.img0 = -1;
}

// Row data of a warp's 32-row slab (grid rows Rw .. Rw + 31) in the transposed domain: lane (rsub = lane / 8,
// chunk = lane % 8) handles rows 4i + rsub, i = 0..7, and four columns per row.  Computed before the accumulator
// is waited for.
struct SlabRows {
    int mi[8];               // output row (index into [M][KN]) of row 4i + rsub, -1 = not an output position
    int m_own;               // the same for row `lane` (the ragged path works row per lane)
    int n_own;               // image of row `lane`
    int Rw, wimg0, split;    // first grid row, its image, first slab row that belongs to the next image
    bool fast, slow;         // how |y| is summed, see slab_rows
};

// |y| sums.  Usual case ("fast"): the slab's 32 consecutive grid rows lie in at most two images (rows below `split`
// in image wimg0, the others in wimg0 + 1) and the values are small enough for 32 of them to add exactly in float
// (|y| < 2^18): a lane adds its values of a block in float per image and keeps running totals as integers (integer
// data: exact, one REDUX at the end) or, with a residual, as doubles.  Otherwise ("slow", rare: images of fewer than
// 32 grid positions, very long K): one double atomic per row and block.
template <bool FUSED>
__device__ __forceinline__ void slab_rows(const ImmaParams& p, int Rw, int PW, int PHW, int lane, SlabRows& sr) {
    const int R = Rw + lane;
    const int n = R / PHW;
    const int rr = R - n * PHW;
    const int oh = rr / PW;
    const int ow = rr - oh * PW;
    const bool row_ok = n < p.N && oh < p.OH && ow < p.OW;
    sr.m_own = row_ok ? (n * p.OH + oh) * p.OW + ow : -1;                  // M < 2^31 is checked on the host
    sr.n_own = n;
#pragma unroll
    for (int i = 0; i < 8; i++) sr.mi[i] = __shfl_sync(0xFFFFFFFFu, sr.m_own, 4 * i + (lane >> 3));
    sr.Rw = Rw;
    sr.wimg0 = Rw / PHW;
    sr.split = (sr.wimg0 + 1) * PHW - Rw;
    const bool want_sum = FUSED && p.abs_sums != nullptr;
    sr.fast = want_sum && p.Kw < (1 << 12) && (Rw + 31) / PHW - sr.wimg0 <= 1;
    sr.slow = want_sum && !sr.fast;
}

// Residual values of the 32-column block at filter nbase, in the transposed layout (res[i] = row 4i + rsub, 4 columns).
__device__ __forceinline__ void slab_load_residual(const ImmaParams& p, const SlabRows& sr, int nbase, int lane, float4 (&res)[8]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        res[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sr.mi[i] >= 0) res[i] = __ldg(reinterpret_cast<const float4*>(p.residual + (long long)sr.mi[i] * p.KN + nbase) + (lane & 7));
    }
}

// Columns [c0, c1) (multiples of 32, relative to the tile's first filter n0) of one 128-row accumulator block whose
// TMEM address (column 0, this warp's lane quarter) is taddr.  The residual of a block is fetched one block ahead -
// for the first block by the caller, before it waits for the accumulator (res / res_loaded) - because a load issued
// when the block is processed costs the warp its whole DRAM latency (measured 1 700 cycles per block).
template <bool FUSED>
__device__ __forceinline__ void slab_columns(const ImmaParams& p, uint32_t taddr, const SlabRows& sr, int n0, int c0, int c1, int PHW,
                                             int lane, uint32_t stage, float4 (&res)[8], bool res_loaded, PendingSums& ps) {
    const bool vec4 = (p.KN & 3) == 0;
    const bool small_acc = p.Kw < (1 << 15);                               // |accumulator| <= 64 * Kw < 2^21: the bias conversion is exact
    const bool has_res = FUSED && p.residual != nullptr;
    const bool want_sum = FUSED && p.abs_sums != nullptr;
    const int rsub = lane >> 3, chunk = lane & 7;
    unsigned isum_own = 0;                                                 // integer data: |y| total of the lane's own row
    double dsum0 = 0.0, dsum1 = 0.0;                                       // float data: totals per image in the transposed domain
#pragma unroll 1
    for (int cb = c0; cb < c1; cb += 32) {
        const int nbase = n0 + cb;
        if (nbase >= p.KN) break;                                          // uniform over the warp
        uint32_t v[32];
        tmem_ld32(taddr + (uint32_t)cb, v);
        if (vec4 && nbase + 32 <= p.KN) {
#pragma unroll
            for (int q = 0; q < 8; q++)
                sts_v4(stage + lane * 128 + ((q ^ (lane & 7)) << 4), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            if (sr.fast && !has_res) {                                     // y is the accumulator itself: sum |acc| of the lane's own row
                unsigned r0 = 0, r1 = 0, r2 = 0, r3 = 0;                   // (row `lane` of the slab), in integers, before the transposition;
#pragma unroll                                                             // four independent |x| + acc chains (one SAD instruction each)
                for (int j = 0; j < 32; j += 4) {
                    r0 = __sad((int)v[j], 0, r0); r1 = __sad((int)v[j + 1], 0, r1);
                    r2 = __sad((int)v[j + 2], 0, r2); r3 = __sad((int)v[j + 3], 0, r3);
                }
                isum_own += sr.m_own >= 0 ? (r0 + r1) + (r2 + r3) : 0u;
            }
            if (has_res && !res_loaded) slab_load_residual(p, sr, nbase, lane, res);
            __syncwarp();
            float4 o[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int r = 4 * i + rsub;
                const int4 raw = lds_v4(stage + r * 128 + ((chunk ^ (r & 7)) << 4));
                if (small_acc) {                                           // int -> float by the 1.5 * 2^23 bias, no I2F
                    o[i].x = __int_as_float(raw.x + 0x4B400000) - 12582912.f; o[i].y = __int_as_float(raw.y + 0x4B400000) - 12582912.f;
                    o[i].z = __int_as_float(raw.z + 0x4B400000) - 12582912.f; o[i].w = __int_as_float(raw.w + 0x4B400000) - 12582912.f;
                } else {
                    o[i].x = (float)raw.x; o[i].y = (float)raw.y; o[i].z = (float)raw.z; o[i].w = (float)raw.w;
                }
            }
            if (has_res) {
#pragma unroll
                for (int i = 0; i < 8; i++) { o[i].x += res[i].x; o[i].y += res[i].y; o[i].z += res[i].z; o[i].w += res[i].w; }
                // the next block's residual, in flight while this block is stored and summed
                res_loaded = vec4 && cb + 32 < c1 && nbase + 64 <= p.KN;
                if (res_loaded) slab_load_residual(p, sr, nbase + 32, lane, res);
            }
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (sr.mi[i] >= 0) reinterpret_cast<float4*>(p.y + (long long)sr.mi[i] * p.KN + nbase)[chunk] = o[i];
            if (sr.fast && has_res) {
                float fs0 = 0.f, fs1 = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float s4 = sr.mi[i] >= 0 ? (fabsf(o[i].x) + fabsf(o[i].y)) + (fabsf(o[i].z) + fabsf(o[i].w)) : 0.f;
                    if (4 * i + rsub < sr.split) fs0 += s4; else fs1 += s4;
                }
                dsum0 += (double)fs0; dsum1 += (double)fs1;
            } else if (sr.slow) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int img = (sr.Rw + 4 * i + rsub) / PHW;
                    if (sr.mi[i] >= 0 && img < p.N)
                        atomicAdd(p.abs_sums + img, (double)(fabsf(o[i].x) + fabsf(o[i].y)) + (double)(fabsf(o[i].z) + fabsf(o[i].w)));
                }
            }
            __syncwarp();
        } else {
            res_loaded = false;
            if (sr.m_own >= 0) {                                           // ragged right edge / odd filter counts: a row per lane
                float* yrow = p.y + (long long)sr.m_own * p.KN;
                const float* rrow = has_res ? p.residual + (long long)sr.m_own * p.KN : nullptr;
                double rsum = 0.0;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (nbase + i < p.KN) {
                        float ov = (float)(int)v[i];
                        if (rrow) ov += __ldg(rrow + nbase + i);
                        yrow[nbase + i] = ov;
                        if (FUSED) rsum += (double)fabsf(ov);
                    }
                }
                if (want_sum && sr.n_own < p.N) atomicAdd(p.abs_sums + sr.n_own, rsum);
            }
        }
    }
    if (sr.fast) {
        flush_pending(p, ps, lane);                                        // totals the caller has not taken yet
        if (has_res) {
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) {
                dsum0 += __shfl_xor_sync(0xFFFFFFFFu, dsum0, sh);
                dsum1 += __shfl_xor_sync(0xFFFFFFFFu, dsum1, sh);
            }
            ps.tot0 = dsum0; ps.tot1 = dsum1;
        } else {                                                           // row totals < 2^26 (|y| < 2^18, at most 256 columns): the warp's fit 32 bits
            ps.tot0 = (double)__reduce_add_sync(0xFFFFFFFFu, lane < sr.split ? isum_own : 0u);
            ps.tot1 = (double)__reduce_add_sync(0xFFFFFFFFu, lane < sr.split ? 0u : isum_own);
        }
        ps.img0 = sr.wimg0;
    }
}

// Persistent, warp-specialised form of the TMA kernel: one CTA per SM walks over tiles; warp 0 (one thread) issues the
// tensor-map copies and runs ahead across tile boundaries, warp 1 (one thread) issues the MMAs into one of two TMEM
// accumulator buffers, warps 4-7 drain the other buffer (tcgen05.ld -> float -> global) - so copies, MMAs and the
// epilogue of consecutive tiles overlap.  Counters g (ring stages), q (patch buffers) and a (accumulator buffers)
// run across tiles; barrier parities follow from them.
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}

#ifdef TAB_PERSIST_PROFILE
// Build-time instrumentation (off in the shipped library): cycles CTA 0's role threads spend in each wait.
__device__ unsigned long long g_persist_prof[16];
#define PWAIT(slot, call) ([&]() { const long long _t = clock64(); const bool _r = (call); prof[slot] += clock64() - _t; return _r; }())
#else
#define PWAIT(slot, call) (call)
#endif

// Bounded wait by a whole warp; the result is the same in every lane.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t addr, uint32_t parity) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(addr, parity));
}
// True in exactly one lane of a converged warp.  Role loops are run by the whole warp with the issuing instructions
// under this predicate, so that loop counters, addresses and descriptors stay warp-uniform values.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

#ifdef TAB_PERSIST_PROFILE
#define PDBG(bit) ((dbg & (bit)) != 0)
#else
#define PDBG(bit) false
#endif

// BRES: the filter block of the CTA (all taps, all channel pairs; needs KN <= TNI) is copied once and stays in shared
// memory; otherwise it streams through a ring of SB stages, one stage per tap and channel pair.
constexpr int PTHREADS = 384;                                              // warps 0-2 producers and MMA, 3 idle, 4-11 epilogue

// UNIT: stride 1 in both directions (one plane; the tap loops are then flat, which matters because the MMA warp's
// instruction stream, not the tensor pipe, limits small tiles).
template <int MT, int TNI, int SB, bool BRES, bool FUSED, bool UNIT>
__global__ void __launch_bounds__(PTHREADS, 1)
conv_umma_persist_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const ImmaParams p, int* __restrict__ status, const int prow, const int nst,
                         const int tiles_m, const int tiles_n, const int dbg) {
    constexpr int BSTAGE = TNI * IROW;
    constexpr int ACOLS = MT * TNI;                                        // columns of one accumulator buffer
    static_assert(2 * ACOLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");
    static_assert(SB <= 8, "eight ring barriers are laid out");
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t sPatch = sbase;                                         // [2][prow][128 B]
    const uint32_t sRing = sbase + 2 * prow * IROW;                        // [nst][TNI][128 B]
    const int tail = 2 * prow * IROW + nst * BSTAGE;
    const uint32_t fullB = sbase + tail, emptyB = fullB + 64;              // [8] each
    const uint32_t fullP = emptyB + 64, emptyP = fullP + 16, accFull = emptyP + 16, accEmpty = accFull + 16;
    const uint32_t tslot = accEmpty + 16;                                  // = fullB + 192
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + tail + 192);
    const uint32_t sStage = sbase + tail + 256;                            // [8 epilogue warps][4 KB]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Activations come as parity planes (stride 1: the one padded image): plane (a, b), a < PA, b < PB, is a
    // [N][PH][PW] grid; tap (kh, kw) reads plane (kh % s1, kw % s2) at row offset (kh / s1) * PW + kw / s2.
    const int s1 = p.s1, s2 = p.s2;
    const int PA = s1 < p.KH ? s1 : p.KH, PB = s2 < p.KW ? s2 : p.KW;
    const int PH = (p.H + 2 * p.p1 + s1 - 1) / s1, PW = (p.W + 2 * p.p2 + s2 - 1) / s2, PHW = PH * PW;
    const int plane_rows = p.N * PHW;
    const int T = p.KH * p.KW, ncp = (p.PC + 1) >> 1;
    const int ntiles = tiles_m * tiles_n;

    if (tid == 0) {
        for (int s = 0; s < 22; s++) mbar_init(fullB + 8 * s, 1);
        mbar_init(accEmpty, 8); mbar_init(accEmpty + 8, 8);                // one arrival per epilogue warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(tslot), "r"((uint32_t)(2 * ACOLS)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic launch: the set-up above overlapped the tail of the previous kernel (the quantiser); from here on its
    // output is read.  The next kernel (the next layer's quantiser) may be scheduled when every CTA has finished its tiles
    // (not earlier: a grid waiting in griddepcontrol.wait was measured to slow the MMA warp of the tiles still running).
    pdl_wait();

#ifdef TAB_PERSIST_PROFILE
    long long prof[3] = {0, 0, 0};
    const long long prof_t0 = clock64();
#endif
    // In every role the whole warp runs the loops and the waits and one elected lane issues the copies, MMAs and
    // commits: loop counters, addresses and descriptors then stay warp-uniform values (a single-thread role was
    // measured to spend 130-170 cycles per MMA on issue alone; this form 45-90).
    // All roles walk the same nest: tile, channel pair cp, plane (a, b), taps of that plane.  One patch is staged
    // per (tile, cp, plane); counters q (patches) and g (ring stages) run across tiles.
    if (warp == 0) {
        // ---- patch producer: runs ahead of the MMAs by up to two patches (across tile boundaries) ----------------
        const int nbox = prow / TMA_BOX_ROWS;
        unsigned q = 0;
        bool dead = false;
        for (int t = blockIdx.x; t < ntiles && !dead; t += gridDim.x) {
            const int R0 = (t / tiles_n) * (UTM * MT);
            for (int cp = 0; cp < ncp && !dead; cp++) {
                for (int pl = 0; pl < PA * PB; pl++, q++) {
                    const unsigned pb = q & 1;
                    if (q >= 2 && !PWAIT(0, mbar_wait_warp(emptyP + 8 * pb, ((q >> 1) - 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 11); break; }
                    if (elect_one()) {
                        if (PDBG(2)) mbar_arrive(fullP + 8 * pb);
                        else {
                            mbar_expect_tx(fullP + 8 * pb, (uint32_t)(nbox * TMA_BOX_ROWS * IROW));
                            for (int b = 0; b < nbox; b++)
                                tma_load_2d(sPatch + (pb * prow + b * TMA_BOX_ROWS) * IROW, &tmA, 2 * cp * 64,
                                            pl * plane_rows + R0 + b * TMA_BOX_ROWS, fullP + 8 * pb);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 2) {
        // ---- filter producer ---------------------------------------------------------------------------------------
        if (BRES) {
            if (elect_one()) {
                mbar_expect_tx(fullB, (uint32_t)(nst * BSTAGE));
                for (int cp = 0; cp < ncp; cp++)
                    for (int tap = 0; tap < T; tap++)
                        tma_load_2d(sRing + (cp * T + tap) * BSTAGE, &tmB, (tap * p.PC + 2 * cp) * 64, 0, fullB);
            }
            __syncwarp();
        } else {
            unsigned g = 0;
            bool dead = false;
            for (int t = blockIdx.x; t < ntiles && !dead; t += gridDim.x) {
                const int n0 = (t % tiles_n) * TNI;
                for (int cp = 0; cp < ncp && !dead; cp++) {
                    if (UNIT) {
                        for (int tap = 0; tap < T; tap++, g++) {
                            const unsigned slot = g % SB;
                            if (g >= (unsigned)SB && !PWAIT(1, mbar_wait_warp(emptyB + 8 * slot, ((g / SB) - 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 12); break; }
                            if (elect_one()) {
                                if (PDBG(4)) mbar_arrive(fullB + 8 * slot);
                                else {
                                    mbar_expect_tx(fullB + 8 * slot, (uint32_t)BSTAGE);
                                    tma_load_2d(sRing + slot * BSTAGE, &tmB, (tap * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
                                }
                            }
                            __syncwarp();
                        }
                    } else
                    for (int pa = 0; pa < PA && !dead; pa++)
                    for (int pbb = 0; pbb < PB && !dead; pbb++)
                    for (int kh = pa; kh < p.KH && !dead; kh += s1)
                    for (int kw = pbb; kw < p.KW; kw += s2, g++) {
                        const unsigned slot = g % SB;
                        if (g >= (unsigned)SB && !PWAIT(1, mbar_wait_warp(emptyB + 8 * slot, ((g / SB) - 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 12); break; }
                        if (elect_one()) {
                            if (PDBG(4)) mbar_arrive(fullB + 8 * slot);
                            else {
                                mbar_expect_tx(fullB + 8 * slot, (uint32_t)BSTAGE);
                                tma_load_2d(sRing + slot * BSTAGE, &tmB, ((kh * p.KW + kw) * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA warp --------------------------------------------------------------------------------------------------
        constexpr uint32_t IDESC = umma_idesc(TNI);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t MB_UNITS = (UTM * IROW) >> 4;                   // next 128-row block of the patch, in 16-byte units
        unsigned g = 0, q = 0, a = 0;
        bool dead = false;
        if (BRES && !PWAIT(2, mbar_wait_warp(fullB, 0))) { dead = true; if (status && lane == 0) atomicExch(status, 15); }
        for (int t = blockIdx.x; t < ntiles && !dead; t += gridDim.x, a++) {
            const unsigned buf = a & 1;
            if (a >= 2 && !PWAIT(0, mbar_wait_warp(accEmpty + 8 * buf, ((a >> 1) - 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 13); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + buf * ACOLS;
            uint32_t accumulate = 0;                                       // 0 for the tile's first MMAs
            for (int cp = 0; cp < ncp && !dead; cp++) {
                const bool four = 2 * cp + 1 < p.PC;                       // both 64-channel words of the pair exist
                // the MMAs of one tap: 2 or 4 K steps of 32 bytes, MT row blocks each
                auto issue_tap = [&](uint64_t da, uint64_t db, uint32_t acc_first) {
#pragma unroll
                    for (int mb = 0; mb < MT; mb++) umma_i8(acc + mb * TNI, da + mb * MB_UNITS, db, IDESC, acc_first);
#pragma unroll
                    for (int mb = 0; mb < MT; mb++) umma_i8(acc + mb * TNI, da + mb * MB_UNITS + 2, db + 2, IDESC, 1u);
                    if (four) {
#pragma unroll
                        for (int mb = 0; mb < MT; mb++) umma_i8(acc + mb * TNI, da + mb * MB_UNITS + 4, db + 4, IDESC, 1u);
#pragma unroll
                        for (int mb = 0; mb < MT; mb++) umma_i8(acc + mb * TNI, da + mb * MB_UNITS + 6, db + 6, IDESC, 1u);
                    }
                };
                if (UNIT) {
                    const unsigned pb = q & 1;
                    if (!PWAIT(1, mbar_wait_warp(fullP + 8 * pb, (q >> 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 14); break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t arow = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;   // descriptor address of the tap's first patch row
                    int kw = 0;
                    if (BRES) {
                        if (elect_one()) {                                 // nothing to wait for between taps: one issue burst
                            for (int tap = 0; tap < T; tap++) {
                                issue_tap(((uint64_t)DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)DESC_HI << 32) | ((sRing + (uint32_t)(cp * T + tap) * BSTAGE) >> 4), (cp > 0 || tap > 0) ? 1u : 0u);
                                if (++kw == p.KW) { kw = 0; arow += (uint32_t)PW * (IROW >> 4); }
                            }
                            umma_commit(emptyP + 8 * pb);
                            if (cp == ncp - 1) umma_commit(accFull + 8 * buf);
                        }
                        __syncwarp();
                    } else {
                        for (int tap = 0; tap < T; tap++, g++) {
                            const unsigned slot = g % SB;
                            if (!PWAIT(2, mbar_wait_warp(fullB + 8 * slot, (g / SB) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 15); break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            if (elect_one()) {
                                issue_tap(((uint64_t)DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)DESC_HI << 32) | ((sRing + slot * BSTAGE) >> 4), (cp > 0 || tap > 0) ? 1u : 0u);
                                umma_commit(emptyB + 8 * slot);
                                if (tap == T - 1) {
                                    umma_commit(emptyP + 8 * pb);
                                    if (cp == ncp - 1) umma_commit(accFull + 8 * buf);
                                }
                            }
                            __syncwarp();
                            if (++kw == p.KW) { kw = 0; arow += (uint32_t)PW * (IROW >> 4); }
                        }
                    }
                    q++;
                } else
                for (int pa = 0; pa < PA && !dead; pa++)
                for (int pbb = 0; pbb < PB && !dead; pbb++, q++) {
                    const unsigned pb = q & 1;
                    if (!PWAIT(1, mbar_wait_warp(fullP + 8 * pb, (q >> 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 14); break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t patch = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;    // descriptor address of the patch
                    const bool last_group = cp == ncp - 1 && pa == PA - 1 && pbb == PB - 1;
                    for (int kh = pa, ih = 0; kh < p.KH && !dead; kh += s1, ih++)
                    for (int kw = pbb, iw = 0; kw < p.KW; kw += s2, iw++) {
                        const bool last_tap = kh + s1 >= p.KH && kw + s2 >= p.KW;
                        uint32_t bsm;
                        if (BRES) bsm = sRing + (uint32_t)(cp * T + kh * p.KW + kw) * BSTAGE;
                        else {
                            const unsigned slot = g % SB;
                            if (!PWAIT(2, mbar_wait_warp(fullB + 8 * slot, (g / SB) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 15); break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            bsm = sRing + slot * BSTAGE;
                        }
                        if (elect_one()) {
                            issue_tap(((uint64_t)DESC_HI << 32) | (patch + (uint32_t)(ih * PW + iw) * (IROW >> 4)),
                                      ((uint64_t)DESC_HI << 32) | (bsm >> 4), accumulate);
                            if (!BRES) umma_commit(emptyB + 8 * (g % SB));
                            if (last_tap) {
                                umma_commit(emptyP + 8 * pb);
                                if (last_group) umma_commit(accFull + 8 * buf);
                            }
                        }
                        __syncwarp();
                        accumulate = 1u;
                        if (!BRES) g++;
                    }
                }
            }
        }
    } else if (warp >= 4) {
        // ---- epilogue warps (TMEM lane quarter = warp % 4) --------------------------------------------------------
        unsigned a = 0;
        bool dead = false;
        PendingSums pending;
        for (int t = blockIdx.x; t < ntiles && !dead; t += gridDim.x, a++) {
            const unsigned buf = a & 1;
            const int R0 = (t / tiles_n) * (UTM * MT), n0 = (t % tiles_n) * TNI;
            // two warps per TMEM lane quarter: they split the row blocks of a two-block tile, else the columns.  Row data
            // and the first block's residual are fetched before the accumulator is waited for.
            const int wg = (warp - 4) >> 2;
            const int emb = MT == 2 ? wg : 0, ec0 = MT == 2 ? 0 : wg * (TNI / 2), ec1 = MT == 2 ? TNI : (wg + 1) * (TNI / 2);
            SlabRows sr;
            slab_rows<FUSED>(p, R0 + emb * UTM + (warp & 3) * 32, PW, PHW, lane, sr);
            float4 res[8];
            bool res_loaded = false;
            if (FUSED && p.residual != nullptr && (p.KN & 3) == 0 && n0 + ec0 + 32 <= p.KN) {
                slab_load_residual(p, sr, n0 + ec0, lane, res);
                res_loaded = true;
            }
            if (!PWAIT(0, mbar_wait_warp(accFull + 8 * buf, (a >> 1) & 1u))) { dead = true; if (status && lane == 0) atomicExch(status, 16); break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!PDBG(1)) slab_columns<FUSED>(p, tmem_base + buf * ACOLS + (uint32_t)(emb * TNI) + ((uint32_t)((warp & 3) * 32) << 16), sr, n0, ec0, ec1, PHW,
                                              lane, sStage + (warp - 4) * 4096, res, res_loaded, pending);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accEmpty + 8 * buf);
            if (FUSED) flush_pending(p, pending, lane);                    // the |y| atomics, off the buffer's critical path
        }
    }
#ifdef TAB_PERSIST_PROFILE
    if (blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 1 || warp == 4 || warp == 2)) {
        const int o = warp == 0 ? 0 : (warp == 1 ? 4 : (warp == 4 ? 8 : 12));
        g_persist_prof[o] = clock64() - prof_t0;
        g_persist_prof[o + 1] = prof[0]; g_persist_prof[o + 2] = prof[1]; g_persist_prof[o + 3] = prof[2];
    }
#endif
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    pdl_launch_dependents();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)(2 * ACOLS)) : "memory");
    }
    if (FUSED) fused_finish(p);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D byte tensor [rows][row_bytes] (row pitch = row_bytes), box = 128 bytes x box_rows, 128-byte swizzle.
// Encoding a map costs tens of microseconds on the host, more than a small convolution takes on the device, and
// callers reuse their buffers: the last few maps are kept, keyed by everything that goes into them.
struct MapKey { const void* base; unsigned long long row_bytes, rows; unsigned box_rows; };
static bool make_map_2d(CUtensorMap* m, const void* base, unsigned long long row_bytes, unsigned long long rows, unsigned box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    constexpr int NCACHE = 32;
    static std::mutex mu;
    static MapKey keys[NCACHE] = {};
    static CUtensorMap maps[NCACHE];
    static int used = 0, next = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++) {
        if (keys[i].base == base && keys[i].row_bytes == row_bytes && keys[i].rows == rows && keys[i].box_rows == box_rows) {
            *m = maps[i];
            return true;
        }
    }
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    if (fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    keys[next] = MapKey{base, row_bytes, rows, box_rows};
    maps[next] = *m;
    next = (next + 1) % NCACHE;
    if (used < NCACHE) used++;
    return true;
}

template <int MT, int TNI, int SB, bool FUSED>
static int launch_umma_tma_f(const CUtensorMap& tmA, const CUtensorMap& tmB, const ImmaParams& p, int* status, int prow, int npb,
                             cudaStream_t stream) {
    constexpr int TMI = UTM * MT;
    const int smem_bytes = npb * prow * IROW + SB * TNI * IROW + 16 * SB + 64 + 1024;
    static int configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || configured[dev] < smem_bytes) {
        e = cudaFuncSetAttribute(conv_umma_tma_kernel<MT, TNI, SB, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = UMMA_SMEM_MAX;
    }
    const long long PH = p.H + 2LL * p.p1, PW = p.W + 2LL * p.p2;
    const long long Mv = (long long)(p.N - 1) * PH * PW + (long long)(p.OH - 1) * PW + p.OW;
    dim3 grid((unsigned)((Mv + TMI - 1) / TMI), (unsigned)((p.KN + TNI - 1) / TNI));
    conv_umma_tma_kernel<MT, TNI, SB, FUSED><<<grid, UTHREADS, smem_bytes, stream>>>(tmA, tmB, p, status, prow, npb);
    return check_launch();
}

template <int MT, int TNI, int SB>
static int launch_umma_tma(const CUtensorMap& tmA, const CUtensorMap& tmB, const ImmaParams& p, int* status, cudaStream_t stream) {
    const long long PW = p.W + 2LL * p.p2;
    const int prow = (int)((UTM * MT + (p.KH - 1) * PW + p.KW - 1 + TMA_BOX_ROWS - 1) / TMA_BOX_ROWS * TMA_BOX_ROWS);
    const int npb = p.PC > 2 ? 2 : 1;
    const long long smem_bytes = (long long)npb * prow * IROW + (long long)SB * TNI * IROW + 16 * SB + 64 + 1024;
    if (smem_bytes > UMMA_SMEM_MAX || p.KH * p.KW < SB) return TAB_E_TOO_LARGE;
    return (p.residual || p.abs_sums) ? launch_umma_tma_f<MT, TNI, SB, true>(tmA, tmB, p, status, prow, npb, stream)
                                      : launch_umma_tma_f<MT, TNI, SB, false>(tmA, tmB, p, status, prow, npb, stream);
}

// Plane grid of a geometry (see the persistent kernel): planes, rows and columns of one plane, patch halo rows.
struct PlaneGrid { long long planes, PH, PW, halo; };
static PlaneGrid plane_grid(const ImmaParams& p) {
    PlaneGrid g;
    const long long A = p.s1 < p.KH ? p.s1 : p.KH, B = p.s2 < p.KW ? p.s2 : p.KW;
    g.planes = A * B;
    g.PH = (p.H + 2LL * p.p1 + p.s1 - 1) / p.s1;
    g.PW = (p.W + 2LL * p.p2 + p.s2 - 1) / p.s2;
    g.halo = ((p.KH - 1) / p.s1) * g.PW + (p.KW - 1) / p.s2;
    return g;
}

static int g_persist_dbg = 0;
void persist_set_debug(int v) { g_persist_dbg = v & 7; }

template <int MT, int TNI, int SB, bool BRES, bool FUSED, bool UNIT>
static int launch_umma_persist_u(const CUtensorMap& tmA, const CUtensorMap& tmB, const ImmaParams& p, int* status, int prow, int nst,
                                 int smem_bytes, cudaStream_t stream) {
    constexpr int TMI = UTM * MT;
    static int configured[64] = {};
    int dev = 0, sms = 148;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (dev < 0 || dev >= 64 || configured[dev] < smem_bytes) {
        e = cudaFuncSetAttribute(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, UNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = UMMA_SMEM_MAX;
    }
    const PlaneGrid pg = plane_grid(p);
    const long long Mv = (long long)(p.N - 1) * pg.PH * pg.PW + (long long)(p.OH - 1) * pg.PW + p.OW;   // last useful virtual row + 1
    const long long tiles_m = (Mv + TMI - 1) / TMI, tiles_n = (p.KN + TNI - 1) / TNI;
    if (tiles_m * tiles_n >= (1LL << 31)) return TAB_E_TOO_LARGE;
    const long long ntiles = tiles_m * tiles_n;
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);
    return launch_pdl(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, UNIT>, dim3(grid), dim3(PTHREADS), (size_t)smem_bytes, stream,
                      tmA, tmB, p, status, prow, nst, (int)tiles_m, (int)tiles_n, g_persist_dbg);
}

template <int MT, int TNI, int SB, bool BRES, bool FUSED>
static int launch_umma_persist_f(const CUtensorMap& tmA, const CUtensorMap& tmB, const ImmaParams& p, int* status, int prow, int nst,
                                 int smem_bytes, cudaStream_t stream) {
    return (p.s1 == 1 && p.s2 == 1) ? launch_umma_persist_u<MT, TNI, SB, BRES, FUSED, true>(tmA, tmB, p, status, prow, nst, smem_bytes, stream)
                                    : launch_umma_persist_u<MT, TNI, SB, BRES, FUSED, false>(tmA, tmB, p, status, prow, nst, smem_bytes, stream);
}

// Shared-memory need of the persistent kernel for a tile shape; resident (out) says whether the filter block stays
// in shared memory.  0 = does not fit.
static long long persist_smem(const ImmaParams& p, int mt, int tn, int sb, bool* resident) {
    const long long prow = (UTM * mt + plane_grid(p).halo + TMA_BOX_ROWS - 1) / TMA_BOX_ROWS * TMA_BOX_ROWS;
    const long long fixed = 2 * prow * IROW + 256 + 8 * 4096 + 1024;
    const long long nres = (long long)p.KH * p.KW * ((p.PC + 1) / 2);     // stages of a resident filter block
    if (p.KN <= tn && fixed + nres * tn * IROW <= UMMA_SMEM_MAX) { *resident = true; return fixed + nres * tn * IROW; }
    *resident = false;
    const long long need = fixed + (long long)sb * tn * IROW;
    return need <= UMMA_SMEM_MAX ? need : 0;
}

template <int MT, int TNI, int SB>
static int launch_umma_persist(const CUtensorMap& tmA, const CUtensorMap& tmB, const ImmaParams& p, int* status, cudaStream_t stream) {
    const int prow = (int)((UTM * MT + plane_grid(p).halo + TMA_BOX_ROWS - 1) / TMA_BOX_ROWS * TMA_BOX_ROWS);
    bool resident = false;
    const long long smem_bytes = persist_smem(p, MT, TNI, SB, &resident);
    if (!smem_bytes) return TAB_E_TOO_LARGE;
    const bool fused = p.residual || p.abs_sums;
    if (resident) {
        const int nres = p.KH * p.KW * ((p.PC + 1) / 2);
        return fused ? launch_umma_persist_f<MT, TNI, SB, true, true>(tmA, tmB, p, status, prow, nres, (int)smem_bytes, stream)
                     : launch_umma_persist_f<MT, TNI, SB, true, false>(tmA, tmB, p, status, prow, nres, (int)smem_bytes, stream);
    }
    return fused ? launch_umma_persist_f<MT, TNI, SB, false, true>(tmA, tmB, p, status, prow, SB, (int)smem_bytes, stream)
                 : launch_umma_persist_f<MT, TNI, SB, false, false>(tmA, tmB, p, status, prow, SB, (int)smem_bytes, stream);
}

// Tile of the persistent kernel for a problem: N tile by filter count; two row blocks per tile when the patch of a
// wide image still fits.  false = no shape fits (wide images with many taps).
static bool persist_plan(const ImmaParams& p, int* mt, int* tn) {
    bool res;
    *tn = p.KN <= 64 ? 64 : (p.KN <= 128 ? 128 : 256);
    if (*tn == 256) { *mt = 1; return persist_smem(p, 1, 256, 4, &res) != 0; }
    const int sb2 = *tn == 64 ? 6 : 4, sb1 = 6;
    if (persist_smem(p, 2, *tn, sb2, &res)) { *mt = 2; return true; }
    *mt = 1;
    return persist_smem(p, 1, *tn, sb1, &res) != 0;
}

static bool tma_shape_ok(const ImmaParams& p) {
    const PlaneGrid pg = plane_grid(p);
    return pg.planes * p.N * pg.PH * pg.PW < (1LL << 31) - 4096;
}

// Whether conv_tma_dispatch(p, 0, ..) will take the problem (asked before the activations are laid out padded).
bool conv_tma_persist_fits(const ImmaParams& p) {
    int mt, tn;
    return tma_shape_ok(p) && persist_plan(p, &mt, &tn);
}

static int* umma_status_ptr();

// GEMM stage of the TMA variant.  p.qx must be the PADDED byte activations [N*PH*PW][Cp]; stride 1 only.
// shape: 0 = choose by filter count; returns TAB_E_TOO_LARGE when the shape does not fit (caller falls back).
// mode 0: persistent kernel or TAB_E_TOO_LARGE; 1: persistent kernel, else the one-tile-per-CTA TMA kernel; 2: the latter only.
// TAB_E_TOO_LARGE = shape not covered (the caller falls back to the kernels on unpadded activations).
int conv_tma_dispatch(const ImmaParams& p, int mode, cudaStream_t stream) {
    const PlaneGrid pg = plane_grid(p);
    const long long rows = pg.planes * p.N * pg.PH * pg.PW;
    const bool unit = p.s1 == 1 && p.s2 == 1;                              // the one-tile-per-CTA kernel knows stride 1 only
    if (!tma_shape_ok(p) || !encode_tiled_fn() || (mode == 2 && !unit)) return TAB_E_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(p.qx) & 15) || (reinterpret_cast<uintptr_t>(p.w8) & 15)) return TAB_E_TOO_LARGE;
    alignas(64) CUtensorMap tmA, tmB;
    const unsigned tn = p.KN <= 64 ? 64 : (p.KN <= 128 ? 128 : 256);
    if (!make_map_2d(&tmA, p.qx, (unsigned long long)p.PC * 64, (unsigned long long)rows, TMA_BOX_ROWS)) return TAB_E_TOO_LARGE;
    if (!make_map_2d(&tmB, p.w8, (unsigned long long)p.Kw * 64, (unsigned long long)p.KN, tn)) return TAB_E_TOO_LARGE;
    int* status = umma_status_ptr();
    if (mode != 2) {
        int mt = 0, ptn = 0;
        if (persist_plan(p, &mt, &ptn)) {
            if (ptn == 64) return mt == 2 ? launch_umma_persist<2, 64, 6>(tmA, tmB, p, status, stream) : launch_umma_persist<1, 64, 6>(tmA, tmB, p, status, stream);
            if (ptn == 128) return mt == 2 ? launch_umma_persist<2, 128, 4>(tmA, tmB, p, status, stream) : launch_umma_persist<1, 128, 6>(tmA, tmB, p, status, stream);
            return launch_umma_persist<1, 256, 4>(tmA, tmB, p, status, stream);
        }
        if (mode == 0 || !unit) return TAB_E_TOO_LARGE;
    }
    if (tn == 64) return launch_umma_tma<2, 64, 4>(tmA, tmB, p, status, stream);
    if (tn == 128) return launch_umma_tma<2, 128, 4>(tmA, tmB, p, status, stream);
    return launch_umma_tma<2, 256, 4>(tmA, tmB, p, status, stream);
}

// Where an expired wait is recorded (0 = never).  In host code the name is only a symbol handle; the device
// address is looked up once per device.
static __device__ int g_umma_status;
static int* g_umma_status_addr[64] = {};

static int* umma_status_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_umma_status_addr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_umma_status) != cudaSuccess) return nullptr;
        g_umma_status_addr[dev] = static_cast<int*>(ptr);
    }
    return g_umma_status_addr[dev];
}

// Reads (and clears) the record of expired waits on the current device; synchronises the device.
int umma_status_read_and_clear() {
    int v = -1, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));
    return v;
}

// GEMM stage on the tcgen05 tensor cores; same contract as the mma.sync dispatch.
//
// Shape choice.  All variants are bound by their loaders, and measured per-CTA times follow
//     time ~ 3.2 ns x (rows copied per K step) x (K steps)  +  a fixed set-up/epilogue cost,
// where a "row" is 128 bytes of one operand row.  The candidates are scored with that model times the number of
// waves the grid needs on the device's SMs, so that small problems (few output rows) get small tiles and fill the
// machine, and large ones get the tiles with the fewest copies per multiply-add.
struct UmmaChoice { int patch, mt, tn; };

int conv_umma_dispatch(const ImmaParams& p, bool padone, int alt, cudaStream_t stream) {
    int* status = umma_status_ptr();
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long PH = p.H + 2LL * p.p1, PW = p.W + 2LL * p.p2;
    const int T = p.KH * p.KW;
    const long long nchunks = (p.Kw + IKW - 1) / IKW, ncp = (p.PC + 1) / 2;
    const long long Mv = (long long)(p.N - 1) * PH * PW + (long long)(p.OH - 1) * PW + p.OW;
    const long long halo = (p.KH - 1) * PW + p.KW - 1;
    const bool patch_ok = p.s1 == 1 && p.s2 == 1 && T >= 4 && (long long)p.N * PH * PW < (1LL << 31) - 4096;
    const double fixed = 1200.0;                                 // set-up + epilogue of one CTA, in row units

    static const UmmaChoice cands[] = {{0, 2, 256}, {0, 1, 256}, {0, 2, 128}, {0, 1, 128}, {0, 2, 64}, {0, 1, 64},
                                       {1, 2, 256}, {1, 2, 128}, {1, 1, 128}, {1, 2, 64}};
    UmmaChoice best = {0, 1, 64};
    double best_cost = 1e300;
    for (const UmmaChoice& c : cands) {
        if (c.tn > 64 && c.tn / 2 >= p.KN) continue;             // a tile twice as wide as the filter count only wastes
        if (alt == 1 && c.patch) continue;                       // A/B switches: im2col staging only / patch staging only
        if (alt == 2 && !c.patch && patch_ok) continue;
        const long long tm = 128LL * c.mt;
        const long long ctas_n = (p.KN + c.tn - 1) / c.tn;
        double cost;
        if (c.patch) {
            if (!patch_ok) continue;
            const long long prow = (tm + halo + 7) / 8 * 8;
            const int npb = p.PC > 2 ? 2 : 1;
            const long long smem = npb * prow * IROW + 4LL * c.tn * IROW + prow * 4 + 8 * 6 + 16 + 1024;
            if (smem > UMMA_SMEM_MAX) continue;
            const long long ctas = ((Mv + tm - 1) / tm) * ctas_n;
            const int per_sm = (c.mt * c.tn <= 256 && 2 * smem <= UMMA_SMEM_MAX) ? 2 : 1;
            const double rows = (double)ncp * (double)(tm + halo + (long long)T * c.tn) + fixed;
            const double waves = (double)((ctas + (long long)sms * per_sm - 1) / ((long long)sms * per_sm));
            cost = waves * rows * (per_sm == 2 ? 1.6 : 1.0);     // two resident CTAs share the SM's copy rate
        } else {
            const long long ctas = ((p.M + tm - 1) / tm) * ctas_n;
            const double rows = (double)nchunks * (double)(tm + c.tn) + fixed;
            cost = (double)((ctas + sms - 1) / sms) * rows;
        }
        if (cost < best_cost) { best_cost = cost; best = c; }
    }
    if (best.patch) {
        int rc = TAB_E_TOO_LARGE;
        if (best.mt == 2 && best.tn == 256) rc = launch_umma_patch<2, 256, 4>(p, padone, status, stream);
        else if (best.mt == 2 && best.tn == 128) rc = launch_umma_patch<2, 128, 4>(p, padone, status, stream);
        else if (best.mt == 1 && best.tn == 128) rc = launch_umma_patch<1, 128, 4>(p, padone, status, stream);
        else if (best.mt == 2 && best.tn == 64) rc = launch_umma_patch<2, 64, 4>(p, padone, status, stream);
        if (rc != TAB_E_TOO_LARGE) return rc;
        best = {0, 1, p.KN <= 64 ? 64 : (p.KN <= 128 ? 128 : 256)};
    }
    if (best.tn == 256) return best.mt == 2 ? launch_umma<2, 256, 3>(p, padone, status, stream)     // 256 x 256, 3 x 65 KB
                                            : launch_umma<1, 256, 4>(p, padone, status, stream);    // 128 x 256, 4 x 49 KB
    if (best.tn == 128) return best.mt == 2 ? launch_umma<2, 128, 4>(p, padone, status, stream)     // 256 x 128, 4 x 49 KB
                                            : launch_umma<1, 128, 6>(p, padone, status, stream);    // 128 x 128, 6 x 33 KB
    return best.mt == 2 ? launch_umma<2, 64, 5>(p, padone, status, stream)                          // 256 x 64,  5 x 41 KB
                        : launch_umma<1, 64, 8>(p, padone, status, stream);                         // 128 x 64,  8 x 25 KB
}

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
    if (mode == 4) {
        // mode 3 with the next slot's barrier probed before the current group is issued (its latency hides behind the MMAs)
        const int warp = threadIdx.x >> 5;
        if (warp == 1) {
            for (unsigned g = 0; g < (unsigned)iters; g++) {
                const unsigned slot = g % S;
                if (g >= (unsigned)S && !mbar_wait(empty + 8 * slot, ((g / S) - 1) & 1u)) { if (status) atomicExch(status, 21); break; }
                __syncwarp();
                if (elect_one()) mbar_arrive(full + 8 * slot);
                __syncwarp();
            }
        } else if (warp == 0) {
            constexpr uint32_t IDESC = umma_idesc(TNI);
            const uint64_t db = umma_desc(sB);
            const long long t0 = clock64();
            bool ready = mbar_wait(full, 0);
            for (unsigned it = 0; it < (unsigned)iters; it++) {
                const unsigned slot = it % S;
                if (!ready && !mbar_wait(full + 8 * slot, (it / S) & 1u)) { if (status) atomicExch(status, 22); break; }
                const unsigned nslot = (it + 1) % S;
                ready = mbar_try(full + 8 * nslot, ((it + 1) / S) & 1u);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                __syncwarp();
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
    } else if (mode == 3) {
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
    umma_probe_kernel<TNI, NA><<<blocks, 128, smem_bytes, stream>>>(sink, iters, umma_status_ptr(), shift_rows, mode);
    return check_launch();
}

// code = shape + 5 * shift + 40 * mode.  shape: 0 = N 64, 1 = N 128, 2 = N 256 (one A tile); 3 = N 64, 4 = N 128 with
// two A tiles sharing each B slice.  shift (0..7): rows by which A starts into its 1024-byte swizzle group.
// Returns the int8 operations of the whole launch through ops_out.
int umma_probe_dispatch(int code, int iters, uint32_t* sink, int blocks, double* ops_out, cudaStream_t stream) {
    const int mode = code / 40, shift_rows = (code % 40) / 5, shape = code % 5;
    if (mode > 4) return TAB_E_BAD_ARGUMENT;
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

#ifdef TAB_PERSIST_PROFILE
int persist_profile_read(unsigned long long* out16) {
    return cudaMemcpyFromSymbol(out16, g_persist_prof, 16 * sizeof(unsigned long long)) == cudaSuccess ? 0 : -1;
}
#endif

}  // namespace tab
