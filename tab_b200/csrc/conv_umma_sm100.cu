// TAB convolution on the 5th-generation tensor cores: a persistent, warp-specialised implicit GEMM that reads the
// activations as the bit-planes tab_quantize_launch writes (TAB_GEMM.cu:196-197) and multiplies them as int8.
//
// Replaces the reference's PadKernel, Img2RowKernel (TAB_GEMM.cuh:73-115) and TNN/TBN/BTN/BNNGEMM (TAB_GEMM.cu:25-147).
// The quantised values {-1,0,+1} times {-1,0,+1} accumulate exactly in int32 (at most KH*KW*C terms), so y = sum a*w
// directly and none of the per-type corrections of the popcount formulas is needed: zero words of binary activations
// decode to +1 (the reference's padding rule), channel tails decode to 0.
//
// One CTA per SM walks over output tiles of 128*MT virtual rows x TN filters (see TcConvParams for the virtual grid):
//   * expander warps (0, 12-15): stage the *patch* of a tile - the 128*MT + halo consecutive virtual rows all its
//     taps read - for one pair of 64-channel words and one stride plane: 16 bytes of (sign, magnitude) per pixel and
//     word are loaded from global memory (padding positions are not loaded at all) and expanded to 64 bytes of int8
//     in the K-major, 128-byte-swizzled layout the MMA descriptors expect.  Two patch buffers; the expanders run up to
//     two patches ahead of the MMAs, across tile boundaries.
//   * warp 2: TMA copies of the filter slice (TN x 128 B per tap and channel pair) into a ring of SB stages, or - when
//     the filters of all taps fit beside the patches (BRES) - once per CTA.
//   * warps 1 and 3 (row block 0 and row block 1 of a tile): tcgen05.mma.cta_group::1.kind::i8, 128 x TN x 32 per
//     instruction.  Tap (kh, kw) of the 128 rows of an MMA is 128 consecutive patch rows starting (kh/s1)*VW + kw/s2 rows
//     into the patch: the A descriptor simply starts there (the 128-byte swizzle is a function of absolute shared-memory
//     address bits).  Two TMEM accumulator buffers.
//   * warps 4-11: epilogue of the other accumulator buffer: tcgen05.ld, then either a transposition through a private
//     shared-memory block so that stores are coalesced, or (TEPI) TMA loads of the residual and TMA stores of the result;
//     int -> float, residual, per-image sums of |y|.
//   * the CTA that finishes last turns the sums into the next layer's thresholds - or, second phase, the whole grid meets
//     at a counter and quantises the result it has just written for the next convolution (quantize_tail).
//   * PAIR: the same roles on clusters of two CTAs with one tcgen05.mma.cta_group::2 stream for both (see the kernel).
// Every mbarrier wait is a bounded try_wait loop; on expiry the role records a code in *status and stops, the other
// roles run into their own limits, every thread still reaches the final barrier, TMEM is freed and the kernel returns.
// The grid-wide counter of the second phase is the only place where a CTA waits for other CTAs (all resident, at most one
// per SM; bounded as well); no kernel here waits on another GPU, and no copy is multicast.
#include <cuda.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include "tab_kernels.cuh"
#include "umma_common.cuh"

namespace tab {

constexpr int PTHREADS = 512;                                              // 16 warps
// Extra expander warps (16 and up): layers without a residual are bound by their expanders.  An expander warp is one
// dependent instruction stream that takes the patch's items 32 at a time, so what counts is how many rounds of items a
// thread has per patch: the patches of strided layers (about 290 items) want nine expander warps to be done in one round.
// The epilogue of these variants fits 96 registers, so up to 21 warps fit the register file.  Measured per filter-block
// width on the ResNet-18-shaped layers: 2 / 4 / 3 extra warps; one more each changed nothing, and on residual layers the
// epilogue is the bound and needs the registers.
__host__ __device__ constexpr int extra_warps(int fused, bool tepi, int tn) { return (fused <= 1 && !tepi) ? (tn == 64 ? 2 : (tn == 128 ? 4 : 3)) : 0; }
// Kernels that can work a tile as two halves of tn/2 filters (their filter boxes hold tn/2 filters): one row block, the
// widest tile, streamed filters, transposing epilogue, single CTAs.
__host__ __device__ constexpr bool split_capable(int mt, int tn, bool resident, bool tepi, bool pair) { return mt == 1 && tn == 256 && !resident && !tepi && !pair; }
constexpr int NXT = 160;                                                   // expander threads: 5 warps, and a sixth (192) where the
                                                                           // second MMA warp has nothing to issue (one row block per tile)
constexpr int XUNROLL = 4;                                                 // (pixel, word) items a thread has in flight

// Build-time diagnostic (-DTAB_PROF, never in the shipped library): cycles one representative warp of each role spends
// in each kind of wait and in its work, summed over CTAs into g_prof, read back by tab_prof_read.
#ifdef TAB_PROF
__device__ unsigned long long g_prof[32];
#define PROF_T0 const long long prof_t0 = clock64()
#define PROF_ADD(slot, on) do { if (on) atomicAdd(&g_prof[slot], (unsigned long long)(clock64() - prof_t0)); } while (0)
#define PROF_MAX(slot, on) do { if (on) atomicMax(&g_prof[slot], (unsigned long long)(clock64() - prof_t0)); } while (0)
__device__ __forceinline__ unsigned long long prof_gtime() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define PROF_GT(slot_min, slot_max, on) do { if (on) { const unsigned long long g = prof_gtime(); atomicMin(&g_prof[slot_min], g); atomicMax(&g_prof[slot_max], g); } } while (0)
#else
#define PROF_MAX(slot, on) do { } while (0)
#define PROF_GT(slot_min, slot_max, on) do { } while (0)
#define PROF_T0 do { } while (0)
#define PROF_ADD(slot, on) do { } while (0)
#endif
template <int SLOT, bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait_prof(bool on, uint32_t addr, uint32_t parity) {
    PROF_T0;
    const bool ok = CLUSTER ? mbar_wait_cluster_warp(addr, parity) : mbar_wait_warp(addr, parity);
    PROF_ADD(SLOT, on);
    return ok;
}

// Called by every thread of every CTA at the end of the kernel, after the CTA's last atomic on abs_sums.
__device__ __forceinline__ void fused_finish(const TcConvParams& p) {
    if (p.ths_out == nullptr) return;
    __threadfence();
    int mine = 0;
    __syncthreads();                                                       // every thread's atomics are issued and fenced
    if (threadIdx.x == 0) mine = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1u);
    const int last = __syncthreads_or(mine);
    if (last) {
        __threadfence();
        for (int n = threadIdx.x; n < p.N; n += blockDim.x) {
            const double sum = __ldcg(p.abs_sums + n);                     // the other CTAs' atomics live in L2
            p.ths_out[n] = (float)((double)p.ths_scale * (sum / p.per_image));
            if (p.self_clean) p.abs_sums[n] = 0.0;
        }
        if (p.self_clean && threadIdx.x == 0) *p.done_counter = 0u;
    }
}

// ---- second phase: the grid quantises its own result for the next convolution ------------------------------------------
// Replaces, for a chained layer, the quantiser launch of the next convolution (TerOnlyKernel / BinOnlyKernel,
// TAB_GEMM.cu:163-247, same encoding).  Every CTA first reports in at a grid-wide counter - all CTAs of the launch are
// resident (one per SM at most), so the wait is for CTAs that are running; it is bounded all the same - then computes the
// thresholds of all images from the complete |y| sums (the arithmetic of fused_finish), and the CTAs share the words of
// the result, last word first (the end of the tensor is what was written last).  Data written by other SMs in this
// launch is read with L2-coherent loads.
constexpr uint32_t GRID_WAIT_LIMIT = 1u << 22;                             // x ~100 ns

__device__ __forceinline__ float4 ld_cg_f4(const float* ptr) {
    float4 r;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(ptr));
    return r;
}
struct F8 { float v[8]; };
__device__ __forceinline__ F8 ld_cg_f8(const float* ptr) {                         // two 128-bit loads
    F8 r;
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]) : "l"(ptr));
    asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7]) : "l"(ptr + 4));
    return r;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* ptr) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(ptr));
    return r;
}

// Eight consecutive channels -> one byte per plane, stored at byte `byte` of the word's planes.
__device__ __forceinline__ void quantize8(const float (&v)[8], float t, int bits, unsigned char* word_out, int byte) {
    if (bits == 2) {
        const float nt = -t;
        unsigned pos = 0, neg = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            pos |= (v[i] > t) ? (1u << i) : 0u;
            neg |= (v[i] < nt) ? (1u << i) : 0u;
        }
        neg &= ~pos;                                                       // the "+1" branch is tested first (TAB_GEMM.cu:184-192)
        word_out[byte] = (unsigned char)neg;                               // sign plane
        word_out[8 + byte] = (unsigned char)(pos | neg);                   // magnitude plane
    } else {
        unsigned b = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) b |= (v[i] < t) ? (1u << i) : 0u;      // TAB_GEMM.cu:231
        word_out[byte] = (unsigned char)b;
    }
}

// What the second phase needs of the kernel's parameter block, handed over by value: taking the block's address for a
// call would move the whole block, which every role reads all the time, from registers and constant memory to the stack.
struct QuantTailArgs {
    const float* y; const int16_t* y16; double* abs_sums; float* ths_out; uint64_t* next_qx; unsigned* grid_bar;
    double per_image; float ths_scale; int self_clean, next_bits, N, M, KN, OH, OW;
};
__device__ __forceinline__ QuantTailArgs quant_tail_args(const TcConvParams& p) {
    QuantTailArgs a;
    a.y = p.y; a.y16 = p.y16; a.abs_sums = p.abs_sums; a.ths_out = p.ths_out; a.next_qx = p.next_qx; a.grid_bar = p.grid_bar;
    a.per_image = p.per_image; a.ths_scale = p.ths_scale; a.self_clean = p.self_clean; a.next_bits = p.next_bits;
    a.N = p.N; a.M = p.M; a.KN = p.KN; a.OH = p.OH; a.OW = p.OW;
    return a;
}
__device__ __noinline__ void quantize_tail(const QuantTailArgs p, float* ths_smem, int* status) {
    const int tid = threadIdx.x;
    const unsigned G = gridDim.x;
    __threadfence();                                                       // this thread's stores and atomics, device-wide
    __syncthreads();
    int flag = 0;
    if (tid == 0) {
        __threadfence();
        atomicAdd(p.grid_bar, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < GRID_WAIT_LIMIT && !ok; i++) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.grid_bar) : "memory");
            ok = seen >= G;
            if (!ok) __nanosleep(100);
        }
        if (!ok && status) atomicExch(status, 21);
        flag = ok ? 1 : 0;
    }
    if (!__syncthreads_or(flag)) return;                                   // the result of the launch is void; the status says so
    for (int n = tid; n < p.N; n += (int)blockDim.x) {
        const double sum = __ldcg(p.abs_sums + n);
        const float t = (float)((double)p.ths_scale * (sum / p.per_image));
        ths_smem[n] = t;
        if (blockIdx.x == 0 && p.ths_out) p.ths_out[n] = t;
    }
    __syncthreads();
    // the CTA that gets here last knows that every CTA has read the sums: it leaves the state block zero again
    flag = 0;
    if (tid == 0) flag = (atomicAdd(p.grid_bar + 1, 1u) == G - 1u) ? 1 : 0;
    if (__syncthreads_or(flag)) {
        if (p.self_clean) for (int n = tid; n < p.N; n += (int)blockDim.x) p.abs_sums[n] = 0.0;
        if (tid == 0) { p.grid_bar[0] = 0u; p.grid_bar[1] = 0u; }
    }
    // words of the result: word w = 64 consecutive channels = elements [64 w, 64 w + 64) of y; 8 lanes per word, 64 words
    // per pass of the CTA, UN passes per step with all loads of a step issued before the first is used (addresses are one
    // base register plus constants)
    if (tid >= 512) return;                                                // 64 words per pass: 512 threads (kernels with extra warps have more)
    const int PC2 = p.KN >> 6, bits = p.next_bits, byte = tid & 7;
    const uint32_t grp = (uint32_t)tid >> 3;
    const uint32_t words = (uint32_t)((long long)p.M * PC2);               // < 2^31, checked on the host
    const FastDiv dimg = make_fastdiv_dev((uint32_t)(p.OH * p.OW * PC2));
    unsigned char* out = reinterpret_cast<unsigned char*>(p.next_qx);
    const size_t obytes = (size_t)8 * bits;                                // bytes of a word's planes
    if (p.y16 != nullptr) {
        constexpr int UN = 16;                                             // 16 x 16 bytes in flight per thread
        constexpr uint32_t SPAN = 64u * UN;
        const long long nsteps = ((long long)words + SPAN - 1) / SPAN;
        for (long long s = nsteps - 1 - (long long)blockIdx.x; s >= 0; s -= G) {
            const uint32_t w0 = (uint32_t)s * SPAN + grp;
            const int16_t* src = p.y16 + (size_t)w0 * 64 + byte * 8;
            const bool full = (uint32_t)s * SPAN + SPAN <= words;
            uint4 raw[UN];
            if (full) {
#pragma unroll
                for (int u = 0; u < UN; u++) raw[u] = ld_cg_u4(src + u * 4096);
            } else {
#pragma unroll
                for (int u = 0; u < UN; u++) if (w0 + 64u * u < words) raw[u] = ld_cg_u4(src + u * 4096);
            }
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const uint32_t w = w0 + 64u * u;
                if (!full && w >= words) continue;
                const uint32_t q[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                float v[8];
#pragma unroll
                for (int i = 0; i < 4; i++) { v[2 * i] = (float)(int16_t)(q[i] & 0xFFFFu); v[2 * i + 1] = (float)(int16_t)(q[i] >> 16); }
                quantize8(v, ths_smem[dimg.div(w)], bits, out + (size_t)w * obytes, byte);
            }
        }
    } else {
        constexpr int UN = 8;                                              // 8 x 32 bytes in flight per thread
        constexpr uint32_t SPAN = 64u * UN;
        const long long nsteps = ((long long)words + SPAN - 1) / SPAN;
        for (long long s = nsteps - 1 - (long long)blockIdx.x; s >= 0; s -= G) {
            const uint32_t w0 = (uint32_t)s * SPAN + grp;
            const float* src = p.y + (size_t)w0 * 64 + byte * 8;
            const bool full = (uint32_t)s * SPAN + SPAN <= words;
            F8 v[UN];
            if (full) {
#pragma unroll
                for (int u = 0; u < UN; u++) v[u] = ld_cg_f8(src + u * 4096);
            } else {
#pragma unroll
                for (int u = 0; u < UN; u++) if (w0 + 64u * u < words) v[u] = ld_cg_f8(src + u * 4096);
            }
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const uint32_t w = w0 + 64u * u;
                if (!full && w >= words) continue;
                quantize8(v[u].v, ths_smem[dimg.div(w)], bits, out + (size_t)w * obytes, byte);
            }
        }
    }
}

// ---- expander: bit-planes -> int8 patch rows ---------------------------------------------------------------------------
// Four quantised values from the low four bits of a magnitude and a sign nibble: bytes 0x00 / 0x01 / 0xFF.
__device__ __forceinline__ uint32_t expand4(uint32_t mnib, uint32_t snib) {
    const uint32_t m01 = (mnib * 0x00204081u) & 0x01010101u;               // bit i -> byte i (the shifted copies do not overlap)
    const uint32_t s01 = (snib * 0x00204081u) & 0x01010101u;
    return m01 | (s01 * 0xFFu);
}

// The (sign, magnitude) words of XUNROLL items of a patch, held in registers between the loads and the expansion.
// Nothing is computed on them before store_items: an instruction that consumes a loaded register would make the thread
// wait for that load, and the point of loading a patch ahead is not to wait.
struct RawItems { uint64_t sg[XUNROLL], mg[XUNROLL]; };

// Loads items base + u*NXT + xt (u < XUNROLL) of the patch at virtual row Rbase of plane (pa, pb), channel words 2*cp and
// 2*cp + 1.  Item = (row, word); the two words of a pixel go to neighbouring threads (32 contiguous bytes).  Padding
// positions are not loaded: they are zero words (ternary: 0; binary: +1 in the real channels).  Binary activations
// have one plane: its word is the sign, the magnitude is all ones.
__device__ __forceinline__ void load_items(const TcConvParams& p, RawItems& raw, int Rbase, int nrows, int cp, int pa, int pb, int base, int xt, int nxt) {
    const bool UNIT = p.s1 == 1 && p.s2 == 1;
    const int nw = (2 * cp + 1 < p.PC) ? 2 : 1;
    const int items = nrows * nw;
    const int VHW = p.VH * p.VW;
#pragma unroll
    for (int u = 0; u < XUNROLL; u++) {
        const int it = base + u * nxt + xt;
        raw.sg[u] = 0;
        raw.mg[u] = p.abits == 1 ? ~0ull : 0ull;
        if (it < items) {
            const int r = nw == 2 ? it >> 1 : it, w = nw == 2 ? it & 1 : 0;
            const uint32_t R = (uint32_t)(Rbase + r);
            const uint32_t n = p.dVHW.div(R);
            const uint32_t rem = R - n * (uint32_t)VHW;
            const uint32_t i = p.dVW.div(rem);
            const uint32_t j = rem - i * (uint32_t)p.VW;
            const int ih = (UNIT ? (int)i : (int)i * p.s1 + pa) - p.p1;
            const int iw = (UNIT ? (int)j : (int)j * p.s2 + pb) - p.p2;
            if ((int)n < p.N && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W) {
                const long long widx = (((long long)n * p.H + ih) * p.W + iw) * p.PC + 2 * cp + w;
                if (p.abits == 2) {
                    const ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2*>(p.qx + 2 * widx));
                    raw.sg[u] = v.x;
                    raw.mg[u] = v.y;
                } else {
                    raw.sg[u] = __ldg(p.qx + widx);
                }
            }
        }
    }
}

// Expands the items load_items fetched into rows of patch buffer `buf` (K-major, 128-byte swizzle: 16-byte unit u of
// row r lives at r*128 + ((u ^ (r & 7)) << 4); buf is 1024-byte aligned).  Channels beyond C become 0.
__device__ __forceinline__ void store_items(const TcConvParams& p, const RawItems& raw, uint32_t buf, int nrows, int cp, int base, int xt, int nxt) {
    const int nw = (2 * cp + 1 < p.PC) ? 2 : 1;
    const int items = nrows * nw;
#pragma unroll
    for (int u = 0; u < XUNROLL; u++) {
        const int it = base + u * nxt + xt;
        if (it < items) {
            const int r = nw == 2 ? it >> 1 : it, w = nw == 2 ? it & 1 : 0;
            const uint32_t rowaddr = buf + (uint32_t)r * IROW;
            const int cvalid = p.C - 64 * (2 * cp + w);                    // real channels in this word (>= 1)
            const uint64_t vmask = cvalid >= 64 ? ~0ull : ((1ull << cvalid) - 1ull);
            const uint64_t mg = raw.mg[u] & vmask, sg = raw.sg[u] & mg;
#pragma unroll
            for (int q = 0; q < 4; q++) {                                  // 16 channels = one 16-byte unit
                const uint32_t m16 = (uint32_t)(mg >> (16 * q)) & 0xFFFFu, s16 = (uint32_t)(sg >> (16 * q)) & 0xFFFFu;
                const uint32_t o0 = expand4(m16 & 15u, s16 & 15u), o1 = expand4((m16 >> 4) & 15u, (s16 >> 4) & 15u);
                const uint32_t o2 = expand4((m16 >> 8) & 15u, (s16 >> 8) & 15u), o3 = expand4(m16 >> 12, s16 >> 12);
                sts_v4(rowaddr + ((uint32_t)((4 * w + q) ^ (r & 7)) << 4), o0, o1, o2, o3);
            }
        }
    }
}

// Position of an expander in the sequence of patches its CTA stages: tile, channel pair, plane.
struct PatchIter {
    int t, cp, pl;
    __device__ __forceinline__ void next(int ncp, int planes, int step) {
        if (++pl == planes) { pl = 0; if (++cp == ncp) { cp = 0; t += step; } }
    }
};

// ---- epilogue ------------------------------------------------------------------------------------------------------------
// tcgen05.ld hands lane r of a warp the 32 columns of accumulator row r; written straight out, one store instruction
// would touch 32 different output rows.  The warp instead passes each 32x32 block through a private 4 KB shared-memory
// buffer (16-byte chunks XOR-swizzled by row, so both directions are conflict-free) and stores it transposed: eight
// lanes cover 128 contiguous bytes of one row, one instruction writes four full lines.  The residual is read the same way.

// |y| sums a warp has computed but not yet added to abs_sums: the global atomic is issued by the caller AFTER it has
// released the accumulator buffer (an mbarrier arrive has release semantics and would otherwise wait for the atomic's
// round trip to L2 on every tile).
struct PendingSums {
    int img0 = -1;
    double tot0 = 0.0, tot1 = 0.0;                                         // for images img0 and img0 + 1
};
__device__ __forceinline__ void flush_pending(const TcConvParams& p, PendingSums& ps, int lane) {
    if (ps.img0 >= 0 && lane == 0) {
        if (ps.tot0 != 0.0 && ps.img0 < p.N) atomicAdd(p.abs_sums + ps.img0, ps.tot0);
        if (ps.tot1 != 0.0 && ps.img0 + 1 < p.N) atomicAdd(p.abs_sums + ps.img0 + 1, ps.tot1);
    }
    ps.img0 = -1;
}

// Row data of a warp's 32-row slab (virtual rows Rw .. Rw + 31) in the transposed domain: lane (rsub = lane / 8,
// chunk = lane % 8) handles rows 4i + rsub, i = 0..7, and four columns per row.  Computed before the accumulator
// is waited for.
struct SlabRows {
    int mi[8];               // output row (index into [M][KN]) of row 4i + rsub, -1 = not an output position
    int m_own;               // the same for row `lane` (the ragged path works row per lane)
    int n_own;               // image of row `lane`
    int Rw, wimg0, split;    // first virtual row, its image, first slab row that belongs to the next image
    bool fast, slow;         // how |y| is summed, see slab_rows
};

// |y| sums.  Usual case ("fast"): the slab's 32 consecutive virtual rows lie in at most two images (rows below `split`
// in image wimg0, the others in wimg0 + 1) and the values are small enough for 32 of them to add exactly in float
// (|y| < 2^18): a lane keeps running totals per image as integers straight from the accumulators (exact, one REDUX at
// the end) or, with a residual - which need not be integer-valued - as doubles, every term converted before it is added.  Otherwise ("slow", rare: images of fewer than
// 32 virtual positions, very long K): one double atomic per row and block.
template <int FUSED>
__device__ __forceinline__ void slab_rows(const TcConvParams& p, int Rw, int lane, SlabRows& sr) {
    const int VHW = p.VH * p.VW;
    const uint32_t R = (uint32_t)(Rw + lane);
    const int n = (int)p.dVHW.div(R);
    const int rr = (int)R - n * VHW;
    const int oh = (int)p.dVW.div((uint32_t)rr);
    const int ow = rr - oh * p.VW;
    const bool row_ok = n < p.N && oh < p.OH && ow < p.OW;
    sr.m_own = row_ok ? (n * p.OH + oh) * p.OW + ow : -1;                  // M < 2^31 is checked on the host
    sr.n_own = n;
#pragma unroll
    for (int i = 0; i < 8; i++) sr.mi[i] = __shfl_sync(0xFFFFFFFFu, sr.m_own, 4 * i + (lane >> 3));
    sr.Rw = Rw;
    sr.wimg0 = (int)p.dVHW.div((uint32_t)Rw);
    sr.split = (sr.wimg0 + 1) * VHW - Rw;
    const bool want_sum = FUSED && p.abs_sums != nullptr;
    sr.fast = want_sum && p.Kw < (1 << 12) && (int)p.dVHW.div((uint32_t)(Rw + 31)) - sr.wimg0 <= 1;
    sr.slow = want_sum && !sr.fast;
}

// Streaming 128-bit load that leaves no line in L1 (the residual is read once).
__device__ __forceinline__ float4 ld_stream_f4(const float4* ptr) {
    float4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(ptr));
    return r;
}

// Residual values of the 32-column block at filter nbase, in the transposed layout (res[i] = row 4i + rsub, 4 columns).
__device__ __forceinline__ void slab_load_residual(const TcConvParams& p, const SlabRows& sr, int nbase, int lane, float4 (&res)[8]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        res[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sr.mi[i] >= 0) res[i] = ld_stream_f4(reinterpret_cast<const float4*>(p.residual + (long long)sr.mi[i] * p.KN + nbase) + (lane & 7));
    }
}

// Columns [c0, c1) (multiples of 32, relative to the tile's first filter n0) of one 128-row accumulator block whose
// TMEM address (column 0, this warp's lane quarter) is taddr.  The residual of a block is fetched one block ahead -
// for the first block by the caller, before it waits for the accumulator (res / res_loaded) - because a load issued
// when the block is processed costs the warp its whole DRAM latency.
template <int FUSED>
__device__ __forceinline__ void slab_columns(const TcConvParams& p, uint32_t taddr, const SlabRows& sr, int n0, int c0, int c1,
                                             int lane, uint32_t stage, float4 (&res)[8], bool res_loaded, PendingSums& ps) {
    const bool vec4 = (p.KN & 3) == 0;
    const bool small_acc = p.Kw < (1 << 15);                               // |accumulator| <= 64 * Kw < 2^21: the bias conversion is exact
    constexpr bool has_res = FUSED == 2;
    const bool want_sum = FUSED && p.abs_sums != nullptr;
    const int rsub = lane >> 3, chunk = lane & 7;
    const int VHW = p.VH * p.VW;
    unsigned isum_own = 0;                                                 // integer data: |y| total of the lane's own row
    double dsum0 = 0.0, dsum1 = 0.0;                                       // float data: totals per image in the transposed domain
#pragma unroll 1
    for (int cb = c0; cb < c1; cb += 32) {
        const int nbase = n0 + cb;
        if (nbase >= p.KN) break;                                          // uniform over the warp
        uint32_t v[32];
        tmem_ld32(taddr + (uint32_t)cb, v);
        if (vec4 && nbase + 32 <= p.KN) {
            // compact output whose rows start on 16-byte boundaries: the block is transposed as 16-bit values (half the
            // shared-memory traffic; on the 64-filter layers that traffic, next to the MMAs' operand reads, is the bound)
            const bool pack16 = !has_res && p.y16 != nullptr && (p.KN & 7) == 0;
            if (pack16) {
#pragma unroll
                for (int q = 0; q < 4; q++)                                // row `lane`: 64 bytes, 16-byte chunk q at (q ^ (lane / 2 % 4))
                    sts_v4(stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4), __byte_perm(v[8 * q], v[8 * q + 1], 0x5410), __byte_perm(v[8 * q + 2], v[8 * q + 3], 0x5410),
                           __byte_perm(v[8 * q + 4], v[8 * q + 5], 0x5410), __byte_perm(v[8 * q + 6], v[8 * q + 7], 0x5410));
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++)
                    sts_v4(stage + lane * 128 + ((q ^ (lane & 7)) << 4), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
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
            if (pack16) {                                                  // four lanes store the 64 bytes of a row, eight rows per instruction
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int r = 8 * i + (lane >> 2), c = lane & 3;
                    const int4 raw = lds_v4(stage + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
                    const int m = __shfl_sync(0xFFFFFFFFu, sr.m_own, r);
                    if (m >= 0) {
                        reinterpret_cast<int4*>(p.y16 + (long long)m * p.KN + nbase)[c] = raw;
                        if (sr.slow) {
                            const int img = (int)p.dVHW.div((uint32_t)(sr.Rw + r));
                            const int q4[4] = {raw.x, raw.y, raw.z, raw.w};
                            int tot = 0;
#pragma unroll
                            for (int j = 0; j < 4; j++) tot += abs((int)(int16_t)(q4[j] & 0xFFFF)) + abs(q4[j] >> 16);
                            if (img < p.N) atomicAdd(p.abs_sums + img, (double)tot);
                        }
                    }
                }
                __syncwarp();
                continue;
            }
            if (!has_res && p.y16 != nullptr) {                            // compact output: the integers themselves, 16 bits each
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = 4 * i + rsub;
                    const int4 raw = lds_v4(stage + r * 128 + ((chunk ^ (r & 7)) << 4));
                    if (sr.mi[i] >= 0) {
                        reinterpret_cast<uint2*>(p.y16 + (long long)sr.mi[i] * p.KN + nbase)[chunk] =
                            make_uint2(__byte_perm((uint32_t)raw.x, (uint32_t)raw.y, 0x5410), __byte_perm((uint32_t)raw.z, (uint32_t)raw.w, 0x5410));
                        if (sr.slow) {
                            const int img = (int)p.dVHW.div((uint32_t)(sr.Rw + r));
                            if (img < p.N) atomicAdd(p.abs_sums + img, (double)abs(raw.x) + (double)abs(raw.y) + (double)abs(raw.z) + (double)abs(raw.w));
                        }
                    }
                }
                __syncwarp();
                continue;
            }
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
                // the residual need not be integer-valued: compensated (Kahan) float sums, two chains per image, whose value
                // and compensation go to the double totals (good to about 1e-14 of the total)
                float sa0 = 0.f, sa1 = 0.f, ca0 = 0.f, ca1 = 0.f, sb0 = 0.f, sb1 = 0.f, cb0 = 0.f, cb1 = 0.f;
                auto kahan = [](float x, float& sv, float& cv) { const float yv = x - cv, tv = sv + yv; cv = (tv - sv) - yv; sv = tv; };
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (sr.mi[i] < 0) continue;
                    if (4 * i + rsub < sr.split) {
                        kahan(fabsf(o[i].x), sa0, ca0); kahan(fabsf(o[i].y), sa1, ca1); kahan(fabsf(o[i].z), sa0, ca0); kahan(fabsf(o[i].w), sa1, ca1);
                    } else {
                        kahan(fabsf(o[i].x), sb0, cb0); kahan(fabsf(o[i].y), sb1, cb1); kahan(fabsf(o[i].z), sb0, cb0); kahan(fabsf(o[i].w), sb1, cb1);
                    }
                }
                dsum0 += ((double)sa0 + (double)sa1) - ((double)ca0 + (double)ca1);
                dsum1 += ((double)sb0 + (double)sb1) - ((double)cb0 + (double)cb1);
            } else if (sr.slow) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int img = (int)p.dVHW.div((uint32_t)(sr.Rw + 4 * i + rsub));
                    if (sr.mi[i] >= 0 && img < p.N)
                        atomicAdd(p.abs_sums + img, ((double)fabsf(o[i].x) + (double)fabsf(o[i].y)) + ((double)fabsf(o[i].z) + (double)fabsf(o[i].w)));
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
                        if (!has_res && p.y16 != nullptr) p.y16[(long long)sr.m_own * p.KN + nbase + i] = (int16_t)(int)v[i];
                        else yrow[nbase + i] = ov;
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
    (void)VHW;
}

// ---- epilogue through TMA (TEPI) ---------------------------------------------------------------------------------------
// With a virtual grid whose row length divides 32 or is a multiple of 32 (TcConvParams::tepi), the 32 virtual rows of a
// warp's slab are one box of the output tensor [N][OH][OW][KN]: 32 positions of one grid row, or 32/VW whole grid rows of
// one image.  The box's positions outside the real output (ow >= OW, oh >= OH, n >= N) are exactly the rows the other
// epilogue drops, and the TMA engine drops them by itself.  So a 32 x 32 block needs no transposition: lane r keeps
// accumulator row r, reads its residual row from the warp's shared-memory buffer (a TMA load that was issued a whole
// block earlier put it there), converts, adds, writes the row back into the same buffer (128-byte swizzle: conflict
// free both ways) and one lane issues the TMA store.  Two buffers per warp: while block b is processed, the store of
// block b-1 drains and the residual of block b+1 arrives.  No address arithmetic per row, no global load or store
// instruction in the warp, and the bytes in flight are bounded by shared memory instead of registers.
struct TepiBox { int c0, c1, c2, c3; bool live; };

// Box of the slab at virtual row Rw, filters from nbase.
__device__ __forceinline__ TepiBox tepi_box(const TcConvParams& p, int Rw, int nbase) {
    const int VHW = p.VH * p.VW;
    const int n = (int)p.dVHW.div((uint32_t)Rw);
    const int rem = Rw - n * VHW;
    const int i = (int)p.dVW.div((uint32_t)rem);
    const int j = rem - i * p.VW;
    TepiBox b;
    b.c0 = nbase; b.c1 = j; b.c2 = i; b.c3 = n;
    b.live = n < p.N && i < p.OH && j < p.OW && nbase < p.KN;              // else nothing of the box is a real output
    return b;
}

// The warp's blocks in order: columns [ec0, ec1) of its slab of tile t (those below KN), then the same of tile t + step, ...
struct TepiIter {
    int t, cb;
    __device__ __forceinline__ void settle(int ec0, int step, int ntiles, int tiles_n, int tni, int KN) {
        while (t < ntiles && (t % tiles_n) * tni + cb >= KN) { t += step; cb = ec0; }
    }
    __device__ __forceinline__ void next(int ec0, int ec1, int step, int ntiles, int tiles_n, int tni, int KN) {
        cb += 32;
        if (cb >= ec1) { cb = ec0; t += step; }
        settle(ec0, step, ntiles, tiles_n, tni, KN);
    }
};

// Requests the residual of a block into buffer `buf` (arrives on mbar), or just arrives when the box is dead.
__device__ __forceinline__ void tepi_request_residual(const void* tmR, const TepiBox& b, uint32_t buf, uint32_t mbar) {
    if (b.live) {
        mbar_expect_tx(mbar, 4096u);
        tma_load_4d(buf, tmR, b.c0, b.c1, b.c2, b.c3, mbar);
    } else {
        mbar_arrive(mbar);
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------------------------
// FUSED: 0 plain; 1 per-image |y| sums and the threshold tail; 2 residual added (sums and tail when asked for).
// BRES: the filter block of the CTA (all taps, all channel pairs; needs KN <= TNI) is copied once and stays in shared
// memory; otherwise it streams through a ring of SB stages, one stage per tap and channel pair.
// TEPI: the epilogue moves the output (and the residual) with TMA boxes; needs the aligned virtual grid (p.tepi).
// Counters g (ring stages), q (patches) and a (accumulator buffers) run across tiles; barrier parities follow from them.
// PAIR: the kernel runs as clusters of two CTAs (see umma_common.cuh): a tile is 256 virtual rows x TNI filters, each CTA
// stages the patch of its own 128 rows and fetches TNI/2 filters of every slice; the even CTA's MMA warp issues the pair's
// MMAs and its commits arrive on the "empty" / "accumulator full" barriers of both CTAs, while the "full" / "accumulator
// empty" barriers it waits on live in the even CTA and collect the arrivals of both.
template <int MT, int TNI, int SB, bool BRES, int FUSED, bool TEPI, bool PAIR = false>
__global__ void __launch_bounds__(PTHREADS + 32 * extra_warps(FUSED, TEPI, TNI), 1)
conv_umma_persist_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmR,
                         const TcConvParams p, int* __restrict__ status,
                         const int prow, const int nrows, const int nst, const int tiles_m, const int tiles_n, const int split_from) {
    static_assert(!PAIR || (MT == 1 && !BRES && !TEPI), "CTA pairs: one row block per CTA, streamed filters, transposing epilogue");
    constexpr bool SPLIT = split_capable(MT, TNI, BRES, TEPI, PAIR);
    constexpr int BROWS = PAIR ? TNI / 2 : TNI;                            // filters of a slice this CTA holds
    constexpr int BSTAGE = BROWS * IROW;
    constexpr int ACOLS = MT * TNI;                                        // columns of one accumulator buffer
    constexpr int NXW = 5 + extra_warps(FUSED, TEPI, TNI) + (MT == 1 ? 1 : 0);   // expander warps: 0, 12 and up, and warp 3 when it has no MMAs to issue
    constexpr int NX = 32 * NXW;
    static_assert(2 * ACOLS <= 512, "two accumulator buffers must fit the 512 TMEM columns");
    static_assert(SB <= 8, "eight ring barriers are laid out");
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw);
    const uint32_t sPatch = sbase;                                         // [2][prow][128 B], prow % 8 == 0
    const uint32_t sRing = sbase + 2 * prow * IROW;                        // [nst][TNI][128 B]
    const int tail = 2 * prow * IROW + nst * BSTAGE;
    const uint32_t fullB = sbase + tail, emptyB = fullB + 64;              // [8] each
    const uint32_t fullP = emptyB + 64, emptyP = fullP + 16, accFull = emptyP + 16, accEmpty = accFull + 16;
    const uint32_t tslot = accEmpty + 16;                                  // = fullB + 192
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + tail + 192);
    volatile int* deadp = reinterpret_cast<volatile int*>(smem + tail + 200);     // set by a role whose bounded wait ran out
    const uint32_t resB = sbase + tail + 256;                              // [8 epilogue warps][2]: residual arrived (TEPI)
    const uint32_t sStage = sbase + tail + 1024;                           // [8 epilogue warps][4 KB, or 2 x 4 KB with TEPI]; 1024-byte aligned

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    PROF_GT(16, 17, tid == 0);                                             // kernel entry
    const int s1 = p.s1, s2 = p.s2;
    const bool UNIT = s1 == 1 && s2 == 1;                                  // one plane: flat tap loops
    const int PA = p.PA, PB = p.PB, VW = p.VW;
    const int T = p.KH * p.KW, ncp = (p.PC + 1) >> 1;
    // SPLIT: the tiles from split_from on (the last, partly filled round of the grid) are worked as two halves of TNI/2
    // filters each, numbered after the whole tiles: twice as many CTAs share the round and it takes about half as long.
    const int sfrom = SPLIT ? split_from : tiles_m * tiles_n;
    const int ntiles = tiles_m * tiles_n + (tiles_m * tiles_n - sfrom);    // work items: whole tiles, then halves (at most one grid of them)
    auto tile_of = [&](int v) { return SPLIT && v >= sfrom ? sfrom + ((v - sfrom) >> 1) : v; };
    auto half_of = [&](int v) { return SPLIT && v >= sfrom ? 1 + ((v - sfrom) & 1) : 0; };    // 0: whole tile, 1 / 2: its halves
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;                  // 0: the CTA whose MMA warp works for the pair
    const int cta0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // first tile of this CTA (pair)
    const int cstep = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;       // tiles between two of its tiles
    // first virtual row of this CTA's part of tile t
    auto tile_row0 = [&](int t) { return PAIR ? ((t / tiles_n) * 2 + (int)crank) * UTM : (tile_of(t) / tiles_n) * (UTM * MT); };

    if (tid == 0) {
        *deadp = 0;
        for (int s = 0; s < 8; s++) mbar_init(fullB + 8 * s, 1);
        mbar_init(fullP, (PAIR ? 2 : 1) * NX); mbar_init(fullP + 8, (PAIR ? 2 : 1) * NX);     // one arrival per expander thread (of both CTAs)
        for (int s = 0; s < 8; s++) mbar_init(emptyB + 8 * s, MT);          // one commit per MMA warp (MT = 2: two warps)
        mbar_init(emptyP, MT); mbar_init(emptyP + 8, MT);
        mbar_init(accFull, MT); mbar_init(accFull + 8, MT);
        mbar_init(accEmpty, PAIR ? 16 : 8); mbar_init(accEmpty + 8, PAIR ? 16 : 8);   // one arrival per epilogue warp (of both CTAs)
        if (TEPI) for (int i = 0; i < 16; i++) mbar_init(resB + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { if (PAIR) tmem_alloc_pair(tslot, (uint32_t)(2 * ACOLS)); else tmem_alloc(tslot, (uint32_t)(2 * ACOLS)); }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();                                          // both CTAs' barriers exist before either arrives on the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic launch: the set-up above overlapped the tail of the previous kernel (the quantiser); from here on its
    // output is read.  The next kernel may be scheduled when every CTA has finished its tiles (not earlier: a grid
    // waiting in griddepcontrol.wait was measured to slow the MMA warp of the tiles still running).
    pdl_wait();
    PROF_GT(18, 19, tid == 0);                                             // dependencies resolved
    PROF_T0;

    // In every role the whole warp runs the loops and the waits and one elected lane issues the copies, MMAs and
    // commits.  All roles walk the same nest: tile, channel pair cp, plane (a, b), taps of that plane.
    if (warp == 0 || warp >= 12 || (MT == 1 && warp == 3)) {
        // ---- expanders: up to two patches ahead of the MMAs (across tile boundaries).  The global loads of a patch are
        //      issued a whole patch earlier than they are used (they need registers, not the patch buffer), so that their
        //      latency - long when the epilogue's stores fill the memory system - is off the critical path. -----------------
        const int xt = (warp == 0 ? 0 : (warp == 3 ? NXW - 1 : warp - 11)) * 32 + lane;
        const bool prof_on = warp == 0 && lane == 0;
        (void)prof_on;
        const int planes = PA * PB, step = cstep;
        PatchIter cur = {cta0, 0, 0};
        unsigned q = 0;
        bool dead = false;
        // One patch: wait for its buffer, expand the words loaded earlier (mine), hand the patch to the MMA warp.
        auto stage_patch = [&](const RawItems& mine) {
            const unsigned pb = q & 1;
            if (q >= 2 && !mbar_wait_prof<0, PAIR>(prof_on, emptyP + 8 * pb, ((q >> 1) - 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 11); *deadp = 1; } return; }
            const uint32_t buf = sPatch + (uint32_t)(pb * prow) * IROW;
            PROF_T0;
            store_items(p, mine, buf, nrows, cur.cp, 0, xt, NX);
            const int items = nrows * ((2 * cur.cp + 1 < p.PC) ? 2 : 1);
            if (items > NX * XUNROLL) {                                    // long patches (large halo): the rest, chunk by chunk
                const int R0 = tile_row0(cur.t);
                const int pa = UNIT ? 0 : cur.pl / PB;
                for (int base = NX * XUNROLL; base < items; base += NX * XUNROLL) {
                    RawItems more;
                    load_items(p, more, R0, nrows, cur.cp, pa, UNIT ? 0 : cur.pl - pa * PB, base, xt, NX);
                    store_items(p, more, buf, nrows, cur.cp, base, xt, NX);
                }
            }
            fence_async_smem();
            if (PAIR) mbar_arrive_cluster(fullP + 8 * pb, 0u); else mbar_arrive(fullP + 8 * pb);
            PROF_ADD(1, prof_on);
            q++;
        };
        auto load_patch = [&](RawItems& into, const PatchIter& at) {
            const int pa = UNIT ? 0 : at.pl / PB;
            if (at.t < ntiles) load_items(p, into, tile_row0(at.t), nrows, at.cp, pa, UNIT ? 0 : at.pl - pa * PB, 0, xt, NX);
        };
        // The words of the next patch are loaded before this one is expanded.  (The hand-over raw = ahead comes after the
        // expansion, when those loads have long arrived: a move of a register whose load is in flight would wait for it.)
        RawItems raw;
        load_patch(raw, cur);
        while (cur.t < ntiles && !dead) {
            PatchIter nxt = cur;
            nxt.next(ncp, planes, step);
            RawItems ahead;
            load_patch(ahead, nxt);
            stage_patch(raw);
            raw = ahead;
            cur = nxt;
        }
    } else if (warp == 2) {
        // ---- filter producer ---------------------------------------------------------------------------------------------
        if (BRES) {
            if (elect_one()) {
                mbar_expect_tx(fullB, (uint32_t)(nst * BSTAGE));
                if (p.PC == 1) {
                    // one 64-byte word per tap: a 128-byte-wide slot holds taps 2j and 2j + 1 (the box of the last slot of
                    // an odd tap count ends beyond the row and is zero-filled there)
                    for (int j = 0; j < nst; j++) tma_load_2d(sRing + j * BSTAGE, &tmB, j * 128, 0, fullB);
                } else {
                    for (int cp = 0; cp < ncp; cp++)
                        for (int tap = 0; tap < T; tap++)
                            tma_load_2d(sRing + (cp * T + tap) * BSTAGE, &tmB, (tap * p.PC + 2 * cp) * 64, 0, fullB);
                }
            }
            __syncwarp();
        } else {
            unsigned g = 0;
            bool dead = false;
            const bool prof_on = lane == 0;
            (void)prof_on;
            for (int t = cta0; t < ntiles && !dead; t += cstep) {
                const int hf = half_of(t);
                const int n0 = (tile_of(t) % tiles_n) * TNI + (PAIR ? (int)crank * BROWS : 0) + (hf == 2 ? TNI / 2 : 0);
                for (int cp = 0; cp < ncp && !dead; cp++) {
                    // same tap order as the MMA warp: plane by plane
                    for (int pa = 0; pa < PA && !dead; pa++)
                    for (int pbb = 0; pbb < PB && !dead; pbb++)
                    for (int kh = pa; kh < p.KH && !dead; kh += s1)
                    for (int kw = pbb; kw < p.KW; kw += s2, g++) {
                        const unsigned slot = g % SB;
                        if (g >= (unsigned)SB && !mbar_wait_prof<2, PAIR>(prof_on, emptyB + 8 * slot, ((g / SB) - 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 12); *deadp = 1; } break; }
                        if (elect_one()) {
                            if (PAIR) {                                    // both halves are counted on the even CTA's barrier
                                if (crank == 0) mbar_expect_tx(fullB + 8 * slot, 2u * (uint32_t)BSTAGE);
                                tma_load_2d_pair(sRing + slot * BSTAGE, &tmB, ((kh * p.KW + kw) * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
                            } else if (SPLIT) {                            // boxes of TNI/2 filters: two for a whole tile
                                const int kx = ((kh * p.KW + kw) * p.PC + 2 * cp) * 64;
                                mbar_expect_tx(fullB + 8 * slot, (uint32_t)(hf ? BSTAGE / 2 : BSTAGE));
                                tma_load_2d(sRing + slot * BSTAGE, &tmB, kx, n0, fullB + 8 * slot);
                                if (!hf) tma_load_2d(sRing + slot * BSTAGE + BSTAGE / 2, &tmB, kx, n0 + TNI / 2, fullB + 8 * slot);
                            } else {
                                mbar_expect_tx(fullB + 8 * slot, (uint32_t)BSTAGE);
                                tma_load_2d(sRing + slot * BSTAGE, &tmB, ((kh * p.KW + kw) * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (warp == 1 || (MT == 2 && warp == 3)) {
        // ---- MMA warps.  One thread cannot issue the MMAs of a stage, its commits and the waits between stages as fast
        //      as the tensor pipe executes them (about 300 cycles per handshake and 80 per MMA against 48-128 cycles of
        //      execution).  With two row blocks per tile (MT = 2) warp 1 issues row block 0 and warp 3 row block 1: separate
        //      accumulators, the same operands and the same barrier phases (both warps follow every stage, so a parity
        //      wait never sees a phase other than the current or the previous one); the "empty" and "accumulator full"
        //      barriers then count one commit from each.  With one row block warp 3 idles. -----------------------------------
        constexpr uint32_t IDESC = PAIR ? umma_idesc_pair(TNI) : umma_idesc(TNI);
        constexpr uint32_t MB_UNITS = (UTM * IROW) >> 4;                   // next 128-row block of the patch, in 16-byte units
        const int mw = warp == 1 ? 0 : 1;
        const bool prof_on = warp == 1 && lane == 0;
        (void)prof_on;
        PROF_T0;
        const int mb_lo = MT == 2 ? mw : 0, mb_hi = MT == 2 ? mw + 1 : 1;  // this warp's row blocks
        unsigned g = 0, q = 0, a = 0;
        bool dead = (MT == 1 && mw == 1) || (PAIR && crank != 0);          // nothing to do for the second warp, nor in the odd CTA of a pair
        if (BRES && !dead && !mbar_wait_prof<5, PAIR>(prof_on, fullB, 0)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 15); *deadp = 1; } }
        // descriptor address of the resident filter slice of (channel pair, tap); with one channel word two taps share a slot
        auto resident_b = [&](int cp, int tap) -> uint32_t {
            return p.PC == 1 ? ((sRing + (uint32_t)(tap >> 1) * BSTAGE) >> 4) + (uint32_t)(tap & 1) * 4u
                             : (sRing + (uint32_t)(cp * T + tap) * BSTAGE) >> 4;
        };
        uint32_t idesc = IDESC;
        auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t acc_flag) {
            if (PAIR) umma_i8_pair(d, da, db, IDESC, acc_flag); else umma_i8(d, da, db, SPLIT ? idesc : IDESC, acc_flag);
        };
        auto commit = [&](uint32_t bar) { if (PAIR) umma_commit_pair(bar); else umma_commit(bar); };
        for (int t = cta0; t < ntiles && !dead; t += cstep, a++) {
            const unsigned buf = a & 1;
            if (a >= 2 && !mbar_wait_prof<3, PAIR>(prof_on, accEmpty + 8 * buf, ((a >> 1) - 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 13); *deadp = 1; } break; }
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * ACOLS;
            if (SPLIT) idesc = half_of(t) ? umma_idesc(TNI / 2) : IDESC;
            uint32_t accumulate = 0;                                       // 0 for the tile's first MMAs
            for (int cp = 0; cp < ncp && !dead; cp++) {
                const bool four = 2 * cp + 1 < p.PC;                       // both 64-channel words of the pair exist
                // the MMAs of one tap: 2 or 4 K steps of 32 bytes, MT row blocks each
                auto issue_tap = [&](uint64_t da, uint64_t db, uint32_t acc_first) {
                    for (int mb = mb_lo; mb < mb_hi; mb++) {
                        const uint32_t d = acc + mb * TNI;
                        const uint64_t dam = da + mb * MB_UNITS;
                        mma(d, dam, db, acc_first);
                        mma(d, dam + 2, db + 2, 1u);
                        if (four) {
                            mma(d, dam + 4, db + 4, 1u);
                            mma(d, dam + 6, db + 6, 1u);
                        }
                    }
                };
                if (UNIT) {
                    const unsigned pb = q & 1;
                    if (!mbar_wait_prof<4, PAIR>(prof_on, fullP + 8 * pb, (q >> 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 14); *deadp = 1; } break; }
                    tc_fence_after();
                    uint32_t arow = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;   // descriptor address of the tap's first patch row
                    int kw = 0;
                    if (BRES) {
                        if (elect_one()) {                                 // nothing to wait for between taps: one issue burst
                            for (int tap = 0; tap < T; tap++) {
                                issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)UMMA_DESC_HI << 32) | resident_b(cp, tap), (cp > 0 || tap > 0) ? 1u : 0u);
                                if (++kw == p.KW) { kw = 0; arow += (uint32_t)VW * (IROW >> 4); }
                            }
                            commit(emptyP + 8 * pb);
                            if (cp == ncp - 1) commit(accFull + 8 * buf);
                        }
                        __syncwarp();
                    } else {
                        for (int tap = 0; tap < T; tap++, g++) {
                            const unsigned slot = g % SB;
                            if (!mbar_wait_prof<5, PAIR>(prof_on, fullB + 8 * slot, (g / SB) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 15); *deadp = 1; } break; }
                            tc_fence_after();
                            if (elect_one()) {
                                issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)UMMA_DESC_HI << 32) | ((sRing + slot * BSTAGE) >> 4), (cp > 0 || tap > 0) ? 1u : 0u);
                                commit(emptyB + 8 * slot);
                                if (tap == T - 1) {
                                    commit(emptyP + 8 * pb);
                                    if (cp == ncp - 1) commit(accFull + 8 * buf);
                                }
                            }
                            __syncwarp();
                            if (++kw == p.KW) { kw = 0; arow += (uint32_t)VW * (IROW >> 4); }
                        }
                    }
                    q++;
                } else
                for (int pa = 0; pa < PA && !dead; pa++)
                for (int pbb = 0; pbb < PB && !dead; pbb++, q++) {
                    const unsigned pb = q & 1;
                    if (!mbar_wait_prof<4, PAIR>(prof_on, fullP + 8 * pb, (q >> 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 14); *deadp = 1; } break; }
                    tc_fence_after();
                    const uint32_t patch = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;    // descriptor address of the patch
                    const bool last_group = cp == ncp - 1 && pa == PA - 1 && pbb == PB - 1;
                    for (int kh = pa, ih = 0; kh < p.KH && !dead; kh += s1, ih++)
                    for (int kw = pbb, iw = 0; kw < p.KW; kw += s2, iw++) {
                        const bool last_tap = kh + s1 >= p.KH && kw + s2 >= p.KW;
                        uint32_t bsm = 0;
                        if (!BRES) {
                            const unsigned slot = g % SB;
                            if (!mbar_wait_prof<5, PAIR>(prof_on, fullB + 8 * slot, (g / SB) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 15); *deadp = 1; } break; }
                            tc_fence_after();
                            bsm = sRing + slot * BSTAGE;
                        }
                        if (elect_one()) {
                            issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (patch + (uint32_t)(ih * VW + iw) * (IROW >> 4)),
                                      ((uint64_t)UMMA_DESC_HI << 32) | (BRES ? resident_b(cp, kh * p.KW + kw) : (bsm >> 4)), accumulate);
                            if (!BRES) commit(emptyB + 8 * (g % SB));
                            if (last_tap) {
                                commit(emptyP + 8 * pb);
                                if (last_group) commit(accFull + 8 * buf);
                            }
                        }
                        __syncwarp();
                        accumulate = 1u;
                        if (!BRES) g++;
                    }
                }
            }
        }
        PROF_ADD(9, prof_on);
    } else if (TEPI) {
        // ---- epilogue warps 4-11 through TMA (TMEM lane quarter = warp % 4) -------------------------------------------
        const int ew = warp - 4, wg = ew >> 2, step = cstep;
        const bool prof_on = warp == 4 && lane == 0;
        (void)prof_on;
        const uint32_t sbuf = sStage + (uint32_t)ew * 8192u;               // two 4 KB block buffers
        const uint32_t mres = resB + 16u * (uint32_t)ew;                   // their "residual arrived" barriers
        const int emb = MT == 2 ? wg : 0, ec0 = MT == 2 ? 0 : wg * (TNI / 2), ec1 = MT == 2 ? TNI : (wg + 1) * (TNI / 2);
        constexpr bool has_res = FUSED == 2;
        const bool want_sum = FUSED && p.abs_sums != nullptr;
        const bool small_acc = p.Kw < (1 << 15);                           // |accumulator| <= 64 * Kw < 2^21: the bias conversion is exact
        const int VHW = p.VH * p.VW;
        auto slab_row = [&](int t) { return (t / tiles_n) * (UTM * MT) + emb * UTM + (warp & 3) * 32; };
        unsigned a = 0, blk = 0;
        bool dead = false;
        PendingSums pending;
        if (has_res && lane == 0) {                                        // the residual of the warp's first block
            TepiIter first = {cta0, ec0};
            first.settle(ec0, step, ntiles, tiles_n, TNI, p.KN);
            if (first.t < ntiles) tepi_request_residual(&tmR, tepi_box(p, slab_row(first.t), (first.t % tiles_n) * TNI + first.cb), sbuf, mres);
        }
        for (int t = cta0; t < ntiles && !dead; t += step, a++) {
            const unsigned buf = a & 1;
            const int n0 = (t % tiles_n) * TNI, Rw = slab_row(t);
            // the lane's own row, for the |y| sums: lanes of image wimg0 and of wimg0 + 1 are totalled separately ("fast":
            // the slab touches at most two images and row totals stay below 2^26), else every lane adds its own total
            const uint32_t R = (uint32_t)(Rw + lane);
            const int n_own = (int)p.dVHW.div(R);
            const int rr = (int)R - n_own * VHW, oh = (int)p.dVW.div((uint32_t)rr), ow = rr - oh * p.VW;
            const bool row_ok = n_own < p.N && oh < p.OH && ow < p.OW;
            const int wimg0 = (int)p.dVHW.div((uint32_t)Rw);
            const bool fast = want_sum && p.Kw < (1 << 12) && (int)p.dVHW.div((uint32_t)(Rw + 31)) - wimg0 <= 1;
            unsigned isum = 0;
            double dsum = 0.0;
            // (No prefetch of the next tile's residual boxes into the L2: the copy engine, which takes every box row by row, is
            //  what bounds this epilogue, and the prefetches were half as many requests again - 5 % of the launch.)
            if (!mbar_wait_prof<6>(prof_on, accFull + 8 * buf, (a >> 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 16); *deadp = 1; } break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + buf * ACOLS + (uint32_t)(emb * TNI) + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 1
            for (int cb = ec0; cb < ec1 && n0 + cb < p.KN; cb += 32, blk++) {
                const unsigned k = blk & 1;
                const uint32_t sb = sbuf + k * 4096u;
                const int nbase = n0 + cb, ncols = min(32, p.KN - nbase);
                uint32_t v[32];
                tmem_ld32(taddr + (uint32_t)cb, v);
                float o[32];
                if (has_res) {
                    if (lane == 0) {
                        // the other buffer's last store must have finished reading it before the next residual lands there
                        bulk_wait_read<0>();
                        TepiIter nx = {t, cb};
                        nx.next(ec0, ec1, step, ntiles, tiles_n, TNI, p.KN);
                        if (nx.t < ntiles)
                            tepi_request_residual(&tmR, tepi_box(p, slab_row(nx.t), (nx.t % tiles_n) * TNI + nx.cb), sbuf + (k ^ 1u) * 4096u, mres + 8u * (k ^ 1u));
                    }
                    if (!mbar_wait_prof<7>(prof_on, mres + 8u * k, (blk >> 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 17); *deadp = 1; } break; }
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const int4 rv = lds_v4(sb + (uint32_t)lane * 128u + ((uint32_t)(q ^ (lane & 7)) << 4));
                        o[4 * q] = __int_as_float(rv.x); o[4 * q + 1] = __int_as_float(rv.y); o[4 * q + 2] = __int_as_float(rv.z); o[4 * q + 3] = __int_as_float(rv.w);
                    }
                } else {
                    if (lane == 0) bulk_wait_read<1>();                    // this buffer's previous store (two blocks ago) has read it
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float f = small_acc ? __int_as_float((int)v[j] + 0x4B400000) - 12582912.f : (float)(int)v[j];
                    o[j] = has_res ? o[j] + f : f;
                }
                if (want_sum && row_ok) {
                    if (!has_res && fast) {
                        // y is the accumulator itself: integers below 2^18, so 32 of them add exactly in float (|.| is free)
                        float f0 = 0.f, f1 = 0.f, f2 = 0.f, f3 = 0.f;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (j < ncols) f0 += fabsf(o[j]);
                            if (j + 1 < ncols) f1 += fabsf(o[j + 1]);
                            if (j + 2 < ncols) f2 += fabsf(o[j + 2]);
                            if (j + 3 < ncols) f3 += fabsf(o[j + 3]);
                        }
                        isum += __float2uint_rn((f0 + f1) + (f2 + f3));
                    } else {
                        // the residual need not be integer-valued: compensated (Kahan) float sums, four chains, whose value and
                        // compensation go to the double total - the total is then good to about 1e-14 of itself
                        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (j < ncols) { const float yv = fabsf(o[j]) - c0, tv = s0 + yv; c0 = (tv - s0) - yv; s0 = tv; }
                            if (j + 1 < ncols) { const float yv = fabsf(o[j + 1]) - c1, tv = s1 + yv; c1 = (tv - s1) - yv; s1 = tv; }
                            if (j + 2 < ncols) { const float yv = fabsf(o[j + 2]) - c2, tv = s2 + yv; c2 = (tv - s2) - yv; s2 = tv; }
                            if (j + 3 < ncols) { const float yv = fabsf(o[j + 3]) - c3, tv = s3 + yv; c3 = (tv - s3) - yv; s3 = tv; }
                        }
                        dsum += (((double)s0 + (double)s1) + ((double)s2 + (double)s3)) - (((double)c0 + (double)c1) + ((double)c2 + (double)c3));
                    }
                }
#pragma unroll
                for (int q = 0; q < 8; q++)
                    sts_v4(sb + (uint32_t)lane * 128u + ((uint32_t)(q ^ (lane & 7)) << 4), __float_as_uint(o[4 * q]), __float_as_uint(o[4 * q + 1]),
                           __float_as_uint(o[4 * q + 2]), __float_as_uint(o[4 * q + 3]));
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const TepiBox bx = tepi_box(p, Rw, nbase);
                    if (bx.live) tma_store_4d(&tmY, bx.c0, bx.c1, bx.c2, bx.c3, sb);
                    bulk_commit();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accEmpty + 8 * buf);
            if (want_sum) {                                                // the |y| atomics, off the buffer's critical path
                flush_pending(p, pending, lane);
                if (fast) {
                    const bool first_img = n_own == wimg0;
                    if (has_res) {
                        double t0 = first_img ? dsum : 0.0, t1 = first_img ? 0.0 : dsum;
#pragma unroll
                        for (int sh = 16; sh > 0; sh >>= 1) { t0 += __shfl_xor_sync(0xFFFFFFFFu, t0, sh); t1 += __shfl_xor_sync(0xFFFFFFFFu, t1, sh); }
                        pending.tot0 = t0; pending.tot1 = t1;
                    } else {
                        pending.tot0 = (double)__reduce_add_sync(0xFFFFFFFFu, first_img ? isum : 0u);
                        pending.tot1 = (double)__reduce_add_sync(0xFFFFFFFFu, first_img ? 0u : isum);
                    }
                    pending.img0 = wimg0;
                    flush_pending(p, pending, lane);
                } else if (row_ok && dsum != 0.0) {
                    atomicAdd(p.abs_sums + n_own, dsum);
                }
            }
        }
        if (lane == 0) bulk_wait_all();                                    // every store of this warp has left shared memory and landed
        __syncwarp();
    } else {
        // ---- epilogue warps 4-11 (TMEM lane quarter = warp % 4) -------------------------------------------------------
        unsigned a = 0;
        bool dead = false;
        PendingSums pending;
        const bool prof_on = warp == 4 && lane == 0;
        (void)prof_on;
        for (int t = cta0; t < ntiles && !dead; t += cstep, a++) {
            const unsigned buf = a & 1;
            const int hf = half_of(t), wcols = hf ? TNI / 2 : TNI;         // columns of the accumulator in use
            const int R0 = tile_row0(t), n0 = (tile_of(t) % tiles_n) * TNI + (hf == 2 ? TNI / 2 : 0);
            // two warps per TMEM lane quarter: they split the row blocks of a two-block tile, else the columns.  Row data
            // and the first block's residual are fetched before the accumulator is waited for.
            const int wg = (warp - 4) >> 2;
            const int emb = MT == 2 ? wg : 0, ec0 = MT == 2 ? 0 : wg * (wcols / 2), ec1 = MT == 2 ? TNI : (wg + 1) * (wcols / 2);
            SlabRows sr;
            slab_rows<FUSED>(p, R0 + emb * UTM + (warp & 3) * 32, lane, sr);
            float4 res[8];
            bool res_loaded = false;
            if (FUSED == 2 && (p.KN & 3) == 0 && n0 + ec0 + 32 <= p.KN) {
                slab_load_residual(p, sr, n0 + ec0, lane, res);
                res_loaded = true;
            }
            if (!mbar_wait_prof<6, PAIR>(prof_on, accFull + 8 * buf, (a >> 1) & 1u)) { dead = true; if (lane == 0) { if (status) atomicExch(status, 16); *deadp = 1; } break; }
            tc_fence_after();
            PROF_T0;
            slab_columns<FUSED>(p, tmem_base + buf * ACOLS + (uint32_t)(emb * TNI) + ((uint32_t)((warp & 3) * 32) << 16), sr, n0, ec0, ec1,
                                lane, sStage + (warp - 4) * 4096, res, res_loaded, pending);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (PAIR) mbar_arrive_cluster(accEmpty + 8 * buf, 0u); else mbar_arrive(accEmpty + 8 * buf); }
            PROF_ADD(8, prof_on);
            if (FUSED) flush_pending(p, pending, lane);                    // the |y| atomics, off the buffer's critical path
        }
    }
    tc_fence_before();
    __syncthreads();
    PROF_ADD(12, tid == 0);
    PROF_MAX(13, tid == 0);
    PROF_GT(20, 21, tid == 0);                                             // tiles done
    if (*deadp != 0) {
        // a wait ran out in this CTA: give copies and MMAs that may still be in flight time to land before this
        // CTA frees its tensor memory and its shared memory goes to another CTA (never taken when the protocol is intact)
        for (int i = 0; i < 200; i++) __nanosleep(1000);
    }
    __syncthreads();
    if (PAIR) cluster_sync_all();                                          // the other CTA no longer reads this one's memory nor arrives on its barriers
    pdl_launch_dependents();
    if (warp == 1) { if (PAIR) tmem_dealloc_pair(tmem_base, (uint32_t)(2 * ACOLS)); else tmem_dealloc(tmem_base, (uint32_t)(2 * ACOLS)); }
    if (FUSED) {
        if (p.next_qx != nullptr) quantize_tail(quant_tail_args(p), reinterpret_cast<float*>(smem), status);   // the patch area is free now
        else fused_finish(p);
    }
    PROF_GT(22, 23, tid == 0);                                             // exit
}

#ifdef TAB_PROF
extern "C" int tab_prof_read(unsigned long long* out, int clear) {
    if (cudaMemcpyFromSymbol(out, g_prof, sizeof(unsigned long long) * 32) != cudaSuccess) return -1;
    if (clear) {
        unsigned long long z[32] = {0};
        z[16] = z[18] = z[20] = z[22] = ~0ull;
        cudaMemcpyToSymbol(g_prof, z, sizeof(z));
    }
    return 0;
}
#endif

// ---- host side -----------------------------------------------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 2-D byte tensor [rows][row_bytes] (row pitch = row_bytes), box = 128 bytes x box_rows, 128-byte swizzle.
// Encoding a map costs tens of microseconds on the host, more than a small convolution takes on the device, and
// callers reuse their buffers: the last few maps are kept, keyed by everything that goes into them.
struct MapKey { const void* base; unsigned long long row_bytes, rows; unsigned box_rows; };
struct MapKey4 { const void* base; int d[4]; int bw, bh; };

// 4-D float tensor [N][OH][OW][KN] (innermost first: KN, OW, OH, N), box = 32 filters x bw positions x bh rows x 1 image,
// 128-byte swizzle, out-of-range elements read as zero.  Needs KN % 4 == 0 and a 16-byte aligned base.
static bool make_map_4d(CUtensorMap* m, const void* base, int KN, int OW, int OH, int N, int bw, int bh);
static bool make_map_2d(CUtensorMap* m, const void* base, unsigned long long row_bytes, unsigned long long rows, unsigned box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    constexpr int NCACHE = 64;
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

static bool make_map_4d(CUtensorMap* m, const void* base, int KN, int OW, int OH, int N, int bw, int bh) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    constexpr int NCACHE = 128;
    static std::mutex mu;
    static MapKey4 keys[NCACHE] = {};
    static CUtensorMap maps[NCACHE];
    static int used = 0, next = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++) {
        const MapKey4& k = keys[i];
        if (k.base == base && k.d[0] == KN && k.d[1] == OW && k.d[2] == OH && k.d[3] == N && k.bw == bw && k.bh == bh) { *m = maps[i]; return true; }
    }
    const cuuint64_t dims[4] = {(cuuint64_t)KN, (cuuint64_t)OW, (cuuint64_t)OH, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)KN * 4, (cuuint64_t)KN * 4 * OW, (cuuint64_t)KN * 4 * OW * OH};
    const cuuint32_t box[4] = {32, (cuuint32_t)bw, (cuuint32_t)bh, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    keys[next] = MapKey4{base, {KN, OW, OH, N}, bw, bh};
    maps[next] = *m;
    next = (next + 1) % NCACHE;
    if (used < NCACHE) used++;
    return true;
}

// Where an expired wait is recorded (0 = never).  In host code the name is only a symbol handle; the device
// address is looked up once per device, under a lock.
static __device__ int g_umma_status;
static int* umma_status_ptr() {
    static std::mutex mu;
    static int* addr[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_umma_status) != cudaSuccess) return nullptr;
        addr[dev] = static_cast<int*>(ptr);
    }
    return addr[dev];
}

int* device_status_word() { return umma_status_ptr(); }

// Reads (and clears) the record of expired waits on the current device; synchronises the device.
int umma_status_read_and_clear() {
    int v = -1, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));
    return v;
}

// Virtual grid of a geometry (see TcConvParams).  aligned: rows of the grid are stretched so that a 32-row slab is one
// box of the output tensor - VW a divisor or a multiple of 32, and, where a slab spans several grid rows, VH a multiple
// of that number (the stretch is more padding, which the expanders and the drop rules already handle).  Returns false
// when that cannot be had (images of fewer than 32 positions).
static bool set_virtual_grid(TcConvParams& p, bool aligned) {
    const bool unit = p.s1 == 1 && p.s2 == 1;
    p.PA = p.s1 < p.KH ? p.s1 : p.KH;
    p.PB = p.s2 < p.KW ? p.s2 : p.KW;
    if (unit) {                                                            // padding shared between neighbours where the output fits
        p.VH = p.OH <= p.H + p.p1 ? p.H + p.p1 : p.H + 2 * p.p1;
        p.VW = p.OW <= p.W + p.p2 ? p.W + p.p2 : p.W + 2 * p.p2;
    } else {
        p.VH = (p.H + 2 * p.p1 + p.s1 - 1) / p.s1;
        p.VW = (p.W + 2 * p.p2 + p.s2 - 1) / p.s2;
    }
    p.tepi = 0;
    if (!aligned) return true;
    if (p.VW >= 32) {
        p.VW = (p.VW + 31) / 32 * 32;
    } else {
        int w = 1;
        while (w < p.VW) w *= 2;
        p.VW = w;
        const int rows = 32 / w;                                           // grid rows per slab
        p.VH = (p.VH + rows - 1) / rows * rows;
    }
    p.tepi = 1;
    return true;
}

// How many clusters of two CTAs of the pair kernel's size the device holds at once (0: none), asked of the occupancy
// calculator once per device.  The launch never asks for more: all its CTAs are resident, which the second phase's
// grid-wide counter relies on.
static int pair_clusters();
static bool pair_launch_possible() { return pair_clusters() >= 1; }

// A tile shape and what it needs.
struct TcPlan { int mt, tn, sb; bool resident, pair; int prow, nrows, nst, smem; long long tiles_m, tiles_n; };

// pair: clusters of two CTAs; a tile is 256 rows (128 per CTA) x tn filters, a ring stage holds tn/2 filters per CTA.
static bool plan_shape(const TcConvParams& p, int mt, int tn, int sb, TcPlan* out, bool pair = false) {
    const long long halo = (long long)((p.KH - 1) / p.s1) * p.VW + (p.KW - 1) / p.s2;
    const long long nrows = 128LL * mt + halo, prow = (nrows + 7) / 8 * 8;
    const long long fixed = 2 * prow * IROW + 1024 + 8 * (p.tepi ? 8192 : 4096) + 1024;   // patches, barriers, epilogue buffers, alignment
    const long long nres = p.PC == 1 ? ((long long)p.KH * p.KW + 1) / 2 : (long long)p.KH * p.KW * ((p.PC + 1) / 2);   // slots of resident filters
    TcPlan pl;
    pl.mt = mt; pl.tn = tn; pl.sb = sb; pl.pair = pair;
    pl.resident = !pair && p.KN <= tn && fixed + nres * tn * IROW <= UMMA_SMEM_MAX;
    const long long smem = pl.resident ? fixed + nres * tn * IROW : fixed + (long long)sb * (pair ? tn / 2 : tn) * IROW;
    if (smem > UMMA_SMEM_MAX) return false;
    pl.prow = (int)prow; pl.nrows = (int)nrows; pl.nst = pl.resident ? (int)nres : sb; pl.smem = (int)smem;
    const long long Mv = (long long)(p.N - 1) * p.VH * p.VW + (long long)(p.OH - 1) * p.VW + p.OW;   // last useful virtual row + 1
    pl.tiles_m = (Mv + 128LL * mt - 1) / (128LL * mt);
    if (pair) pl.tiles_m = (pl.tiles_m + 1) / 2;
    pl.tiles_n = (p.KN + tn - 1) / tn;
    if (pl.tiles_m * pl.tiles_n >= (1LL << 31) - 65536) return false;      // tile and work-item indices are ints
    *out = pl;
    return true;
}

// Tile for a problem on the grid p holds; false = no shape fits (very wide images with many taps).
// Measured on the ResNet-18-shaped layers at batch 256 (every shape forced in turn): the widest tile the filter count
// fills is fastest - the MMA warps pay about 300 cycles per ring stage whatever the stage holds, so wide MMAs amortise
// it - and two row blocks per tile beat one where they fit (the two MMA warps then issue in parallel).  A problem that
// gives the SMs less than half a wave of such tiles takes the next narrower tile instead.
static bool tc_plan(const TcConvParams& p, int sms, TcPlan* best) {
    static const int cands[5][3] = {{1, 256, 4}, {2, 128, 4}, {1, 128, 6}, {2, 64, 6}, {1, 64, 6}};
    const int tn0 = p.KN <= 64 ? 64 : (p.KN <= 128 ? 128 : 256);
    // Wide filter blocks on CTA pairs: a lone CTA would have to take in a 32 KB filter slice per 512 cycles of MMAs, which is
    // all an SM can take in from the L2; a pair splits every slice between its two CTAs.  (Strided layers, bound by their
    // four or more patches per tile, and layers with a residual, bound by their epilogue, measured no faster on pairs.)
#ifdef TAB_TUNE
    // Build-time diagnostic (-DTAB_TUNE, never in the shipped library): the tile is taken from the environment, "mt,tn,pair".
    if (const char* env = getenv("TAB_TILE")) {
        int mt = 0, tn = 0, pair = 0;
        if (sscanf(env, "%d,%d,%d", &mt, &tn, &pair) == 3) {
            if (pair) return tn == 256 && mt == 1 && !p.tepi && p.residual == nullptr && plan_shape(p, 1, 256, 8, best, true);
            for (const auto& c : cands)
                if (c[0] == mt && c[1] == tn) return plan_shape(p, mt, tn, c[2], best);
            return false;
        }
    }
#endif
    TcPlan lone;
    const bool fits_whole = plan_shape(p, 1, 256, 4, &lone) && lone.resident;      // a block that stays in shared memory is fetched once anyway
    if (tn0 == 256 && !p.tepi && !fits_whole && p.PA * p.PB == 1 && p.KH * p.KW > 1 && p.residual == nullptr && pair_launch_possible() &&
        plan_shape(p, 1, 256, 8, best, true) &&
        best->tiles_m * best->tiles_n * 2 > sms) return true;              // with a round of tiles for the pairs or less, single CTAs measured faster
    bool found = false;
    for (const auto& c : cands) {
        if (c[1] > tn0) continue;
        TcPlan pl;
        if (!plan_shape(p, c[0], c[1], c[2], &pl)) continue;
        if (!found) { *best = pl; found = true; }
        if (pl.tiles_m * pl.tiles_n * 2 > sms) { *best = pl; break; }      // enough tiles: take it; else keep looking for more tiles
        if (pl.tiles_m * pl.tiles_n > best->tiles_m * best->tiles_n) *best = pl;
    }
    return found;
}

static bool grid_in_range(const TcConvParams& p) {
    const long long rows = (long long)p.N * p.VH * p.VW;
    return rows < (1LL << 31) - 65536;
}

// Chooses the virtual grid and the tile.  The TMA epilogue (aligned grid) is taken where it measured faster: layers with
// a residual whose arithmetic is light against their bytes (at most 64 filters and 1024 terms per output), where the
// transposing epilogue's residual loads and stores leave the memory system idle half of the time.
static bool tc_prepare(TcConvParams& p, int sms, TcPlan* pl) {
    if ((long long)p.N * p.H * p.W >= (1LL << 31) || (long long)p.M >= (1LL << 31) - 512) return false;
    if ((long long)p.KH * p.KW * p.PC >= (1LL << 20)) return false;
    const bool tepi_ok = (p.KN & 3) == 0 && !(reinterpret_cast<uintptr_t>(p.y) & 15) && !(reinterpret_cast<uintptr_t>(p.residual) & 15) &&
                         (long long)p.KN * p.OW * p.OH * 4 < (1LL << 40);
    bool tepi_pays = p.residual != nullptr && p.y16 == nullptr && p.KN <= 64 && (long long)p.KH * p.KW * p.C <= 1024;
#ifdef TAB_TUNE
    if (const char* env = getenv("TAB_TEPI")) tepi_pays = p.residual != nullptr && p.y16 == nullptr && atoi(env) != 0;
#endif
    bool have = false;
    if (tepi_ok && tepi_pays) {
        TcConvParams q = p;
        if (set_virtual_grid(q, true) && grid_in_range(q) && tc_plan(q, sms, pl)) { p = q; have = true; }
    }
    if (!have) {
        set_virtual_grid(p, false);
        if (!grid_in_range(p) || !tc_plan(p, sms, pl)) return false;
    }
    p.dVHW = make_fastdiv((uint32_t)(p.VH * p.VW));
    p.dVW = make_fastdiv((uint32_t)p.VW);
    return true;
}

// First tile that is worked as two halves (see SPLIT in the kernel), ntiles = none: a last round of the persistent grid
// that fills at most half of it is split, so that it takes about half as long.
static long long split_point(long long ntiles, int sms, bool capable) {
#ifdef TAB_TUNE
    if (const char* env = getenv("TAB_SPLIT")) if (atoi(env) == 0) return ntiles;      // build-time diagnostic only
#endif
    const long long grid = ntiles < sms ? ntiles : sms, rest = grid > 0 ? ntiles % grid : 0;
    return capable && ntiles > grid && rest != 0 && 2 * rest <= grid ? ntiles - rest : ntiles;
}

template <int MT, int TNI, int SB, bool BRES, int FUSED, bool TEPI, bool PAIR = false>
static int launch_persist_u(const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcConvParams& p, const TcPlan& pl,
                            int sms, int* status, cudaStream_t stream) {
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            e = cudaFuncSetAttribute(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, TEPI, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX);
            if (e != cudaSuccess) return record_cuda_error(e);
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    const long long ntiles = pl.tiles_m * pl.tiles_n;
    if (PAIR) {
        const long long pairs = std::min<long long>(sms / 2, pair_clusters());
        const unsigned grid = 2u * (unsigned)(ntiles < pairs ? ntiles : pairs);
        return launch_pdl_cluster(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, TEPI, PAIR>, dim3(grid), dim3(PTHREADS + 32 * extra_warps(FUSED, TEPI, TNI)), (size_t)pl.smem, stream, 2u,
                                  tmB, tmY, tmR, p, status, pl.prow, pl.nrows, pl.nst, (int)pl.tiles_m, (int)pl.tiles_n, (int)ntiles);
    }
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);
    const long long split_from = split_point(ntiles, sms, split_capable(MT, TNI, BRES, TEPI, PAIR));
    return launch_pdl(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, TEPI, PAIR>, dim3(grid), dim3(PTHREADS + 32 * extra_warps(FUSED, TEPI, TNI)), (size_t)pl.smem, stream,
                      tmB, tmY, tmR, p, status, pl.prow, pl.nrows, pl.nst, (int)pl.tiles_m, (int)pl.tiles_n, (int)split_from);
}

template <int MT, int TNI, int SB>
static int launch_persist(const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR, const TcConvParams& p, const TcPlan& pl,
                          int sms, int* status, cudaStream_t stream) {
    const int fused = p.residual ? 2 : (p.abs_sums ? 1 : 0);
    const bool tepi = p.tepi != 0;
#define TAB_LAUNCH(BR, FU, TE) return launch_persist_u<MT, TNI, SB, BR, FU, TE>(tmB, tmY, tmR, p, pl, sms, status, stream)
    if (pl.pair) {
        if constexpr (MT == 1 && TNI == 256) {
            if (fused == 2) return TAB_E_TOO_LARGE;                        // the planner does not pair layers with a residual
            if (fused == 1) return launch_persist_u<1, 256, SB, false, 1, false, true>(tmB, tmY, tmR, p, pl, sms, status, stream);
            return launch_persist_u<1, 256, SB, false, 0, false, true>(tmB, tmY, tmR, p, pl, sms, status, stream);
        } else {
            return TAB_E_TOO_LARGE;
        }
    }
#define TAB_LAUNCH_F(BR, TE) do { if (fused == 2) TAB_LAUNCH(BR, 2, TE); if (fused == 1) TAB_LAUNCH(BR, 1, TE); TAB_LAUNCH(BR, 0, TE); } while (0)
    if (pl.resident) { if (tepi) TAB_LAUNCH_F(true, true); TAB_LAUNCH_F(true, false); }
    if (tepi) TAB_LAUNCH_F(false, true);
    TAB_LAUNCH_F(false, false);
#undef TAB_LAUNCH_F
#undef TAB_LAUNCH
}

static int pair_clusters() {
    static std::mutex mu;
    static int known[64] = {};                                             // 0 unknown, else clusters + 1
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!known[dev]) {
        auto kernel = conv_umma_persist_kernel<1, 256, 8, false, 0, false, true>;
        int clusters = 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2); cfg.blockDim = dim3(PTHREADS + 32 * extra_warps(0, false, 256)); cfg.dynamicSmemBytes = UMMA_SMEM_MAX;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        const bool ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX) == cudaSuccess &&
                        cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1;
        if (!ok) cudaGetLastError();
        known[dev] = ok ? clusters + 1 : 1;
    }
    return known[dev] - 1;
}

static thread_local char g_last_kernel[112] = "none";
const char* tc_last_kernel() { return g_last_kernel; }
void tc_forget_last_kernel() { snprintf(g_last_kernel, sizeof(g_last_kernel), "none"); }

static bool operands_aligned(const TcConvParams& p) {
    return !((reinterpret_cast<uintptr_t>(p.w8) & 15) || (reinterpret_cast<uintptr_t>(p.qx) & (p.abits == 2 ? 15 : 7)));
}

// Whether tc_conv_dispatch will take the problem (asked before the quantiser is given the weight expansion to do).
bool tc_conv_covers(TcConvParams p) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    TcPlan pl;
    return encode_tiled_fn() && operands_aligned(p) && tc_prepare(p, sms, &pl);
}

// GEMM stage on the tensor cores.  TAB_E_TOO_LARGE when the shape is not covered (the caller falls back to the
// popcount kernel, which reads the same bit-planes).
int tc_conv_dispatch(TcConvParams p, cudaStream_t stream) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    TcPlan pl;
    if (!encode_tiled_fn() || !operands_aligned(p) || !tc_prepare(p, sms, &pl)) return TAB_E_TOO_LARGE;
    alignas(64) CUtensorMap tmB, tmY, tmR;
    // filter boxes: a pair's CTA and a kernel that can work tiles in halves fetch half a tile's filters per copy
    const bool half_box = pl.pair || split_capable(pl.mt, pl.tn, pl.resident, p.tepi != 0, pl.pair);
    if (!make_map_2d(&tmB, p.w8, (unsigned long long)p.Kw * 64, (unsigned long long)p.KN, (unsigned)(half_box ? pl.tn / 2 : pl.tn))) return TAB_E_TOO_LARGE;
    tmY = tmB; tmR = tmB;                                                   // placeholders when the epilogue does not use them
    if (p.tepi) {
        const int bw = p.VW >= 32 ? 32 : p.VW, bh = 32 / bw;
        if (!make_map_4d(&tmY, p.y, p.KN, p.OW, p.OH, p.N, bw, bh)) return TAB_E_TOO_LARGE;
        if (p.residual && !make_map_4d(&tmR, p.residual, p.KN, p.OW, p.OH, p.N, bw, bh)) return TAB_E_TOO_LARGE;
    }
    int* status = umma_status_ptr();
    const bool halves = split_point(pl.tiles_m * pl.tiles_n, sms, half_box && !pl.pair) < pl.tiles_m * pl.tiles_n;
    snprintf(g_last_kernel, sizeof(g_last_kernel), "conv_umma_persist_kernel<%d,%d,%d,%d,%d,%d%s> grid %dx%d%s%s", pl.mt, pl.tn, pl.sb, (int)pl.resident,
             p.residual ? 2 : (p.abs_sums ? 1 : 0), p.tepi, pl.pair ? ",pair" : "", p.VH, p.VW, halves ? " halves" : "", p.next_qx ? " +next" : "");
    if (pl.pair) return launch_persist<1, 256, 8>(tmB, tmY, tmR, p, pl, sms, status, stream);
    if (pl.tn == 64) return pl.mt == 2 ? launch_persist<2, 64, 6>(tmB, tmY, tmR, p, pl, sms, status, stream) : launch_persist<1, 64, 6>(tmB, tmY, tmR, p, pl, sms, status, stream);
    if (pl.tn == 128) return pl.mt == 2 ? launch_persist<2, 128, 4>(tmB, tmY, tmR, p, pl, sms, status, stream) : launch_persist<1, 128, 6>(tmB, tmY, tmR, p, pl, sms, status, stream);
    return launch_persist<1, 256, 4>(tmB, tmY, tmR, p, pl, sms, status, stream);
}

}  // namespace tab
