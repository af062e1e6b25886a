// TAB convolution on the 5th-generation tensor cores: a persistent, warp-specialised implicit GEMM that reads the
// activations as the bit-planes tab_quantize_launch writes (TAB_GEMM.cu:196-197) and multiplies them as int8.
//
// Replaces the reference's PadKernel, Img2RowKernel (TAB_GEMM.cuh:73-115) and TNN/TBN/BTN/BNNGEMM (TAB_GEMM.cu:25-147).
// The quantised values {-1,0,+1} times {-1,0,+1} accumulate exactly in int32 (at most KH*KW*C terms), so y = sum a*w
// directly and none of the per-type corrections of the popcount formulas is needed: zero words of binary activations
// decode to +1 (the reference's padding rule), channel tails decode to 0.
//
// One CTA per SM walks over output tiles of 128*MT virtual rows x TN filters (see TcConvParams for the virtual grid):
//   * expander warps (0, 3, 12-15): stage the *patch* of a tile - the 128*MT + halo consecutive virtual rows all its
//     taps read - for one pair of 64-channel words and one stride plane: 16 bytes of (sign, magnitude) per pixel and
//     word are loaded from global memory (padding positions are not loaded at all) and expanded to 64 bytes of int8
//     in the K-major, 128-byte-swizzled layout the MMA descriptors expect.  Two patch buffers; the expanders run up to
//     two patches ahead of the MMAs, across tile boundaries.
//   * warp 2: TMA copies of the filter slice (TN x 128 B per tap and channel pair) into a ring of SB stages, or - when
//     the filters of all taps fit beside the patches (BRES) - once per CTA.
//   * warp 1: tcgen05.mma.cta_group::1.kind::i8, 128 x TN x 32 per instruction.  Tap (kh, kw) of the 128 rows of an MMA
//     is 128 consecutive patch rows starting (kh/s1)*VW + kw/s2 rows into the patch: the A descriptor simply starts
//     there (the 128-byte swizzle is a function of absolute shared-memory address bits).  Two TMEM accumulator buffers.
//   * warps 4-11: epilogue of the other accumulator buffer: tcgen05.ld, transposition through a private shared-memory
//     block so that stores are coalesced, int -> float, residual, per-image sums of |y|, stores.
//   * the CTA that finishes last turns the sums into the next layer's thresholds.
// Every mbarrier wait is a bounded try_wait loop; on expiry the role records a code in *status and stops, the other
// roles run into their own limits, every thread still reaches the final barrier, TMEM is freed and the kernel returns.
// No kernel here waits on another CTA or GPU, and no copy is multicast.
#include <cuda.h>
#include <algorithm>
#include <cstdio>
#include <mutex>
#include "tab_kernels.cuh"
#include "umma_common.cuh"

namespace tab {

constexpr int PTHREADS = 512;                                              // 16 warps
constexpr int NXT = 192;                                                   // expander threads (6 warps)
constexpr int XUNROLL = 4;                                                 // (pixel, word) items a thread has in flight

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
template <bool UNIT>
__device__ __forceinline__ void load_items(const TcConvParams& p, RawItems& raw, int Rbase, int nrows, int cp, int pa, int pb, int base, int xt) {
    const int nw = (2 * cp + 1 < p.PC) ? 2 : 1;
    const int items = nrows * nw;
    const int VHW = p.VH * p.VW;
#pragma unroll
    for (int u = 0; u < XUNROLL; u++) {
        const int it = base + u * NXT + xt;
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
__device__ __forceinline__ void store_items(const TcConvParams& p, const RawItems& raw, uint32_t buf, int nrows, int cp, int base, int xt) {
    const int nw = (2 * cp + 1 < p.PC) ? 2 : 1;
    const int items = nrows * nw;
#pragma unroll
    for (int u = 0; u < XUNROLL; u++) {
        const int it = base + u * NXT + xt;
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
template <bool FUSED>
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

// Residual values of the 32-column block at filter nbase, in the transposed layout (res[i] = row 4i + rsub, 4 columns).
__device__ __forceinline__ void slab_load_residual(const TcConvParams& p, const SlabRows& sr, int nbase, int lane, float4 (&res)[8]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        res[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sr.mi[i] >= 0) res[i] = __ldg(reinterpret_cast<const float4*>(p.residual + (long long)sr.mi[i] * p.KN + nbase) + (lane & 7));
    }
}

// Columns [c0, c1) (multiples of 32, relative to the tile's first filter n0) of one 128-row accumulator block whose
// TMEM address (column 0, this warp's lane quarter) is taddr.  The residual of a block is fetched one block ahead -
// for the first block by the caller, before it waits for the accumulator (res / res_loaded) - because a load issued
// when the block is processed costs the warp its whole DRAM latency.
template <bool FUSED>
__device__ __forceinline__ void slab_columns(const TcConvParams& p, uint32_t taddr, const SlabRows& sr, int n0, int c0, int c1,
                                             int lane, uint32_t stage, float4 (&res)[8], bool res_loaded, PendingSums& ps) {
    const bool vec4 = (p.KN & 3) == 0;
    const bool small_acc = p.Kw < (1 << 15);                               // |accumulator| <= 64 * Kw < 2^21: the bias conversion is exact
    const bool has_res = FUSED && p.residual != nullptr;
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
            if (sr.fast && has_res) {                                     // the residual need not be integer-valued: every term in double
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const double s4 = sr.mi[i] >= 0 ? ((double)fabsf(o[i].x) + (double)fabsf(o[i].y)) + ((double)fabsf(o[i].z) + (double)fabsf(o[i].w)) : 0.0;
                    if (4 * i + rsub < sr.split) dsum0 += s4; else dsum1 += s4;
                }
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
    (void)VHW;
}

// ---- the kernel ------------------------------------------------------------------------------------------------------------
// BRES: the filter block of the CTA (all taps, all channel pairs; needs KN <= TNI) is copied once and stays in shared
// memory; otherwise it streams through a ring of SB stages, one stage per tap and channel pair.
// UNIT: stride 1 in both directions (one plane; the tap loops are then flat, which matters because the MMA warp's
// instruction stream, not the tensor pipe, limits small tiles).
// Counters g (ring stages), q (patches) and a (accumulator buffers) run across tiles; barrier parities follow from them.
template <int MT, int TNI, int SB, bool BRES, bool FUSED, bool UNIT>
__global__ void __launch_bounds__(PTHREADS, 1)
conv_umma_persist_kernel(const __grid_constant__ CUtensorMap tmB, const TcConvParams p, int* __restrict__ status,
                         const int prow, const int nrows, const int nst, const int tiles_m, const int tiles_n) {
    constexpr int BSTAGE = TNI * IROW;
    constexpr int ACOLS = MT * TNI;                                        // columns of one accumulator buffer
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
    const uint32_t sStage = sbase + tail + 256;                            // [8 epilogue warps][4 KB]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int s1 = p.s1, s2 = p.s2;
    const int PA = p.PA, PB = p.PB, VW = p.VW;
    const int T = p.KH * p.KW, ncp = (p.PC + 1) >> 1;
    const int ntiles = tiles_m * tiles_n;

    if (tid == 0) {
        for (int s = 0; s < 16; s++) mbar_init(fullB + 8 * s, 1);          // fullB[8], emptyB[8]
        mbar_init(fullP, NXT); mbar_init(fullP + 8, NXT);                  // one arrival per expander thread
        mbar_init(emptyP, 1); mbar_init(emptyP + 8, 1);
        mbar_init(accFull, 1); mbar_init(accFull + 8, 1);
        mbar_init(accEmpty, 8); mbar_init(accEmpty + 8, 8);                // one arrival per epilogue warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tslot, (uint32_t)(2 * ACOLS));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic launch: the set-up above overlapped the tail of the previous kernel (the quantiser); from here on its
    // output is read.  The next kernel may be scheduled when every CTA has finished its tiles (not earlier: a grid
    // waiting in griddepcontrol.wait was measured to slow the MMA warp of the tiles still running).
    pdl_wait();

    // In every role the whole warp runs the loops and the waits and one elected lane issues the copies, MMAs and
    // commits.  All roles walk the same nest: tile, channel pair cp, plane (a, b), taps of that plane.
    if (warp == 0 || warp == 3 || warp >= 12) {
        // ---- expanders: up to two patches ahead of the MMAs (across tile boundaries).  The global loads of a patch are
        //      issued a whole patch earlier than they are used (they need registers, not the patch buffer), so that their
        //      latency - long when the epilogue's stores fill the memory system - is off the critical path. -----------------
        const int xt = (warp == 0 ? 0 : (warp == 3 ? 1 : warp - 10)) * 32 + lane;
        const int planes = PA * PB, step = (int)gridDim.x;
        PatchIter cur = {(int)blockIdx.x, 0, 0};
        RawItems raw;
        if (cur.t < ntiles) load_items<UNIT>(p, raw, (cur.t / tiles_n) * (UTM * MT), nrows, 0, 0, 0, 0, xt);
        unsigned q = 0;
        bool dead = false;
        while (cur.t < ntiles && !dead) {
            PatchIter nxt = cur;
            nxt.next(ncp, planes, step);
            RawItems ahead;
            const int npa = UNIT ? 0 : nxt.pl / PB;
            if (nxt.t < ntiles) load_items<UNIT>(p, ahead, (nxt.t / tiles_n) * (UTM * MT), nrows, nxt.cp, npa, UNIT ? 0 : nxt.pl - npa * PB, 0, xt);
            const unsigned pb = q & 1;
            if (q >= 2 && !mbar_wait_warp(emptyP + 8 * pb, ((q >> 1) - 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 11); break; }
            const uint32_t buf = sPatch + (uint32_t)(pb * prow) * IROW;
            store_items(p, raw, buf, nrows, cur.cp, 0, xt);
            const int items = nrows * ((2 * cur.cp + 1 < p.PC) ? 2 : 1);
            if (items > NXT * XUNROLL) {                                   // long patches (large halo): the rest, chunk by chunk
                const int R0 = (cur.t / tiles_n) * (UTM * MT);
                const int pa = UNIT ? 0 : cur.pl / PB;
                for (int base = NXT * XUNROLL; base < items; base += NXT * XUNROLL) {
                    RawItems more;
                    load_items<UNIT>(p, more, R0, nrows, cur.cp, pa, UNIT ? 0 : cur.pl - pa * PB, base, xt);
                    store_items(p, more, buf, nrows, cur.cp, base, xt);
                }
            }
            fence_async_smem();
            mbar_arrive(fullP + 8 * pb);
            raw = ahead;
            cur = nxt;
            q++;
        }
    } else if (warp == 2) {
        // ---- filter producer ---------------------------------------------------------------------------------------------
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
                    // same tap order as the MMA warp: plane by plane
                    for (int pa = 0; pa < PA && !dead; pa++)
                    for (int pbb = 0; pbb < PB && !dead; pbb++)
                    for (int kh = pa; kh < p.KH && !dead; kh += s1)
                    for (int kw = pbb; kw < p.KW; kw += s2, g++) {
                        const unsigned slot = g % SB;
                        if (g >= (unsigned)SB && !mbar_wait_warp(emptyB + 8 * slot, ((g / SB) - 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 12); break; }
                        if (elect_one()) {
                            mbar_expect_tx(fullB + 8 * slot, (uint32_t)BSTAGE);
                            tma_load_2d(sRing + slot * BSTAGE, &tmB, ((kh * p.KW + kw) * p.PC + 2 * cp) * 64, n0, fullB + 8 * slot);
                        }
                        __syncwarp();
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA warp --------------------------------------------------------------------------------------------------
        constexpr uint32_t IDESC = umma_idesc(TNI);
        constexpr uint32_t MB_UNITS = (UTM * IROW) >> 4;                   // next 128-row block of the patch, in 16-byte units
        unsigned g = 0, q = 0, a = 0;
        bool dead = false;
        if (BRES && !mbar_wait_warp(fullB, 0)) { dead = true; if (status && lane == 0) atomicExch(status, 15); }
        for (int t = blockIdx.x; t < ntiles && !dead; t += gridDim.x, a++) {
            const unsigned buf = a & 1;
            if (a >= 2 && !mbar_wait_warp(accEmpty + 8 * buf, ((a >> 1) - 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 13); break; }
            tc_fence_after();
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
                    if (!mbar_wait_warp(fullP + 8 * pb, (q >> 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 14); break; }
                    tc_fence_after();
                    uint32_t arow = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;   // descriptor address of the tap's first patch row
                    int kw = 0;
                    if (BRES) {
                        if (elect_one()) {                                 // nothing to wait for between taps: one issue burst
                            for (int tap = 0; tap < T; tap++) {
                                issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)UMMA_DESC_HI << 32) | ((sRing + (uint32_t)(cp * T + tap) * BSTAGE) >> 4), (cp > 0 || tap > 0) ? 1u : 0u);
                                if (++kw == p.KW) { kw = 0; arow += (uint32_t)VW * (IROW >> 4); }
                            }
                            umma_commit(emptyP + 8 * pb);
                            if (cp == ncp - 1) umma_commit(accFull + 8 * buf);
                        }
                        __syncwarp();
                    } else {
                        for (int tap = 0; tap < T; tap++, g++) {
                            const unsigned slot = g % SB;
                            if (!mbar_wait_warp(fullB + 8 * slot, (g / SB) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 15); break; }
                            tc_fence_after();
                            if (elect_one()) {
                                issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (arow + (uint32_t)kw * (IROW >> 4)),
                                          ((uint64_t)UMMA_DESC_HI << 32) | ((sRing + slot * BSTAGE) >> 4), (cp > 0 || tap > 0) ? 1u : 0u);
                                umma_commit(emptyB + 8 * slot);
                                if (tap == T - 1) {
                                    umma_commit(emptyP + 8 * pb);
                                    if (cp == ncp - 1) umma_commit(accFull + 8 * buf);
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
                    if (!mbar_wait_warp(fullP + 8 * pb, (q >> 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 14); break; }
                    tc_fence_after();
                    const uint32_t patch = (sPatch + (uint32_t)(pb * prow) * IROW) >> 4;    // descriptor address of the patch
                    const bool last_group = cp == ncp - 1 && pa == PA - 1 && pbb == PB - 1;
                    for (int kh = pa, ih = 0; kh < p.KH && !dead; kh += s1, ih++)
                    for (int kw = pbb, iw = 0; kw < p.KW; kw += s2, iw++) {
                        const bool last_tap = kh + s1 >= p.KH && kw + s2 >= p.KW;
                        uint32_t bsm;
                        if (BRES) bsm = sRing + (uint32_t)(cp * T + kh * p.KW + kw) * BSTAGE;
                        else {
                            const unsigned slot = g % SB;
                            if (!mbar_wait_warp(fullB + 8 * slot, (g / SB) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 15); break; }
                            tc_fence_after();
                            bsm = sRing + slot * BSTAGE;
                        }
                        if (elect_one()) {
                            issue_tap(((uint64_t)UMMA_DESC_HI << 32) | (patch + (uint32_t)(ih * VW + iw) * (IROW >> 4)),
                                      ((uint64_t)UMMA_DESC_HI << 32) | (bsm >> 4), accumulate);
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
    } else {
        // ---- epilogue warps 4-11 (TMEM lane quarter = warp % 4) -------------------------------------------------------
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
            slab_rows<FUSED>(p, R0 + emb * UTM + (warp & 3) * 32, lane, sr);
            float4 res[8];
            bool res_loaded = false;
            if (FUSED && p.residual != nullptr && (p.KN & 3) == 0 && n0 + ec0 + 32 <= p.KN) {
                slab_load_residual(p, sr, n0 + ec0, lane, res);
                res_loaded = true;
            }
            if (!mbar_wait_warp(accFull + 8 * buf, (a >> 1) & 1u)) { dead = true; if (status && lane == 0) atomicExch(status, 16); break; }
            tc_fence_after();
            slab_columns<FUSED>(p, tmem_base + buf * ACOLS + (uint32_t)(emb * TNI) + ((uint32_t)((warp & 3) * 32) << 16), sr, n0, ec0, ec1,
                                lane, sStage + (warp - 4) * 4096, res, res_loaded, pending);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(accEmpty + 8 * buf);
            if (FUSED) flush_pending(p, pending, lane);                    // the |y| atomics, off the buffer's critical path
        }
    }
    tc_fence_before();
    __syncthreads();
    pdl_launch_dependents();
    if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)(2 * ACOLS));
    if (FUSED) fused_finish(p);
}

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

// Reads (and clears) the record of expired waits on the current device; synchronises the device.
int umma_status_read_and_clear() {
    int v = -1, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int));
    return v;
}

// Virtual grid of a geometry (see TcConvParams).
static void set_virtual_grid(TcConvParams& p) {
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
}

// A tile shape with what it needs and what it is expected to cost.
struct TcPlan { int mt, tn, sb; bool resident; int prow, nrows, nst, smem; long long tiles_m, tiles_n; double cost; };

static bool plan_shape(const TcConvParams& p, int mt, int tn, int sb, int sms, bool has_res, TcPlan* out) {
    const long long halo = (long long)((p.KH - 1) / p.s1) * p.VW + (p.KW - 1) / p.s2;
    const long long nrows = 128LL * mt + halo, prow = (nrows + 7) / 8 * 8;
    const long long fixed = 2 * prow * IROW + 256 + 8 * 4096 + 1024;
    const long long T = (long long)p.KH * p.KW, ncp = (p.PC + 1) / 2;
    const long long nres = T * ncp;
    TcPlan pl;
    pl.mt = mt; pl.tn = tn; pl.sb = sb;
    pl.resident = p.KN <= tn && fixed + nres * tn * IROW <= UMMA_SMEM_MAX;
    const long long smem = pl.resident ? fixed + nres * tn * IROW : fixed + (long long)sb * tn * IROW;
    if (smem > UMMA_SMEM_MAX || (!pl.resident && T * ncp * p.PA * p.PB < 1)) return false;
    pl.prow = (int)prow; pl.nrows = (int)nrows; pl.nst = pl.resident ? (int)nres : sb; pl.smem = (int)smem;
    const long long Mv = (long long)(p.N - 1) * p.VH * p.VW + (long long)(p.OH - 1) * p.VW + p.OW;   // last useful virtual row + 1
    pl.tiles_m = (Mv + 128LL * mt - 1) / (128LL * mt);
    pl.tiles_n = (p.KN + tn - 1) / tn;
    if (pl.tiles_m * pl.tiles_n >= (1LL << 31)) return false;
    // Cost in SM cycles: rounds of tiles x the slowest of a tile's three pipelines (they overlap across tiles):
    // MMAs (128 x tn x 32 takes 48 / 64 / 128 cycles for tn = 64 / 128 / 256; a ring stage also costs the MMA warp a
    // handshake and moves tn*128 bytes of filters at about 64 B/clk), the epilogue (output and residual bytes at
    // about 24 B/clk per SM) and the expanders (about 1.5 cycles per byte of patch with four warps).
    const double mma_clk = tn == 64 ? 48.0 : (tn == 128 ? 64.0 : 128.0);
    const double words = (double)p.PC;                                      // K steps of 32 bytes per tap: 2 per word
    const double mma_tile = (double)T * words * 2.0 * mt * mma_clk;
    const double stage_over = pl.resident ? 0.0 : (double)T * (double)ncp * std::max(0.0, std::max(300.0 + 45.0 * 4 * mt, tn * 2.0) - 4.0 * mt * mma_clk);
    const double epi_tile = 128.0 * mt * std::min(tn, p.KN) * 4.0 * (has_res ? 2.0 : 1.0) / 24.0;
    const double exp_tile = (double)nrows * 64.0 * words * p.PA * p.PB * 1.5 / 64.0 * 1.0;
    const double tile = std::max(std::max(mma_tile + stage_over, epi_tile), exp_tile) + 600.0;
    const double rounds = (double)((pl.tiles_m * pl.tiles_n + sms - 1) / sms);
    pl.cost = rounds * tile + 4000.0;
    *out = pl;
    return true;
}

// Best tile for a problem; false = no shape fits (very wide images with many taps).
static bool tc_plan(const TcConvParams& p, int sms, bool has_res, TcPlan* best) {
    static const int cands[5][3] = {{2, 64, 6}, {1, 64, 6}, {2, 128, 4}, {1, 128, 6}, {1, 256, 4}};
    bool found = false;
    for (const auto& c : cands) {
        if (c[1] > 64 && c[1] / 2 >= p.KN) continue;                       // a tile twice as wide as the filter count only wastes
        TcPlan pl;
        if (!plan_shape(p, c[0], c[1], c[2], sms, has_res, &pl)) continue;
        if (!found || pl.cost < best->cost) { *best = pl; found = true; }
    }
    return found;
}

template <int MT, int TNI, int SB, bool BRES, bool FUSED, bool UNIT>
static int launch_persist_u(const CUtensorMap& tmB, const TcConvParams& p, const TcPlan& pl, int sms, int* status, cudaStream_t stream) {
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            e = cudaFuncSetAttribute(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, UNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, UMMA_SMEM_MAX);
            if (e != cudaSuccess) return record_cuda_error(e);
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    const long long ntiles = pl.tiles_m * pl.tiles_n;
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);
    return launch_pdl(conv_umma_persist_kernel<MT, TNI, SB, BRES, FUSED, UNIT>, dim3(grid), dim3(PTHREADS), (size_t)pl.smem, stream,
                      tmB, p, status, pl.prow, pl.nrows, pl.nst, (int)pl.tiles_m, (int)pl.tiles_n);
}

template <int MT, int TNI, int SB>
static int launch_persist(const CUtensorMap& tmB, const TcConvParams& p, const TcPlan& pl, int sms, int* status, cudaStream_t stream) {
    const bool fused = p.residual || p.abs_sums;
    const bool unit = p.s1 == 1 && p.s2 == 1;
#define TAB_LAUNCH(BR, FU, UN) return launch_persist_u<MT, TNI, SB, BR, FU, UN>(tmB, p, pl, sms, status, stream)
    if (pl.resident) {
        if (fused) { if (unit) TAB_LAUNCH(true, true, true); TAB_LAUNCH(true, true, false); }
        if (unit) TAB_LAUNCH(true, false, true);
        TAB_LAUNCH(true, false, false);
    }
    if (fused) { if (unit) TAB_LAUNCH(false, true, true); TAB_LAUNCH(false, true, false); }
    if (unit) TAB_LAUNCH(false, false, true);
    TAB_LAUNCH(false, false, false);
#undef TAB_LAUNCH
}

// Whether tc_conv_dispatch will take the problem, and - through kernel_name - which tile it would run.
static bool tc_prepare(TcConvParams& p, int sms, TcPlan* pl) {
    set_virtual_grid(p);
    const long long rows = (long long)p.N * p.VH * p.VW;
    if (rows >= (1LL << 31) - 65536 || (long long)p.N * p.H * p.W >= (1LL << 31) || (long long)p.M >= (1LL << 31) - 512) return false;
    if ((long long)p.KH * p.KW * p.PC >= (1LL << 20)) return false;
    p.dVHW = make_fastdiv((uint32_t)(p.VH * p.VW));
    p.dVW = make_fastdiv((uint32_t)p.VW);
    return tc_plan(p, sms, p.residual != nullptr, pl);
}

static thread_local char g_last_kernel[96] = "none";
const char* tc_last_kernel() { return g_last_kernel; }
void tc_forget_last_kernel() { snprintf(g_last_kernel, sizeof(g_last_kernel), "none"); }

// Whether tc_conv_dispatch will take the problem (asked before the quantiser is given the weight expansion to do).
bool tc_conv_covers(TcConvParams p) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    TcPlan pl;
    if (!encode_tiled_fn() || !tc_prepare(p, sms, &pl)) return false;
    return !((reinterpret_cast<uintptr_t>(p.w8) & 15) || (reinterpret_cast<uintptr_t>(p.qx) & (p.abits == 2 ? 15 : 7)));
}

// GEMM stage on the tensor cores.  TAB_E_TOO_LARGE when the shape is not covered (the caller falls back to the
// popcount kernel, which reads the same bit-planes).
int tc_conv_dispatch(TcConvParams p, cudaStream_t stream) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    TcPlan pl;
    if (!encode_tiled_fn() || !tc_prepare(p, sms, &pl)) return TAB_E_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(p.w8) & 15) || (reinterpret_cast<uintptr_t>(p.qx) & (p.abits == 2 ? 15 : 7))) return TAB_E_TOO_LARGE;
    alignas(64) CUtensorMap tmB;
    if (!make_map_2d(&tmB, p.w8, (unsigned long long)p.Kw * 64, (unsigned long long)p.KN, (unsigned)pl.tn)) return TAB_E_TOO_LARGE;
    int* status = umma_status_ptr();
    snprintf(g_last_kernel, sizeof(g_last_kernel), "conv_umma_persist_kernel<%d,%d,%d,%d,%d,%d>", pl.mt, pl.tn, pl.sb, (int)pl.resident,
             (int)(p.residual || p.abs_sums), (int)(p.s1 == 1 && p.s2 == 1));
    if (pl.tn == 64) return pl.mt == 2 ? launch_persist<2, 64, 6>(tmB, p, pl, sms, status, stream) : launch_persist<1, 64, 6>(tmB, p, pl, sms, status, stream);
    if (pl.tn == 128) return pl.mt == 2 ? launch_persist<2, 128, 4>(tmB, p, pl, sms, status, stream) : launch_persist<1, 128, 6>(tmB, p, pl, sms, status, stream);
    return launch_persist<1, 256, 4>(tmB, p, pl, sms, status, stream);
}

}  // namespace tab
