// TAB convolution on the integer tensor cores: quantised values {-1,0,+1} held as int8, implicit-im2col
// GEMM with s8 x s8 -> s32 MMA.  Bit-exact with the popcount formulation: every product is in {-1,0,1}
// and the int32 accumulation of at most KH*KW*C terms is exact, so y = sum a*w directly and none of the
// per-type corrections of the popcount kernels (TAB_GEMM.cu:25-147: "- 2*cnt", btn[kn], NUM) is needed.
//
// Why this path exists next to conv_sm100.cu: on B200 a 1-bit MMA is not native (mma.sync ... b1 and.popc
// is expanded by the compiler into byte operands + integer MMA: ncu shows 37 % IMMA pipe, 69 % ALU, 55 % LSU
// for a register-only loop, 423 TOP/s), the POPC unit issues 16 lanes/clk/SM (about 145-290 TOP/s for
// ternary data), while the s8 MMA sustains > 1100 TOP/s from registers.  Feeding the tensor cores with
// expanded bytes is therefore the faster exact route for all four types.
//
// Stages (all on the caller's stream, scratch in the caller's workspace):
//   1. quantize_int8_kernel   fp32 NHWC -> int8 NHWC with the channel dimension padded to a multiple of
//                             64 (pad bytes 0): replaces TerOnly/BinOnlyKernel (TAB_GEMM.cu:163-247) for
//                             this path; same compares, same thresholds.
//   2. expand_weights_kernel  packed QW [KN][KH*KW*PC][wb] -> int8 [KN][KH*KW*PC][64]; channel tails -> 0.
//   3. conv_imma_kernel       CTA tile TM pixels x TN filters, 4 warps, warp tile 64 x 64,
//                             mma.sync.m16n8k32.s8; K walked in chunks of two 64-channel words (128 B per
//                             row, XOR-swizzled so that ldmatrix is conflict-free), 2- or 3-stage cp.async ring;
//                             the loader does padding (zero fill for ternary activations, +1 fill for
//                             binary activations: a zero word means +1 there) and im2col by address.
#include "tab_kernels.cuh"
#include "conv_int8.cuh"

namespace tab {

// ------------------------------------------------------------------------------------------------
// 1. fp32 -> int8 {-1,0,+1}
// ------------------------------------------------------------------------------------------------
constexpr int Q8THREADS = 256;

__device__ __forceinline__ int q_ternary(float v, float t, float nt) { return v > t ? 1 : (v < nt ? -1 : 0); }
__device__ __forceinline__ int q_binary(float v, float t) { return v < t ? -1 : 1; }

// Four quantised values as the four bytes of a word.  `set` gives a compare as an all-ones/zero word in one instruction
// (false for NaN, like the reference's `>` and `<`), two byte permutes per pair of words gather the low bytes, so a word
// costs 8 compares + 6 permutes + 2 logic operations instead of a select, shift and OR per value.
// ternary = (pos & 0x01) | (neg & ~pos)  (the "+1" branch is tested first); binary = neg | 0x01 (flag -> 0xFF = -1, else +1).
// `valid` = number of real channels among the four (the rest are channel padding and must be 0).
__device__ __forceinline__ uint32_t cmp_mask_gt(float a, float b) {
    uint32_t d;
    asm("set.gt.u32.f32 %0, %1, %2;" : "=r"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ uint32_t cmp_mask_lt(float a, float b) {
    uint32_t d;
    asm("set.lt.u32.f32 %0, %1, %2;" : "=r"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ uint32_t low_bytes4(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
    return __byte_perm(__byte_perm(m0, m1, 0x0040), __byte_perm(m2, m3, 0x0040), 0x5410);
}
template <int BITS>
__device__ __forceinline__ uint32_t q_word(const float* v, float t, float nt, int valid) {
    uint32_t r;
    if (BITS == 2) {
        const uint32_t pos = low_bytes4(cmp_mask_gt(v[0], t), cmp_mask_gt(v[1], t), cmp_mask_gt(v[2], t), cmp_mask_gt(v[3], t));
        const uint32_t neg = low_bytes4(cmp_mask_lt(v[0], nt), cmp_mask_lt(v[1], nt), cmp_mask_lt(v[2], nt), cmp_mask_lt(v[3], nt));
        r = (pos & 0x01010101u) | (neg & ~pos);
    } else {
        r = low_bytes4(cmp_mask_lt(v[0], t), cmp_mask_lt(v[1], t), cmp_mask_lt(v[2], t), cmp_mask_lt(v[3], t)) | 0x01010101u;
    }
    if (valid < 4) r &= valid <= 0 ? 0u : (0xFFFFFFFFu >> (8 * (4 - valid)));
    return r;
}

// grid = (chunks, N); one thread per 16 consecutive channels of a pixel (one 16-byte store).
// groups_per_pixel = Cp/16; VEC: C % 16 == 0 and x 32-byte aligned -> two 256-bit loads per thread.
template <int BITS, bool VEC>
__global__ void __launch_bounds__(Q8THREADS)
quantize_int8_kernel(const float* __restrict__ x, const float* __restrict__ ths, int8_t* __restrict__ q,
                     long long pixels_per_image, int C, int Cp) {
    const int n = blockIdx.y;
    const float t = __ldg(ths + n), nt = -t;
    const int gpp = Cp >> 4;
    const long long groups = pixels_per_image * gpp;
    const float* xi = x + (long long)n * pixels_per_image * C;
    int8_t* qi = q + (long long)n * pixels_per_image * Cp;
    for (long long g = (long long)blockIdx.x * Q8THREADS + threadIdx.x; g < groups; g += (long long)gridDim.x * Q8THREADS) {
        const long long pix = g / gpp;
        const int c0 = (int)(g - pix * gpp) << 4;
        const float* src = xi + pix * C + c0;
        float v[16];
        if (VEC && c0 + 16 <= C) {
#pragma unroll
            for (int h = 0; h < 2; h++)
                asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                             : "=f"(v[8 * h + 0]), "=f"(v[8 * h + 1]), "=f"(v[8 * h + 2]), "=f"(v[8 * h + 3]),
                               "=f"(v[8 * h + 4]), "=f"(v[8 * h + 5]), "=f"(v[8 * h + 6]), "=f"(v[8 * h + 7])
                             : "l"(src + 8 * h));
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = (c0 + i < C) ? __ldg(src + i) : 0.f;
        }
        uint32_t o[4];
#pragma unroll
        for (int w = 0; w < 4; w++) {
            uint32_t r = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
                const int i = 4 * w + b;
                int qv = (BITS == 2) ? q_ternary(v[i], t, nt) : q_binary(v[i], t);
                if (c0 + i >= C) qv = 0;                       // channel padding carries no value
                r |= (uint32_t)(qv & 0xFF) << (8 * b);
            }
            o[w] = r;
        }
        *reinterpret_cast<uint4*>(qi + pix * Cp + c0) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Same quantiser writing the layout of the TMA-fed GEMM: the zero-padded (or +1-padded, for binary activations) image,
// split into the s1 x s2 "parity planes" a strided convolution reads:  [plane (a, b)][N][PH2][PW2][Cp], where plane
// pixel (i, j) is padded pixel (s1*i + a, s2*j + b) and only planes that hold a tap exist (a < A = min(s1, KH),
// b < B = min(s2, KW)).  Tap (kh, kw) of output (oh, ow) is then pixel (oh + kh/s1, ow + kw/s2) of plane
// (kh % s1, kw % s2): stride 1 inside every plane.  With stride 1 this is the padded image itself.  One thread per
// 16 channels of a plane pixel; border pixels get the padding value in the real channels, 0 in the channel padding.
struct QLayout { int p1, p2, s1, s2, A, B, PH2, PW2; };

// One thread per (filter, word k, 16-channel group) of the packed weights: 16 bytes of {-1,0,+1}.
template <int WB>
__device__ __forceinline__ void expand_group(const uint64_t* __restrict__ qw, int8_t* __restrict__ w8, long long idx, int PC, int C) {
    const long long word = idx >> 2;
    const int grp = (int)(idx & 3);
    const int pc = (int)(word % PC);
    const int cbase = pc * 64 + grp * 16;
    uint32_t s16, m16;
    if (WB == 2) {
        s16 = (uint32_t)(qw[word * 2] >> (grp * 16)) & 0xFFFFu;
        m16 = (uint32_t)(qw[word * 2 + 1] >> (grp * 16)) & 0xFFFFu;
    } else {
        s16 = (uint32_t)(qw[word] >> (grp * 16)) & 0xFFFFu;     // bit = 1 means -1
        m16 = 0xFFFFu;
    }
    uint32_t o[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        uint32_t r = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int i = 4 * w + b;
            int v = ((m16 >> i) & 1u) ? (((s16 >> i) & 1u) ? -1 : 1) : 0;
            if (cbase + i >= C) v = 0;
            r |= (uint32_t)(v & 0xFF) << (8 * b);
        }
        o[w] = r;
    }
    *reinterpret_cast<uint4*>(w8 + word * 64 + grp * 16) = make_uint4(o[0], o[1], o[2], o[3]);
}

// Inside a convolution call the same launch also does the call's small set-up jobs, so that they cost no launch of
// their own: all CTAs share the expansion of the packed weights to bytes, and the first CTA of every image clears
// that image's |y| sum (and the first of all the completion counter) for the GEMM's epilogue.
struct PrepExtras {
    int images;                  // grid rows (= images)
    double* zero_sums;           // [images] or null
    unsigned* zero_counter;      // or null
    const uint64_t* qw;          // packed weights, or null
    int8_t* w8;
    long long words;             // KN*KH*KW*PC
    int wbits;
};

template <int BITS, bool VEC>
__global__ void __launch_bounds__(Q8THREADS, 8)
quantize_int8_padded_kernel(const float* __restrict__ x, const float* __restrict__ ths, int8_t* __restrict__ q,
                            int H, int W, int C, int Cp, const QLayout L, const PrepExtras ex) {
    const int n = blockIdx.y;
    // Programmatic launch: nothing is read or written before the previous kernel of the stream (the GEMM that produced
    // x and the thresholds, and that may still be reading the scratch this launch overwrites) has completed; the next
    // kernel may be scheduled once every CTA of this one is done (a waiting grid polls, so it is not let in earlier).
    pdl_wait();
    if (ex.qw != nullptr) {                                                // the weights, spread over all CTAs of the launch
        const int PC = Cp >> 6;
        const long long stride = (long long)gridDim.x * gridDim.y * Q8THREADS;
        for (long long idx = ((long long)blockIdx.y * gridDim.x + blockIdx.x) * Q8THREADS + threadIdx.x; idx < ex.words * 4; idx += stride) {
            if (ex.wbits == 2) expand_group<2>(ex.qw, ex.w8, idx, PC, C);
            else expand_group<1>(ex.qw, ex.w8, idx, PC, C);
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (ex.zero_sums) ex.zero_sums[n] = 0.0;
        if (n == 0 && ex.zero_counter) *ex.zero_counter = 0u;
    }
    const float t = __ldg(ths + n), nt = -t;
    const int gpp = Cp >> 4;
    const long long plane_pix = (long long)L.PH2 * L.PW2;
    const long long groups = (long long)L.A * L.B * plane_pix * gpp;
    const float* xi = x + (long long)n * H * W * C;
    const long long plane_stride = (long long)gridDim.y * plane_pix;      // pixels of one plane over all images
    const bool small = groups < (1LL << 31);                               // 32-bit index arithmetic (always, in practice)
    const bool one_plane = L.A * L.B == 1;
    for (long long g = (long long)blockIdx.x * Q8THREADS + threadIdx.x; g < groups; g += (long long)gridDim.x * Q8THREADS) {
        int c0, plane, i, j;
        long long pix;
        if (small) {
            const unsigned ug = (unsigned)g, upix = ug / (unsigned)gpp;
            c0 = (int)(ug - upix * (unsigned)gpp) << 4;
            const unsigned upl = one_plane ? 0u : upix / (unsigned)plane_pix;
            const unsigned up = upix - upl * (unsigned)plane_pix;
            plane = (int)upl;
            i = (int)(up / (unsigned)L.PW2);
            j = (int)(up - (unsigned)i * (unsigned)L.PW2);
            pix = up;
        } else {
            const long long pixall = g / gpp;
            c0 = (int)(g - pixall * gpp) << 4;
            plane = (int)(pixall / plane_pix);
            pix = pixall - plane * plane_pix;
            i = (int)(pix / L.PW2);
            j = (int)(pix - (long long)i * L.PW2);
        }
        const int pa = plane / L.B, pb = plane - pa * L.B;
        const int ih = L.s1 * i + pa - L.p1, iw = L.s2 * j + pb - L.p2;
        int8_t* qi = q + (plane * plane_stride + (long long)n * plane_pix) * Cp;
        uint32_t o[4];
        if ((unsigned)ih < (unsigned)H && (unsigned)iw < (unsigned)W) {
            const float* src = xi + ((long long)ih * W + iw) * C + c0;
            float v[16];
            if (VEC && c0 + 16 <= C) {
#pragma unroll
                for (int h = 0; h < 2; h++)
                    asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=f"(v[8 * h + 0]), "=f"(v[8 * h + 1]), "=f"(v[8 * h + 2]), "=f"(v[8 * h + 3]),
                                   "=f"(v[8 * h + 4]), "=f"(v[8 * h + 5]), "=f"(v[8 * h + 6]), "=f"(v[8 * h + 7])
                                 : "l"(src + 8 * h));
            } else {
#pragma unroll
                for (int e = 0; e < 16; e++) v[e] = (c0 + e < C) ? __ldg(src + e) : 0.f;
            }
            if (VEC && c0 + 16 <= C) {
#pragma unroll
                for (int w = 0; w < 4; w++) o[w] = q_word<BITS>(v + 4 * w, t, nt, 4);
            } else {
#pragma unroll
                for (int w = 0; w < 4; w++) o[w] = q_word<BITS>(v + 4 * w, t, nt, C - c0 - 4 * w);
            }
        } else {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t r = 0;
#pragma unroll
                for (int b = 0; b < 4; b++)
                    if (BITS == 1 && c0 + 4 * w + b < C) r |= 1u << (8 * b);     // binary activations pad with +1
                o[w] = r;
            }
        }
        *reinterpret_cast<uint4*>(qi + pix * Cp + c0) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// 2. packed weights -> int8
// ------------------------------------------------------------------------------------------------
// One thread per (filter, word k, 16-channel group).  words = KN*Kw.
template <int WB>
__global__ void expand_weights_kernel(const uint64_t* __restrict__ qw, int8_t* __restrict__ w8,
                                      long long words, int PC, int C) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= words * 4) return;
    expand_group<WB>(qw, w8, idx, PC, C);
}

// ------------------------------------------------------------------------------------------------
// 3. implicit-im2col s8 GEMM
// ------------------------------------------------------------------------------------------------
constexpr int ITHREADS = 128;                // 4 warps, each a 64 x 64 output tile
constexpr int PATCH_SMEM_BUDGET = 110 * 1024; // dynamic shared memory of the patch variant: two CTAs per SM

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void imma(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}


// Epilogue shared by the GEMM kernels: int32 -> float32, [M][KN].
// FUSED adds the residual and accumulates sum |y| per image: a warp's 64 rows touch at most three
// images when an image has >= 32 output pixels, so each lane keeps three partial sums, the warp
// reduces them with shuffles and lane 0 issues at most three double atomics; smaller images fall
// back to one atomic per row.
template <bool FUSED>
__device__ __forceinline__ void imma_epilogue(const ImmaParams& p, const int (&acc)[4][8][4], int m0, int n0,
                                              int wm, int wn, int lane) {
    const int g = lane >> 2, t4 = lane & 3;
    const bool pair_ok = (p.KN & 1) == 0;
    const int ohw = p.OH * p.OW;
    const int wrow0 = m0 + wm * 64;
    const int wimg0 = FUSED ? wrow0 / ohw : 0;
    const bool few = ohw >= 32;
    const int wb1 = (wimg0 + 1) * ohw, wb2 = wb1 + ohw;          // first rows of the warp's 2nd and 3rd image
    float part[3] = {0.f, 0.f, 0.f};                             // per lane: <= 8 rows x 16 values, exact in fp32 for integer data
#pragma unroll
    for (int mi = 0; mi < 4; mi++) {
#pragma unroll
        for (int hrow = 0; hrow < 2; hrow++) {
            const int m = wrow0 + mi * 16 + g + hrow * 8;
            if (m >= p.M) continue;
            float* __restrict__ yrow = p.y + (long long)m * p.KN;
            const float* __restrict__ rrow = (FUSED && p.residual) ? p.residual + (long long)m * p.KN : nullptr;
            // all residual loads of the row first (they must not wait behind the stores)
            float2 res[8];
#pragma unroll
            for (int ni = 0; ni < 8; ni++) {
                const int n = n0 + wn * 64 + ni * 8 + 2 * t4;
                res[ni] = make_float2(0.f, 0.f);
                if (FUSED && rrow) {
                    if (pair_ok && n + 1 < p.KN) res[ni] = __ldg(reinterpret_cast<const float2*>(rrow + n));
                    else {
                        if (n < p.KN) res[ni].x = __ldg(rrow + n);
                        if (n + 1 < p.KN) res[ni].y = __ldg(rrow + n + 1);
                    }
                }
            }
            float rsum = 0.f;
#pragma unroll
            for (int ni = 0; ni < 8; ni++) {
                const int n = n0 + wn * 64 + ni * 8 + 2 * t4;
                const float v0 = (float)acc[mi][ni][2 * hrow] + res[ni].x, v1 = (float)acc[mi][ni][2 * hrow + 1] + res[ni].y;
                if (pair_ok && n + 1 < p.KN) {
                    *reinterpret_cast<float2*>(yrow + n) = make_float2(v0, v1);
                    if (FUSED) rsum += fabsf(v0) + fabsf(v1);
                } else {
                    if (n < p.KN) { yrow[n] = v0; if (FUSED) rsum += fabsf(v0); }
                    if (n + 1 < p.KN) { yrow[n + 1] = v1; if (FUSED) rsum += fabsf(v1); }
                }
            }
            if (FUSED && p.abs_sums) {
                if (few) {
                    const int d = (m >= wb1) + (m >= wb2);
                    part[0] += d == 0 ? rsum : 0.f;
                    part[1] += d == 1 ? rsum : 0.f;
                    part[2] += d == 2 ? rsum : 0.f;
                } else {
                    atomicAdd(p.abs_sums + m / ohw, (double)rsum);
                }
            }
        }
    }
    if (FUSED && p.abs_sums && few) {
#pragma unroll
        for (int i = 0; i < 3; i++) {
            double d = (double)part[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
            if (lane == 0 && d != 0.0 && wimg0 + i < p.N) atomicAdd(p.abs_sums + wimg0 + i, d);
        }
    }
}

// WM x WN warps (WM*WN == 4); CTA tile (64*WM) x (64*WN).  PADONE: out-of-image taps hold +1 (binary
// activations) instead of 0.
//
// Loader: a 64-byte row-word is copied by four consecutive lanes (16 bytes each), so a warp reads eight
// fully used 64-byte segments per cp.async instruction.  Each thread owns one (word-in-chunk, 16-byte unit)
// pair and walks the rows r = tid/8 + 16 e; the per-row geometry (first tap's input coordinates and the
// image offset) sits in shared memory, written once per CTA.
template <int WM, int WN, int ISTAGES, bool PADONE, bool FUSED>
__global__ void __launch_bounds__(ITHREADS, 2)
conv_imma_kernel(const ImmaParams p) {
    constexpr int TMI = 64 * WM, TNI = 64 * WN;
    constexpr int STAGE = (TMI + TNI) * IROW;
    constexpr int RING = ISTAGES * STAGE;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    int4* rowinfo = reinterpret_cast<int4*>(smem + RING);        // {first-tap pixel index, tap mask lo, hi, row valid}

    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * TMI;
    const int n0 = blockIdx.y * TNI;
    const int Cp = p.PC * 64;

    // Per output pixel: pixel index of its first tap (may be negative: it is only used when the tap's bit
    // in the validity mask is set) and a 64-bit mask with bit kh*KW+kw = "that tap lies inside the image".
    for (int r = tid; r < TMI; r += ITHREADS) {
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
    __syncthreads();

    // ---- loader state: this thread copies unit l_q of word l_wi of every chunk ----------------------------
    const int l_unit = tid & 7, l_wi = l_unit >> 2, l_q = l_unit & 3;
    const int l_row0 = tid >> 3;                                 // rows l_row0 + 16 e
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
#pragma unroll 4
        for (int e = 0; e < TMI / 16; e++) {
            const int row = l_row0 + 16 * e;
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
#pragma unroll 4
        for (int e = 0; e < TNI / 16; e++) {
            const int row = l_row0 + 16 * e;
            const bool v = kvalid && (n0 + row) < p.KN;
            const int8_t* src = v ? bbase + (long long)row * p.Kw * 64 : p.w8;
            cp16(sB + swz(row, l_unit), src, v);
        }
        l_k += IKW;
        l_pc += IKW;
        while (l_pc >= p.PC) { l_pc -= p.PC; if (++l_kw == p.KW) { l_kw = 0; ++l_kh; } }
        asm volatile("cp.async.commit_group;");
    };

    // ---- compute mapping ----------------------------------------------------------------------------
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = warp % WM, wn = warp / WM;
    // ldmatrix row/unit of this lane inside a 16-row (A) or 16-column (B) block
    const int a_lrow = (lane & 7) + ((lane >> 3) & 1) * 8, a_lu = lane >> 4;
    const int b_lrow = (lane & 7) + (lane >> 4) * 8, b_lu = (lane >> 3) & 1;
    // row * IROW and (row & 7) are the same for every k-step: keep them, the unit index changes
    uint32_t a_rowoff[4], b_rowoff[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        a_rowoff[i] = (uint32_t)((wm * 64 + i * 16 + a_lrow) * IROW);
        b_rowoff[i] = (uint32_t)(TMI * IROW + (wn * 64 + i * 16 + b_lrow) * IROW);
    }
    const int a_x = a_lrow & 7, b_x = b_lrow & 7;               // (row & 7): 16-row blocks start at multiples of 16

    int acc[4][8][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0;

    uint32_t af[2][4][4], bf[2][8][2];
    auto load_frags = [&](uint32_t sA, int j, int buf) {
#pragma unroll
        for (int mi = 0; mi < 4; mi++)
            ldsm4(sA + a_rowoff[mi] + (((2 * j + a_lu) ^ a_x) << 4), af[buf][mi][0], af[buf][mi][1], af[buf][mi][2], af[buf][mi][3]);
#pragma unroll
        for (int nj = 0; nj < 4; nj++)
            ldsm4(sA + b_rowoff[nj] + (((2 * j + b_lu) ^ b_x) << 4), bf[buf][2 * nj][0], bf[buf][2 * nj][1],
                  bf[buf][2 * nj + 1][0], bf[buf][2 * nj + 1][1]);
    };

    const int nchunks = (p.Kw + IKW - 1) / IKW;
#pragma unroll
    for (int s = 0; s < ISTAGES - 1; s++) {
        if (s < nchunks) load_chunk(s); else asm volatile("cp.async.commit_group;");
    }
    for (int c = 0; c < nchunks; c++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(ISTAGES - 2));
        __syncthreads();
        const uint32_t sA = sbase + (c % ISTAGES) * STAGE;
        load_frags(sA, 0, 0);
        if (c + ISTAGES - 1 < nchunks) load_chunk((c + ISTAGES - 1) % ISTAGES); else asm volatile("cp.async.commit_group;");
#pragma unroll
        for (int j = 0; j < IROW / 32; j++) {                   // k32 steps inside the chunk
            if (j + 1 < IROW / 32) load_frags(sA, j + 1, (j + 1) & 1);   // next step's fragments first
#pragma unroll
            for (int mi = 0; mi < 4; mi++)
#pragma unroll
                for (int ni = 0; ni < 8; ni++) imma(acc[mi][ni], af[j & 1][mi], bf[j & 1][ni][0], bf[j & 1][ni][1]);
        }
    }
    asm volatile("cp.async.wait_group 0;");

    imma_epilogue<FUSED>(p, acc, m0, n0, wm, wn, lane);
    if (FUSED) fused_finish(p);
}

// ------------------------------------------------------------------------------------------------
// Patch variant: the A operand is not staged as an im2col tile (which copies every input pixel once
// per tap) but as the patch of input pixels the CTA's output rows touch, one 64-byte row per pixel and
// per 64-channel word; ldmatrix gathers the im2col rows from it by address.  For a 3x3 kernel this cuts
// the activation copies (and the loader's instructions, which dominated the im2col variant) about 6x.
//
// Pixels are indexed on the zero-padded input grid, L = (n*PH + ph)*PW + pw.  Output row m with first tap
// L0(m) = (n*PH + oh*s1)*PW + ow*s2 reads tap (kh,kw) at L0(m) + kh*PW + kw, so the patch of a tile is the
// contiguous range [L0(first row), L0(last row) + (KH-1)*PW + KW-1]; padding pixels are filled with 0
// (or +1 for binary activations).  K order: 64-channel word (outer), tap (inner); two taps per ring
// stage of B.  pmax = largest patch over all tiles (computed on the host).
template <int WM, int WN, bool PADONE, bool FUSED>
__global__ void __launch_bounds__(ITHREADS, 2)
conv_imma_patch_kernel(const ImmaParams p, const int pmax) {
    constexpr int TMI = 64 * WM, TNI = 64 * WN, ISTAGES = 3;
    constexpr int BSTAGE = TNI * IROW;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t sPatch = sbase + ISTAGES * BSTAGE;            // [2][pmax][64 B]
    int* patch_src = reinterpret_cast<int*>(smem + ISTAGES * BSTAGE + 2 * pmax * 64);   // [pmax]

    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * TMI;
    const int n0 = blockIdx.y * TNI;
    const int Cp = p.PC * 64;
    const int PH = p.H + 2 * p.p1, PW = p.W + 2 * p.p2;
    const int ohw = p.OH * p.OW;
    const int T = p.KH * p.KW, CT = (T + 1) >> 1;                // taps, ring stages per channel word

    auto first_tap = [&](int m) {
        const int n = m / ohw;
        const int r = m - n * ohw;
        const int oh = r / p.OW;
        const int ow = r - oh * p.OW;
        return (n * PH + oh * p.s1) * PW + ow * p.s2;
    };
    const int m_last = min(m0 + TMI, p.M) - 1;
    const int Lmin = first_tap(m0);
    const int P = min(first_tap(m_last) + (p.KH - 1) * PW + p.KW - Lmin, pmax);

    // source pixel (index into [N][H][W]) of every patch pixel, -1 for padding
    for (int i = tid; i < P; i += ITHREADS) {
        const int L = Lmin + i;
        const int n = L / (PH * PW);
        const int r = L - n * PH * PW;
        const int ph = r / PW;
        const int pw = r - ph * PW;
        const int ih = ph - p.p1, iw = pw - p.p2;
        const bool inside = ((unsigned)ih < (unsigned)p.H) && ((unsigned)iw < (unsigned)p.W) && n < p.N;
        patch_src[i] = inside ? (n * p.H + ih) * p.W + iw : -1;
    }
    __syncthreads();

    // ---- loaders ----------------------------------------------------------------------------------------
    const int l_unit = tid & 7, l_wi = l_unit >> 2, l_q = l_unit & 3, l_row0 = tid >> 3;
    auto load_b = [&](int c, int stage) {                        // ring stage: taps 2ct, 2ct+1 of word cc
        const int cc = c / CT, ct = c - cc * CT;
        const int tap = 2 * ct + l_wi;
        const bool kvalid = tap < T;
        const uint32_t sB = sbase + stage * BSTAGE;
        const int8_t* bbase = p.w8 + ((long long)n0 * p.Kw + (long long)tap * p.PC + cc) * 64 + l_q * 16;
#pragma unroll 4
        for (int e = 0; e < TNI / 16; e++) {
            const int row = l_row0 + 16 * e;
            const bool v = kvalid && (n0 + row) < p.KN;
            const int8_t* src = v ? bbase + (long long)row * p.Kw * 64 : p.w8;
            cp16(sB + swz(row, l_unit), src, v);
        }
    };
    auto load_patch = [&](int cc) {                              // all pixels of the patch, 64-channel word cc
        const uint32_t buf = sPatch + (cc & 1) * pmax * 64;
        const int8_t* abase = p.qx + (long long)cc * 64 + (tid & 3) * 16;
        for (int i = tid; i < P * 4; i += ITHREADS) {
            const int pix = i >> 2;
            const int sp = patch_src[pix];
            const uint32_t dst = buf + pix * 64 + ((((tid & 3) ^ (pix >> 1)) & 3) << 4);
            if (PADONE && sp < 0) sts16(dst, 0x01010101u);
            else cp16(dst, sp >= 0 ? abase + (long long)sp * Cp : p.qx, sp >= 0);
        }
    };

    // ---- compute mapping ----------------------------------------------------------------------------------
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = warp % WM, wn = warp / WM;
    const int a_lrow = (lane & 7) + ((lane >> 3) & 1) * 8, a_lu = lane >> 4;
    const int b_lrow = (lane & 7) + (lane >> 4) * 8, b_lu = (lane >> 3) & 1;
    int a_rel[4];                                                // patch index of this lane's ldmatrix rows, tap (0,0)
    uint32_t b_rowoff[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + wm * 64 + i * 16 + a_lrow;
        a_rel[i] = (m < p.M) ? first_tap(m) - Lmin : 0;
        b_rowoff[i] = (uint32_t)((wn * 64 + i * 16 + b_lrow) * IROW);
    }
    const int b_x = b_lrow & 7;

    int acc[4][8][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0;

    uint32_t af[2][4][4], bf[2][8][2];
    // fragments of k32 step j (0..3) of a stage: tap = first tap of the stage + j/2, half j%2 of the 64-byte word
    auto load_frags = [&](uint32_t sB, uint32_t pbuf, int toff0, int toff1, int j, int buf) {
        const int toff = (j >> 1) ? toff1 : toff0;
#pragma unroll
        for (int mi = 0; mi < 4; mi++) {
            const int pix = a_rel[mi] + toff;
            const uint32_t addr = pbuf + pix * 64 + ((((2 * (j & 1) + a_lu) ^ (pix >> 1)) & 3) << 4);
            ldsm4(addr, af[buf][mi][0], af[buf][mi][1], af[buf][mi][2], af[buf][mi][3]);
        }
#pragma unroll
        for (int nj = 0; nj < 4; nj++)
            ldsm4(sB + b_rowoff[nj] + (((2 * j + b_lu) ^ b_x) << 4), bf[buf][2 * nj][0], bf[buf][2 * nj][1],
                  bf[buf][2 * nj + 1][0], bf[buf][2 * nj + 1][1]);
    };

    const int nchunks = p.PC * CT;
#pragma unroll
    for (int s = 0; s < ISTAGES - 1; s++) {
        if (s < nchunks) {
            if (s % CT == 0) load_patch(s / CT);                 // CT >= 2: only s == 0 here
            load_b(s, s);
        }
        asm volatile("cp.async.commit_group;");
    }
    for (int c = 0; c < nchunks; c++) {
        asm volatile("cp.async.wait_group %0;" ::"n"(ISTAGES - 2));
        __syncthreads();
        const int cc = c / CT, ct = c - cc * CT;
        const uint32_t sB = sbase + (c % ISTAGES) * BSTAGE;
        const uint32_t pbuf = sPatch + (cc & 1) * pmax * 64;
        const int tap0 = 2 * ct, tap1 = min(2 * ct + 1, T - 1);
        const int kh0 = tap0 / p.KW, kh1 = tap1 / p.KW;
        const int toff0 = kh0 * PW + (tap0 - kh0 * p.KW), toff1 = kh1 * PW + (tap1 - kh1 * p.KW);
        const int nsteps = (2 * ct + 1 < T) ? 4 : 2;              // an odd tap count leaves the last stage half empty
        load_frags(sB, pbuf, toff0, toff1, 0, 0);
        {
            const int cn = c + ISTAGES - 1;
            if (cn < nchunks) {
                if (cn % CT == 0) load_patch(cn / CT);
                load_b(cn, cn % ISTAGES);
            }
            asm volatile("cp.async.commit_group;");
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (j < nsteps) {
                if (j + 1 < nsteps) load_frags(sB, pbuf, toff0, toff1, j + 1, (j + 1) & 1);
#pragma unroll
                for (int mi = 0; mi < 4; mi++)
#pragma unroll
                    for (int ni = 0; ni < 8; ni++) imma(acc[mi][ni], af[j & 1][mi], bf[j & 1][ni][0], bf[j & 1][ni][1]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;");
    imma_epilogue<FUSED>(p, acc, m0, n0, wm, wn, lane);
    if (FUSED) fused_finish(p);
}

// Largest patch (in pixels) over all tiles of TMI output rows; 0 when pixel indices would not fit an int.
static int patch_pixels_max(int TMI, int N, int H, int W, int OH, int OW, int KH, int KW, int p1, int p2, int s1, int s2) {
    const long long PH = H + 2LL * p1, PW = W + 2LL * p2;
    if ((long long)N * PH * PW >= (1LL << 31)) return 0;
    const long long M = (long long)N * OH * OW, ohw = (long long)OH * OW;
    auto first_tap = [&](long long m) {
        const long long n = m / ohw, r = m - n * ohw, oh = r / OW, ow = r - oh * OW;
        return (n * PH + oh * s1) * PW + ow * s2;
    };
    // the pattern of tile starts repeats with period lcm(TMI, ohw) rows: scanning one period is exact
    long long period = ohw;
    {
        long long a = TMI, b = ohw;
        while (b) { const long long t = a % b; a = b; b = t; }
        period = (long long)TMI / a * ohw;
    }
    const long long scan = period < M ? period : M;
    long long best = 0;
    for (long long m0 = 0; m0 < scan; m0 += TMI) {
        const long long ml = (m0 + TMI < M ? m0 + TMI : M) - 1;
        const long long P = first_tap(ml) + (KH - 1) * PW + KW - first_tap(m0);
        if (P > best) best = P;
    }
    // the last (partial) tile of the whole problem is never larger than a full one starting at the same row
    return best < (1LL << 24) ? (int)best : 0;
}

template <int WM, int WN, bool PADONE, bool FUSED>
static int launch_patch_f(const ImmaParams& p, int pmax, cudaStream_t stream) {
    constexpr int TMI = 64 * WM, TNI = 64 * WN;
    const int smem_bytes = 3 * TNI * IROW + 2 * pmax * 64 + pmax * 4;
    static int configured[64] = {};                               // largest size configured so far, per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || configured[dev] < smem_bytes) {
        e = cudaFuncSetAttribute(conv_imma_patch_kernel<WM, WN, PADONE, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, PATCH_SMEM_BUDGET);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = PATCH_SMEM_BUDGET;
    }
    dim3 grid((unsigned)((p.M + TMI - 1) / TMI), (unsigned)((p.KN + TNI - 1) / TNI));
    conv_imma_patch_kernel<WM, WN, PADONE, FUSED><<<grid, ITHREADS, smem_bytes, stream>>>(p, pmax);
    return check_launch();
}

template <int WM, int WN, bool PADONE>
static int launch_patch(const ImmaParams& p, int pmax, cudaStream_t stream) {
    return (p.residual || p.abs_sums) ? launch_patch_f<WM, WN, PADONE, true>(p, pmax, stream)
                                      : launch_patch_f<WM, WN, PADONE, false>(p, pmax, stream);
}

template <int WM, int WN, int ISTAGES, bool PADONE, bool FUSED>
static int launch_imma_f(const ImmaParams& p, cudaStream_t stream) {
    constexpr int TMI = 64 * WM, TNI = 64 * WN;
    constexpr int smem_bytes = ISTAGES * (TMI + TNI) * IROW + TMI * 16;
    // once per device and instantiation (kept out of the steady-state launch path, e.g. stream capture)
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(conv_imma_kernel<WM, WN, ISTAGES, PADONE, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return record_cuda_error(e);
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid((unsigned)((p.M + TMI - 1) / TMI), (unsigned)((p.KN + TNI - 1) / TNI));
    conv_imma_kernel<WM, WN, ISTAGES, PADONE, FUSED><<<grid, ITHREADS, smem_bytes, stream>>>(p);
    return check_launch();
}

template <int WM, int WN, int ISTAGES, bool PADONE>
static int launch_imma(const ImmaParams& p, cudaStream_t stream) {
    return (p.residual || p.abs_sums) ? launch_imma_f<WM, WN, ISTAGES, PADONE, true>(p, stream)
                                      : launch_imma_f<WM, WN, ISTAGES, PADONE, false>(p, stream);
}

int conv_umma_dispatch(const ImmaParams& p, bool padone, int alt, cudaStream_t stream);
int conv_tma_dispatch(const ImmaParams& p, int mode, cudaStream_t stream);
bool conv_tma_persist_fits(const ImmaParams& p);

// 0 = default choice, 1 = mma.sync with im2col staging, 2 = mma.sync (patch or im2col), 3 = tcgen05 (for A/B tests)
static int g_imma_variant = 0;
static const bool g_tma_default = true;   // persistent TMA-fed kernel where it applies (measured ahead of the others)

// Pixels per image of the activation scratch: the padded image, or its parity planes (rounded up per plane).
static size_t scratch_pixels(int H, int W, int KH, int KW, int p1, int p2, int s1, int s2) {
    const size_t padded = (H + 2 * (size_t)p1) * (W + 2 * (size_t)p2);
    const size_t A = s1 < KH ? s1 : KH, B = s2 < KW ? s2 : KW;
    const size_t planes = A * B * ((H + 2 * (size_t)p1 + s1 - 1) / s1) * ((W + 2 * (size_t)p2 + s2 - 1) / s2);
    return padded > planes ? padded : planes;
}

size_t imma_workspace_bytes(int N, int H, int W, int C, int KN, int KH, int KW, int p1, int p2, int s1, int s2) {
    const size_t Cp = (size_t)packed_channels(C) * 64;
    const size_t a = ((size_t)N * scratch_pixels(H, W, KH, KW, p1, p2, s1, s2) * Cp + 255) / 256 * 256;
    const size_t b = ((size_t)KN * KH * KW * Cp + 255) / 256 * 256;
    return a + b + 256;                          // + completion counter of the fused tail
}

static int imma_limits(int N, int H, int W, int C, int KN, int KH, int KW, long long oh, long long ow) {
    const long long M = (long long)N * oh * ow, Kw = (long long)KH * KW * packed_channels(C);
    if (M >= (1LL << 31) - 512 || Kw >= (1LL << 24) || (long long)N * H * W >= (1LL << 31) ||
        (KN + 63) / 64 > 65535 || N > 65535 || KH * KW > 64)
        return TAB_E_TOO_LARGE;
    return TAB_OK;
}

int quantize_int8_dispatch(const float* x, const float* ths, int8_t* qx8, int bits, int N, int H, int W, int C,
                           cudaStream_t stream) {
    const int Cp = packed_channels(C) * 64;
    const long long pixels = (long long)H * W;
    if (N == 0 || pixels == 0) return TAB_OK;
    if (N > 65535) return TAB_E_TOO_LARGE;
    const long long groups = pixels * (Cp / 16);
    long long per = (groups + Q8THREADS - 1) / Q8THREADS;
    const long long cap = (148LL * 8 * 4 + N - 1) / N;
    if (per > cap) per = cap;
    if (per < 1) per = 1;
    dim3 grid((unsigned)per, (unsigned)N);
    const bool vec = (C % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 31) == 0) && ((pixels * C) % 8 == 0);
    if (bits == 2) {
        if (vec) quantize_int8_kernel<2, true><<<grid, Q8THREADS, 0, stream>>>(x, ths, qx8, pixels, C, Cp);
        else quantize_int8_kernel<2, false><<<grid, Q8THREADS, 0, stream>>>(x, ths, qx8, pixels, C, Cp);
    } else {
        if (vec) quantize_int8_kernel<1, true><<<grid, Q8THREADS, 0, stream>>>(x, ths, qx8, pixels, C, Cp);
        else quantize_int8_kernel<1, false><<<grid, Q8THREADS, 0, stream>>>(x, ths, qx8, pixels, C, Cp);
    }
    return check_launch();
}

int expand_weights_dispatch(const int64_t* qw, int8_t* w8, int wbits, int KN, int KH, int KW, int C, cudaStream_t stream) {
    const int PC = packed_channels(C);
    const long long words = (long long)KN * KH * KW * PC;
    if (words == 0) return TAB_OK;
    if (words * 4 >= (1LL << 31) * 256) return TAB_E_TOO_LARGE;
    const unsigned blocks = (unsigned)((words * 4 + 255) / 256);
    const uint64_t* q = reinterpret_cast<const uint64_t*>(qw);
    if (wbits == 2) expand_weights_kernel<2><<<blocks, 256, 0, stream>>>(q, w8, words, PC, C);
    else expand_weights_kernel<1><<<blocks, 256, 0, stream>>>(q, w8, words, PC, C);
    return check_launch();
}

// GEMM stage alone on byte operands.  binary_act: activations are {-1,+1} (out-of-image taps count as +1).
int conv_int8_dispatch(const int8_t* qx8, const int8_t* w8, float* y, int binary_act,
                       int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW,
                       cudaStream_t stream, const float* residual, double* abs_sums, const FusedTail* tail) {
    const int PC = packed_channels(C);
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (oh <= 0 || ow <= 0 || N == 0 || KN == 0) return TAB_OK;
    int rc = imma_limits(N, H, W, C, KN, KH, KW, oh, ow);
    if (rc != TAB_OK) return rc;
    ImmaParams p;
    p.qx = qx8; p.w8 = w8; p.y = y; p.residual = residual; p.abs_sums = abs_sums;
    p.N = N; p.H = H; p.W = W; p.PC = PC; p.KN = KN; p.KH = KH; p.KW = KW;
    p.OH = (int)oh; p.OW = (int)ow; p.p1 = p1; p.p2 = p2; p.s1 = s1; p.s2 = s2;
    p.M = (int)((long long)N * oh * ow); p.Kw = KH * KW * PC;
    if (tail && tail->ths_out && abs_sums) {
        p.ths_out = tail->ths_out; p.ths_scale = tail->scale; p.done_counter = tail->counter;
        p.per_image = (double)KN * (double)oh * (double)ow;
    }
    const bool padone = binary_act && (p1 > 0 || p2 > 0);
    // 256 x 64 tiles when there are at most 64 filters, 128 x 128 tiles otherwise.  The patch variant is used
    // when the kernel has at least 3 taps, the largest patch fits the shared-memory budget and it copies at
    // most half of what the im2col variant would; else the im2col variant (1x1 kernels, large strides).
    // more than 64 filters: tcgen05 kernel; up to 64 filters the mma.sync kernel with patch staging is still ahead
    // (very short K - fewer than four ring stages - does not amortise the tcgen05 kernel's set-up)
    if (g_imma_variant == 3 || g_imma_variant == 4 || g_imma_variant == 5 || (g_imma_variant == 0 && KN > 64 && p.Kw >= 8))
        return conv_umma_dispatch(p, padone, g_imma_variant == 4 ? 1 : (g_imma_variant == 5 ? 2 : 0), stream);
    const bool narrow = KN <= 64;
    const int TMI = narrow ? 256 : 128, TNI = narrow ? 64 : 128, T = KH * KW;
    if (T >= 3 && g_imma_variant != 1) {
        const int pmax = patch_pixels_max(TMI, N, H, W, (int)oh, (int)ow, KH, KW, p1, p2, s1, s2);
        const long long need = 3LL * TNI * IROW + 2LL * pmax * 64 + 4LL * pmax;
        if (pmax > 0 && need <= PATCH_SMEM_BUDGET && 2LL * pmax <= (long long)TMI * T) {
            if (narrow) return padone ? launch_patch<4, 1, true>(p, pmax, stream) : launch_patch<4, 1, false>(p, pmax, stream);
            return padone ? launch_patch<2, 2, true>(p, pmax, stream) : launch_patch<2, 2, false>(p, pmax, stream);
        }
    }
    if (narrow) return padone ? launch_imma<4, 1, 2, true>(p, stream) : launch_imma<4, 1, 2, false>(p, stream);
    return padone ? launch_imma<2, 2, 3, true>(p, stream) : launch_imma<2, 2, 3, false>(p, stream);
}

void imma_set_variant(int v) { g_imma_variant = v; }

// Plane layout of a convolution geometry (see QLayout).
static QLayout plane_layout(int H, int W, int KH, int KW, int p1, int p2, int s1, int s2) {
    QLayout L;
    L.p1 = p1; L.p2 = p2; L.s1 = s1; L.s2 = s2;
    L.A = s1 < KH ? s1 : KH; L.B = s2 < KW ? s2 : KW;
    L.PH2 = (H + 2 * p1 + s1 - 1) / s1; L.PW2 = (W + 2 * p2 + s2 - 1) / s2;
    return L;
}

static int quantize_prep_dispatch(const float* x, const float* ths, int8_t* qx8, int bits, int N, int H, int W, int C,
                                  const QLayout& L, const PrepExtras& ex, cudaStream_t stream) {
    if (N >= 65535) return TAB_E_TOO_LARGE;
    const int Cp = packed_channels(C) * 64;
    const long long groups = (long long)L.A * L.B * L.PH2 * L.PW2 * (Cp / 16);
    if (N == 0 || groups == 0) return TAB_OK;
    // CTAs per image: at most four full waves of 8 CTAs per SM over all images, and every CTA the same number of
    // grid-stride iterations (a ragged last iteration or a fifth, nearly empty wave costs a whole wave's time).
    const long long steps = (groups + Q8THREADS - 1) / Q8THREADS;
    long long cap = (148LL * 8 * 4) / N;
    if (cap < 1) cap = 1;
    long long per = steps;
    if (per > cap) {
        const long long iters = (steps + cap - 1) / cap;
        per = (steps + iters - 1) / iters;
    }
    dim3 grid((unsigned)per, (unsigned)N);
    const bool vec = (C % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 31) == 0) && (((long long)H * W * C) % 8 == 0);
    if (bits == 2) {
        if (vec) return launch_pdl(quantize_int8_padded_kernel<2, true>, grid, dim3(Q8THREADS), 0, stream, x, ths, qx8, H, W, C, Cp, L, ex);
        return launch_pdl(quantize_int8_padded_kernel<2, false>, grid, dim3(Q8THREADS), 0, stream, x, ths, qx8, H, W, C, Cp, L, ex);
    }
    if (vec) return launch_pdl(quantize_int8_padded_kernel<1, true>, grid, dim3(Q8THREADS), 0, stream, x, ths, qx8, H, W, C, Cp, L, ex);
    return launch_pdl(quantize_int8_padded_kernel<1, false>, grid, dim3(Q8THREADS), 0, stream, x, ths, qx8, H, W, C, Cp, L, ex);
}

// Quantise to the padded plane layout of a convolution geometry (QLayout).  Binary activations (bits 1) get +1 in
// the border.  N < 65535.
int quantize_int8_padded_dispatch(const float* x, const float* ths, int8_t* qx8, int bits, int N, int H, int W, int C,
                                  int KH, int KW, int p1, int p2, int s1, int s2, cudaStream_t stream) {
    PrepExtras none = {};
    none.images = N;
    return quantize_prep_dispatch(x, ths, qx8, bits, N, H, W, C, plane_layout(H, W, KH, KW, p1, p2, s1, s2), none, stream);
}

// GEMM stage on activations in the padded plane layout: the TMA-fed tcgen05 kernels.
// TAB_E_TOO_LARGE when the shape is not covered.
int conv_int8_padded_dispatch(const int8_t* qx8p, const int8_t* w8, float* y, int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                              int KN, int KH, int KW, cudaStream_t stream, const float* residual, double* abs_sums) {
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (oh <= 0 || ow <= 0 || N == 0 || KN == 0) return TAB_OK;
    int rc = imma_limits(N, H, W, C, KN, KH, KW, oh, ow);
    if (rc != TAB_OK) return rc;
    if (N >= 65535) return TAB_E_TOO_LARGE;
    ImmaParams p;
    p.qx = qx8p; p.w8 = w8; p.y = y; p.residual = residual; p.abs_sums = abs_sums;
    p.N = N; p.H = H; p.W = W; p.PC = packed_channels(C); p.KN = KN; p.KH = KH; p.KW = KW;
    p.OH = (int)oh; p.OW = (int)ow; p.p1 = p1; p.p2 = p2; p.s1 = s1; p.s2 = s2;
    p.M = (int)((long long)N * oh * ow); p.Kw = KH * KW * p.PC;
    return conv_tma_dispatch(p, g_imma_variant == 7 ? 2 : 1, stream);
}

// Scratch layout: padded byte activations | byte weights | 256 bytes holding the completion counter of the fused tail.
// next_ths (optional, with abs_sums): the GEMM's last CTA writes next_scale * abs_sums[n] / (KN*OH*OW) there.
// abs_sums is cleared by this call.  Three launches at most: quantise (+ weight expansion + clears), GEMM.
int conv_imma_dispatch(const float* x, const int64_t* qw, const float* ths, float* y, void* workspace, int type,
                       int p1, int p2, int s1, int s2, int N, int H, int W, int C, int KN, int KH, int KW,
                       cudaStream_t stream, const float* residual, double* abs_sums, float* next_ths, float next_scale) {
    const int Cp = packed_channels(C) * 64;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1, ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (oh <= 0 || ow <= 0 || N == 0 || KN == 0) return TAB_OK;
    int rc = imma_limits(N, H, W, C, KN, KH, KW, oh, ow);
    if (rc != TAB_OK) return rc;
    if (N >= 65535) return TAB_E_TOO_LARGE;
    int8_t* qx8 = reinterpret_cast<int8_t*>(workspace);
    int8_t* w8 = qx8 + ((size_t)N * scratch_pixels(H, W, KH, KW, p1, p2, s1, s2) * Cp + 255) / 256 * 256;
    unsigned* counter = reinterpret_cast<unsigned*>(w8 + ((size_t)KN * KH * KW * Cp + 255) / 256 * 256);
    FusedTail tail = {};
    if (next_ths && abs_sums) { tail.ths_out = next_ths; tail.scale = next_scale; tail.counter = counter; }
    PrepExtras ex = {};
    ex.images = N;
    ex.zero_sums = abs_sums;
    ex.zero_counter = tail.ths_out ? counter : nullptr;
    ex.qw = reinterpret_cast<const uint64_t*>(qw); ex.w8 = w8;
    ex.words = (long long)KN * KH * KW * packed_channels(C);
    ex.wbits = weight_bits(type);
    // Persistent TMA-fed tcgen05 kernel on the padded plane layout (any stride); at least 4 taps unless there is no
    // padding at all (with fewer, the padded grid costs more than the patch saves); at least 45 % of the plane grid
    // useful.  A strided 1x1 convolution has the single plane of the pixels it reads.
    bool quantized = false;
    {
        const QLayout L = plane_layout(H, W, KH, KW, p1, p2, s1, s2);
        const long long rows = (long long)L.A * L.B * N * L.PH2 * L.PW2;
        const double useful = (double)oh * ow / ((double)L.PH2 * L.PW2);
        ImmaParams p;
        p.qx = qx8; p.w8 = w8; p.y = y; p.residual = residual; p.abs_sums = abs_sums;
        p.N = N; p.H = H; p.W = W; p.PC = packed_channels(C); p.KN = KN; p.KH = KH; p.KW = KW;
        p.OH = (int)oh; p.OW = (int)ow; p.p1 = p1; p.p2 = p2; p.s1 = s1; p.s2 = s2;
        p.M = (int)((long long)N * oh * ow); p.Kw = KH * KW * p.PC;
        if (tail.ths_out) {
            p.ths_out = tail.ths_out; p.ths_scale = tail.scale; p.done_counter = tail.counter;
            p.per_image = (double)KN * (double)oh * (double)ow;
        }
        const bool unit = s1 == 1 && s2 == 1;
        const bool shape = (KH * KW >= 4 || (p1 == 0 && p2 == 0)) && rows < (1LL << 31) - 4096;
        const bool want = shape && (((g_imma_variant == 6 || g_imma_variant == 7) && unit) ||
                                    ((g_imma_variant == 0 || g_imma_variant == 6) && g_tma_default && useful >= 0.45 && conv_tma_persist_fits(p)));
        if (want) {
            rc = quantize_prep_dispatch(x, ths, qx8, act_bits(type), N, H, W, C, L, ex, stream);
            if (rc != TAB_OK) return rc;
            quantized = unit && p1 == 0 && p2 == 0;   // then the layout is the one the other kernels read
            rc = conv_tma_dispatch(p, g_imma_variant == 7 ? 2 : (g_imma_variant == 6 ? 1 : 0), stream);
            if (rc != TAB_E_TOO_LARGE) return rc;     // shape not covered after all: continue with the unpadded form
        }
    }
    if (!quantized) {
        rc = quantize_prep_dispatch(x, ths, qx8, act_bits(type), N, H, W, C, plane_layout(H, W, 1, 1, 0, 0, 1, 1), ex, stream);
        if (rc != TAB_OK) return rc;
    }
    return conv_int8_dispatch(qx8, w8, y, act_bits(type) == 1, p1, p2, s1, s2, N, H, W, C, KN, KH, KW, stream, residual, abs_sums, &tail);
}

}  // namespace tab
