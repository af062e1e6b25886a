// TAB convolution as an implicit-im2col, bit-packed popcount GEMM on the integer pipes of sm_100a.
//
// Replaces PadKernel (TAB_GEMM.cuh:73-89), Img2RowKernel (:92-115), GEMMWithCuda (:22-66) and the four
// GEMM kernels TNNGEMM/TBNGEMM/BTNGEMM/BNNGEMM (TAB_GEMM.cu:25-147).  Nothing is materialised: the
// activation tile of each CTA is gathered straight from the packed [N][H][W][PC][ab] tensor with
// cp.async, out-of-image taps are zero-filled (zero words = value 0 for ternary activations and +1 for
// binary activations, exactly what the reference's zero-bordered pad buffer holds), and the weight
// tile is the contiguous [KN][KH*KW*PC][wb] rows of QW.
//
// GEMM view: M = N*OH*OW output pixels, KN filters, Kw = KH*KW*PC 64-bit words per plane.
//   type 0 TNN  y = sum popc(ma&mw) - 2*sum popc((sa^sw)&ma&mw)
//   type 1 TBN  y = sum popc(ma)    - 2*sum popc((sa^bw)&ma)
//   type 2 BTN  y = btn[kn]         - 2*sum popc((ba^sw)&mw)
//   type 3 BNN  y = KH*KW*C         - 2*sum popc(ba^bw)
//
// Tiling: a CTA of 256 threads owns 128 pixels x 64 filters; a warp owns 64 x 16; a lane owns
// pixels {pg + 8i} and filters {fg + 4j} (pg = lane/4, fg = lane%4), 32 outputs.  K is walked in chunks
// of KCH words, double-buffered in shared memory (cp.async groups).  Inside a chunk the words of one
// output are reduced four 64-bit words (eight 32-bit lanes) at a time through a carry-save adder tree
// (LOP3 full adders: 8 words -> ones, ones, twos, fours), so that 4 POPC replace 8: POPC issues at
// 16 lanes/clk/SM against 64 for LOP3, and this split keeps both pipes about equally busy.
#include "tab_kernels.cuh"

namespace tab {

constexpr int TM = 128;        // pixels per CTA
constexpr int TN = 64;         // filters per CTA
constexpr int KCH = 12;        // 64-bit words (per plane) per K chunk
constexpr int CTHREADS = 256;
constexpr int RM = 8;          // pixels per lane
constexpr int RN = 4;          // filters per lane
constexpr int STAGES = 2;

struct ConvParams {
    const uint64_t* qx;        // [N][H][W][PC][AB]
    const uint64_t* qw;        // [KN][KH*KW*PC][WB]
    const int* btn;            // [KN] (type 2)
    float* y;                  // [M][KN]
    int N, H, W, PC, KN, KH, KW, OH, OW, p1, p2, s1, s2;
    int M, Kw, NUM;
    int qw16;                  // qw is 16-byte aligned
    // Accumulation weights, passed as run-time values on purpose: "acc += w * popc" then stays an
    // integer multiply-add (FMA pipe) instead of being strength-reduced into shifts/adds on the ALU pipe,
    // which the LOP3 work already saturates.  wpos = {1,2,4,8,16}, wneg = {-2,-4,-8,-16,-32}.
    int wpos[5];
    int wneg[5];
};

template <int TYPE> struct Planes {
    static constexpr int AB = (TYPE == 2 || TYPE == 3) ? 1 : 2;
    static constexpr int WB = (TYPE == 1 || TYPE == 3) ? 1 : 2;
    static constexpr int SA = KCH * AB * 8 + 16;   // row strides in bytes: = 16 (mod 32), so that eight
    static constexpr int SB = KCH * WB * 8 + 16;   // consecutive rows hit eight different 16-byte bank groups
    static constexpr int STAGE_BYTES = TM * SA + TN * SB;
};

__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 8 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

// Full adder on 32 independent bit positions: two LOP3.
__device__ __forceinline__ void csa(uint32_t a, uint32_t b, uint32_t c, uint32_t& sum, uint32_t& carry) {
    sum = a ^ b ^ c;
    carry = (a & b) | (c & (a | b));
}

__device__ __forceinline__ void mad_acc(int& acc, int p, int w) {
    asm("mad.lo.s32 %0, %1, %2, %0;" : "+r"(acc) : "r"(p), "r"(w));
}

// acc += sum_i w[LVL] * popc(x[i]) for N words of weight 2^LVL, after carry-save compression: triples
// at a level go through a full adder (sum stays, carry moves one level up) until fewer than three
// words remain at every level; only those survivors are POPC'ed.  N words cost about N/2 POPC.
// cy holds C pending words of the next level.  Everything unrolls at compile time.
template <int N, int C, int LVL> struct CsaTree {
    static __device__ __forceinline__ void run(const uint32_t* x, const uint32_t* cy, int& acc, const int* w) {
        if constexpr (N >= 3) {
            constexpr int K = N / 3, R = N - 2 * K;
            uint32_t same[R], cy2[C + K];
#pragma unroll
            for (int c = 0; c < C; c++) cy2[c] = cy[c];
#pragma unroll
            for (int k = 0; k < K; k++) csa(x[3 * k], x[3 * k + 1], x[3 * k + 2], same[k], cy2[C + k]);
#pragma unroll
            for (int r = 0; r < N - 3 * K; r++) same[K + r] = x[3 * K + r];
            CsaTree<R, C + K, LVL>::run(same, cy2, acc, w);
        } else {
#pragma unroll
            for (int i = 0; i < N; i++) mad_acc(acc, __popc(x[i]), w[LVL]);
            if constexpr (C > 0) CsaTree<C, 0, LVL + 1>::run(cy, nullptr, acc, w);
        }
    }
};

// acc += w[0] * sum popc(x[i]); CSA selects the compressed or the one-POPC-per-word form.
template <int NU, bool CSA> __device__ __forceinline__ void popc_accumulate(const uint32_t (&x)[NU], int& acc, const int* w) {
    if constexpr (CSA) {
        CsaTree<NU, 0, 0>::run(x, nullptr, acc, w);
    } else {
#pragma unroll
        for (int i = 0; i < NU; i++) mad_acc(acc, __popc(x[i]), w[0]);
    }
}

// Read NW 64-bit words from shared memory (8-byte aligned; 16-byte loads when AL16).
template <int NW, bool AL16> __device__ __forceinline__ void lds_words(const unsigned char* p, uint32_t (&r)[2 * NW]) {
    if constexpr (AL16 && (NW % 2 == 0)) {
#pragma unroll
        for (int i = 0; i < NW / 2; i++) {
            const uint4 v = *reinterpret_cast<const uint4*>(p + 16 * i);
            r[4 * i + 0] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NW; i++) {
            const uint2 v = *reinterpret_cast<const uint2*>(p + 8 * i);
            r[2 * i + 0] = v.x; r[2 * i + 1] = v.y;
        }
    }
}

// One group of G consecutive k-words for the whole 8x4 register tile of a lane.
// a_rows / b_rows point at this lane's first pixel / filter row, at the group's first word.
template <int TYPE, int G, bool CSA>
__device__ __forceinline__ void compute_group(const unsigned char* a_rows, const unsigned char* b_rows,
                                              int (&acc)[RM][RN], int (&pcount)[RM], int kb, int fg,
                                              const int* wpos, const int* wneg) {
    using P = Planes<TYPE>;
    constexpr int AB = P::AB, WB = P::WB, NU = 2 * G;
    // register image of the weights: [filter][word g][plane][lo,hi] as stored (planes interleaved per word)
    uint32_t wreg[RN][2 * G * WB];
#pragma unroll
    for (int j = 0; j < RN; j++)
        lds_words<G * WB, (WB == 2) || (G % 2 == 0)>(b_rows + j * 4 * P::SB, wreg[j]);

#pragma unroll
    for (int i = 0; i < RM; i++) {
        uint32_t areg[2 * G * AB];
        lds_words<G * AB, (AB == 2) || (G % 2 == 0)>(a_rows + i * 8 * P::SA, areg);
        if (TYPE == 1) {
            // sum popc(ma): the four lanes that share this pixel each take the words with k%4 == fg
#pragma unroll
            for (int g = 0; g < G; g++)
                if (((kb + g) & 3) == fg) pcount[i] += __popc(areg[4 * g + 2]) + __popc(areg[4 * g + 3]);
        }
#pragma unroll
        for (int j = 0; j < RN; j++) {
            uint32_t u[NU];
            if (TYPE == 0) {
                uint32_t t[NU];
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t sa = areg[4 * g + h], ma = areg[4 * g + 2 + h];
                        const uint32_t sw = wreg[j][4 * g + h], mw = wreg[j][4 * g + 2 + h];
                        t[2 * g + h] = ma & mw;
                        u[2 * g + h] = (sa ^ sw) & t[2 * g + h];
                    }
                popc_accumulate<NU, CSA>(t, acc[i][j], wpos);
            } else if (TYPE == 1) {
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        u[2 * g + h] = (areg[4 * g + h] ^ wreg[j][2 * g + h]) & areg[4 * g + 2 + h];
            } else if (TYPE == 2) {
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        u[2 * g + h] = (areg[2 * g + h] ^ wreg[j][4 * g + h]) & wreg[j][4 * g + 2 + h];
            } else {
#pragma unroll
                for (int g = 0; g < G; g++)
#pragma unroll
                    for (int h = 0; h < 2; h++) u[2 * g + h] = areg[2 * g + h] ^ wreg[j][2 * g + h];
            }
            popc_accumulate<NU, CSA>(u, acc[i][j], wneg);
        }
    }
}

template <int TYPE, bool CSA>
__global__ void __launch_bounds__(CTHREADS, 2)
conv_popc_kernel(const ConvParams p) {
    using P = Planes<TYPE>;
    constexpr int AB = P::AB, WB = P::WB;
    extern __shared__ __align__(16) unsigned char smem[];

    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * TM;
    const int n0 = blockIdx.y * TN;

    // ---- loader state: A (activation rows, implicit im2col) ------------------------------------
    const int a_row = tid & (TM - 1);
    const int a_kphase = tid >> 7;                    // 0 or 1: this thread copies words k = kphase + 2e
    int a_ih0, a_iw0;
    const uint64_t* a_img;
    bool a_ok;
    {
        const int m = m0 + a_row;
        a_ok = m < p.M;
        const int mm = a_ok ? m : 0;
        const int ohw = p.OH * p.OW;
        const int n = mm / ohw;
        const int r = mm - n * ohw;
        const int oh = r / p.OW;
        const int ow = r - oh * p.OW;
        a_ih0 = oh * p.s1 - p.p1;
        a_iw0 = ow * p.s2 - p.p2;
        a_img = p.qx + (long long)n * p.H * p.W * p.PC * AB;
    }
    int a_kh, a_kw, a_pc;                             // decode of the next word this thread copies
    {
        const int tap = a_kphase / p.PC;
        a_pc = a_kphase - tap * p.PC;
        a_kh = tap / p.KW;
        a_kw = tap - a_kh * p.KW;
    }
    // ---- loader state: B (weight rows) ---------------------------------------------------------
    const int b_row = tid & (TN - 1);
    const int b_kphase = tid >> 6;                    // 0..3: words k = kphase + 4e
    const bool b_ok = (n0 + b_row) < p.KN;
    const uint64_t* b_src = p.qw + (long long)(b_ok ? n0 + b_row : 0) * p.Kw * WB;

    const uint32_t smem_u32 = (uint32_t)__cvta_generic_to_shared(smem);

    auto load_chunk = [&](int chunk, int stage) {
        const int k0 = chunk * KCH;
        const uint32_t sA = smem_u32 + stage * P::STAGE_BYTES;
        const uint32_t sB = sA + TM * P::SA;
#pragma unroll
        for (int e = 0; e < KCH / 2; e++) {
            const int kl = a_kphase + 2 * e;
            const int ih = a_ih0 + a_kh, iw = a_iw0 + a_kw;
            const bool v = a_ok && (a_kh < p.KH) && ((unsigned)ih < (unsigned)p.H) && ((unsigned)iw < (unsigned)p.W);
            const uint64_t* src = v ? a_img + ((long long)(ih * p.W + iw) * p.PC + a_pc) * AB : p.qx;
            const uint32_t dst = sA + a_row * P::SA + kl * AB * 8;
            if (AB == 2) cp_async_16(dst, src, v); else cp_async_8(dst, src, v);
            a_pc += 2;
            while (a_pc >= p.PC) {
                a_pc -= p.PC;
                if (++a_kw == p.KW) { a_kw = 0; ++a_kh; }
            }
        }
#pragma unroll
        for (int e = 0; e < KCH / 4; e++) {
            const int kl = b_kphase + 4 * e;
            const int k = k0 + kl;
            const bool v = b_ok && (k < p.Kw);
            const uint64_t* src = v ? b_src + (long long)k * WB : p.qw;
            const uint32_t dst = sB + b_row * P::SB + kl * WB * 8;
            if (WB == 2) {
                if (p.qw16) cp_async_16(dst, src, v);
                else { cp_async_8(dst, src, v); cp_async_8(dst + 8, v ? src + 1 : src, v); }
            } else {
                cp_async_8(dst, src, v);
            }
        }
        cp_async_commit();
    };

    // ---- compute mapping -----------------------------------------------------------------------
    const int warp = tid >> 5, lane = tid & 31;
    const int wm = warp & 1, wn = warp >> 1;
    const int fg = lane & 3, pg = lane >> 2;
    const int a_lane_row = wm * 64 + pg;              // + 8*i
    const int b_lane_row = wn * 16 + fg;              // + 4*j

    int acc[RM][RN];
    int pcount[RM];
#pragma unroll
    for (int i = 0; i < RM; i++) {
        pcount[i] = 0;
#pragma unroll
        for (int j = 0; j < RN; j++) acc[i][j] = 0;
    }

    const int nchunks = (p.Kw + KCH - 1) / KCH;
    load_chunk(0, 0);
    for (int c = 0; c < nchunks; c++) {
        const int stage = c & 1;
        if (c + 1 < nchunks) { load_chunk(c + 1, stage ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();

        const unsigned char* sA = smem + stage * P::STAGE_BYTES;
        const unsigned char* sB = sA + TM * P::SA;
        const unsigned char* a_rows = sA + a_lane_row * P::SA;
        const unsigned char* b_rows = sB + b_lane_row * P::SB;
        const int kc = min(KCH, p.Kw - c * KCH);
        if (CSA) {
            const int ng = kc >> 2;
            for (int g = 0; g < ng; g++)
                compute_group<TYPE, 4, true>(a_rows + g * 4 * AB * 8, b_rows + g * 4 * WB * 8, acc, pcount, g * 4, fg, p.wpos, p.wneg);
            const int kb = ng * 4;
            const unsigned char* ar = a_rows + kb * AB * 8;
            const unsigned char* br = b_rows + kb * WB * 8;
            switch (kc & 3) {
                case 1: compute_group<TYPE, 1, true>(ar, br, acc, pcount, kb, fg, p.wpos, p.wneg); break;
                case 2: compute_group<TYPE, 2, true>(ar, br, acc, pcount, kb, fg, p.wpos, p.wneg); break;
                case 3: compute_group<TYPE, 3, true>(ar, br, acc, pcount, kb, fg, p.wpos, p.wneg); break;
                default: break;
            }
        } else {
            for (int k = 0; k < kc; k++)
                compute_group<TYPE, 1, false>(a_rows + k * AB * 8, b_rows + k * WB * 8, acc, pcount, k, fg, p.wpos, p.wneg);
        }
        __syncthreads();
    }

    // ---- epilogue: type correction, exact int -> float, store [M][KN] -----------------------------
    if (TYPE == 1) {
#pragma unroll
        for (int i = 0; i < RM; i++) {
            pcount[i] += __shfl_xor_sync(0xFFFFFFFFu, pcount[i], 1);
            pcount[i] += __shfl_xor_sync(0xFFFFFFFFu, pcount[i], 2);
        }
    }
    int fbase[RN];
#pragma unroll
    for (int j = 0; j < RN; j++) {
        const int f = n0 + b_lane_row + 4 * j;
        fbase[j] = (TYPE == 2) ? ((f < p.KN) ? __ldg(p.btn + f) : 0) : (TYPE == 3 ? p.NUM : 0);
    }
#pragma unroll
    for (int i = 0; i < RM; i++) {
        const int m = m0 + a_lane_row + 8 * i;
        if (m >= p.M) continue;
        float* yrow = p.y + (long long)m * p.KN;
#pragma unroll
        for (int j = 0; j < RN; j++) {
            const int f = n0 + b_lane_row + 4 * j;
            if (f < p.KN) yrow[f] = (float)(acc[i][j] + fbase[j] + (TYPE == 1 ? pcount[i] : 0));
        }
    }
}

template <int TYPE, bool CSA>
static int launch_conv(const ConvParams& p, cudaStream_t stream) {
    using P = Planes<TYPE>;
    const int smem_bytes = STAGES * P::STAGE_BYTES;
    static bool configured[16] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (dev < 16 && !configured[dev]) {
        e = cudaFuncSetAttribute(conv_popc_kernel<TYPE, CSA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return record_cuda_error(e);
        configured[dev] = true;
    } else if (dev >= 16) {
        e = cudaFuncSetAttribute(conv_popc_kernel<TYPE, CSA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return record_cuda_error(e);
    }
    dim3 grid((unsigned)((p.M + TM - 1) / TM), (unsigned)((p.KN + TN - 1) / TN));
    conv_popc_kernel<TYPE, CSA><<<grid, CTHREADS, smem_bytes, stream>>>(p);
    return check_launch();
}

int conv_packed_dispatch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y, int type,
                         int p1, int p2, int s1, int s2, int N, int H, int W, int C,
                         int KN, int KH, int KW, cudaStream_t stream, bool use_csa) {
    ConvParams p;
    p.qx = reinterpret_cast<const uint64_t*>(qx);
    p.qw = reinterpret_cast<const uint64_t*>(qw);
    p.btn = btn;
    p.y = y;
    p.N = N; p.H = H; p.W = W; p.PC = packed_channels(C);
    p.KN = KN; p.KH = KH; p.KW = KW;
    p.p1 = p1; p.p2 = p2; p.s1 = s1; p.s2 = s2;
    const long long oh = ((long long)H + 2LL * p1 - KH + 1) / s1;
    const long long ow = ((long long)W + 2LL * p2 - KW + 1) / s2;
    if (oh <= 0 || ow <= 0 || N == 0 || KN == 0) return TAB_OK;      // empty output
    const long long M = (long long)N * oh * ow;
    const long long Kw = (long long)KH * KW * p.PC;
    if (M >= (1LL << 31) - TM || Kw >= (1LL << 28) || (long long)KH * KW * C >= (1LL << 30) ||
        (long long)H * W >= (1LL << 31) || (KN + TN - 1) / TN > 65535)
        return TAB_E_TOO_LARGE;
    p.OH = (int)oh; p.OW = (int)ow; p.M = (int)M; p.Kw = (int)Kw; p.NUM = KH * KW * C;
    p.qw16 = (reinterpret_cast<uintptr_t>(qw) & 15) == 0;
    for (int i = 0; i < 5; i++) { p.wpos[i] = 1 << i; p.wneg[i] = -(2 << i); }
    switch (type) {
        case 0: return use_csa ? launch_conv<0, true>(p, stream) : launch_conv<0, false>(p, stream);
        case 1: return use_csa ? launch_conv<1, true>(p, stream) : launch_conv<1, false>(p, stream);
        case 2: return use_csa ? launch_conv<2, true>(p, stream) : launch_conv<2, false>(p, stream);
        case 3: return use_csa ? launch_conv<3, true>(p, stream) : launch_conv<3, false>(p, stream);
        default: return TAB_E_BAD_ARGUMENT;
    }
}

}  // namespace tab
