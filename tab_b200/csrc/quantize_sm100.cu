// Threshold-quantise fp32 NHWC data into bit-planes packed 64 channels per 64-bit word, in one pass,
// with the per-n popcount of the magnitude plane folded in.
//
// Replaces the reference's TerOnlyKernel (TAB_GEMM.cu:163-208), BinOnlyKernel (:211-247) and
// BTN_Weight (:150-160).  Encoding (TAB_GEMM.cu:184-206, :231-245): ternary x > t -> (sign 0, mag 1),
// else x < -t -> (1, 1), else (0, 0); binary bit = (x < t); channel c is bit c%64 of word c/64.
//
// The kernel is HBM-bound: 4 bytes read per element, 2 or 1 bits written.  Fast path (C % 64 == 0,
// 32-byte aligned input): eight lanes own one 64-channel word; each lane issues QUNROLL independent
// 256-bit loads before it touches any of them, so a resident SM keeps > 200 KB in flight; a lane turns
// its 8 channels into one byte per plane with compares and predicated ORs and stores those bytes
// itself - no shuffles, votes or redux (a first version merged nibbles with redux.sync and was bound
// by that instruction's pipe at 37 % of DRAM bandwidth).
// General path (any C, any alignment): one warp per word, two coalesced 32-bit loads per lane, the
// two 32-bit halves come straight out of __ballot_sync.
//
// Inside a convolution call the same launch also does the call's small set-up jobs (QuantExtras), so that they cost no
// launch of their own: all CTAs share the expansion of the packed weights to the bytes the tensor-core kernel
// multiplies, and the first CTA of every image clears that image's |y| sum (the first of all the completion counter).
#include <mutex>
#include "tab_kernels.cuh"

namespace tab {

constexpr int QTHREADS = 256;
constexpr int QUNROLL = 4;                                   // independent 256-bit loads per lane
constexpr int QWORDS_PER_ITER = (QTHREADS / 8) * QUNROLL;    // 128 words = 32 KB of fp32 per CTA step

struct f8 { float v[8]; };

// One thread per (filter, word k, 16-channel group) of packed weights [KN][KH*KW*PC][WB]: 16 bytes of {-1,0,+1}
// into [KN][KH*KW*PC][64]; channels beyond C become 0.
template <int WB>
__device__ __forceinline__ void expand_group(const uint64_t* __restrict__ qw, int8_t* __restrict__ w8, long long idx, int PC, int C) {
    const long long word = idx >> 2;
    const int grp = (int)(idx & 3);
    const int pc = (int)(word % PC);
    const int cbase = pc * 64 + grp * 16;
    uint32_t s16, m16;
    if (WB == 2) {
        m16 = (uint32_t)(qw[word * 2 + 1] >> (grp * 16)) & 0xFFFFu;
        s16 = (uint32_t)(qw[word * 2] >> (grp * 16)) & m16;
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

template <int WB>
__global__ void expand_weights_kernel(const uint64_t* __restrict__ qw, int8_t* __restrict__ w8, long long words, int PC, int C) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= words * 4) return;
    expand_group<WB>(qw, w8, idx, PC, C);
}

// Runs at the top of both quantiser kernels.  Programmatic launch: nothing is read or written before the previous
// kernel of the stream (which produced x and the thresholds, and may still be reading the scratch this launch
// overwrites) has completed.
__device__ __forceinline__ void quant_prologue(const QuantExtras& ex, int n) {
    pdl_wait();
    if (ex.qw != nullptr) {                                                // the weights, spread over all CTAs of the launch
        const long long stride = (long long)gridDim.x * gridDim.y * blockDim.x;
        for (long long idx = ((long long)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x; idx < ex.words * 4; idx += stride) {
            if (ex.wbits == 2) expand_group<2>(ex.qw, ex.w8, idx, ex.PC, ex.C);
            else expand_group<1>(ex.qw, ex.w8, idx, ex.PC, ex.C);
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (ex.zero_sums) ex.zero_sums[n] = 0.0;
        if (n == 0 && ex.zero_counter) *ex.zero_counter = 0u;
    }
}

// Sixteen consecutive channels held as 16-bit integers (the compact output of a convolution): one 256-bit load.
struct u8w { uint32_t v[8]; };
__device__ __forceinline__ u8w ld_stream_u8(const int16_t* p) {
    u8w r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7]) : "l"(p));
    return r;
}

// 256-bit streaming load (sm_100): a lane reads 8 consecutive channels, a warp 1 KB contiguous.
__device__ __forceinline__ f8 ld_stream_f8(const float* p) {
    f8 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]),
                   "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7]) : "l"(p));
    return r;
}

// grid = (ctas_per_image, N).  words_per_image = H*W*PC with PC = C/64.
// Eight lanes own one 64-channel word: lane b of the group quantises channels 8b..8b+7 and stores byte b
// of the sign and of the magnitude word itself, so no cross-lane traffic is needed at all.
// IN16: x holds 16-bit integers instead of floats (same element order).
template <int BITS, bool IN16>
__global__ void __launch_bounds__(QTHREADS)
quantize_c64_kernel(const void* __restrict__ x, const float* __restrict__ ths,
                    uint64_t* __restrict__ qx, int* __restrict__ btn, long long words_per_image, const QuantExtras ex) {
    // Last image first, and within an image the last chunk first: the tensor usually was written front to back by the
    // kernel before this one, so its end is what the L2 still holds.
    const int n = (int)(gridDim.y - 1u - blockIdx.y);
    const unsigned bx = gridDim.x - 1u - blockIdx.x;
    quant_prologue(ex, n);
    const float t = __ldg(ths + n);
    const float nt = -t;
    const int byte = threadIdx.x & 7;
    const int grp = threadIdx.x >> 3;                         // word slot within the CTA: 0..31
    const float* xi = reinterpret_cast<const float*>(x) + (IN16 ? 0 : (long long)n * words_per_image * 64);
    const int16_t* xs = reinterpret_cast<const int16_t*>(x) + (IN16 ? (long long)n * words_per_image * 64 : 0);
    unsigned char* qi = reinterpret_cast<unsigned char*>(qx + (long long)n * words_per_image * BITS);
    int cnt = 0;

    if (IN16) {
        // 16-bit input: four lanes own a word, a lane loads its 16 channels as one 256-bit load (the same bytes per load and
        // per thread in flight as the fp32 path) and stores 16 bits per plane.  Inside the chain this form measured 1 us per
        // launch faster than 128-bit loads, twice as many of them, by eight lanes per word.
        constexpr int WORDS16 = (QTHREADS / 4) * QUNROLL;                  // 256 words per CTA step
        const int q4 = threadIdx.x & 3, g4 = threadIdx.x >> 2;
        for (long long w0 = (long long)bx * WORDS16; w0 < words_per_image; w0 += (long long)gridDim.x * WORDS16) {
            u8w raw[QUNROLL];
#pragma unroll
            for (int u = 0; u < QUNROLL; u++) {
                const long long w = w0 + u * (QTHREADS / 4) + g4;
                if (w < words_per_image) raw[u] = ld_stream_u8(xs + w * 64 + q4 * 16);
            }
#pragma unroll
            for (int u = 0; u < QUNROLL; u++) {
                const long long w = w0 + u * (QTHREADS / 4) + g4;
                if (w >= words_per_image) continue;
                unsigned pos = 0, neg = 0, bin = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float lo = (float)(int16_t)(raw[u].v[i] & 0xFFFFu), hi = (float)(int16_t)(raw[u].v[i] >> 16);
                    if (BITS == 2) {
                        pos |= (lo > t) ? (1u << (2 * i)) : 0u;      neg |= (lo < nt) ? (1u << (2 * i)) : 0u;
                        pos |= (hi > t) ? (1u << (2 * i + 1)) : 0u;  neg |= (hi < nt) ? (1u << (2 * i + 1)) : 0u;
                    } else {
                        bin |= (lo < t) ? (1u << (2 * i)) : 0u;      bin |= (hi < t) ? (1u << (2 * i + 1)) : 0u;
                    }
                }
                if (BITS == 2) {
                    neg &= ~pos;
                    const unsigned mag = pos | neg;
                    unsigned short* o = reinterpret_cast<unsigned short*>(qi + w * 16) + q4;
                    o[0] = (unsigned short)neg;
                    o[4] = (unsigned short)mag;
                    cnt += __popc(mag);
                } else {
                    reinterpret_cast<unsigned short*>(qi + w * 8)[q4] = (unsigned short)bin;
                }
            }
        }
    }
    constexpr int UN = QUNROLL;
    constexpr int WORDS = (QTHREADS / 8) * UN;
    for (long long w0 = (long long)bx * WORDS; !IN16 && w0 < words_per_image; w0 += (long long)gridDim.x * WORDS) {
        f8 v[UN];
        long long w[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            w[u] = w0 + u * (QTHREADS / 8) + grp;
            if (w[u] < words_per_image) v[u] = ld_stream_f8(xi + w[u] * 64 + byte * 8);
        }
#pragma unroll
        for (int u = 0; u < UN; u++) {
            if (w[u] >= words_per_image) continue;
            const f8 val = v[u];
            if (BITS == 2) {
                unsigned pos = 0, neg = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    pos |= (val.v[i] > t) ? (1u << i) : 0u;
                    neg |= (val.v[i] < nt) ? (1u << i) : 0u;
                }
                neg &= ~pos;                                   // the "+1" branch is tested first
                const unsigned mag = pos | neg;
                unsigned char* o = qi + w[u] * 16 + byte;
                o[0] = (unsigned char)neg;                     // sign plane, byte `byte` of the word
                o[8] = (unsigned char)mag;                     // magnitude plane
                cnt += __popc(mag);
            } else {
                unsigned b = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) b |= (val.v[i] < t) ? (1u << i) : 0u;
                qi[w[u] * 8 + byte] = (unsigned char)b;
            }
        }
    }

    if (BITS == 2 && btn != nullptr) {
        __shared__ int wsum[QTHREADS / 32];
        cnt = __reduce_add_sync(0xFFFFFFFFu, cnt);
        if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = cnt;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
#pragma unroll
            for (int i = 0; i < QTHREADS / 32; i++) tot += wsum[i];
            if (tot) atomicAdd(btn + n, tot);                 // integer: order-independent, exact
        }
    }
    pdl_launch_dependents();                                  // the next kernel may be scheduled once every CTA got here
}

// One warp per output word; works for every C and alignment.  grid = (ctas_per_image, N).
template <int BITS, bool IN16>
__global__ void __launch_bounds__(QTHREADS)
quantize_generic_kernel(const void* __restrict__ x, const float* __restrict__ ths,
                        uint64_t* __restrict__ qx, int* __restrict__ btn,
                        long long pixels_per_image, int C, int PC, const QuantExtras ex) {
    const int n = blockIdx.y;
    quant_prologue(ex, n);
    const float t = __ldg(ths + n);
    const float nt = -t;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const long long words_per_image = pixels_per_image * PC;
    const float* xi = reinterpret_cast<const float*>(x) + (IN16 ? 0 : (long long)n * pixels_per_image * C);
    const int16_t* xs = reinterpret_cast<const int16_t*>(x) + (IN16 ? (long long)n * pixels_per_image * C : 0);
    uint64_t* qi = qx + (long long)n * words_per_image * BITS;
    int cnt = 0;

    for (long long w = (long long)blockIdx.x * (QTHREADS / 32) + warp; w < words_per_image;
         w += (long long)gridDim.x * (QTHREADS / 32)) {
        const long long pix = w / PC;
        const int pc = (int)(w - pix * PC);
        const int c0 = pc * 64 + lane, c1 = c0 + 32;
        const float* row = xi + pix * C;
        const int16_t* rows = xs + pix * C;
        const bool in0 = c0 < C, in1 = c1 < C;
        const float a = in0 ? (IN16 ? (float)__ldg(rows + c0) : __ldg(row + c0)) : 0.f;
        const float b = in1 ? (IN16 ? (float)__ldg(rows + c1) : __ldg(row + c1)) : 0.f;
        if (BITS == 2) {
            const bool pa = in0 && a > t, pb = in1 && b > t;
            const bool na = in0 && !pa && a < nt, nb = in1 && !pb && b < nt;
            const unsigned s_lo = __ballot_sync(0xFFFFFFFFu, na), s_hi = __ballot_sync(0xFFFFFFFFu, nb);
            const unsigned m_lo = __ballot_sync(0xFFFFFFFFu, pa || na), m_hi = __ballot_sync(0xFFFFFFFFu, pb || nb);
            if (lane == 0) {
                uint2* o = reinterpret_cast<uint2*>(qi + w * 2);
                o[0] = make_uint2(s_lo, s_hi);
                o[1] = make_uint2(m_lo, m_hi);
                cnt += __popc(m_lo) + __popc(m_hi);
            }
        } else {
            const unsigned b_lo = __ballot_sync(0xFFFFFFFFu, in0 && a < t);
            const unsigned b_hi = __ballot_sync(0xFFFFFFFFu, in1 && b < t);
            if (lane == 0) *reinterpret_cast<uint2*>(qi + w) = make_uint2(b_lo, b_hi);
        }
    }
    if (BITS == 2 && btn != nullptr && lane == 0 && cnt) atomicAdd(btn + n, cnt);
    pdl_launch_dependents();
}

int quantize_dispatch(const void* x, const float* ths, int64_t* qx, int32_t* btn, int bits,
                      int N, int H, int W, int C, cudaStream_t stream, const QuantExtras* extras, bool in16) {
    const QuantExtras ex = extras ? *extras : QuantExtras{};
    const long long pixels = (long long)H * W;
    const int PC = (C + 63) / 64;
    const long long wpi = pixels * PC;
    if (N == 0 || wpi == 0) return TAB_OK;
    if (N > 65535) {
        // grid.y is limited to 65535: process in slabs of images.
        for (int n0 = 0; n0 < N; n0 += 65535) {
            const int nn = (N - n0 < 65535) ? (N - n0) : 65535;
            int rc = quantize_dispatch(reinterpret_cast<const char*>(x) + (long long)n0 * pixels * C * (in16 ? 2 : 4), ths + n0,
                                       qx + (long long)n0 * wpi * bits, btn ? btn + n0 : nullptr,
                                       bits, nn, H, W, C, stream, n0 == 0 ? extras : nullptr, in16);
            if (rc != TAB_OK) return rc;
        }
        return TAB_OK;
    }
    const bool fast = (C % 64 == 0) && ((reinterpret_cast<uintptr_t>(x) & 31) == 0);
    uint64_t* q = reinterpret_cast<uint64_t*>(qx);
    if (fast) {
        // CTAs per image: every CTA the same whole number of 128-word steps (a ragged last step, or a nearly empty extra
        // wave, costs a whole step's time), at most about six waves of eight CTAs per SM over all images
        const long long words_per_step = in16 ? 2 * QWORDS_PER_ITER : QWORDS_PER_ITER;
        const long long steps = (wpi + words_per_step - 1) / words_per_step;
        const long long cap = 148LL * 8 * 6;
        const long long iters = ((long long)N * steps + cap - 1) / cap;    // steps per CTA
        long long per_image = (steps + iters - 1) / iters;
        if (per_image < 1) per_image = 1;
        dim3 grid((unsigned)per_image, (unsigned)N);
        if (in16) {
            if (bits == 2) return launch_pdl(quantize_c64_kernel<2, true>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, wpi, ex);
            return launch_pdl(quantize_c64_kernel<1, true>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, wpi, ex);
        }
        if (bits == 2) return launch_pdl(quantize_c64_kernel<2, false>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, wpi, ex);
        return launch_pdl(quantize_c64_kernel<1, false>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, wpi, ex);
    } else {
        long long steps = (wpi + (QTHREADS / 32) - 1) / (QTHREADS / 32);
        long long per_image = steps;
        const long long target_total = 148LL * 8 * 8;
        if ((long long)N * per_image > target_total) {
            per_image = (target_total + N - 1) / N;
            if (per_image < 1) per_image = 1;
            if (per_image > steps) per_image = steps;
        }
        dim3 grid((unsigned)per_image, (unsigned)N);
        if (in16) {
            if (bits == 2) return launch_pdl(quantize_generic_kernel<2, true>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, pixels, C, PC, ex);
            return launch_pdl(quantize_generic_kernel<1, true>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, pixels, C, PC, ex);
        }
        if (bits == 2) return launch_pdl(quantize_generic_kernel<2, false>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, pixels, C, PC, ex);
        return launch_pdl(quantize_generic_kernel<1, false>, grid, dim3(QTHREADS), 0, stream, x, ths, q, btn, pixels, C, PC, ex);
    }
}

// ---- thresholds and bit-planes of a tensor in one launch ----------------------------------------------------------------
// What every caller of Quantize does first - thresholds[n] = scale * mean|x[n]| (the reference leaves it to framework ops) -
// and the quantisation against them, as two phases of one persistent grid: per-image sums of |x| (double atomics), a
// grid-wide counter (all CTAs are resident: the grid is sized by the occupancy calculator; the wait is bounded and
// reports in *status), then every CTA quantises, last unit first, the units it has just summed - the end of its share is
// what the L2 still holds.  A unit is one CTA step of 128 words of one image.
constexpr uint32_t QA_WAIT_LIMIT = 1u << 22;

template <int BITS>
__global__ void __launch_bounds__(QTHREADS)
quantize_auto_kernel(const float* __restrict__ x, float scale, double* __restrict__ sums, unsigned* __restrict__ bar,
                     float* __restrict__ ths_out, uint64_t* __restrict__ qx, long long words_per_image, int steps_per_image,
                     long long units, int N, int* __restrict__ status) {
    pdl_wait();
    const int byte = threadIdx.x & 7, grp = threadIdx.x >> 3;
    const double per_image = (double)words_per_image * 64.0;
    __shared__ double wsum[QTHREADS / 32];
    __shared__ float s_t;
    // phase 1: sums
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const long long n = u / steps_per_image;
        const long long w0 = (u - n * steps_per_image) * QWORDS_PER_ITER;
        const float* xi = x + n * words_per_image * 64;
        f8 v[QUNROLL];
        bool live[QUNROLL];
#pragma unroll
        for (int k = 0; k < QUNROLL; k++) {
            const long long w = w0 + k * (QTHREADS / 8) + grp;
            live[k] = w < words_per_image;
            if (live[k]) v[k] = ld_stream_f8(xi + w * 64 + byte * 8);
        }
        double acc = 0.0;
#pragma unroll
        for (int k = 0; k < QUNROLL; k++)
            if (live[k]) {
                const float* q = v[k].v;
                acc += (((double)fabsf(q[0]) + (double)fabsf(q[1])) + ((double)fabsf(q[2]) + (double)fabsf(q[3]))) +
                       (((double)fabsf(q[4]) + (double)fabsf(q[5])) + ((double)fabsf(q[6]) + (double)fabsf(q[7])));
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        __syncthreads();                                      // wsum of the previous unit has been read
        if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
#pragma unroll
            for (int i = 0; i < QTHREADS / 32; i++) t += wsum[i];
            atomicAdd(sums + n, t);
        }
    }
    // grid-wide counter
    __threadfence();
    __syncthreads();
    int flag = 0;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        bool ok = false;
        for (uint32_t i = 0; i < QA_WAIT_LIMIT && !ok; i++) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
            ok = seen >= gridDim.x;
            if (!ok) __nanosleep(100);
        }
        if (!ok && status) atomicExch(status, 22);
        flag = ok ? 1 : 0;
    }
    if (!__syncthreads_or(flag)) return;
    if (blockIdx.x == 0 && ths_out)
        for (int n = threadIdx.x; n < N; n += QTHREADS) ths_out[n] = (float)((double)scale * (__ldcg(sums + n) / per_image));
    // phase 2: the CTA's units again, last first
    const long long mine = units > blockIdx.x ? (units - 1 - blockIdx.x) / gridDim.x : -1;      // index of its last unit
    for (long long k = mine; k >= 0; k--) {
        const long long u = blockIdx.x + k * gridDim.x;
        const long long n = u / steps_per_image;
        const long long w0 = (u - n * steps_per_image) * QWORDS_PER_ITER;
        __syncthreads();
        if (threadIdx.x == 0) s_t = (float)((double)scale * (__ldcg(sums + n) / per_image));
        __syncthreads();
        const float t = s_t, nt = -t;
        const float* xi = x + n * words_per_image * 64;
        unsigned char* qi = reinterpret_cast<unsigned char*>(qx + n * words_per_image * BITS);
        f8 v[QUNROLL];
        long long w[QUNROLL];
#pragma unroll
        for (int q = 0; q < QUNROLL; q++) {
            w[q] = w0 + q * (QTHREADS / 8) + grp;
            if (w[q] < words_per_image) v[q] = ld_stream_f8(xi + w[q] * 64 + byte * 8);
        }
#pragma unroll
        for (int q = 0; q < QUNROLL; q++) {
            if (w[q] >= words_per_image) continue;
            if (BITS == 2) {
                unsigned pos = 0, neg = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    pos |= (v[q].v[i] > t) ? (1u << i) : 0u;
                    neg |= (v[q].v[i] < nt) ? (1u << i) : 0u;
                }
                neg &= ~pos;
                unsigned char* o = qi + w[q] * 16 + byte;
                o[0] = (unsigned char)neg;
                o[8] = (unsigned char)(pos | neg);
            } else {
                unsigned b = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) b |= (v[q].v[i] < t) ? (1u << i) : 0u;
                qi[w[q] * 8 + byte] = (unsigned char)b;
            }
        }
    }
    // the CTA that gets here last leaves the state block zero again (every CTA has read the sums it needs)
    __syncthreads();
    flag = 0;
    if (threadIdx.x == 0) flag = (atomicAdd(bar + 1, 1u) == gridDim.x - 1u) ? 1 : 0;
    if (__syncthreads_or(flag)) {
        for (int n = threadIdx.x; n < N; n += QTHREADS) sums[n] = 0.0;
        if (threadIdx.x == 0) { bar[0] = 0u; bar[1] = 0u; }
    }
    pdl_launch_dependents();
}

// TAB_E_TOO_LARGE: the caller runs the separate launches instead (C not a multiple of 64, unaligned x).
int quantize_auto_dispatch(const float* x, float scale, double* sums, unsigned* bar, float* ths_out, int64_t* qx, int bits,
                           int N, int H, int W, int C, int* status, cudaStream_t stream) {
    const long long wpi = (long long)H * W * (C / 64);
    if (C % 64 != 0 || (reinterpret_cast<uintptr_t>(x) & 31) || wpi == 0 || N == 0) return TAB_E_TOO_LARGE;
    const long long spi = (wpi + QWORDS_PER_ITER - 1) / QWORDS_PER_ITER;
    if (spi >= (1LL << 31)) return TAB_E_TOO_LARGE;
    const long long units = spi * N;
    static std::mutex mu;
    static int capacity[64][2] = {};                          // resident CTAs per device, per bitwidth
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TAB_E_TOO_LARGE;
    int cap = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        int& c = capacity[dev][bits == 2 ? 1 : 0];
        if (!c) {
            int per_sm = 0, sms = 0;
            cudaError_t e = bits == 2 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_auto_kernel<2>, QTHREADS, 0)
                                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_auto_kernel<1>, QTHREADS, 0);
            if (e != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return record_cuda_error(cudaGetLastError());
            c = per_sm * sms;
        }
        cap = c;
    }
    if (cap < 1) return TAB_E_TOO_LARGE;
    const unsigned grid = (unsigned)(units < cap ? units : cap);
    uint64_t* q = reinterpret_cast<uint64_t*>(qx);
    if (bits == 2) return launch_pdl(quantize_auto_kernel<2>, dim3(grid), dim3(QTHREADS), 0, stream, x, scale, sums, bar, ths_out, q, wpi, (int)spi, units, N, status);
    return launch_pdl(quantize_auto_kernel<1>, dim3(grid), dim3(QTHREADS), 0, stream, x, scale, sums, bar, ths_out, q, wpi, (int)spi, units, N, status);
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

}  // namespace tab
