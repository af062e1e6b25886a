// Building blocks of the tcgen05 (5th-generation tensor core) kernels: mbarrier, TMA and tcgen05 wrappers in inline
// PTX, the shared-memory and instruction descriptors of kind::i8 MMAs, and the parameter block of the convolution.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tab {

constexpr int UTM = 128;                     // rows of one MMA (= TMEM lanes)
constexpr int IROW = 128;                    // bytes of K per shared-memory operand row (two 64-channel words)
constexpr uint32_t UMMA_WAIT_LIMIT = 1u << 16;       // about a quarter of a second per wait
constexpr int UMMA_SMEM_MAX = 227 * 1024;    // dynamic shared memory a kernel may ask for (one CTA per SM)

// Exact n / d for 0 <= n < 2^31 by one multiply-high and a shift (d >= 1), set up on the host.
struct FastDiv {
    uint32_t mul, shr, d;
#ifdef __CUDACC__
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, mul) >> shr; }
#endif
};
#ifdef __CUDACC__
__device__ __forceinline__ FastDiv make_fastdiv_dev(uint32_t d) {
    FastDiv f = {0u, 0u, d};
    if (d > 1) {
        const uint32_t l = 32u - (uint32_t)__clz((int)(d - 1));           // ceil(log2 d)
        const uint32_t p = 31 + l;
        f.mul = (uint32_t)(((1ull << p) + d - 1) / d);
        f.shr = p - 32;
    }
    return f;
}
#endif
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f = {0u, 0u, d};
    if (d > 1) {
        uint32_t l = 0;
        while ((1ull << l) < d) l++;                                       // ceil(log2 d)
        const uint32_t p = 31 + l;
        f.mul = (uint32_t)(((1ull << p) + d - 1) / d);
        f.shr = p - 32;
    }
    return f;
}

// One convolution as the tensor-core kernel sees it.
//
// Activations are the bit-planes tab_quantize_launch writes, [N][H][W][PC][planes] 64-bit words (TAB_GEMM.cu:196-197);
// weights are bytes {-1,0,+1}, [KN][KH*KW*PC][64], channel tails 0.  Output positions are enumerated on a *virtual grid*
// per plane: VH x VW positions per image, virtual row R = (n*VH + i)*VW + j.
//   stride 1 (one plane): VH = H + p1, VW = W + p2; position (i, j) is padded pixel (i, j), i.e. input pixel
//     (i - p1, j - p2), and a pixel with i < p1 or j < p2 is padding.  The right padding of a row is the left padding of
//     the next one and the bottom padding of an image is the top padding of the next (all padding holds one value), so
//     tap (kh, kw) of output (oh, ow) is virtual row R(oh, ow) + kh*VW + kw.
//   stride (s1, s2): planes (a, b), a < min(s1, KH), b < min(s2, KW); VH = ceil((H + 2*p1)/s1), VW likewise; position
//     (i, j) of plane (a, b) is padded pixel (s1*i + a, s2*j + b); tap (kh, kw) reads plane (kh % s1, kw % s2) at row
//     offset (kh / s1)*VW + kw / s2.
// Output (n, oh, ow) is virtual row (n*VH + oh)*VW + ow of any plane; rows with oh >= OH or ow >= OW are computed and dropped.
struct TcConvParams {
    const uint64_t* qx;      // activation bit-planes
    const int8_t* w8;        // byte weights
    float* y;                // [M][KN]
    int16_t* y16;            // when not null the result goes here as int16 instead (no residual; |y| <= KH*KW*C must fit)
    const float* residual;   // [M][KN] added to the result, or null
    double* abs_sums;        // [N]: += sum |y| per image, or null
    int N, H, W, C, PC, KN, KH, KW, OH, OW, p1, p2, s1, s2;
    int M, Kw;
    int abits;               // planes of the activations: 2 ternary, 1 binary
    int VH, VW, PA, PB;      // virtual grid of one plane; planes
    int tepi;                // the grid is aligned for the TMA epilogue: a 32-row slab is one box of the output tensor
    FastDiv dVHW, dVW;
    // Optional tail: the CTA that finishes last turns the sums into the next layer's thresholds,
    // ths_out[n] = ths_scale * abs_sums[n] / per_image, and (self_clean) leaves abs_sums and the counter zero again.
    float* ths_out;
    float ths_scale;
    double per_image;
    unsigned* done_counter;  // zero before the launch
    int self_clean;
    // Optional second phase (needs abs_sums and ths_scale): when every CTA has finished its tiles, the grid quantises the
    // result it has just written (y, or y16) against those thresholds into next_qx, bit-planes [M][KN/64][next_bits] as
    // tab_quantize_launch would write them - the next convolution's input, without a kernel of its own and read back
    // while most of it is still in the L2.  KN % 64 == 0.  grid_bar: two words, zero before the launch, zero again after.
    uint64_t* next_qx;
    int next_bits;
    unsigned* grid_bar;
};

#ifdef __CUDACC__

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count) : "memory");
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
// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < UMMA_WAIT_LIMIT; i++)
        if (mbar_try(addr, parity)) return true;
    return false;
}
// Bounded wait by a whole warp; the result is the same in every lane.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t addr, uint32_t parity) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(addr, parity));
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// True in exactly one lane of a converged warp.  Role loops are run by the whole warp with the issuing instructions
// under this predicate, so that loop counters, addresses and descriptors stay warp-uniform values.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// Tiled 2-D tensor-map copy into this CTA's shared memory, completing on an mbarrier.  No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(tmap), "r"(mbar), "r"(x), "r"(y) : "memory");
}
// 4-D tiled copies (float tensors [N][OH][OW][KN], innermost coordinate first).  A load fills out-of-range elements of
// its box with zeros and always delivers the whole box; a store writes only the in-range part of its box.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 :: "r"(dst), "l"(tmap), "r"(mbar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, int c0, int c1, int c2, int c3, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :: "l"(tmap), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk-store groups have not finished READING their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// Waits until all of this thread's bulk-store groups have completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Generic-proxy writes to shared memory made visible to the async proxy (the tensor core reads operands through it).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// High word of a shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart,
// descriptor version 1.  The low word is the operand's shared-memory address >> 4 (18-bit window).
constexpr uint32_t UMMA_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return ((uint64_t)UMMA_DESC_HI << 32) | ((smem_addr & 0x3FFFFu) >> 4);
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
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(cols) : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: lane r of the warp receives row r.
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
// ---- CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) ----------------------------------------------------
// One MMA instruction, issued by the even CTA of the pair, multiplies 256 rows - 128 from each CTA's shared memory, at the
// same offset in both - by N filters of which each CTA holds N/2 (same offset again); each CTA's tensor memory receives the
// accumulators of its own 128 rows.  A CTA thus fetches half of every filter slice.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of all CTAs of the cluster (every thread must execute it).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at this shared-memory offset in CTA `rank` of the cluster (may be the caller's own).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t mbar, uint32_t rank) {
    asm volatile("{\n\t.reg .b32 ra;\n\t"
                 "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
                 "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(mbar), "r"(rank) : "memory");
}
// Bounded wait, by a whole warp, on a barrier that threads of the other CTA arrive on.
__device__ __forceinline__ bool mbar_wait_cluster_warp(uint32_t addr, uint32_t parity) {
    bool ok = false;
    for (uint32_t i = 0; i < UMMA_WAIT_LIMIT && !ok; i++) {
        uint32_t r;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(r) : "r"(addr), "r"(parity) : "memory");
        ok = r != 0;
    }
    return __all_sync(0xFFFFFFFFu, ok);
}
// This CTA's half of a filter slice; the bytes are counted on the even CTA's barrier (bit 24 of a shared::cluster
// address is the CTA's rank within the pair).  No multicast: each CTA copies its own half.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(tmap), "r"(mbar & 0xFEFFFFFFu), "r"(x), "r"(y) : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)((2 * UTM) >> 4) << 24);
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the pair's MMAs issued so far have completed, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(mbar), "h"((uint16_t)3) : "memory");
}
// Executed by the same warp of both CTAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(cols) : "memory");
}

__device__ __forceinline__ void sts_v4(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ int4 lds_v4(uint32_t a) {
    int4 r;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(a) : "memory");
    return r;
}

#endif  // __CUDACC__

}  // namespace tab
