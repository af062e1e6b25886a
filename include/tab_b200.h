/*
 * tab_b200 — C ABI of the B200 (sm_100a) implementation of TAB's ternary/binary inference hot path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the given CUDA stream and
 * returns immediately (no host synchronisation).  Return value: 0 on success, a negative TAB_E_* code
 * otherwise; nothing is thrown across this boundary.  None of the *_launch functions allocates or
 * frees device memory: scratch is a caller-provided workspace.  The library keeps no mutable global state
 * besides per-thread settings, a per-device error record and caches of immutable driver objects.
 *
 * Data formats (identical to the reference CUDA backend):
 *   x    float32, N·H·W·C elements in N,H,W,C order                       (TAB_GEMM.cu:184,231)
 *   ths  float32[N], one threshold per image / per filter                   (TAB_GPU.cpp:23,49)
 *   qx   int64  [N][H][W][PC][bits], PC = ceil(C/64); channel c is bit c%64 (LSB first) of word c/64;
 *        bits == 2: plane 0 = sign (1 means -1), plane 1 = magnitude (1 means non-zero);
 *        bits == 1: the single plane holds 1 for -1 and 0 for +1           (TAB_GEMM.cu:184-206,231-245)
 *   btn  int32  [N], popcount of the magnitude plane of every n            (TAB_GEMM.cu:150-160)
 *   y    float32, physical order [N][OH][OW][KN] (the reference relabels this buffer as
 *        shape {N,KN,OH,OW} without permuting it)                           (TAB_GEMM.cu:53,509,526)
 */
#ifndef TAB_B200_H_
#define TAB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same object as cudaStream_t; declared here so that C callers need no CUDA headers. */
typedef struct CUstream_st* tab_stream_t;

enum {
    TAB_OK = 0,
    TAB_E_BAD_ARGUMENT = -1,   /* a size, type or bitwidth is out of range */
    TAB_E_NULL_POINTER = -2,   /* a required pointer is NULL */
    TAB_E_WORKSPACE = -3,      /* workspace smaller than tab_conv2d_workspace_bytes() or misaligned */
    TAB_E_CUDA = -4,           /* the CUDA runtime reported an error; see tab_last_cuda_error() */
    TAB_E_TOO_LARGE = -5,      /* a size exceeds what an entry point supports */
    TAB_E_ALIGNMENT = -6       /* a pointer is not aligned to its element type */
};

/* Human-readable text for a TAB_E_* code (static storage). */
const char* tab_error_string(int code);
/* cudaError_t value of the most recent CUDA failure seen by this library on the calling thread. */
int tab_last_cuda_error(void);
/* Library version: major*10000 + minor*100 + patch. */
int tab_version(void);

/*
 * Threshold-quantise and bit-pack (replaces QuanWithCuda_TAB, TAB_GEMM.cu:250-322, and its kernels
 * TerOnlyKernel :163-208, BinOnlyKernel :211-247, BTN_Weight :150-160).
 * bitwidth == 1 -> binary {+1,-1} (bit = x < ths[n]); anything else -> ternary {+1,0,-1}
 * (x > ths[n] -> +1, else x < -ths[n] -> -1, else 0).
 * qx receives N·H·W·PC·bits words; btn receives N counts (zero for bitwidth 1).  btn may be NULL, in
 * which case the counts are not produced.  btn is cleared by this call; it need not be pre-zeroed.
 */
int tab_quantize_launch(const float* x, const float* ths, int64_t* qx, int32_t* btn,
                        int bitwidth, int N, int H, int W, int C, tab_stream_t stream);

/*
 * Bytes of scratch tab_conv2d_launch needs for these sizes, whichever compute path is selected: the activations'
 * bit-planes (N*H*W*ceil(C/64) words per plane), the byte-expanded weights of the tensor-core path and a 256-byte
 * completion counter.  Same geometry arguments, in the same order, as tab_conv2d_launch.  Returns 0 for invalid arguments.
 */
size_t tab_conv2d_workspace_bytes(int type, int p1, int p2, int s1, int s2,
                                  int N, int H, int W, int C, int KN, int KH, int KW);

/*
 * Compute path of the convolution entry points, per calling thread (results are identical bit for bit):
 *   TAB_PATH_AUTO (default)   the bit-planes are expanded to int8 inside a persistent tcgen05 kernel (s8 MMA, exact);
 *                             shapes that kernel does not cover fall back to TAB_PATH_POPCOUNT
 *   TAB_PATH_POPCOUNT         bit-packed LOP3/POPC kernel with a carry-save popcount tree - the reference's formulation
 *                             (TAB_GEMM.cu:25-147); this is also what tab_conv2d_packed_launch runs
 *   TAB_PATH_POPCOUNT_PLAIN   the same kernel with one POPC per word
 * Returns the previous setting, or TAB_E_BAD_ARGUMENT.
 */
enum { TAB_PATH_AUTO = 0, TAB_PATH_POPCOUNT = 1, TAB_PATH_POPCOUNT_PLAIN = 2 };
int tab_conv2d_set_path(int path);
/* Name and tile of the kernel the calling thread's most recent tensor-core convolution launched ("none" before the first, or
   when the last convolution ran the popcount kernel), e.g. "conv_umma_persist_kernel<1,256,4,0,2,0> grid 15x15 halves +next":
   template arguments (row blocks per tile, filters per tile, ring stages, resident filters, fused epilogue, TMA epilogue,
   ",pair" on clusters of two CTAs), the virtual grid per image, " halves" when the last round of tiles is worked as half-width
   tiles, " +next" when the launch also quantises its result for the next layer.  Static storage per thread. */
const char* tab_last_conv_kernel(void);
/*
 * Every wait inside the tensor-core kernel and inside tab_quantize_auto_launch's kernel is bounded; a wait that ran out makes
 * the kernel record a code and return early, leaving its outputs incomplete.  This call synchronises the current device,
 * returns that code (0 = none; 11-17: a role of the tensor-core kernel gave up on an mbarrier; 21, 22: the grid-wide
 * meeting point of tab_conv2d_bits_next_launch / tab_quantize_auto_launch, which needs the launch's CTAs resident together -
 * other work occupying the device for tenths of a second can cause it) and clears it.  A non-zero code invalidates the
 * outputs of every launch on the device since the previous call.
 */
int tab_device_status(void);

/*
 * Quantise activations, then convolve with pre-quantised weights as an implicit-im2col GEMM
 * (replaces ConvWithCuda_TAB, TAB_GEMM.cu:325-527: TerOnly/BinOnlyKernel, PadKernel TAB_GEMM.cuh:73-89,
 * Img2RowKernel :92-115, GEMMWithCuda :22-66 and TNN/TBN/BTN/BNNGEMM TAB_GEMM.cu:25-147).
 * type: 0 TNN, 1 TBN, 2 BTN, 3 BNN.  qw is the tab_quantize_launch output of the weights
 * [KN][KH][KW][C] at bitwidth 2 for types 0,2 and bitwidth 1 for types 1,3.  btn (int32[KN]) is read
 * for type 2 only and may be NULL otherwise.  OH = (H + 2*p1 - KH + 1) / s1, OW likewise (integer
 * division, TAB_GEMM.cu:354-357).  y receives N*OH*OW*KN floats.  workspace must be 256-byte aligned.
 * Two launches: the quantiser (which also expands the weights to bytes) and the GEMM.  The first tensor-core call on a
 * device looks up a driver entry point and a device symbol: make it outside any stream capture.
 */
int tab_conv2d_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                      float* y, void* workspace, size_t workspace_bytes, int type,
                      int p1, int p2, int s1, int s2,
                      int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream);

/*
 * tab_conv2d_launch with two optional fusions for chained layers (no counterpart in the reference, whose
 * callers add residuals and compute the next thresholds with framework ops):
 *   residual  float32 [N][OH][OW][KN] or NULL: y = conv(x) + residual
 *   abs_sums  double [N] or NULL: receives sum |y[n]| per image (cleared by this call); pass it to
 *             tab_threshold_from_sums_launch to obtain scale*mean|y| as the next layer's thresholds.
 * On the tensor-core path both happen in the GEMM epilogue (no extra pass over y); otherwise one extra
 * pass is made.  Sums are exact (and independent of scheduling) for integer-valued data.
 */
int tab_conv2d_fused_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                            float* y, void* workspace, size_t workspace_bytes, int type,
                            int p1, int p2, int s1, int s2,
                            int N, int H, int W, int C, int KN, int KH, int KW,
                            const float* residual, double* abs_sums, tab_stream_t stream);
/*
 * tab_conv2d_fused_launch that also finishes the next layer's thresholds (no counterpart in the reference):
 *   next_ths   float [N] or NULL: receives next_scale * abs_sums[n] / (KN*OH*OW), i.e. next_scale * mean|y[n]|;
 *              needs abs_sums.  On the tensor-core path the GEMM kernel's last CTA writes it, so a chained layer
 *              costs two launches; on the other paths it is tab_threshold_from_sums_launch after the sums.
 */
int tab_conv2d_chain_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                            float* y, void* workspace, size_t workspace_bytes, int type,
                            int p1, int p2, int s1, int s2,
                            int N, int H, int W, int C, int KN, int KH, int KW,
                            const float* residual, double* abs_sums, float* next_ths, float next_scale,
                            tab_stream_t stream);
/* ths[n] = scale * sums[n] / per_image. */
int tab_threshold_from_sums_launch(const double* sums, float* ths, float scale, int N, long long per_image,
                                   tab_stream_t stream);

/*
 * Same convolution on activations that are already bit-packed (the qx layout above with bits = 2 for
 * types 0,1 and bits = 1 for types 2,3), by the bit-packed LOP3/POPC kernel.  This is the GEMM stage of the
 * reference on its own (GEMMWithCuda, TAB_GEMM.cuh:22-66, with padding and im2row folded in); it needs no workspace.
 */
int tab_conv2d_packed_launch(const int64_t* qx, const int64_t* qw, const int32_t* btn, float* y,
                             int type, int p1, int p2, int s1, int s2,
                             int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream);

/*
 * The stages of the tensor-core path on their own, for callers that keep prepared weights between calls (weights
 * are constant during inference) or feed several convolutions from one quantised tensor.  No counterpart in the
 * reference, which re-reads packed weights and re-quantises fp32 activations in every call (TAB_GEMM.cu:419-426).
 *
 *   tab_expand_weights_launch   tab_quantize_launch's packed weights (bitwidth 1 or 2) -> int8 {-1,0,+1},
 *                               [KN][KH][KW][Cp] with Cp = 64*ceil(C/64), channel padding 0; w8 16-byte aligned.
 *   tab_conv2d_bits_launch      the GEMM stage: activations as tab_quantize_launch wrote them (qx, bitwidth 2 for types
 *                               0,1 and 1 for types 2,3; 16-byte aligned), weights from tab_expand_weights_launch.
 *                               y and residual 16-byte aligned.  Optional chaining as in tab_conv2d_chain_launch:
 *                               y = conv + residual; next_ths[n] = next_scale * mean|y[n]|, which needs `state`:
 *                               tab_conv2d_state_bytes(N) bytes, 8-byte aligned, that the caller zeroes once
 *                               (cudaMemsetAsync) before its first use; every call leaves it zeroed again, so one state
 *                               block serves any number of calls that are ordered on a stream.  One launch.
 *                               Returns TAB_E_TOO_LARGE for shapes the tensor-core kernel does not cover (a patch of
 *                               128 + (KH-1)/s1*VW + (KW-1)/s2 rows of 128 bytes that does not fit shared memory beside
 *                               the filters, or index ranges beyond 2^31): use tab_conv2d_packed_launch for those.
 */
int tab_expand_weights_launch(const int64_t* qw, int8_t* w8, int bitwidth, int KN, int KH, int KW, int C,
                              tab_stream_t stream);
size_t tab_conv2d_state_bytes(int N);
int tab_conv2d_bits_launch(const int64_t* qx, const int8_t* w8, float* y, int type, int p1, int p2, int s1, int s2,
                           int N, int H, int W, int C, int KN, int KH, int KW,
                           const float* residual, void* state, float* next_ths, float next_scale, tab_stream_t stream);
/*
 * Compact intermediate for chained layers (no counterpart in the reference, whose every tensor between layers is fp32):
 * a convolution's result is integer-valued with |y| <= KH*KW*C, so where its only reader is the next layer's quantiser it
 * can travel as int16 - half the bytes written and read back.  The results are the same numbers.
 *   tab_conv2d_bits_i16_launch   tab_conv2d_bits_launch without a residual, writing int16 [N][OH][OW][KN] (16-byte aligned);
 *                                TAB_E_TOO_LARGE when KH*KW*C > 32767
 *   tab_quantize_i16_launch      tab_quantize_launch on such a tensor (same compares, on the integers converted to float);
 *                                no btn output
 */
int tab_conv2d_bits_i16_launch(const int64_t* qx, const int8_t* w8, int16_t* y16, int type, int p1, int p2, int s1, int s2,
                               int N, int H, int W, int C, int KN, int KH, int KW,
                               void* state, float* next_ths, float next_scale, tab_stream_t stream);
int tab_quantize_i16_launch(const int16_t* x, const float* ths, int64_t* qx, int bitwidth, int N, int H, int W, int C,
                            tab_stream_t stream);
/*
 * Quantize with the thresholds every caller of the reference computes first, ths[n] = scale * mean|x[n]| (the notebook does it
 * with framework reductions before calling Quantize, TAB_GPU.cpp:53-58 takes them as an argument): one launch sums |x| per
 * image, meets at a counter in the state block (a bounded wait, as in tab_conv2d_bits_next_launch), writes the thresholds
 * to ths [N] and the bit-planes to qx, [N][H][W][ceil(C/64)][bitwidth] as tab_quantize_launch does (no btn output).  state:
 * tab_conv2d_state_bytes(N) bytes, zero before the call and zero again after it.  C not a multiple of 64 or x not 32-byte
 * aligned: the same result from three launches.  x is only read.
 */
int tab_quantize_auto_launch(const float* x, float scale, void* state, float* ths, int64_t* qx, int bitwidth,
                             int N, int H, int W, int C, tab_stream_t stream);
/*
 * A chained layer that also hands the next convolution its input: after the GEMM stage (tab_conv2d_bits_launch, or the int16
 * form when y_is_int16) the same launch computes the next thresholds and quantises the result against them into next_qx,
 * [N][OH][OW][ceil(KN/64)][next_bitwidth] 64-bit words - exactly what tab_quantize_launch(y, next_ths, next_qx, ...) writes
 * (TerOnlyKernel / BinOnlyKernel, TAB_GEMM.cu:163-247), without that launch and while most of y is still in the L2.  The CTAs of
 * the grid meet at a counter in the state block in between (a bounded wait; all of them are resident, at most one per SM, as
 * long as no other work holds SMs of the device for as long as the wait's limit of some tenths of a second).  When KN is not a
 * multiple of 64, N > 8192 or next_qx is not 16-byte aligned, the quantiser runs as a launch of its own behind the GEMM stage;
 * the result is the same.  state, next_ths, next_qx are required; residual only with fp32 output.
 */
int tab_conv2d_bits_next_launch(const int64_t* qx, const int8_t* w8, void* y, int y_is_int16, int type, int p1, int p2, int s1, int s2,
                                int N, int H, int W, int C, int KN, int KH, int KW,
                                const float* residual, void* state, float* next_ths, float next_scale,
                                int64_t* next_qx, int next_bitwidth, tab_stream_t stream);

/*
 * tab_conv2d_launch without a workspace argument.  No counterpart in the reference (its host code calls
 * cudaMalloc/cudaFree for scratch on every convolution, TAB_GEMM.cu:391-407,522-524).
 *
 * For callers that cannot allocate device memory: programs whose GPU memory belongs entirely to another
 * component's pool, language bindings that can forward buffers they were given but not create new
 * ones, and loops where an allocation's implicit device synchronisation is not acceptable.  The
 * bit-packed activations go into a fixed array of TAB_STATIC_SCRATCH_BYTES that is part of the library
 * image on every GPU that loads it (held until the process exits).  This function calls no cudaMalloc,
 * cudaFree or other allocating routine.
 *
 * Limits and rules:
 *   - N*H*W*ceil(C/64)*planes*8 bytes (planes = 2 for types 0,1; 1 for types 2,3) must not exceed
 *     TAB_STATIC_SCRATCH_BYTES, else TAB_E_TOO_LARGE is returned and nothing is launched.
 *   - The first call on each device looks up the array's device address (a one-time set-up under a lock);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU
 *     (different streams without an ordering between them, or different host threads) race on it and
 *     give wrong results; serialise them on one stream or with events.
 *   - The array keeps whatever the last call left; this function overwrites every word it later reads,
 *     so no clearing is needed between calls.
 *   - This entry point always runs the bit-packed LOP3/POPC kernel (TAB_PATH_POPCOUNT, about 150 binary TOP/s on a
 *     B200 against several hundred for the tensor-core path of tab_conv2d_launch): the tensor-core path also needs
 *     byte-expanded weights, which would not fit a modest fixed array.
 * Arguments, checks, error codes and results are otherwise exactly those of tab_conv2d_launch.
 */
#define TAB_STATIC_SCRATCH_BYTES (16u << 20)
int tab_conv2d_static_launch(const float* x, const int64_t* qw, const float* ths, const int32_t* btn,
                             float* y, int type, int p1, int p2, int s1, int s2,
                             int N, int H, int W, int C, int KN, int KH, int KW, tab_stream_t stream);

/*
 * Chaining helper: y += residual (skipped when residual is NULL), then ths[n] = scale * mean|y[n]| over
 * the per_image floats of image n - the threshold the next layer's quantiser takes.  sums is scratch
 * for N doubles (cleared by this call).  Convolution outputs are integer-valued, so the double sums are
 * exact and the thresholds do not depend on scheduling.  The reference leaves residuals and thresholds
 * to the caller (its notebook computes them with framework ops): no counterpart there.
 */
int tab_residual_threshold_launch(float* y, const float* residual, float* ths, double* sums,
                                  float scale, int N, long long per_image, tab_stream_t stream);

/*
 * Register-only micro-benchmark of the pipes used by the convolution, for roofline
 * denominators: runs `iters` rounds on a grid that fills the device and writes elapsed-independent
 * checksums to `sink` (at least tab_pipe_probe_sink_bytes() bytes).  kind: 0 = 32-bit POPC,
 * 1 = LOP3, 2 = s8 mma.sync m16n8k32, 3 / 4 = 1-bit mma.sync m16n8k256 and.popc / xor.popc, 5 / 6 / 7 = tcgen05.mma kind::i8
 * 128 x 64 / 128 / 256 x 32 issued back to back from shared memory.  *ops_out receives the number of lane-level
 * instructions of that kind issued (kinds 2-7: multiply-adds * 2); the caller times the call with CUDA events.  Has no
 * counterpart in the reference.
 */
size_t tab_pipe_probe_sink_bytes(void);
int tab_pipe_probe_launch(int kind, int iters, void* sink, double* ops_out, tab_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TAB_B200_H_ */
