// Helpers for chaining TAB convolutions: residual add and the per-image threshold scale*mean|x| that
// the next layer's quantiser needs, in one pass over the activations.  The reference leaves both to
// the caller (its demo notebook computes thresholds with framework ops), so these have no counterpart
// there.  Sums are accumulated in double with integer-like exactness: convolution outputs are
// integer-valued, so every partial sum is exactly representable and the result does not depend on
// the order of the atomic adds.
#include "tab_kernels.cuh"

namespace tab {

constexpr int RTHREADS = 256;

template <bool VEC, bool ADD>
__global__ void __launch_bounds__(RTHREADS)
residual_abs_sum_kernel(float* __restrict__ y, const float* __restrict__ r, double* __restrict__ sums,
                        long long per_image) {
    const int n = blockIdx.y;
    float* yi = y + (long long)n * per_image;
    const float* ri = ADD ? r + (long long)n * per_image : nullptr;
    double acc = 0.0;
    const long long stride = (long long)gridDim.x * RTHREADS;
    if (VEC) {
        const long long n4 = per_image >> 2;
        float4* y4 = reinterpret_cast<float4*>(yi);
        const float4* r4 = reinterpret_cast<const float4*>(ri);
        // four loads in flight per thread (a streaming pass lives on the bytes it has in flight); the sum takes the
        // elements in the same order as a one-at-a-time loop
        for (long long i0 = (long long)blockIdx.x * RTHREADS + threadIdx.x; i0 < n4; i0 += 4 * stride) {
            float4 v[4], q[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const long long i = i0 + u * stride;
                if (i < n4) { v[u] = y4[i]; if (ADD) q[u] = __ldg(r4 + i); }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const long long i = i0 + u * stride;
                if (i >= n4) break;
                if (ADD) {
                    v[u].x += q[u].x; v[u].y += q[u].y; v[u].z += q[u].z; v[u].w += q[u].w;
                    y4[i] = v[u];
                }
                acc += ((double)fabsf(v[u].x) + (double)fabsf(v[u].y)) + ((double)fabsf(v[u].z) + (double)fabsf(v[u].w));
            }
        }
    } else {
        for (long long i = (long long)blockIdx.x * RTHREADS + threadIdx.x; i < per_image; i += stride) {
            float v = yi[i];
            if (ADD) { v += __ldg(ri + i); yi[i] = v; }
            acc += (double)fabsf(v);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    __shared__ double wsum[RTHREADS / 32];
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
#pragma unroll
        for (int i = 0; i < RTHREADS / 32; i++) t += wsum[i];
        if (sums) atomicAdd(sums + n, t);
    }
}

__global__ void threshold_finalize_kernel(const double* __restrict__ sums, float* __restrict__ ths,
                                          float scale, double per_image, int N) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n < N) ths[n] = (float)((double)scale * (sums[n] / per_image));
}

}  // namespace tab

namespace tab {

// y += residual (optional), sums[n] += sum |y[n]| (sums may be null when only the addition is wanted).
int residual_abs_sum_dispatch(float* y, const float* residual, double* sums, int N, long long per_image, cudaStream_t s) {
    if (per_image <= 0 || N <= 0) return TAB_OK;
    const bool vec = (per_image % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(residual) & 15) == 0);
    const long long items = vec ? per_image / 4 : per_image;
    long long per = (items + RTHREADS * 4 - 1) / (RTHREADS * 4);
    const long long cap = (148LL * 8 * 2 + N - 1) / N;
    if (per > cap) per = cap;
    if (per < 1) per = 1;
    for (int n0 = 0; n0 < N; n0 += 65535) {
        const int nn = (N - n0 < 65535) ? N - n0 : 65535;
        dim3 grid((unsigned)per, (unsigned)nn);
        float* yy = y + (long long)n0 * per_image;
        const float* rr = residual ? residual + (long long)n0 * per_image : nullptr;
        double* ss = sums ? sums + n0 : nullptr;
        if (vec) {
            if (rr) residual_abs_sum_kernel<true, true><<<grid, RTHREADS, 0, s>>>(yy, rr, ss, per_image);
            else residual_abs_sum_kernel<true, false><<<grid, RTHREADS, 0, s>>>(yy, rr, ss, per_image);
        } else {
            if (rr) residual_abs_sum_kernel<false, true><<<grid, RTHREADS, 0, s>>>(yy, rr, ss, per_image);
            else residual_abs_sum_kernel<false, false><<<grid, RTHREADS, 0, s>>>(yy, rr, ss, per_image);
        }
        int rc = check_launch();
        if (rc != TAB_OK) return rc;
    }
    return TAB_OK;
}

}  // namespace tab

using namespace tab;

extern "C" int tab_threshold_from_sums_launch(const double* sums, float* ths, float scale, int N, long long per_image,
                                              tab_stream_t stream) {
    if (N < 0 || per_image < 0) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (!sums || !ths) return TAB_E_NULL_POINTER;
    threshold_finalize_kernel<<<(N + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        sums, ths, scale, per_image > 0 ? (double)per_image : 1.0, N);
    return check_launch();
}


extern "C" int tab_residual_threshold_launch(float* y, const float* residual, float* ths, double* sums,
                                             float scale, int N, long long per_image, tab_stream_t stream) {
    if (N < 0 || per_image < 0) return TAB_E_BAD_ARGUMENT;
    if (N == 0) return TAB_OK;
    if (!ths || !sums || (per_image > 0 && !y)) return TAB_E_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(y) & 3) || (reinterpret_cast<uintptr_t>(residual) & 3) ||
        (reinterpret_cast<uintptr_t>(ths) & 3) || (reinterpret_cast<uintptr_t>(sums) & 7))
        return TAB_E_ALIGNMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(sums, 0, sizeof(double) * (size_t)N, s);
    if (e != cudaSuccess) return record_cuda_error(e);
    int rc = residual_abs_sum_dispatch(y, residual, sums, N, per_image, s);
    if (rc != TAB_OK) return rc;
    threshold_finalize_kernel<<<(N + 255) / 256, 256, 0, s>>>(sums, ths, scale, per_image > 0 ? (double)per_image : 1.0, N);
    return check_launch();
}
