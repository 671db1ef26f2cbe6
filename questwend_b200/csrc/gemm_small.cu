// Matrix product for a few rows:  y[M,N] = x[M,K] W[N,K]^T (+ residual), 32-bit sums.
// W is read once, row by row, with 16-byte loads; one warp forms one output column for
// up to 8 rows of x at a time.  This is the weight-streaming product of a decode step
// with a small batch (the reference uses its own mul_mat_vec_f / mul_mat_f there,
// ggml-cuda/mmvf.cu, mmf.cuh, chosen in ggml-cuda.cu:1812-1866).  x and W share a dtype
// (float or bfloat16); y and the residual are float; y may be the residual itself.
#include "common.cuh"

template <typename T, int MT, bool VECTOR>
__global__ void gemm_small_kernel(const T* __restrict__ x, const T* __restrict__ W, const float* residual,
                                  float* y, int M0, int M, int N, int K) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int VEC = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= N) return;
    const T* wrow = W + (size_t)n * K;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    if (VECTOR) {
        const int nchunk = K / VEC;
        const Vec16<T>* wv = reinterpret_cast<const Vec16<T>*>(wrow);
        for (int c = lane; c < nchunk; c += 32) {
            float wf[VEC];
            wv[c].get(wf);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (M0 + m < M) {
                    float xf[VEC];
                    reinterpret_cast<const Vec16<T>*>(x + (size_t)(M0 + m) * K)[c].get(xf);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[m] += wf[e] * xf[e];
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float w = to_f32(wrow[k]);
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (M0 + m < M) acc[m] += w * to_f32(x[(size_t)(M0 + m) * K + k]);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float total = warp_sum(acc[m]);
        if (lane == 0 && M0 + m < M) {
            const size_t at = (size_t)(M0 + m) * N + n;
            y[at] = residual ? residual[at] + total : total;
        }
    }
}

template <typename T>
static int launch_small(const void* x, const void* W, const float* residual, float* y, int M, int N, int K,
                        cudaStream_t stream) {
    constexpr int VEC = Vec16<T>::N;
    const bool vec = (K % VEC == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0);
    const int warps = 8;
    const int grid = (N + warps - 1) / warps;
    for (int m0 = 0; m0 < M; m0 += 8) {
        const int left = M - m0;
#define QWB_SMALL(MT)                                                                                             \
    do {                                                                                                          \
        if (vec) qwb_launch(gemm_small_kernel<T, MT, true>, grid, warps * 32, 0, stream, (const T*)x, (const T*)W, residual, y, m0, M, N, K); \
        else qwb_launch(gemm_small_kernel<T, MT, false>, grid, warps * 32, 0, stream, (const T*)x, (const T*)W, residual, y, m0, M, N, K);    \
    } while (0)
        if (left >= 5) QWB_SMALL(8);
        else if (left >= 3) QWB_SMALL(4);
        else if (left == 2) QWB_SMALL(2);
        else QWB_SMALL(1);
#undef QWB_SMALL
        if (int rc = qwb_check_launch("gemm_small")) return rc;
    }
    return 0;
}

extern "C" int qwb_gemm_small(const void* x, const void* W, const float* residual, float* y, int dtype, int M,
                              int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return qwb_fail(QWB_ERR_ARG, "gemm_small: bad inner size %d", K);
    if (M > 64) return qwb_fail(QWB_ERR_ARG, "gemm_small: %d rows; this kernel is for at most 64", M);
    if (dtype == QWB_DT_F32) return launch_small<float>(x, W, residual, y, M, N, K, stream);
    if (dtype == QWB_DT_BF16) return launch_small<bf16>(x, W, residual, y, M, N, K, stream);
    return qwb_fail(QWB_ERR_ARG, "gemm_small: unknown dtype %d", dtype);
}
