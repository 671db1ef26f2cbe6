// Embedding gather, RMS norm (with the residual sum folded in) and the gated SiLU
// product.  The residual stream and the sums of squares are 32-bit in both engines.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// h[t,:] = float(E[id_t,:]).  A row gather without scaling (the reference:
// core/runtime.cpp:1001, ggml-cuda/getrows.cu:73-102).  An id outside [0, V) writes a
// row of zeros and records the first such token in *bad_token (if given).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                    float* __restrict__ out, int D, int V, int* bad_token) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * D;
    if (id < 0 || id >= V) {
        if (bad_token && threadIdx.x == 0) atomicCAS(bad_token, -1, t);
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * D;
    constexpr int VEC = Vec16<T>::N;
    if (D % VEC == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0) {      // 16 bytes of the row a load
        const Vec16<T>* src = reinterpret_cast<const Vec16<T>*>(row);
        for (int i = threadIdx.x; i < D / VEC; i += blockDim.x) {
            float v[VEC];
            src[i].get(v);
#pragma unroll
            for (int e = 0; e < VEC; e += 4)
                *reinterpret_cast<float4*>(o + (size_t)i * VEC + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
        return;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int qwb_embed_gather(const int* ids, const void* table, int table_dtype, float* out,
                                int T, int D, int V, int* bad_token, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D <= 0 || V <= 0) return qwb_fail(QWB_ERR_ARG, "embed_gather: bad sizes D=%d V=%d", D, V);
    const int block = D >= 1024 ? 256 : 128;
    if (table_dtype == QWB_DT_F32)
        qwb_launch(embed_gather_kernel<float>, T, block, 0, stream, ids, (const float*)table, out, D, V, bad_token);
    else if (table_dtype == QWB_DT_BF16)
        qwb_launch(embed_gather_kernel<bf16>, T, block, 0, stream, ids, (const bf16*)table, out, D, V, bad_token);
    else
        return qwb_fail(QWB_ERR_ARG, "embed_gather: unknown dtype %d", table_dtype);
    return qwb_check_launch("embed_gather");
}

// ---------------------------------------------------------------------------------
// RMS norm over rows of D:  y = v * rsqrt(mean(v^2) + eps) * w,  v = x (+ delta).
// (the reference: core/runtime.cpp:1018-1019, ggml-cuda/norm.cu:76-155.)
//   x      [rows_in, D] float   the residual stream
//   delta  [rows_in, D] float   optional: the sum x + delta is formed in 32-bit first
//   planes [P, rows_in, D] float optional, instead of delta: a product that its kernel left as sums over pieces of k
//                                (gemm_ring's split form); columns 16 t .. 16 t + 15 have plane_count[t] <= 4 planes, which
//                                are added onto x in the order of the planes
//   sum_out[rows_in, D] float   optional: where x + delta is written (may be x itself)
//   rows   [n_rows] int         optional: row r of the output is made from row rows[r]
//   out    [n_rows, D]  float or bfloat16
// One block per output row; the row is kept in shared memory between the two passes.
// ---------------------------------------------------------------------------------
template <typename TOut> struct Pack4;
template <> struct Pack4<float> {
    static __device__ __forceinline__ void store(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <> struct Pack4<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float a, float b, float c, float d) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};

// VEC: rows are a multiple of 4 wide and 16-byte aligned, so everything moves four values at a time.
#define RMS_MAX_PLANES 4
#define RMS_W_FIRST 4             // pieces of the weight a thread asks for before the wait (rows of up to 4,096: all of it)
#define RMS_PLANE_COLS 16
template <typename TOut, bool VEC>
__global__ void rmsnorm_kernel(const float* x, const float* delta, const float* planes,
                               const unsigned char* __restrict__ plane_count, size_t plane_stride,
                               float* sum_out, const float* __restrict__ w, TOut* __restrict__ out,
                               const int* __restrict__ rows, int D, float eps) {
    pdl_launch_dependents();            // the trigger first: the kernel after this one may start before the one before it ends
    // the norm's weight is nobody's output: a thread's first pieces of it are on their way before the wait
    float4 w_first[RMS_W_FIRST];
    if (VEC) {
#pragma unroll
        for (int k = 0; k < RMS_W_FIRST; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            w_first[k] = i < D / 4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * D;
    float ss = 0.f;
    if (VEC) {
        const float4* x4 = reinterpret_cast<const float4*>(x + src);
        const float4* d4 = delta ? reinterpret_cast<const float4*>(delta + src) : nullptr;
        float4* s4 = sum_out ? reinterpret_cast<float4*>(sum_out + src) : nullptr;
        float4* c4 = reinterpret_cast<float4*>(row_cache);
        for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
            // plain loads (x and delta are not __restrict__: never the read-only path, see pdl_wait); with __ldcg a norm
            // of 8 rows of 4,096 took 1.4 us longer under the ring fill of the product that follows (and with a thread's four
            // loads issued together, before the first store, a step took 0.5 % longer)
            float4 v = x4[i];
            if (d4) { const float4 d = d4[i]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
            if (planes) {
                const int n_planes = plane_count[4 * i / RMS_PLANE_COLS];
                const float4* p4 = reinterpret_cast<const float4*>(planes + src) + i;
                float4 d[RMS_MAX_PLANES];
#pragma unroll
                for (int p = 0; p < RMS_MAX_PLANES; ++p)
                    if (p < n_planes) d[p] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p4) + p * plane_stride);
#pragma unroll
                for (int p = 0; p < RMS_MAX_PLANES; ++p)
                    if (p < n_planes) { v.x += d[p].x; v.y += d[p].y; v.z += d[p].z; v.w += d[p].w; }
            }
            if (s4) s4[i] = v;
            c4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = x[src + i];
            if (delta) v += delta[src + i];
            if (planes)
                for (int p = 0, n_planes = plane_count[i / RMS_PLANE_COLS]; p < n_planes; ++p) v += planes[p * plane_stride + src + i];
            if (sum_out) sum_out[src + i] = v;
            row_cache[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, red);
    const float scale = rsqrtf(total / (float)D + eps);
    TOut* o = out + (size_t)r * D;
    if (VEC) {
        const float4* c4 = reinterpret_cast<const float4*>(row_cache);
        const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
        for (int k = 0; k < RMS_W_FIRST; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < D / 4) {
                const float4 v = c4[i], g = w_first[k];
                Pack4<TOut>::store(o + 4 * i, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
            }
        }
        for (int i = threadIdx.x + RMS_W_FIRST * blockDim.x; i < D / 4; i += blockDim.x) {
            const float4 v = c4[i], g = w4[i];
            Pack4<TOut>::store(o + 4 * i, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = from_f32<TOut>(row_cache[i] * scale * w[i]);
    }
}

// Rows of up to 4 x ITERS x 256 values (ITERS 4 or 8: up to 4,096 or 8,192): the row stays in the threads' registers
// between the two passes (a thread's loads are issued together; 2,048 rows of 4,096: 8.6 us against 11.8 through shared
// memory; a decode step of 8 rows 0.5 % faster).
template <typename TOut, int ITERS>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* x, const float* delta, const float* planes, const unsigned char* __restrict__ plane_count,
                    size_t plane_stride, float* sum_out, const float* __restrict__ w, TOut* __restrict__ out,
                    const int* __restrict__ rows, int D, float eps) {
    pdl_launch_dependents();            // the trigger first, and the weight asked for before the wait: as in rmsnorm_kernel
    float4 g[ITERS];
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int i = threadIdx.x + k * 256;
        g[k] = i < D / 4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * D;
    const float4* x4 = reinterpret_cast<const float4*>(x + src);
    const float4* d4 = delta ? reinterpret_cast<const float4*>(delta + src) : nullptr;
    float4 v[ITERS];
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int i = threadIdx.x + k * 256;
        v[k] = i < D / 4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (d4) {
#pragma unroll
        for (int k = 0; k < ITERS; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < D / 4) { const float4 d = d4[i]; v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w; }
        }
    }
    if (planes) {                       // a product left as sums over pieces of k: a column's planes, in their order
#pragma unroll
        for (int k = 0; k < ITERS; ++k) {
            const int i = threadIdx.x + k * 256;
            if (i < D / 4) {
                const int n_planes = plane_count[4 * i / RMS_PLANE_COLS];
                const float* p4 = planes + src + 4 * (size_t)i;
                float4 pv[RMS_MAX_PLANES];
#pragma unroll
                for (int p = 0; p < RMS_MAX_PLANES; ++p)
                    if (p < n_planes) pv[p] = *reinterpret_cast<const float4*>(p4 + p * plane_stride);
#pragma unroll
                for (int p = 0; p < RMS_MAX_PLANES; ++p)
                    if (p < n_planes) { v[k].x += pv[p].x; v[k].y += pv[p].y; v[k].z += pv[p].z; v[k].w += pv[p].w; }
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int i = threadIdx.x + k * 256;
        if (sum_out && i < D / 4) reinterpret_cast<float4*>(sum_out + src)[i] = v[k];
        ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
    const float scale = rsqrtf(block_sum(ss, red) / (float)D + eps);
    TOut* o = out + (size_t)r * D;
#pragma unroll
    for (int k = 0; k < ITERS; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < D / 4)
            Pack4<TOut>::store(o + 4 * i, v[k].x * scale * g[k].x, v[k].y * scale * g[k].y, v[k].z * scale * g[k].z, v[k].w * scale * g[k].w);
    }
}

template <typename TOut>
static int launch_rmsnorm(const float* x, const float* delta, const float* planes, const unsigned char* plane_count,
                          size_t plane_stride, float* sum_out, const float* w, TOut* out, const int* rows,
                          int n_rows, int D, float eps, size_t smem, cudaStream_t stream) {
    const bool vec = D % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                     (!delta || (uintptr_t)delta % 16 == 0) && (!sum_out || (uintptr_t)sum_out % 16 == 0) &&
                     (!planes || ((uintptr_t)planes % 16 == 0 && plane_stride % 4 == 0));
    const int work = vec ? D / 4 : D;
    const int block = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    cudaError_t e = cudaSuccess;
    if (vec && D / 4 <= 4 * 256) {
        qwb_launch_link(n_rows, QWB_LINK_ROWS_NORM, rmsnorm_rows_kernel<TOut, 4>, n_rows, 256, 0, stream, x, delta, planes, plane_count, plane_stride, sum_out, w, out, rows, D, eps);
    } else if (vec && D / 4 <= 8 * 256) {
        qwb_launch_link(n_rows, QWB_LINK_ROWS_NORM, rmsnorm_rows_kernel<TOut, 8>, n_rows, 256, 0, stream, x, delta, planes, plane_count, plane_stride, sum_out, w, out, rows, D, eps);
    } else if (vec) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<TOut, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "rmsnorm: %s", cudaGetErrorString(e));
        qwb_launch_link(n_rows, QWB_LINK_ROWS_NORM, rmsnorm_kernel<TOut, true>, n_rows, block, smem, stream, x, delta, planes, plane_count, plane_stride, sum_out, w, out, rows, D, eps);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(rmsnorm_kernel<TOut, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "rmsnorm: %s", cudaGetErrorString(e));
        qwb_launch(rmsnorm_kernel<TOut, false>, n_rows, block, smem, stream, x, delta, planes, plane_count, plane_stride, sum_out, w, out, rows, D, eps);
    }
    return qwb_check_launch("rmsnorm");
}

static int rmsnorm_any(const float* x, const float* delta, const float* planes, const unsigned char* plane_count,
                       size_t plane_stride, float* sum_out, const float* w, void* out, int out_dtype, const int* rows,
                       int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (D <= 0) return qwb_fail(QWB_ERR_ARG, "rmsnorm: bad width %d", D);
    const size_t smem = (size_t)D * sizeof(float);
    if (smem > 200 * 1024) return qwb_fail(QWB_ERR_ARG, "rmsnorm: width %d does not fit in shared memory (max %d)", D, 200 * 1024 / 4);
    if (out_dtype == QWB_DT_F32)
        return launch_rmsnorm<float>(x, delta, planes, plane_count, plane_stride, sum_out, w, (float*)out, rows, n_rows, D, eps, smem, stream);
    if (out_dtype == QWB_DT_BF16)
        return launch_rmsnorm<bf16>(x, delta, planes, plane_count, plane_stride, sum_out, w, (bf16*)out, rows, n_rows, D, eps, smem, stream);
    return qwb_fail(QWB_ERR_ARG, "rmsnorm: unknown dtype %d", out_dtype);
}

extern "C" int qwb_rmsnorm(const float* x, const float* delta, float* sum_out, const float* w,
                           void* out, int out_dtype, const int* rows, int n_rows, int D, float eps,
                           cudaStream_t stream) {
    return rmsnorm_any(x, delta, nullptr, nullptr, 0, sum_out, w, out, out_dtype, rows, n_rows, D, eps, stream);
}

// The same with a product in planes instead of delta: planes [n_planes, rows_in, D], plane_count [ceil(D / 16)] bytes.
extern "C" int qwb_rmsnorm_planes(const float* x, const float* planes, const unsigned char* plane_count, int n_planes,
                                  int rows_in, float* sum_out, const float* w, void* out, int out_dtype, const int* rows,
                                  int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_planes < 1 || n_planes > RMS_MAX_PLANES)
        return qwb_fail(QWB_ERR_ARG, "rmsnorm: %d planes; this kernel adds up to %d", n_planes, RMS_MAX_PLANES);
    return rmsnorm_any(x, nullptr, planes, plane_count, (size_t)rows_in * D, sum_out, w, out, out_dtype, rows, n_rows, D, eps, stream);
}

// x[t, :] += the planes of a product (as above), for a consumer that is not this norm.
__global__ void add_planes_kernel(float* x, const float* planes, const unsigned char* __restrict__ plane_count,
                                  size_t plane_stride, size_t n, int D) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        for (int p = 0, n_planes = plane_count[(i % D) / RMS_PLANE_COLS]; p < n_planes; ++p) v += planes[p * plane_stride + i];
        x[i] = v;
    }
}

extern "C" int qwb_add_planes(float* x, const float* planes, const unsigned char* plane_count, int T, int D, cudaStream_t stream) {
    if (T <= 0 || D <= 0) return 0;
    const size_t n = (size_t)T * D;
    const int block = 256, grid = (int)((n + block - 1) / block < 1184 ? (n + block - 1) / block : 1184);
    qwb_launch(add_planes_kernel, grid, block, 0, stream, x, planes, plane_count, n, n, D);
    return qwb_check_launch("add_planes");
}

// ---------------------------------------------------------------------------------
// a[t,f] = silu(g[t,f]) * u[t,f], silu(x) = x / (1 + exp(-x)), from one [T, 2F] float
// matrix (the reference: core/runtime.cpp:1074-1076, ggml-cuda/unary.cuh:96-98).
// interleave 0: the first F columns are the gate and the last F the up projection;
// interleave G > 0 (F a multiple of G): for every G features, their G gates and then their G ups.
// ---------------------------------------------------------------------------------
template <typename TOut>
__global__ void silu_mul_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int T, int F, int interleave) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)T * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F, f = i - t * F;
        const size_t gate_at = interleave > 0 ? (f / interleave) * 2 * interleave + f % interleave : f;
        const float g = gu[t * 2 * F + gate_at];
        const float u = gu[t * 2 * F + gate_at + (interleave > 0 ? interleave : F)];
        out[i] = from_f32<TOut>(g / (1.f + expf(-g)) * u);
    }
}

// The same for gates and ups interleaved in eights (the layout that the products with a fused epilogue want): a thread
// takes 8 features: 64 bytes of gates and ups in four 16-byte loads, one store of 8 values.  64 rows of 12,288 features:
// 3.2 us against 5.5 with a value a thread.
template <typename TOut>
__global__ void silu_mul_eights_kernel(const float* __restrict__ gu, TOut* __restrict__ out, int T, int F) {
    pdl_wait();
    pdl_launch_dependents();
    const int groups = F >> 3;
    const size_t n = (size_t)T * groups;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / groups, grp = i - t * groups;
        const float4* src = reinterpret_cast<const float4*>(gu + (t * 2 * F + grp * 16));
        const float4 g0 = src[0], g1 = src[1], u0 = src[2], u1 = src[3];
        TOut* dst = out + t * F + grp * 8;
        Pack4<TOut>::store(dst, g0.x / (1.f + expf(-g0.x)) * u0.x, g0.y / (1.f + expf(-g0.y)) * u0.y,
                           g0.z / (1.f + expf(-g0.z)) * u0.z, g0.w / (1.f + expf(-g0.w)) * u0.w);
        Pack4<TOut>::store(dst + 4, g1.x / (1.f + expf(-g1.x)) * u1.x, g1.y / (1.f + expf(-g1.y)) * u1.y,
                           g1.z / (1.f + expf(-g1.z)) * u1.z, g1.w / (1.f + expf(-g1.w)) * u1.w);
    }
}

extern "C" int qwb_silu_mul(const float* gate_up, void* out, int out_dtype, int T, int F, int interleave, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (F <= 0) return qwb_fail(QWB_ERR_ARG, "silu_mul: bad width %d", F);
    if (interleave < 0 || (interleave > 0 && F % interleave))
        return qwb_fail(QWB_ERR_ARG, "silu_mul: %d features cannot be interleaved in groups of %d", F, interleave);
    const size_t n = (size_t)T * F;
    const int block = 256;
    if (interleave == 8 && F % 8 == 0 && (uintptr_t)gate_up % 16 == 0 && (uintptr_t)out % 16 == 0 &&
        (out_dtype == QWB_DT_F32 || out_dtype == QWB_DT_BF16)) {
        const size_t groups = n / 8;
        const int g8 = (int)((groups + block - 1) / block < 148 * 16 ? (groups + block - 1) / block : 148 * 16);
        if (out_dtype == QWB_DT_F32) qwb_launch(silu_mul_eights_kernel<float>, g8, block, 0, stream, gate_up, (float*)out, T, F);
        else qwb_launch(silu_mul_eights_kernel<bf16>, g8, block, 0, stream, gate_up, (bf16*)out, T, F);
        return qwb_check_launch("silu_mul");
    }
    const int grid = (int)((n + block - 1) / block < 148 * 16 ? (n + block - 1) / block : 148 * 16);
    if (out_dtype == QWB_DT_F32)
        qwb_launch(silu_mul_kernel<float>, grid, block, 0, stream, gate_up, (float*)out, T, F, interleave);
    else if (out_dtype == QWB_DT_BF16)
        qwb_launch(silu_mul_kernel<bf16>, grid, block, 0, stream, gate_up, (bf16*)out, T, F, interleave);
    else
        return qwb_fail(QWB_ERR_ARG, "silu_mul: unknown dtype %d", out_dtype);
    return qwb_check_launch("silu_mul");
}

// out[i] += delta[i]: the residual sum on its own, for blocks that end without a norm.
__global__ void add_inplace_kernel(float* __restrict__ out, const float* __restrict__ delta, size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] += delta[i];
}

extern "C" int qwb_add_inplace(float* out, const float* delta, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int block = 256;
    const long long want = (n + block - 1) / block;
    const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
    qwb_launch(add_inplace_kernel, grid, block, 0, stream, out, delta, (size_t)n);
    return qwb_check_launch("add_inplace");
}

// After a decode step that sampled on the device: the sampled token becomes the next
// step's input, every sequence is one token longer, the step counter goes up, and the
// token enters the sequence's penalty window (a ring of `window` ids).
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* token_ids, int* tok_pos, int* pos0,
                                      int* seq_len, unsigned int* step_counter, int* recent, int* n_seen,
                                      int window, int B) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b == 0 && step_counter) *step_counter += 1;
    if (b >= B) return;
    const int tok = sampled[b];
    token_ids[b] = tok;
    tok_pos[b] += 1;
    pos0[b] += 1;
    seq_len[b] += 1;
    if (recent && window > 0) {
        recent[(size_t)b * window + (n_seen[b] % window)] = tok;
        n_seen[b] += 1;
    }
}

extern "C" int qwb_decode_advance(const int* sampled, int* token_ids, int* tok_pos, int* pos0, int* seq_len,
                                  unsigned int* step_counter, int* recent, int* n_seen, int window, int B,
                                  cudaStream_t stream) {
    if (B <= 0) return 0;
    qwb_launch(decode_advance_kernel, (B + 127) / 128, 128, 0, stream, sampled, token_ids, tok_pos, pos0, seq_len,
                                                               step_counter, recent, n_seen, window, B);
    return qwb_check_launch("decode_advance");
}
