// Rotary position encoding and the write into the paged key/value cache.
//
// Two kernels.  rope_table makes cos/sin of every token's angles once per step (all
// layers and heads share them); qk_norm_rope_store then, per token and head, takes the
// 32-bit output of the fused Q/K/V projection, applies the per-head RMS norm (Q and K),
// rotates the pairs (i, i + n_rot/2) (Q and K), writes Q for the attention kernel and
// stores K and V at the token's place in the cache.  The reference runs these as
// rms_norm + mul + rope (+ set_rows) (core/runtime.cpp:1047-1051, 693-706;
// ggml-cuda/rope.cu:676-754).
#include "common.cuh"

// angle[t,i] = pos[t] * inv_freq[i], in double: positions of thousands keep their digits.
__global__ void rope_table_kernel(const int* __restrict__ pos, const double* __restrict__ inv_freq,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int T, int half) {
    pdl_wait();
    pdl_launch_dependents();
    const int n = T * half;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int t = i / half, j = i - t * half;
        double s, c;
        sincos((double)pos[t] * inv_freq[j], &s, &c);
        cos_out[i] = (float)c;
        sin_out[i] = (float)s;
    }
}

extern "C" int qwb_rope_table(const int* pos, const double* inv_freq, float* cos_out, float* sin_out,
                              int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const int n = T * half, block = 128;
    int grid = (n + block - 1) / block;
    if (grid > 148 * 8) grid = 148 * 8;
    qwb_launch(rope_table_kernel, grid, block, 0, stream, pos, inv_freq, cos_out, sin_out, T, half);
    return qwb_check_launch("rope_table");
}

// One warp per (token, head).  Heads 0..Hq-1 are queries, then Hkv key heads, then Hkv
// value heads, in the order of the fused projection's columns.
//   qkv        [T, (Hq + 2 Hkv) * hd] float
//   q_weight, k_weight [hd] float, or null for no norm
//   cos_t, sin_t [T, rot/2] float
//   tok_seq, tok_pos [T]: the batch row and the position of each token
//   page_table [B, table_width]: the pages of each batch row, in order
//   q_out      [T, Hq, hd]
//   k_pool, v_pool [n_pages, Hkv, page_size, hd]
template <typename TOut>
__global__ void qk_norm_rope_store_kernel(const float* __restrict__ qkv, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, const int* __restrict__ tok_seq,
                                          const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                          TOut* __restrict__ q_out, TOut* __restrict__ k_pool, TOut* __restrict__ v_pool,
                                          int Hq, int Hkv, int hd, int rot, float eps, int page_size,
                                          int table_width, int store_kv) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int n_heads = Hq + 2 * Hkv;
    if (head >= n_heads) return;
    const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
    if (!is_q && !store_kv) return;
    const float* src = qkv + ((size_t)t * n_heads + head) * hd;

    TOut* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * Hq + head) * hd;
    } else {
        const int kvh = is_k ? head - Hq : head - Hq - Hkv;
        const int p = tok_pos[t];
        const int page = page_table[(size_t)tok_seq[t] * table_width + p / page_size];
        TOut* pool = is_k ? k_pool : v_pool;
        dst = pool + (((size_t)page * Hkv + kvh) * page_size + (p % page_size)) * hd;
    }

    const float* nw = is_q ? q_weight : (is_k ? k_weight : nullptr);
    float scale = 1.f;
    if (nw) {
        float ss = 0.f;
        for (int i = lane; i < hd; i += 32) { const float v = src[i]; ss += v * v; }
        ss = warp_sum(ss);
        scale = rsqrtf(ss / (float)hd + eps);
    }
    if (is_q || is_k) {
        const int half = rot >> 1;
        const float* c = cos_t + (size_t)t * half;
        const float* s = sin_t + (size_t)t * half;
        for (int i = lane; i < half; i += 32) {
            float a = src[i] * scale, b = src[i + half] * scale;
            if (nw) { a *= nw[i]; b *= nw[i + half]; }
            dst[i] = from_f32<TOut>(a * c[i] - b * s[i]);
            dst[i + half] = from_f32<TOut>(a * s[i] + b * c[i]);
        }
        for (int i = rot + lane; i < hd; i += 32) {
            float a = src[i] * scale;
            if (nw) a *= nw[i];
            dst[i] = from_f32<TOut>(a);
        }
    } else {
        for (int i = lane; i < hd; i += 32) dst[i] = from_f32<TOut>(src[i]);
    }
}

template <typename TOut> struct Pack4Store;
template <> struct Pack4Store<float> {
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4Store<bf16> {
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

// The same for head size 128 rotated over all 128 values, the common case.  Half a warp takes a head: lane L of the 16
// holds values 4L..4L+3 and 64+4L..64+4L+3, so that a value and its rotation partner (64 places away) lie in one lane
// and only the sum of squares crosses lanes (four shuffles).  A block takes one token: its eight warps share the
// token's pairs of heads (warp w: pairs w, w + 8, ...), up to three pairs' loads on their way before the first is used
// (all of a warp's for a token of 48 heads), the token's cos and sin, position and page looked up once.  A v head runs
// through the same arithmetic with a factor, weights and cosines of one and sines of zero: x * 1 - x' * 0 is x.
// 2,048 tokens of 32 + 2 x 8 heads: 16.8 us (4.5 TB/s); with a whole warp per head and the partner by shuffle 19.7 us (the kernel
// issued instructions 58 % of the time and moved 29 % of what the memory can), with a block per four heads 27.6 us.
#define RK_WARPS 8
#define RK_PAIRS_AT_ONCE 3
template <typename TOut>
__global__ void __launch_bounds__(RK_WARPS * 32)
qk_norm_rope_store_hd128_kernel(const float* __restrict__ qkv, const float* __restrict__ q_weight,
                                const float* __restrict__ k_weight, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, const int* __restrict__ tok_seq,
                                const int* __restrict__ tok_pos, const int* __restrict__ page_table,
                                TOut* __restrict__ q_out, TOut* __restrict__ k_pool, TOut* __restrict__ v_pool,
                                int Hq, int Hkv, float eps, int page_size, int table_width, int store_kv) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int hd = 128;
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
    const int n_heads = store_kv ? Hq + 2 * Hkv : Hq;               // without the cache write only q is made
    const int n_all = Hq + 2 * Hkv;
    const float4* row = reinterpret_cast<const float4*>(qkv + (size_t)t * n_all * hd);
    const float4 c = reinterpret_cast<const float4*>(cos_t + (size_t)t * (hd / 2))[l16];
    const float4 sn = reinterpret_cast<const float4*>(sin_t + (size_t)t * (hd / 2))[l16];
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f), zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 wq_lo = one, wq_hi = one, wk_lo = one, wk_hi = one;
    if (q_weight) { wq_lo = reinterpret_cast<const float4*>(q_weight)[l16]; wq_hi = reinterpret_cast<const float4*>(q_weight)[16 + l16]; }
    if (k_weight) { wk_lo = reinterpret_cast<const float4*>(k_weight)[l16]; wk_hi = reinterpret_cast<const float4*>(k_weight)[16 + l16]; }
    const int p = tok_pos[t];
    const size_t page = (size_t)page_table[(size_t)tok_seq[t] * table_width + p / page_size];
    const int pair_step = RK_WARPS * gridDim.y;     // few tokens: gridDim.y blocks share a token's heads
    const int n_pairs = (n_heads + 1) >> 1;
    for (int p0 = blockIdx.y * RK_WARPS + warp; p0 < n_pairs; p0 += pair_step * RK_PAIRS_AT_ONCE) {
        float4 lo[RK_PAIRS_AT_ONCE], hi[RK_PAIRS_AT_ONCE];
#pragma unroll
        for (int i = 0; i < RK_PAIRS_AT_ONCE; ++i) {
            const int head = 2 * (p0 + i * pair_step) + half;
            if (head < n_heads) {
                lo[i] = row[(size_t)head * (hd / 4) + l16];
                hi[i] = row[(size_t)head * (hd / 4) + 16 + l16];
            } else {
                lo[i] = hi[i] = zero;
            }
        }
#pragma unroll
        for (int i = 0; i < RK_PAIRS_AT_ONCE; ++i) {
            const int pair = p0 + i * pair_step;
            if (pair >= n_pairs) break;                            // the same for the whole warp
            const int head = 2 * pair + half;
            const bool live = head < n_heads, is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
            const bool normed = live && (is_q ? q_weight != nullptr : (is_k && k_weight != nullptr));
            float4 a = lo[i], b = hi[i];
            float ss = a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);             // within the 16 lanes of the head
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            ss += __shfl_xor_sync(0xffffffffu, ss, 8);
            if (normed) {
                const float scale = rsqrtf(ss / (float)hd + eps);
                const float4 w_lo = is_q ? wq_lo : wk_lo, w_hi = is_q ? wq_hi : wk_hi;
                a = make_float4(a.x * scale * w_lo.x, a.y * scale * w_lo.y, a.z * scale * w_lo.z, a.w * scale * w_lo.w);
                b = make_float4(b.x * scale * w_hi.x, b.y * scale * w_hi.y, b.z * scale * w_hi.z, b.w * scale * w_hi.w);
            }
            float4 ya = a, yb = b;
            if (is_q || is_k) {
                ya = make_float4(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
                yb = make_float4(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y, a.z * sn.z + b.z * c.z, a.w * sn.w + b.w * c.w);
            }
            if (live) {
                TOut* dst;
                if (is_q) {
                    dst = q_out + ((size_t)t * Hq + head) * hd;
                } else {
                    const int kvh = is_k ? head - Hq : head - Hq - Hkv;
                    dst = (is_k ? k_pool : v_pool) + ((page * Hkv + kvh) * page_size + (p % page_size)) * hd;
                }
                Pack4Store<TOut>::store(dst + 4 * l16, ya);
                Pack4Store<TOut>::store(dst + 64 + 4 * l16, yb);
            }
        }
    }
}

extern "C" int qwb_qk_norm_rope_store(const float* qkv, const float* q_weight, const float* k_weight,
                                      const float* cos_t, const float* sin_t, const int* tok_seq,
                                      const int* tok_pos, const int* page_table, void* q_out, void* k_pool,
                                      void* v_pool, int dtype, int T, int Hq, int Hkv, int hd, int rot,
                                      float eps, int page_size, int table_width, int store_kv,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    if (Hq <= 0 || Hkv <= 0 || hd <= 0 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0 || table_width <= 0)
        return qwb_fail(QWB_ERR_ARG, "qk_norm_rope_store: bad sizes Hq=%d Hkv=%d hd=%d rot=%d page=%d width=%d",
                        Hq, Hkv, hd, rot, page_size, table_width);
    const int warps = 4;
    dim3 grid(T, (Hq + 2 * Hkv + warps - 1) / warps);
    if (grid.y > 65535) return qwb_fail(QWB_ERR_ARG, "qk_norm_rope_store: too many heads (%d)", Hq + 2 * Hkv);
    const bool fast = hd == 128 && rot == 128 && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                      (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 && (uintptr_t)cos_t % 16 == 0 &&
                      (uintptr_t)sin_t % 16 == 0 && (!q_weight || (uintptr_t)q_weight % 16 == 0) &&
                      (!k_weight || (uintptr_t)k_weight % 16 == 0);
    // hd128 kernel: a block a token; with few tokens up to six blocks share a token's heads, so that there are blocks for the SMs
    int share = 1;
    if (T < 592) {
        share = (592 + T - 1) / T;
        const int most = ((Hq + 2 * Hkv + 1) / 2 + RK_WARPS - 1) / RK_WARPS;
        if (share > most) share = most;
    }
    if (fast && dtype == QWB_DT_F32)
        qwb_launch(qk_norm_rope_store_hd128_kernel<float>, dim3(T, share), RK_WARPS * 32, 0, stream, qkv, q_weight, k_weight, cos_t, sin_t,
                   tok_seq, tok_pos, page_table, (float*)q_out, (float*)k_pool, (float*)v_pool, Hq, Hkv, eps, page_size,
                   table_width, store_kv);
    else if (fast && dtype == QWB_DT_BF16)
        qwb_launch(qk_norm_rope_store_hd128_kernel<bf16>, dim3(T, share), RK_WARPS * 32, 0, stream, qkv, q_weight, k_weight, cos_t, sin_t,
                   tok_seq, tok_pos, page_table, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, Hq, Hkv, eps, page_size,
                   table_width, store_kv);
    else if (dtype == QWB_DT_F32)
        qwb_launch(qk_norm_rope_store_kernel<float>, grid, warps * 32, 0, stream, 
            qkv, q_weight, k_weight, cos_t, sin_t, tok_seq, tok_pos, page_table, (float*)q_out, (float*)k_pool,
            (float*)v_pool, Hq, Hkv, hd, rot, eps, page_size, table_width, store_kv);
    else if (dtype == QWB_DT_BF16)
        qwb_launch(qk_norm_rope_store_kernel<bf16>, grid, warps * 32, 0, stream, 
            qkv, q_weight, k_weight, cos_t, sin_t, tok_seq, tok_pos, page_table, (bf16*)q_out, (bf16*)k_pool,
            (bf16*)v_pool, Hq, Hkv, hd, rot, eps, page_size, table_width, store_kv);
    else
        return qwb_fail(QWB_ERR_ARG, "qk_norm_rope_store: unknown dtype %d", dtype);
    return qwb_check_launch("qk_norm_rope_store");
}
