// Attention over the paged key/value cache: softmax(q k^T / sqrt(hd) + mask) v with
// grouped heads (query head h reads key/value head h / (Hq/Hkv)), causal, with an
// optional window (key j is visible to the query at position p when p - window < j <= p).
// The reference: core/runtime.cpp:681-734 (scale :690, mask :3152-3158) and
// ggml-cuda/fattn*.  Scores, the running maximum and sum, and the output accumulator
// are 32-bit; the cache and the query are float or bfloat16.
//
//   attn_prefill      any number of new tokens per sequence, keys read from the cache
//                     (the new tokens' keys are already stored there)
//   attn_decode_split one new token per sequence, the keys cut into runs of
//                     `split_tokens`, one block per run; the run length does not depend on
//                     the batch, so a sequence's result does not either
//   attn_decode_combine merges the runs' partial results
//
// Cache layout: k_pool, v_pool [n_pages, Hkv, page_size, hd]; page_table [B, table_width]
// lists each batch row's pages in order.
#include "common.cuh"

#define QWB_MAX_HEAD_DIM 256

// ---------------------------------------------------------------------------------
// prefill: one block per (tile of BQ queries, query head, sequence); 4 warps, each
// warp owns BQ/4 queries; keys come in tiles of 32 (one key per lane).
// ---------------------------------------------------------------------------------
template <typename T, int NC>   // NC = ceil(hd / 32) rounded up to 2, 4 or 8
__global__ void attn_prefill_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                    const int* __restrict__ page_table, const int* __restrict__ cu_seqlens,
                                    const int* __restrict__ pos0, T* __restrict__ out, int Hq, int Hkv, int hd,
                                    int page_size, int table_width, float scale, int window) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BQ = 16, BK = 32, QPW = 4;
    extern __shared__ float smem[];
    float* Qs = smem;                         // [BQ][hd], already scaled
    float* Ks = Qs + BQ * hd;                 // [BK][hd + 1]
    float* Vs = Ks + BK * (hd + 1);           // [BK][hd]

    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BQ;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    if (q0 >= n_new) return;
    const int kvh = h / (Hq / Hkv);
    const int p0 = pos0[b];
    const int nq = min(BQ, n_new - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int idx = threadIdx.x; idx < BQ * hd; idx += blockDim.x) {
        const int i = idx / hd, d = idx - i * hd;
        Qs[idx] = i < nq ? to_f32(q[((size_t)(t0 + q0 + i) * Hq + h) * hd + d]) * scale : 0.f;
    }

    float m[QPW], l[QPW], acc[QPW][NC];
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
    }

    const int k_last = p0 + q0 + nq - 1;                                  // last key any query of the tile sees
    const int k_first = window > 0 ? max(0, p0 + q0 - window + 1) : 0;    // first key the first query sees
    const int* pages = page_table + (size_t)b * table_width;

    for (int kt = (k_first / BK) * BK; kt <= k_last; kt += BK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < BK * hd; idx += blockDim.x) {
            const int j = idx / hd, d = idx - j * hd, key = kt + j;
            float kv = 0.f, vv = 0.f;
            if (key <= k_last) {
                const size_t at = (((size_t)pages[key / page_size] * Hkv + kvh) * page_size + key % page_size) * hd + d;
                kv = to_f32(k_pool[at]);
                vv = to_f32(v_pool[at]);
            }
            Ks[j * (hd + 1) + d] = kv;
            Vs[j * hd + d] = vv;
        }
        __syncthreads();

        float s[QPW];
#pragma unroll
        for (int i = 0; i < QPW; ++i) s[i] = 0.f;
        const float* krow = Ks + lane * (hd + 1);
        for (int d = 0; d < hd; ++d) {
            const float kd = krow[d];
#pragma unroll
            for (int i = 0; i < QPW; ++i) s[i] += Qs[(warp * QPW + i) * hd + d] * kd;
        }
        const int key = kt + lane;
        float p[QPW];
#pragma unroll
        for (int i = 0; i < QPW; ++i) {
            const int qi = warp * QPW + i;
            const int qp = p0 + q0 + qi;
            const bool ok = qi < nq && key <= qp && (window <= 0 || key > qp - window);
            const float si = ok ? s[i] : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(si));
            if (m_new == -INFINITY) { p[i] = 0.f; continue; }       // nothing visible so far (whole warp agrees)
            const float alpha = expf(m[i] - m_new);                 // m = -inf gives 0
            p[i] = ok ? expf(si - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(p[i]);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
        }
        for (int j = 0; j < BK; ++j) {
            float pj[QPW];
#pragma unroll
            for (int i = 0; i < QPW; ++i) pj[i] = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int d = lane + 32 * c;
                if (d < hd) {
                    const float v = Vs[j * hd + d];
#pragma unroll
                    for (int i = 0; i < QPW; ++i) acc[i][c] += pj[i] * v;
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < QPW; ++i) {
        const int qi = warp * QPW + i;
        if (qi >= nq) continue;
        const float inv = 1.f / l[i];
        T* o = out + ((size_t)(t0 + q0 + qi) * Hq + h) * hd;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int d = lane + 32 * c;
            if (d < hd) o[d] = from_f32<T>(acc[i][c] * inv);
        }
    }
}

template <typename T>
static int launch_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                          const int* cu_seqlens, const int* pos0, void* out, int B, int max_new, int Hq, int Hkv,
                          int hd, int page_size, int table_width, float scale, int window, cudaStream_t stream) {
    const size_t smem = ((size_t)16 * hd + 32 * (hd + 1) + 32 * hd) * sizeof(float);
    dim3 grid((max_new + 15) / 16, Hq, B);
    const int nc = (hd + 31) / 32;
#define QWB_LAUNCH_PREFILL(NC)                                                                                   \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<T, NC>,                                     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
            if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_prefill: %s", cudaGetErrorString(e));      \
        }                                                                                                        \
        qwb_launch(attn_prefill_kernel<T, NC>, grid, 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, \
            page_table, cu_seqlens, pos0, (T*)out, Hq, Hkv, hd, page_size, table_width, scale, window);          \
    } while (0)
    if (nc <= 2) QWB_LAUNCH_PREFILL(2);
    else if (nc <= 4) QWB_LAUNCH_PREFILL(4);
    else QWB_LAUNCH_PREFILL(8);
#undef QWB_LAUNCH_PREFILL
    return qwb_check_launch("attn_prefill");
}

static int check_attn_sizes(const char* what, int Hq, int Hkv, int hd, int page_size, int table_width) {
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return qwb_fail(QWB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", what, Hq, Hkv);
    if (hd <= 0 || hd % 16 || hd > QWB_MAX_HEAD_DIM)
        return qwb_fail(QWB_ERR_ARG, "%s: head size %d is not a multiple of 16 in [16, %d]", what, hd, QWB_MAX_HEAD_DIM);
    if (page_size <= 0 || table_width <= 0) return qwb_fail(QWB_ERR_ARG, "%s: bad page size %d or table width %d", what, page_size, table_width);
    return 0;
}

extern "C" int qwb_attn_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                                const int* cu_seqlens, const int* pos0, void* out, int dtype, int B, int max_new,
                                int Hq, int Hkv, int hd, int page_size, int table_width, float scale, int window,
                                cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_attn_sizes("attn_prefill", Hq, Hkv, hd, page_size, table_width)) return rc;
    if (B > 65535 || Hq > 65535) return qwb_fail(QWB_ERR_ARG, "attn_prefill: batch %d or heads %d above 65535", B, Hq);
    if (dtype == QWB_DT_F32)
        return launch_prefill<float>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, Hq, Hkv, hd,
                                     page_size, table_width, scale, window, stream);
    if (dtype == QWB_DT_BF16)
        return launch_prefill<bf16>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, Hq, Hkv, hd,
                                    page_size, table_width, scale, window, stream);
    return qwb_fail(QWB_ERR_ARG, "attn_prefill: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// decode: one new token per sequence.  Block = (run of keys, key/value head and slice of
// its query heads, sequence), 128 threads.  Per page of the run: the page's K and V
// tiles go to shared memory; thread (key, head slice) forms the scores; one warp per
// head updates the running maximum and sum; thread d accumulates p v for all heads.
// ---------------------------------------------------------------------------------
#define QWB_DECODE_GT 8      // query heads per block

__device__ __forceinline__ void decode_run_range(int len, int window, int split_tokens, int max_runs, int* first, int* end) {
    // runs [first, end) hold at least one visible key of a sequence of `len` keys.  The caller sizes the grid and the
    // scratch for `max_runs` runs; a sequence longer than max_runs * split_tokens keys (a caller's mistake: the lengths
    // are on the device, the launcher cannot check them) is cut there, so that no block reads or writes beyond the
    // scratch it was given.
    const int k_first = window > 0 ? max(0, len - window) : 0;
    *first = min(k_first / split_tokens, max_runs);
    *end = min((len + split_tokens - 1) / split_tokens, max_runs);
}

template <typename T>
__global__ void attn_decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                         const int* __restrict__ page_table, const int* __restrict__ seq_len,
                                         float* __restrict__ part_acc, float* __restrict__ part_m, float* __restrict__ part_l,
                                         T* __restrict__ out, int Hq, int Hkv, int hd, int page_size, int table_width,
                                         float scale, int window, int split_tokens, int max_runs) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int GT = QWB_DECODE_GT, VEC = Vec16<T>::N;
    const int b = blockIdx.z, run = blockIdx.x;
    const int len = seq_len[b];
    int run_first, run_end;
    decode_run_range(len, window, split_tokens, max_runs, &run_first, &run_end);
    if (run < run_first || run >= run_end) return;

    const int G = Hq / Hkv, slices = (G + GT - 1) / GT;
    const int kvh = blockIdx.y / slices, g0 = (blockIdx.y % slices) * GT;
    const int gcount = min(GT, G - g0);
    const int h0 = kvh * G + g0;                        // first query head of this block

    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* Kt = reinterpret_cast<T*>(smem_raw);             // [page_size][hd]
    T* Vt = Kt + (size_t)page_size * hd;                // [page_size][hd]
    float* qs = reinterpret_cast<float*>(Vt + (size_t)page_size * hd);   // [GT][hd], scaled
    float* sc = qs + GT * hd;                           // [GT][page_size]
    float* m_s = sc + GT * page_size;                   // [GT]
    float* l_s = m_s + GT;
    float* a_s = l_s + GT;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int idx = tid; idx < GT * hd; idx += blockDim.x) {
        const int g = idx / hd, d = idx - g * hd;
        qs[idx] = g < gcount ? to_f32(q[((size_t)b * Hq + h0 + g) * hd + d]) * scale : 0.f;
    }
    if (tid < GT) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; a_s[tid] = 1.f; }

    float acc[GT][2];
#pragma unroll
    for (int g = 0; g < GT; ++g) acc[g][0] = acc[g][1] = 0.f;

    const int k_lo = window > 0 ? max(0, len - window) : 0;          // first visible key
    const int tok_begin = run * split_tokens, tok_end = min(len, tok_begin + split_tokens);
    const int* pages = page_table + (size_t)b * table_width;
    const int key_slices = blockDim.x / page_size;                    // threads per key (>= 1)
    const int my_key = tid % page_size, my_slice = tid / page_size;
    const int nchunk = hd / VEC;

    for (int base = tok_begin; base < tok_end; base += page_size) {
        if (base + page_size <= k_lo) continue;                       // a page wholly before the window
        const int n_keys = min(page_size, tok_end - base);
        const size_t tile = ((size_t)pages[base / page_size] * Hkv + kvh) * page_size * hd;
        __syncthreads();                                              // the last page's tiles are no longer read
        {
            const uint4* ksrc = reinterpret_cast<const uint4*>(k_pool + tile);
            const uint4* vsrc = reinterpret_cast<const uint4*>(v_pool + tile);
            uint4* kdst = reinterpret_cast<uint4*>(Kt);
            uint4* vdst = reinterpret_cast<uint4*>(Vt);
            const int n16 = n_keys * hd / VEC;
            for (int i = tid; i < n16; i += blockDim.x) { kdst[i] = ksrc[i]; vdst[i] = vsrc[i]; }
        }
        __syncthreads();

        // scores: thread (key, slice) handles heads slice, slice + key_slices, ...
        if (my_slice < key_slices && my_key < n_keys) {
            float s[GT];
#pragma unroll
            for (int g = 0; g < GT; ++g) s[g] = 0.f;
            const Vec16<T>* krow = reinterpret_cast<const Vec16<T>*>(Kt + (size_t)my_key * hd);
            for (int c = 0; c < nchunk; ++c) {
                const int ch = (my_key + c) % nchunk;                 // rotate: spread keys over the banks
                float kf[VEC];
                krow[ch].get(kf);
#pragma unroll
                for (int gi = 0; gi < GT; ++gi) {
                    const int g = my_slice + gi * key_slices;
                    if (g < gcount) {
                        const float* qg = qs + g * hd + ch * VEC;
#pragma unroll
                        for (int e = 0; e < VEC; ++e) s[gi] += qg[e] * kf[e];
                    }
                }
            }
            const bool ok = base + my_key >= k_lo;
#pragma unroll
            for (int gi = 0; gi < GT; ++gi) {
                const int g = my_slice + gi * key_slices;
                if (g < gcount) sc[g * page_size + my_key] = ok ? s[gi] : -INFINITY;
            }
        }
        __syncthreads();

        // running maximum and sum, one warp per head
        for (int g = warp; g < gcount; g += (blockDim.x >> 5)) {
            float mx = -INFINITY;
            for (int j = lane; j < n_keys; j += 32) mx = fmaxf(mx, sc[g * page_size + j]);
            mx = warp_max(mx);
            const float m_old = m_s[g], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < n_keys; j += 32) {
                const float sj = sc[g * page_size + j];
                const float pj = (m_new == -INFINITY || sj == -INFINITY) ? 0.f : expf(sj - m_new);
                sc[g * page_size + j] = pj;
                sum += pj;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
                a_s[g] = alpha;
                l_s[g] = l_s[g] * alpha + sum;
                m_s[g] = m_new;
            }
        }
        __syncthreads();

        // p v: thread d (and d + 128) for all heads
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int d = tid + c * 128;
            if (d < hd) {
#pragma unroll
                for (int g = 0; g < GT; ++g) if (g < gcount) acc[g][c] *= a_s[g];
                for (int j = 0; j < n_keys; ++j) {
                    const float v = to_f32(Vt[(size_t)j * hd + d]);
#pragma unroll
                    for (int g = 0; g < GT; ++g) if (g < gcount) acc[g][c] += sc[g * page_size + j] * v;
                }
            }
        }
    }
    __syncthreads();

    const bool single = (run_end - run_first) == 1;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int d = tid + c * 128;
        if (d >= hd) continue;
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            if (g >= gcount) continue;
            const int h = h0 + g;
            if (single) out[((size_t)b * Hq + h) * hd + d] = from_f32<T>(acc[g][c] / l_s[g]);
            else part_acc[(((size_t)b * Hq + h) * max_runs + run) * hd + d] = acc[g][c];
        }
    }
    if (!single && tid < gcount) {
        const size_t at = ((size_t)b * Hq + h0 + tid) * max_runs + run;
        part_m[at] = m_s[tid];
        part_l[at] = l_s[tid];
    }
}

// out = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M), M = max_r m_r; runs in index order.
template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_m,
                                           const float* __restrict__ part_l, const int* __restrict__ seq_len,
                                           T* __restrict__ out, int Hq, int hd, int window, int split_tokens, int max_runs) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x, b = blockIdx.y;
    int run_first, run_end;
    decode_run_range(seq_len[b], window, split_tokens, max_runs, &run_first, &run_end);
    if (run_end - run_first <= 1) return;                  // the split kernel wrote the result itself
    const size_t row = ((size_t)b * Hq + h) * max_runs;
    float M = -INFINITY;
    for (int r = run_first; r < run_end; ++r) M = fmaxf(M, part_m[row + r]);
    float L = 0.f;
    for (int r = run_first; r < run_end; ++r) L += part_l[row + r] * expf(part_m[row + r] - M);
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.f;
        for (int r = run_first; r < run_end; ++r) a += part_acc[(row + r) * hd + d] * expf(part_m[row + r] - M);
        out[((size_t)b * Hq + h) * hd + d] = from_f32<T>(a / L);
    }
}

extern "C" long long qwb_attn_decode_scratch_floats(int B, int Hq, int hd, int max_runs) {
    // part_acc [B,Hq,max_runs,hd] then part_m and part_l [B,Hq,max_runs]
    return (long long)B * Hq * max_runs * (hd + 2);
}

template <typename T>
static int launch_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* seq_len,
                         float* scratch, void* out, int B, int Hq, int Hkv, int hd, int page_size, int table_width,
                         float scale, int window, int split_tokens, int max_runs, cudaStream_t stream) {
    constexpr int GT = QWB_DECODE_GT;
    const size_t smem = 2 * (size_t)page_size * hd * sizeof(T) + ((size_t)GT * hd + GT * page_size + 3 * GT) * sizeof(float);
    if (smem > 200 * 1024)
        return qwb_fail(QWB_ERR_ARG, "attn_decode: page size %d with head size %d needs %zu bytes of shared memory (max %d)",
                        page_size, hd, smem, 200 * 1024);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_decode: %s", cudaGetErrorString(e));
    }
    float* part_acc = scratch;
    float* part_m = scratch + (size_t)B * Hq * max_runs * hd;
    float* part_l = part_m + (size_t)B * Hq * max_runs;
    const int G = Hq / Hkv, slices = (G + GT - 1) / GT;
    dim3 grid(max_runs, Hkv * slices, B);
    qwb_launch(attn_decode_split_kernel<T>, grid, 128, smem, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, page_table,
        seq_len, part_acc, part_m, part_l, (T*)out, Hq, Hkv, hd, page_size, table_width, scale, window, split_tokens, max_runs);
    if (int rc = qwb_check_launch("attn_decode_split")) return rc;
    if (max_runs > 1) {
        qwb_launch(attn_decode_combine_kernel<T>, dim3(Hq, B), 128, 0, stream, part_acc, part_m, part_l, seq_len, (T*)out, Hq, hd,
                                                                     window, split_tokens, max_runs);
        return qwb_check_launch("attn_decode_combine");
    }
    return 0;
}

// q [B, Hq, hd]; seq_len [B] counts the new token; out [B, Hq * hd]; scratch holds
// qwb_attn_decode_scratch_floats(B, Hq, hd, max_runs) floats; max_runs >= ceil(longest
// sequence / split_tokens); split_tokens is a multiple of page_size.
extern "C" int qwb_attn_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                               const int* seq_len, float* scratch, void* out, int dtype, int B, int Hq, int Hkv, int hd,
                               int page_size, int table_width, float scale, int window, int split_tokens, int max_runs,
                               cudaStream_t stream) {
    if (B <= 0) return 0;
    if (int rc = check_attn_sizes("attn_decode", Hq, Hkv, hd, page_size, table_width)) return rc;
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128)
        return qwb_fail(QWB_ERR_ARG, "attn_decode: page size %d is not 16, 32, 64 or 128", page_size);
    if (split_tokens <= 0 || split_tokens % page_size || max_runs <= 0)
        return qwb_fail(QWB_ERR_ARG, "attn_decode: run of %d keys is not a multiple of the page size %d, or %d runs", split_tokens, page_size, max_runs);
    if (B > 65535 || Hq > 65535) return qwb_fail(QWB_ERR_ARG, "attn_decode: batch %d or heads %d above 65535", B, Hq);
    if (max_runs > 1 && !scratch) return qwb_fail(QWB_ERR_ARG, "attn_decode: %d runs need scratch memory", max_runs);
    if (dtype == QWB_DT_F32)
        return launch_decode<float>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, hd, page_size,
                                    table_width, scale, window, split_tokens, max_runs, stream);
    if (dtype == QWB_DT_BF16)
        return launch_decode<bf16>(q, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, hd, page_size,
                                   table_width, scale, window, split_tokens, max_runs, stream);
    return qwb_fail(QWB_ERR_ARG, "attn_decode: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------
// The same decode attention with its scratch inside the library (attention_noalloc.h).
// ---------------------------------------------------------------------------------
#include "attention_noalloc.h"

#define QWB_NOALLOC_MAX_DEVICES 64

// In host code this name is only a handle of the symbol, never a device address: a kernel is
// given the address that cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) float qwb_noalloc_scratch[QWB_NOALLOC_SCRATCH_FLOATS];
static float* qwb_noalloc_scratch_ptr[QWB_NOALLOC_MAX_DEVICES];     // per device, looked up once

extern "C" long long qwb_attn_decode_noalloc_capacity(void) { return QWB_NOALLOC_SCRATCH_FLOATS; }

extern "C" int qwb_attn_decode_noalloc(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                                       const int* seq_len, void* out, int dtype, int B, int Hq, int Hkv, int hd,
                                       int page_size, int table_width, float scale, int window, int split_tokens,
                                       int max_runs, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (Hq <= 0 || hd <= 0 || max_runs <= 0)
        return qwb_fail(QWB_ERR_ARG, "attn_decode_noalloc: bad sizes Hq=%d hd=%d max_runs=%d", Hq, hd, max_runs);
    const long long need = qwb_attn_decode_scratch_floats(B, Hq, hd, max_runs);
    if (max_runs > 1 && need > (long long)QWB_NOALLOC_SCRATCH_FLOATS)
        return qwb_fail(QWB_ERR_ARG,
                        "attn_decode_noalloc: %d sequences x %d heads x %d runs x (%d + 2) = %lld floats of scratch, the "
                        "built-in array holds %lld; use qwb_attn_decode with scratch of your own",
                        B, Hq, max_runs, hd, need, (long long)QWB_NOALLOC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= QWB_NOALLOC_MAX_DEVICES)
        return qwb_fail(QWB_ERR_ARG, "attn_decode_noalloc: device %d is beyond the %d this library keeps track of", device,
                        QWB_NOALLOC_MAX_DEVICES);
    if (!qwb_noalloc_scratch_ptr[device]) {                         // set-up, once per device
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, qwb_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return qwb_fail(QWB_ERR_CUDA, "attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        qwb_noalloc_scratch_ptr[device] = p;
    }
    return qwb_attn_decode(q, k_pool, v_pool, page_table, seq_len, qwb_noalloc_scratch_ptr[device], out, dtype, B, Hq, Hkv,
                           hd, page_size, table_width, scale, window, split_tokens, max_runs, stream);
}
