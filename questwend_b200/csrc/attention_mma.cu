// Tensor-core attention over the paged bfloat16 cache, for head sizes 64 and 128.
//
// Same contract as attention.cu (causal, grouped heads, optional window, pages of 64 keys);
// those kernels stay the path for float32 and for other head sizes.  Here the scores
// S = Q K^T and the output O = P V run on mma.m16n8k16 (bf16 in, 32-bit out), with the
// running maximum, the sum and O kept in 32-bit registers (the reference's tensor-core
// kernel does the same on mma.sync, ggml-cuda/fattn-mma-f16.cuh).
//
// A block serves one key/value head.  Its rows are (token, query head of the group) pairs, so
// the heads that share the key/value head share every K and V tile that is loaded (the
// reference packs heads the same way, ggml-cuda/fattn.cu:91-110).  A K or V tile is one
// (page, head) block of the cache: 64 keys x hd, contiguous, copied to shared memory with
// 16-byte cp.async and stored with its 16-byte chunks XOR-swizzled by the row, so that
// ldmatrix reads without bank conflicts.  K feeds the mma as is; V goes through
// ldmatrix.trans.  Rows of a tile beyond the sequence's keys are zeroed (V) or masked (K).
//
//   prefill: 4 warps x 16 rows = 64 rows per block (64 / group tokens), all warps walk the
//            same tiles, double buffered.
//   decode : one token per sequence; the rows are the group's heads (padded to 16); a
//            block is one warp that takes a run of the sequence's pages; the runs' partial
//            results are merged by a combine kernel.  A run's length follows from the
//            sequence's own length alone, so a result does not depend on the batch.
#include "common.cuh"

#define AM_TILE 64          // keys per tile = tokens per cache page
#define AM_WARPS 4

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem_ptr) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* smem_ptr) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copy one (page, head) block of K or V, [64][HD] bf16, into a swizzled shared tile.  Rows from
// `n_valid` on are zeroed (their cache memory may hold anything).  `nthreads` threads take part.
template <int HD>
__device__ __forceinline__ void load_tile(bf16* tile, const bf16* src, int n_valid, int tid, int nthreads) {
    constexpr int CPR = HD / 8;                       // 16-byte chunks per row
    for (int i = tid; i < AM_TILE * CPR; i += nthreads) {
        const int row = i / CPR, c = i % CPR;
        bf16* dst = tile + row * HD + ((c ^ (row & 7)) << 3);
        if (row < n_valid) cp_async16(dst, src + row * HD + (c << 3));
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// One warp, 16 rows, one tile of 64 keys: S = Q K^T, mask, online softmax, O += P V, in two halves so that a caller
// can wait for K and for V separately and start the next tile's copies in between.
//   qf     Q fragments of the warp's 16 rows: [HD/16][4]
//   key0   position of the tile's first key; row_pos[2]: positions of rows g and g + 8 (-1: row unused)
//   len    keys of the sequence; window (0: none)
//   m, l   running maximum and (this thread's share of the) sum for rows g and g + 8;  o: [HD/8][4]
//   KEYS, key_off: the warp takes the KEYS keys (a multiple of 16) of the tile that start at key_off
//   s, base: the masked scores and the rows' new maxima (scaled), handed from the first half to the second
template <int HD, int KEYS>
__device__ __forceinline__ void tile_scores(const uint32_t (*qf)[4], const bf16* Kt, int key0, const int* row_pos, int len,
                                            int window, float sl2, float* m, float* l, float (*o)[4], int lane, int key_off,
                                            float (*s)[4], float* base) {
    constexpr int KS = HD / 16, NT = KEYS / 8, DT = HD / 8;
    const int t = lane & 3;
#pragma unroll
    for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const int mi = lane >> 3, mr = lane & 7;          // ldmatrix: which matrix this lane addresses, and its row
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
            const int key = key_off + 8 * (j + (mi >> 1)) + mr, chunk = 2 * ks + (mi & 1);
            uint32_t b[4];
            ldmatrix_x4(b, Kt + key * HD + ((chunk ^ (key & 7)) << 3));
            mma_16816(s[j], qf[ks], b[0], b[1]);
            mma_16816(s[j + 1], qf[ks], b[2], b[3]);
        }
    }
    // mask and running maximum
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int key = key0 + key_off + 8 * j + 2 * t + (r & 1);
            const int qp = row_pos[r >> 1];
            const bool ok = qp >= 0 && key <= qp && key < len && (window <= 0 || key > qp - window);
            s[j][r] = ok ? s[j][r] : -INFINITY;
            mx[r >> 1] = fmaxf(mx[r >> 1], s[j][r]);
        }
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        base[h] = m_new == -INFINITY ? 0.f : m_new * sl2;
        alpha[h] = exp2f(m[h] * sl2 - base[h]);       // m = -inf gives 0
        m[h] = m_new;
        l[h] *= alpha[h];
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
        o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
        o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
    }
}

// probabilities, then O += P V
template <int HD, int KEYS>
__device__ __forceinline__ void tile_pv(const bf16* Vt, const float (*s)[4], const float* base, float sl2, float* l,
                                        float (*o)[4], int lane, int key_off) {
    constexpr int DT = HD / 8;
    const int mi = lane >> 3, mr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KEYS / 16; ++kk) {
        uint32_t pf[4];
        float p[2][4];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                p[u][r] = exp2f(s[2 * kk + u][r] * sl2 - base[r >> 1]);
                l[r >> 1] += p[u][r];
            }
        pf[0] = pack_bf16(p[0][0], p[0][1]);
        pf[1] = pack_bf16(p[0][2], p[0][3]);
        pf[2] = pack_bf16(p[1][0], p[1][1]);
        pf[3] = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
        for (int jd = 0; jd < DT; jd += 2) {
            const int key = key_off + 16 * kk + 8 * (mi & 1) + mr, chunk = jd + (mi >> 1);
            uint32_t b[4];
            ldmatrix_x4_trans(b, Vt + key * HD + ((chunk ^ (key & 7)) << 3));
            mma_16816(o[jd], pf, b[0], b[1]);
            mma_16816(o[jd + 1], pf, b[2], b[3]);
        }
    }
}

// Both halves in a row, for a caller whose K and V tiles are both in shared memory already.
template <int HD>
__device__ __forceinline__ void tile_step(const uint32_t (*qf)[4], const bf16* Kt, const bf16* Vt, int key0, const int* row_pos,
                                          int len, int window, float sl2, float* m, float* l, float (*o)[4], int lane) {
    float s[AM_TILE / 8][4], base[2];
    tile_scores<HD, AM_TILE>(qf, Kt, key0, row_pos, len, window, sl2, m, l, o, lane, 0, s, base);
    tile_pv<HD, AM_TILE>(Vt, s, base, sl2, l, o, lane, 0);
}

// Q fragments of rows (g, g + 8) of a warp; q_lo / q_hi point at the rows' hd values (or null).
template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t (*qf)[4], const bf16* q_lo, const bf16* q_hi, int lane) {
    const int t = lane & 3;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
        const int d = 16 * ks + 2 * t;
        qf[ks][0] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + d) : 0u;
        qf[ks][1] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + d) : 0u;
        qf[ks][2] = q_lo ? *reinterpret_cast<const uint32_t*>(q_lo + d + 8) : 0u;
        qf[ks][3] = q_hi ? *reinterpret_cast<const uint32_t*>(q_hi + d + 8) : 0u;
    }
}

// ---------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(AM_WARPS * 32)
attn_mma_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                        const int* __restrict__ page_table, const int* __restrict__ cu_seqlens, const int* __restrict__ pos0,
                        bf16* __restrict__ out, int Hq, int Hkv, int table_width, float scale, int window, int Gc, int chunks) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* tiles = reinterpret_cast<bf16*>(smem_raw);                 // [2 buffers][K, V][64][HD]
    const int b = blockIdx.z;
    const int kvh = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const int G = Hq / Hkv;
    const int tok_per_block = (AM_WARPS * 16) / Gc;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    // The last tokens see the most keys: their blocks start first (blocks start in the order of x, then y; the head is x),
    // so that the long blocks do not form the tail of the launch.
    const int q0 = (int)(gridDim.y - 1 - blockIdx.y) * tok_per_block;
    if (q0 >= n_new) return;
    const int p0 = pos0[b];
    const int len = p0 + n_new;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // rows of this thread: r = warp * 16 + g (+ 8) -> (token q0 + r / Gc, head chunk * Gc + r % Gc)
    int row_pos[2];
    const bf16* qrow[2];
    bf16* orow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + g + 8 * h;
        const int tok = q0 + r / Gc, head_in = chunk * Gc + r % Gc;
        const bool ok = r < tok_per_block * Gc && tok < n_new && head_in < G;
        row_pos[h] = ok ? p0 + tok : -1;
        const size_t at = ((size_t)(t0 + tok) * Hq + kvh * G + head_in) * HD;
        qrow[h] = ok ? q + at : nullptr;
        orow[h] = ok ? out + at : nullptr;
    }
    uint32_t qf[HD / 16][4];
    load_q_frags<HD>(qf, qrow[0], qrow[1], lane);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    const int last_tok = min(n_new, q0 + tok_per_block) - 1;
    const int k_last = p0 + last_tok;                                          // last key any row sees
    const int k_first = window > 0 ? max(0, p0 + q0 - window + 1) : 0;
    const int tile_first = k_first / AM_TILE, tile_last = k_last / AM_TILE;
    const int* pages = page_table + (size_t)b * table_width;
    const float sl2 = scale * 1.4426950408889634f;

    auto issue = [&](int tile, int buf) {
        const size_t src = ((size_t)pages[tile] * Hkv + kvh) * AM_TILE * HD;
        const int n_valid = min(AM_TILE, len - tile * AM_TILE);
        bf16* kt = tiles + (size_t)buf * 2 * AM_TILE * HD;
        load_tile<HD>(kt, k_pool + src, n_valid, threadIdx.x, blockDim.x);
        load_tile<HD>(kt + AM_TILE * HD, v_pool + src, n_valid, threadIdx.x, blockDim.x);
        cp_async_commit();
    };
    issue(tile_first, 0);
    for (int tile = tile_first; tile <= tile_last; ++tile) {
        const int buf = (tile - tile_first) & 1;
        if (tile < tile_last) { issue(tile + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const bf16* kt = tiles + (size_t)buf * 2 * AM_TILE * HD;
        // a warp whose rows all lie before this tile has nothing to see in it
        const int warp_last_tok = min(last_tok, q0 + (warp * 16 + 15) / Gc);
        if (tile * AM_TILE <= p0 + warp_last_tok)
            tile_step<HD>(qf, kt, kt + AM_TILE * HD, tile * AM_TILE, row_pos, len, window, sl2, m, l, o, lane);
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!orow[h]) continue;
        const float inv = 1.f / l[h];
#pragma unroll
        for (int d = 0; d < HD / 8; ++d)
            *reinterpret_cast<uint32_t*>(orow[h] + 8 * d + 2 * t) = pack_bf16(o[d][2 * h] * inv, o[d][2 * h + 1] * inv);
    }
}

// ---------------------------------------------------------------------------------
// decode: block = (run of keys, key/value head and head chunk, sequence), a single warp that takes the run's pages
// one after the other.  It holds 32 KB of shared memory, so seven blocks share an SM and one's loads overlap
// another's arithmetic; its partial result goes straight from registers to the scratch that the combine kernel reads.
// How long a run is depends on the sequence's own length only (never on the batch): short sequences are cut into
// single pages, longer ones into about `runs_target` runs of up to `run_pages_max` pages, which keeps the number
// of partial results, and the work of combining them, small against the keys read.
// ---------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int run_pages_for(int len, int runs_target, int run_pages_max) {
    const int pages = (len + AM_TILE - 1) / AM_TILE;
    const int want = (pages + runs_target - 1) / runs_target;
    return want < 1 ? 1 : (want > run_pages_max ? run_pages_max : want);
}

// The most runs that any sequence of up to max_len keys is cut into (the grid's width and the scratch's size).
static int max_runs_for(int max_len, int runs_target, int run_pages_max) {
    const int pages = (max_len + AM_TILE - 1) / AM_TILE;
    if (pages <= runs_target) return pages < 1 ? 1 : pages;
    if (pages <= runs_target * run_pages_max) return runs_target;
    return (pages + run_pages_max - 1) / run_pages_max;
}

// FUSED: the step's own q, k and v come as the q/k/v projection left them (32-bit, [B, (Hq + 2 Hkv) * HD], q heads first),
// and the kernel does what a kernel of its own did before: per-head norm of q and k, rotation, and the cache write of
// the new key and value.  Every block forms the rotated q of its heads itself (a rotation pair, d and d + HD / 2, lies in
// one thread's fragment registers); the block whose run holds the new token forms k and v, writes them to the cache
// and puts them into its shared tiles, where the copy from the cache brought what was there before.
struct FusedQKV {
    const float* qkv;
    const float* q_w;           // per-head norm weights [HD], or null: no norm
    const float* k_w;
    const float* cos_t;         // [B, HD / 2] of each sequence's new position, or null: no rotation
    const float* sin_t;
    bf16* k_pool;               // the cache, to be written
    bf16* v_pool;
    float eps;
    int store_kv;               // 0: the cache belongs to another layer's run and has the new token already
};

template <int HD>
__device__ __forceinline__ void fused_q_frags(uint32_t (*qf)[4], const FusedQKV& f, const float* row_lo, const float* row_hi,
                                              int b, int lane) {
    constexpr int KS = HD / 16, HALF = HD / 2;
    const int t = lane & 3;
    const float* rows[2] = {row_lo, row_hi};
    float v[2][KS][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float ss = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = 16 * ks + 2 * t;
            const float2 a = rows[h] ? __ldcg(reinterpret_cast<const float2*>(rows[h] + d)) : make_float2(0.f, 0.f);
            const float2 c = rows[h] ? __ldcg(reinterpret_cast<const float2*>(rows[h] + d + 8)) : make_float2(0.f, 0.f);
            v[h][ks][0] = a.x; v[h][ks][1] = a.y; v[h][ks][2] = c.x; v[h][ks][3] = c.y;
            ss += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
        }
        if (f.q_w) {                                      // the row's 4 threads hold its HD values between them
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            const float scale = rsqrtf(ss / (float)HD + f.eps);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int d = 16 * ks + 2 * t;
                const float2 wa = *reinterpret_cast<const float2*>(f.q_w + d), wc = *reinterpret_cast<const float2*>(f.q_w + d + 8);
                v[h][ks][0] = v[h][ks][0] * scale * wa.x; v[h][ks][1] = v[h][ks][1] * scale * wa.y;
                v[h][ks][2] = v[h][ks][2] * scale * wc.x; v[h][ks][3] = v[h][ks][3] * scale * wc.y;
            }
        }
    }
    if (f.cos_t) {
        const float* cs = f.cos_t + (size_t)b * HALF;
        const float* sn = f.sin_t + (size_t)b * HALF;
#pragma unroll
        for (int ks = 0; ks < KS / 2; ++ks) {
            const int d = 16 * ks + 2 * t;
            const float2 ca = *reinterpret_cast<const float2*>(cs + d), cc = *reinterpret_cast<const float2*>(cs + d + 8);
            const float2 sa = *reinterpret_cast<const float2*>(sn + d), sc = *reinterpret_cast<const float2*>(sn + d + 8);
            const float c4[4] = {ca.x, ca.y, cc.x, cc.y}, s4[4] = {sa.x, sa.y, sc.x, sc.y};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = v[h][ks][j], hi = v[h][ks + KS / 2][j];
                    v[h][ks][j] = lo * c4[j] - hi * s4[j];
                    v[h][ks + KS / 2][j] = lo * s4[j] + hi * c4[j];
                }
        }
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        qf[ks][0] = pack_bf16(v[0][ks][0], v[0][ks][1]);
        qf[ks][1] = pack_bf16(v[1][ks][0], v[1][ks][1]);
        qf[ks][2] = pack_bf16(v[0][ks][2], v[0][ks][3]);
        qf[ks][3] = pack_bf16(v[1][ks][2], v[1][ks][3]);
    }
}

// The new token's key (is_k: with norm and rotation) or value, as bfloat16: lane L gets the values d0 = L * HD / 32 ...
template <int HD>
__device__ __forceinline__ void fused_new_row(const FusedQKV& f, const float* src, bool is_k, int b, int lane, float* y) {
    constexpr int PER = HD / 32, HALF = HD / 2;
    const int d0 = lane * PER;
#pragma unroll
    for (int e = 0; e < PER; ++e) y[e] = __ldcg(src + d0 + e);        // written by the kernel before: past the read-only cache
    if (!is_k) return;
    if (f.k_w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < PER; ++e) ss += y[e] * y[e];
        ss = warp_sum(ss);
        const float scale = rsqrtf(ss / (float)HD + f.eps);
#pragma unroll
        for (int e = 0; e < PER; ++e) y[e] = y[e] * scale * f.k_w[d0 + e];
    }
    if (f.cos_t) {
        const int dr = d0 % HALF;                         // lanes 16.. hold the second half: their partners are lanes 0..15
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, y[e], 16);
            const float c = f.cos_t[(size_t)b * HALF + dr + e], sn = f.sin_t[(size_t)b * HALF + dr + e];
            y[e] = lane < 16 ? y[e] * c - other * sn : other * sn + y[e] * c;
        }
    }
}

template <int HD, bool FUSED, bool K_TWO>
__global__ void __launch_bounds__(32)
attn_mma_decode_kernel(const FusedQKV fused, const bf16* q, const bf16* k_pool, const bf16* v_pool,
                       const int* __restrict__ page_table, const int* __restrict__ seq_len, float* __restrict__ part_acc,
                       float* __restrict__ part_m, float* __restrict__ part_l, bf16* __restrict__ out, int Hq, int Hkv,
                       int table_width, float scale, int window, int runs_target, int run_pages_max, int max_runs, int Gc,
                       int chunks) {
    constexpr bool k_two = K_TWO;
    // Launched with programmatic stream serialization, the block may start while the kernel before it still runs.
    // FUSED, that kernel is the q/k/v projection, and what the block needs first does not come from it: the sequences'
    // lengths and page tables were set before the step, and the keys and values of earlier tokens in earlier steps.  So
    // the run's first page is on its way before the wait; q, and the new token's key and value, are read after it, with
    // loads that do not go through the read-only cache (q, k_pool and v_pool are not __restrict__ for that reason: what
    // the kernel before wrote while this one was resident must not be read as constant data).  Not FUSED, the kernel
    // before it wrote the new key and value into the cache, so the wait comes first.
    const bool page_first = FUSED && fused.store_kv;     // a cache that another layer's kernel fills in this step: wait first
    if (!page_first) pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // blocks start in the order of x, then y, then z: the run is z, so that the runs that only longer sequences have
    // (blocks that find nothing to do) start last and keep no block with keys waiting
    const int b = blockIdx.y, run = blockIdx.z;
    const int len = seq_len[b];
    const int split_tokens = run_pages_for(len, runs_target, run_pages_max) * AM_TILE;
    const int k_lo = window > 0 ? max(0, len - window) : 0;
    const int run_first = k_lo / split_tokens, run_end = min(max_runs, (len + split_tokens - 1) / split_tokens);
    if (run < run_first || run >= run_end) return;
    const int kvh = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
    const int G = Hq / Hkv;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    bf16* my_tiles = reinterpret_cast<bf16*>(smem_raw);                         // K then V

    const int tok_begin = run * split_tokens, tok_end = min(len, tok_begin + split_tokens);
    const int* pages = page_table + (size_t)b * table_width;
    const float sl2 = scale * 1.4426950408889634f;
    // The run's pages one after the other, through one K and one V buffer: as soon as the scores of a page are formed
    // its K buffer takes the next page's K, and after O += P V its V buffer the next page's V, so that the copies of
    // page i + 1 run under the arithmetic of page i.  The first page's copies go out before anything else.
    // k_two (the host gives the block a third tile when all blocks still find room on the SMs): K has two buffers, so
    // that the next page's K is asked for a page ahead - the second page's with the first, before anything else - and
    // only V waits for its buffer.  The arithmetic is the same either way.
    bf16* k_tiles[2] = {my_tiles, k_two ? my_tiles + 2 * AM_TILE * HD : my_tiles};
    bf16* v_tile = my_tiles + AM_TILE * HD;
    int base_tok = max(tok_begin, (k_lo / AM_TILE) * AM_TILE);                 // pages wholly before the window are skipped
    if (base_tok < tok_end) {
        const size_t src = ((size_t)pages[base_tok / AM_TILE] * Hkv + kvh) * AM_TILE * HD;
        const int n_valid = min(AM_TILE, len - base_tok);
        load_tile<HD>(k_tiles[0], k_pool + src, n_valid, lane, 32);
        cp_async_commit();
        load_tile<HD>(v_tile, v_pool + src, n_valid, lane, 32);
        cp_async_commit();
        if (k_two && base_tok + AM_TILE < tok_end) {
            const int next_tok = base_tok + AM_TILE;
            const size_t src1 = ((size_t)pages[next_tok / AM_TILE] * Hkv + kvh) * AM_TILE * HD;
            load_tile<HD>(k_tiles[1], k_pool + src1, min(AM_TILE, len - next_tok), lane, 32);
            cp_async_commit();
        }
    }

    if (page_first) pdl_wait();
    int row_pos[2];
    uint32_t qf[HD / 16][4];
    {
        const int n_all = Hq + 2 * Hkv;
        const bf16* qrow[2];
        const float* frow[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = g + 8 * h, head_in = chunk * Gc + r;
            const bool ok = r < Gc && head_in < G;
            row_pos[h] = ok ? len - 1 : -1;
            qrow[h] = ok && !FUSED ? q + ((size_t)b * Hq + kvh * G + head_in) * HD : nullptr;
            frow[h] = ok && FUSED ? fused.qkv + ((size_t)b * n_all + kvh * G + head_in) * HD : nullptr;
        }
        if (FUSED) fused_q_frags<HD>(qf, fused, frow[0], frow[1], b, lane);
        else load_q_frags<HD>(qf, qrow[0], qrow[1], lane);
    }
    // FUSED: the new token's key and value, if its place lies in this run: into the cache (one block per key/value head
    // writes) and, below, into the shared tiles of its page
    const int new_pos = len - 1;
    const bool has_new = FUSED && fused.store_kv && new_pos >= tok_begin && new_pos < tok_end;
    float new_k[HD / 32], new_v[HD / 32];
    if (has_new) {
        const int n_all = Hq + 2 * Hkv;
        fused_new_row<HD>(fused, fused.qkv + ((size_t)b * n_all + Hq + kvh) * HD, true, b, lane, new_k);
        fused_new_row<HD>(fused, fused.qkv + ((size_t)b * n_all + Hq + Hkv + kvh) * HD, false, b, lane, new_v);
        if (chunk == 0) {
            const size_t at = (((size_t)pages[new_pos / AM_TILE] * Hkv + kvh) * AM_TILE + new_pos % AM_TILE) * HD + lane * (HD / 32);
#pragma unroll
            for (int e = 0; e < HD / 32; e += 2) {
                *reinterpret_cast<uint32_t*>(fused.k_pool + at + e) = pack_bf16(new_k[e], new_k[e + 1]);
                *reinterpret_cast<uint32_t*>(fused.v_pool + at + e) = pack_bf16(new_v[e], new_v[e + 1]);
            }
        }
    }
    // the new row's place in a shared tile (rows of HD values, 16-byte pieces XOR-swizzled by the row)
    auto patch = [&](bf16* tile, const float* y) {
        const int row = new_pos % AM_TILE, d0 = lane * (HD / 32);
        bf16* dst = tile + row * HD + (((d0 >> 3) ^ (row & 7)) << 3) + (d0 & 7);
#pragma unroll
        for (int e = 0; e < HD / 32; e += 2) *reinterpret_cast<uint32_t*>(dst + e) = pack_bf16(y[e], y[e + 1]);
    };
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    if constexpr (!K_TWO) {
    for (; base_tok < tok_end; base_tok += AM_TILE) {
        bf16* k_tile = k_tiles[0];
        const int next_tok = base_tok + AM_TILE;
        const bool more = next_tok < tok_end;
        size_t src = 0;
        int n_valid = 0;
        if (more) {
            src = ((size_t)pages[next_tok / AM_TILE] * Hkv + kvh) * AM_TILE * HD;
            n_valid = min(AM_TILE, len - next_tok);
        }
        float s[AM_TILE / 8][4], sbase[2];
        cp_async_wait<1>();                                                     // this page's K has landed (its V may not have)
        __syncwarp();
        const bool new_here = has_new && new_pos >= base_tok && new_pos < base_tok + AM_TILE;
        if (new_here) { patch(k_tile, new_k); __syncwarp(); }
        tile_scores<HD, AM_TILE>(qf, k_tile, base_tok, row_pos, len, window, sl2, m, l, o, lane, 0, s, sbase);
        __syncwarp();                                                           // every lane is done reading K
        if (more) {
            load_tile<HD>(k_tile, k_pool + src, n_valid, lane, 32);
            cp_async_commit();
            cp_async_wait<1>();                                                 // all but the copy just started: this page's V
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        if (new_here) { patch(v_tile, new_v); __syncwarp(); }
        tile_pv<HD, AM_TILE>(v_tile, s, sbase, sl2, l, o, lane, 0);
        __syncwarp();                                                           // every lane is done reading V
        if (more) {
            load_tile<HD>(v_tile, v_pool + src, n_valid, lane, 32);
            cp_async_commit();
        }
    }
    } else {
    for (int page_i = 0; base_tok < tok_end; base_tok += AM_TILE, ++page_i) {
        const int next_tok = base_tok + AM_TILE;
        const bool more = next_tok < tok_end, more2 = next_tok + AM_TILE < tok_end;
        bf16* k_tile = k_tiles[page_i & 1];
        size_t src = 0;
        int n_valid = 0;
        if (more) {
            src = ((size_t)pages[next_tok / AM_TILE] * Hkv + kvh) * AM_TILE * HD;
            n_valid = min(AM_TILE, len - next_tok);
        }
        float s[AM_TILE / 8][4], sbase[2];
        // this page's K has landed (its V may not have; with two K buffers neither the next page's K, asked for before V)
        if (k_two && more) cp_async_wait<2>(); else cp_async_wait<1>();
        __syncwarp();
        const bool new_here = has_new && new_pos >= base_tok && new_pos < base_tok + AM_TILE;
        if (new_here) { patch(k_tile, new_k); __syncwarp(); }
        tile_scores<HD, AM_TILE>(qf, k_tile, base_tok, row_pos, len, window, sl2, m, l, o, lane, 0, s, sbase);
        __syncwarp();                                                           // every lane is done reading K
        bool started = false;                                                   // a copy of K started just now
        if (k_two) {
            if (more2) {                                                        // the page after the next into this page's buffer
                const int tok2 = next_tok + AM_TILE;
                const size_t src2 = ((size_t)pages[tok2 / AM_TILE] * Hkv + kvh) * AM_TILE * HD;
                load_tile<HD>(k_tile, k_pool + src2, min(AM_TILE, len - tok2), lane, 32);
                cp_async_commit();
                started = true;
            }
        } else if (more) {
            load_tile<HD>(k_tile, k_pool + src, n_valid, lane, 32);
            cp_async_commit();
            started = true;
        }
        if (started) cp_async_wait<1>(); else cp_async_wait<0>();               // all but the copy just started: this page's V
        __syncwarp();
        if (new_here) { patch(v_tile, new_v); __syncwarp(); }
        tile_pv<HD, AM_TILE>(v_tile, s, sbase, sl2, l, o, lane, 0);
        __syncwarp();                                                           // every lane is done reading V
        if (more) {
            load_tile<HD>(v_tile, v_pool + src, n_valid, lane, 32);
            cp_async_commit();
        }
    }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const bool single = (run_end - run_first) == 1;
    // the warp's registers are the run's result
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h, head_in = chunk * Gc + r;
        if (r >= Gc || head_in >= G) continue;
        const int head = kvh * G + head_in;
        if (single) {
            const float inv = 1.f / l[h];
            bf16* dst = out + ((size_t)b * Hq + head) * HD;
#pragma unroll
            for (int d = 0; d < HD / 8; ++d)
                *reinterpret_cast<uint32_t*>(dst + 8 * d + 2 * t) = pack_bf16(o[d][2 * h] * inv, o[d][2 * h + 1] * inv);
        } else {
            const size_t at = ((size_t)b * Hq + head) * max_runs + run;
            float* dst = part_acc + at * HD;
#pragma unroll
            for (int d = 0; d < HD / 8; ++d)
                *reinterpret_cast<float2*>(dst + 8 * d + 2 * t) = make_float2(o[d][2 * h], o[d][2 * h + 1]);
            if (t == 0) { part_m[at] = m[h] * scale; part_l[at] = l[h]; }   // the combine kernel works with scaled scores
        }
    }
}

// out = sum_r acc_r e^(m_r - M) / sum_r l_r e^(m_r - M) over the runs, in index order (as in attention.cu).
// A warp per (head, sequence), four heads a block: lane r holds run r's maximum and sum (16 runs at a time), every lane 2
// or 4 columns of every partial result (one 8- or 16-byte load a run), all of a round's loads on their way before the
// first is used.  (One block of 128 threads per (head, sequence), a column a thread, took 3.7 us at 8 sequences and 8.0
// at 64, where this takes 3.6 and 4.5; a decode step of 8 sequences got 1.3 % faster, one of 64 2 %.)
#define AM_COMBINE_THREADS 128
template <int VEC>                     // columns per lane: hd = 32 * VEC
__global__ void __launch_bounds__(AM_COMBINE_THREADS)
attn_mma_combine_warp_kernel(const float* part_acc, const float* part_m, const float* part_l, const int* __restrict__ seq_len,
                             bf16* __restrict__ out, int Hq, int window, int runs_target, int run_pages_max, int max_runs) {
    pdl_launch_dependents();            // the trigger first: the kernel after this one may start while attention still runs
    pdl_wait();
    constexpr int hd = 32 * VEC;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x * (AM_COMBINE_THREADS / 32) + warp, b = blockIdx.y;
    if (h >= Hq) return;
    const int len = seq_len[b];
    const int split_tokens = run_pages_for(len, runs_target, run_pages_max) * AM_TILE;
    const int k_lo = window > 0 ? max(0, len - window) : 0;
    const int run_first = k_lo / split_tokens, run_end = min(max_runs, (len + split_tokens - 1) / split_tokens);
    const int n_runs = run_end - run_first;
    if (n_runs <= 1) return;                              // a single run wrote the output itself
    const size_t row = ((size_t)b * Hq + h) * max_runs + run_first;
    float a[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) a[v] = 0.f;
    float L = 0.f, M = -INFINITY;
    // the maximum over all runs first (32 at a time), then the weighted sums in run order; with up to 16 runs (the
    // usual case) the one round's own loads give the maximum, so that nothing is asked for twice or one after the other
    for (int r0 = 0; n_runs > 16 && r0 < n_runs; r0 += 32) {
        float m = r0 + lane < n_runs ? __ldcg(part_m + row + r0 + lane) : -INFINITY;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        M = fmaxf(M, m);
    }
    for (int r0 = 0; r0 < n_runs; r0 += 16) {
        const int n_here = min(16, n_runs - r0);
        const float my_m = lane < n_here ? __ldcg(part_m + row + r0 + lane) : -INFINITY;
        const float my_l = lane < n_here ? __ldcg(part_l + row + r0 + lane) : 0.f;
        float acc[16][VEC];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < n_here) {
                const float* src = part_acc + (row + r0 + i) * hd + lane * VEC;
                if (VEC == 4) {
                    const float4 t = __ldcg(reinterpret_cast<const float4*>(src));
                    acc[i][0] = t.x; acc[i][1] = t.y; acc[i][VEC - 2] = t.z; acc[i][VEC - 1] = t.w;
                } else {
                    const float2 t = __ldcg(reinterpret_cast<const float2*>(src));
                    acc[i][0] = t.x; acc[i][1] = t.y;
                }
            }
        }
        if (n_runs <= 16) {
            M = my_m;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        }
        const float my_w = lane < n_here ? expf(my_m - M) : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < n_here) {
                const float w = __shfl_sync(0xffffffffu, my_w, i), l = __shfl_sync(0xffffffffu, my_l, i);
                L += l * w;
#pragma unroll
                for (int v = 0; v < VEC; ++v) a[v] += acc[i][v] * w;
            }
        }
    }
    bf16* dst = out + ((size_t)b * Hq + h) * hd + lane * VEC;
#pragma unroll
    for (int v = 0; v < VEC; v += 2) *reinterpret_cast<uint32_t*>(dst + v) = pack_bf16(a[v] / L, a[v + 1] / L);
}

static int group_chunk(int G) { return G < 16 ? G : 16; }

template <int HD>
static int launch_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                          const int* pos0, void* out, int B, int max_new, int Hq, int Hkv, int table_width, float scale,
                          int window, cudaStream_t stream) {
    const int G = Hq / Hkv, Gc = group_chunk(G), chunks = (G + Gc - 1) / Gc;
    const int tok_per_block = (AM_WARPS * 16) / Gc;
    const size_t smem = (size_t)2 * 2 * AM_TILE * HD * sizeof(bf16);
    cudaError_t e = cudaFuncSetAttribute(attn_mma_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_mma_prefill: %s", cudaGetErrorString(e));
    dim3 grid(Hkv * chunks, (max_new + tok_per_block - 1) / tok_per_block, B);
    if (grid.y > 65535) return qwb_fail(QWB_ERR_ARG, "attn_mma_prefill: %d new tokens of a sequence are more than the grid takes", max_new);
    qwb_launch(attn_mma_prefill_kernel<HD>, grid, AM_WARPS * 32, smem, stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool,
        page_table, cu_seqlens, pos0, (bf16*)out, Hq, Hkv, table_width, scale, window, Gc, chunks);
    return qwb_check_launch("attn_mma_prefill");
}

static int check_sizes(const char* what, int Hq, int Hkv, int hd, int page_size, int B) {
    if (hd != 64 && hd != 128) return qwb_fail(QWB_ERR_ARG, "%s: head size %d is not 64 or 128", what, hd);
    if (page_size != AM_TILE) return qwb_fail(QWB_ERR_ARG, "%s: page size %d is not %d", what, page_size, AM_TILE);
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return qwb_fail(QWB_ERR_ARG, "%s: %d query heads are not a multiple of %d key/value heads", what, Hq, Hkv);
    if (B > 65535 || Hq > 65535) return qwb_fail(QWB_ERR_ARG, "%s: batch %d or heads %d above 65535", what, B, Hq);
    return 0;
}

// bfloat16 only.  Arguments as qwb_attn_prefill.
extern "C" int qwb_attn_mma_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                                    const int* cu_seqlens, const int* pos0, void* out, int B, int max_new, int Hq, int Hkv,
                                    int hd, int page_size, int table_width, float scale, int window, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (int rc = check_sizes("attn_mma_prefill", Hq, Hkv, hd, page_size, B)) return rc;
    if (hd == 64) return launch_prefill<64>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, Hq, Hkv, table_width, scale, window, stream);
    return launch_prefill<128>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, max_new, Hq, Hkv, table_width, scale, window, stream);
}

static int am_sm_count() {
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    return n_sm;
}

template <int HD, bool FUSED>
static int launch_decode(const FusedQKV& fused, const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                         const int* seq_len, float* scratch, void* out, int B, int Hq, int Hkv, int table_width, float scale,
                         int window, int runs_target, int run_pages_max, int max_runs, cudaStream_t stream) {
    const int G = Hq / Hkv, Gc = group_chunk(G), chunks = (G + Gc - 1) / Gc;
    // A third tile (two for K) while every block of the grid still finds room: 4 blocks of 48 KB an SM.  Decode steps at
    // the Qwen3-8B sizes: the same with one or two sequences of 1,024 keys, 2 % faster with 4; 5 % faster with 4 of
    // 4,096 and 2.7 % with one of 16,384.  With 8 sequences and a bound of 2,048 keys the grid has 1,024 blocks: 1.7 %
    // faster while they have 1,040 keys (576 blocks with keys), 7 % slower at 4,096 (all 1,024): so by the grid, which is
    // all that the host knows.  The kernel without it keeps its loop as it was: one loop for both cost a step of 8
    // sequences 0.7 %.
    // QWB200_ATTN_K2=0 switches it off, for measurements.
    static const bool k_two_allowed = [] { const char* e = getenv("QWB200_ATTN_K2"); return !(e && e[0] == '0'); }();
    const bool k_two = k_two_allowed && (long long)Hkv * chunks * B * max_runs <= 4LL * am_sm_count();
    const size_t smem = (size_t)(k_two ? 3 : 2) * AM_TILE * HD * sizeof(bf16);
    float* part_acc = scratch;
    float* part_m = scratch + (size_t)B * Hq * max_runs * HD;
    float* part_l = part_m + (size_t)B * Hq * max_runs;
    dim3 grid(Hkv * chunks, B, max_runs);
    // early: see the kernel's first lines
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_mma_decode: %s", cudaGetErrorString(e));
        qwb_launch_early(kernel, grid, 32, smem, stream, fused, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, page_table, seq_len,
                         part_acc, part_m, part_l, (bf16*)out, Hq, Hkv, table_width, scale, window, runs_target, run_pages_max, max_runs,
                         Gc, chunks);
        return 0;
    };
    if (int rc = k_two ? go(attn_mma_decode_kernel<HD, FUSED, true>) : go(attn_mma_decode_kernel<HD, FUSED, false>)) return rc;
    if (int rc = qwb_check_launch("attn_mma_decode")) return rc;
    if (max_runs > 1) {
        // (launched early with more sequences, even with its trigger after its wait, a step of 8 got 1 % slower)
        qwb_launch_link(B, QWB_LINK_ROWS_MERGE, attn_mma_combine_warp_kernel<HD / 32>, dim3((Hq + AM_COMBINE_THREADS / 32 - 1) / (AM_COMBINE_THREADS / 32), B),
                        AM_COMBINE_THREADS, 0, stream, part_acc, part_m, part_l, seq_len, (bf16*)out, Hq, window, runs_target, run_pages_max, max_runs);
        return qwb_check_launch("attn_mma_combine");
    }
    return 0;
}

// The most runs that a sequence of up to max_len keys is cut into under (runs_target, run_pages_max): the host sizes the
// scratch with it, B * Hq * runs * (hd + 2) floats.
extern "C" int qwb_attn_mma_decode_runs(int max_len, int runs_target, int run_pages_max) {
    if (max_len <= 0 || runs_target <= 0 || run_pages_max <= 0) return 0;
    return max_runs_for(max_len, runs_target, run_pages_max);
}

static int check_decode(int B, int Hq, int Hkv, int hd, int page_size, int runs_target, int run_pages_max, int max_len,
                        const float* scratch, int* max_runs) {
    if (int rc = check_sizes("attn_mma_decode", Hq, Hkv, hd, page_size, B)) return rc;
    if (runs_target <= 0 || run_pages_max <= 0 || max_len <= 0)
        return qwb_fail(QWB_ERR_ARG, "attn_mma_decode: %d runs of up to %d pages for up to %d keys", runs_target, run_pages_max, max_len);
    *max_runs = max_runs_for(max_len, runs_target, run_pages_max);
    if (*max_runs > 65535) return qwb_fail(QWB_ERR_ARG, "attn_mma_decode: %d runs of keys; at most 65535", *max_runs);
    if ((size_t)*max_runs * sizeof(float) > 40 * 1024) return qwb_fail(QWB_ERR_ARG, "attn_mma_decode: %d runs of keys are too many to combine", *max_runs);
    if (*max_runs > 1 && !scratch) return qwb_fail(QWB_ERR_ARG, "attn_mma_decode: %d runs need scratch memory", *max_runs);
    return 0;
}

// bfloat16 only.  Arguments as qwb_attn_decode, but for how the keys are cut into runs: a sequence of p pages is cut into
// runs of clamp(ceil(p / runs_target), 1, run_pages_max) pages (runs_target 1 gives runs of exactly run_pages_max pages);
// max_len bounds every entry of seq_len.  scratch: B * Hq * runs(max_len) * (hd + 2) floats, unused with a single run.
extern "C" int qwb_attn_mma_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                                   const int* seq_len, float* scratch, void* out, int B, int Hq, int Hkv, int hd, int page_size,
                                   int table_width, float scale, int window, int runs_target, int run_pages_max, int max_len,
                                   cudaStream_t stream) {
    if (B <= 0) return 0;
    int max_runs = 0;
    if (int rc = check_decode(B, Hq, Hkv, hd, page_size, runs_target, run_pages_max, max_len, scratch, &max_runs)) return rc;
    FusedQKV none = {};
    if (hd == 64) return launch_decode<64, false>(none, q, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, table_width, scale, window, runs_target, run_pages_max, max_runs, stream);
    return launch_decode<128, false>(none, q, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, table_width, scale, window, runs_target, run_pages_max, max_runs, stream);
}

// The same with the step's q, k and v taken from the q/k/v projection's 32-bit output qkv [B, (Hq + 2 Hkv) * hd]: per-head
// norm of q and k (weights [hd], or null), rotation of all hd values by cos/sin [B, hd / 2] (or null), and, with store_kv,
// the new key and value written into the cache at each sequence's position seq_len - 1, all inside the attention kernel.
extern "C" int qwb_attn_mma_decode_fused(const float* qkv, const float* q_weight, const float* k_weight, const float* cos_t,
                                         const float* sin_t, float eps, int store_kv, void* k_pool, void* v_pool,
                                         const int* page_table, const int* seq_len, float* scratch, void* out, int B, int Hq,
                                         int Hkv, int hd, int page_size, int table_width, float scale, int window,
                                         int runs_target, int run_pages_max, int max_len, cudaStream_t stream) {
    if (B <= 0) return 0;
    int max_runs = 0;
    if (int rc = check_decode(B, Hq, Hkv, hd, page_size, runs_target, run_pages_max, max_len, scratch, &max_runs)) return rc;
    if (!qkv || (uintptr_t)qkv % 8 || (q_weight && (uintptr_t)q_weight % 8) || (cos_t && ((uintptr_t)cos_t % 8 || (uintptr_t)sin_t % 8)))
        return qwb_fail(QWB_ERR_ARG, "attn_mma_decode_fused: qkv, norm weights and cos/sin must be 8-byte aligned");
    if ((cos_t == nullptr) != (sin_t == nullptr)) return qwb_fail(QWB_ERR_ARG, "attn_mma_decode_fused: cos and sin come together");
    FusedQKV f = {qkv, q_weight, k_weight, cos_t, sin_t, (bf16*)k_pool, (bf16*)v_pool, eps, store_kv};
    if (hd == 64) return launch_decode<64, true>(f, nullptr, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, table_width, scale, window, runs_target, run_pages_max, max_runs, stream);
    return launch_decode<128, true>(f, nullptr, k_pool, v_pool, page_table, seq_len, scratch, out, B, Hq, Hkv, table_width, scale, window, runs_target, run_pages_max, max_runs, stream);
}
