// Prefill attention on the fifth-generation tensor cores (tcgen05), bfloat16, head sizes 64 and 128, groups of
// up to 64 query heads per key/value head, pages of 64 keys.  Same contract as attn_prefill in attention.cu.
//
// A block serves (128 / G tokens, rounded down) x (the G query heads of one key/value head) rows, up to 128; with a
// G that does not divide 128 the last rows of the 128 stay unused.  Per tile of 64 keys (one cache page of that head):
//     S = Q K^T      tcgen05.mma, Q and K from shared memory (TMA, 128-byte swizzle), S in tensor memory (64 columns, two
//                    buffers: the tensor core is up to two tiles ahead of the softmax)
//     P = softmax    four warps, one thread per row: read S, mask, running maximum and sum in 32-bit, write P as
//                    bfloat16 into shared memory in the layout the tensor core reads
//     O += P V       tcgen05.mma, P and V from shared memory, O accumulates in tensor memory (HD columns).  V is read as
//                    it lies in the cache ([key][d], d contiguous): the "MN-major" operand form.
// O lives in tensor memory across the tiles.  It carries a reference maximum per row; when a tile raises a row's
// maximum by more than 2^8 the row's O and sum are rescaled (read, scale, write back), else the old reference stays
// and the probabilities are simply larger than 1 for a while: the result is the same, most tiles need no rescale.
// Warp 0 loads (one lane), warp 1 issues the products (one lane) and owns the tensor memory, warps 2-5 do the softmax
// and the final write.  Every wait is bounded; a wait that runs out raises *error and the block runs to its end.
//
// Keys of the last page beyond the sequence's length are masked in S; their V rows are multiplied by P = 0, so the
// cache must hold finite numbers there (the cache is zeroed when it is made, and later holds only values that were
// keys and values once).
#include "common.cuh"

#include <cuda.h>

#define AT_ROWS 128
#define AT_KEYS 64
#define AT_THREADS 192
#define AT_KV_STAGES 2
#define AT_SPIN_LIMIT (1u << 22)
#define AT_RESCALE_LOG2 8.f

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < AT_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(at_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void at_tma_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void at_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void at_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 2^x by the hardware approximation (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Operand descriptors, 128-byte swizzle, descriptor version 1.
//   K-major (rows of 64 bfloat16 = 128 bytes, the contraction runs along the row): groups of 8 rows are 1024 bytes apart.
__device__ __forceinline__ uint64_t at_desc_kmajor(const void* tile) {
    return (uint64_t)((at_smem(tile) & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
//   MN-major (each row of 128 bytes holds 64 consecutive values of the non-contracted dimension for one index of the
//   contraction): the next 64 values of the non-contracted dimension are `lbo_bytes` away, the next 8 indices of the
//   contraction 1024 bytes.
__device__ __forceinline__ uint64_t at_desc_mnmajor(const void* tile, uint32_t lbo_bytes) {
    return (uint64_t)((at_smem(tile) & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D float, A and B bfloat16; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t at_idesc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int HD>
struct AtSmem {
    static constexpr int ATOMS = HD / 64;                                  // 128-byte pieces of a row of Q, K or V
    static constexpr size_t Q_BYTES = (size_t)AT_ROWS * HD * 2;            // ATOMS blocks of [128 rows][128 bytes]
    static constexpr size_t KV_BYTES = (size_t)AT_KEYS * HD * 2;           // ATOMS blocks of [64 keys][128 bytes]
    static constexpr size_t P_BYTES = (size_t)AT_ROWS * AT_KEYS * 2;       // [128 rows][128 bytes]
    static constexpr size_t BYTES = Q_BYTES + 2 * AT_KV_STAGES * KV_BYTES + P_BYTES + 128;   // 128: barriers, tensor-memory slot
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS)
attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ pos0, bf16* __restrict__ out, int Hq, int Hkv,
                       int table_width, float scale, int window, int G, int* error) {
    constexpr int ATOMS = AtSmem<HD>::ATOMS;
    constexpr uint32_t KV_BYTES = AtSmem<HD>::KV_BYTES;
    constexpr uint32_t TMEM_COLS = 256;                                     // S: 2 x 64 columns, O: HD columns
    // The tiles need 1024-byte alignment (128-byte swizzle).  No padding to reach it: at head size 128 the block's
    // 113 KB then leave room for a second block on the SM, whose products run while this block's softmax does.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if (at_smem(smem_raw) & 1023u) {                      // never seen; refuse rather than compute with a wrong layout
        if (threadIdx.x == 0) atomicExch(error, 7);
        return;
    }
    unsigned char* q_tile = smem_raw;
    unsigned char* k_tiles = q_tile + AtSmem<HD>::Q_BYTES;
    unsigned char* v_tiles = k_tiles + AT_KV_STAGES * KV_BYTES;
    unsigned char* p_tile = v_tiles + AT_KV_STAGES * KV_BYTES;
    uint64_t* q_full = reinterpret_cast<uint64_t*>(p_tile + AtSmem<HD>::P_BYTES);
    uint64_t* k_full = q_full + 1;                       // K and V have barriers of their own: a K buffer is free as soon
    uint64_t* k_empty = k_full + AT_KV_STAGES;           // as its scores are formed, long before its tile's V buffer is
    uint64_t* v_full = k_empty + AT_KV_STAGES;
    uint64_t* v_empty = v_full + AT_KV_STAGES;
    uint64_t* s_full = v_empty + AT_KV_STAGES;           // [2]: the two S buffers
    uint64_t* s_empty = s_full + 2;                      // [2]
    uint64_t* p_full = s_empty + 2;
    uint64_t* o_full = p_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.z, kvh = blockIdx.x;
    const int tok_per_block = AT_ROWS / G;
    const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
    // The last tokens see the most keys: their blocks go first, so that the long blocks do not form the tail of the launch.
    // Blocks start in the order of blockIdx.x, then y: the key/value head is x, so that the longest blocks of every head
    // start before any short one.
    const int q0 = (int)(gridDim.y - 1 - blockIdx.y) * tok_per_block;
    if (q0 >= n_new) return;
    const int p0 = pos0[b];
    const int len = p0 + n_new;
    const int last_tok = min(n_new, q0 + tok_per_block) - 1;
    const int k_last = p0 + last_tok;
    const int k_first = window > 0 ? max(0, p0 + q0 - window + 1) : 0;
    const int tile_first = k_first / AT_KEYS, tile_last = k_last / AT_KEYS;
    const int n_tiles = tile_last - tile_first + 1;
    const int* pages = page_table + (size_t)b * table_width;

    if (threadIdx.x == 0) {
        at_bar_init(q_full, 1);
        for (int s = 0; s < AT_KV_STAGES; ++s) {
            at_bar_init(&k_full[s], 1); at_bar_init(&k_empty[s], 1);
            at_bar_init(&v_full[s], 1); at_bar_init(&v_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) { at_bar_init(&s_full[i], 1); at_bar_init(&s_empty[i], 4); }
        at_bar_init(p_full, 4);
        at_bar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem_s = *tmem_slot;                 // S: two buffers, columns [0, 64) and [64, 128)
    const uint32_t tmem_o = tmem_s + 128;               // O: columns [128, 128 + HD)

    pdl_wait();
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            at_expect_tx(q_full, (uint32_t)(tok_per_block * G * HD * 2));      // the box's bytes: with G no divisor of 128, fewer than 128 rows
            for (int a = 0; a < ATOMS; ++a)             // rows (token, head of the group): a box of [128 / G tokens][G heads][64 d]
                at_tma_3d(q_tile + (size_t)a * AT_ROWS * 128, &map_q, q_full, a * 64, kvh * G, t0 + q0);
            // K of tile j + 1 goes out before V of tile j: its buffer is free earlier (after the scores of tile j - 1,
            // not after the product of tile j - 2), and the tensor core wants it earlier (the scores run two tiles ahead).
            bool ok = true;
            int k_issued = 0, v_issued = 0;
            auto load = [&](int j, bool is_k) -> bool {
                const int s = j % AT_KV_STAGES;
                uint64_t* empty = is_k ? &k_empty[s] : &v_empty[s];
                uint64_t* full = is_k ? &k_full[s] : &v_full[s];
                if (j >= AT_KV_STAGES && !at_wait(empty, ((j / AT_KV_STAGES) - 1) & 1)) return false;
                const int row0 = (pages[tile_first + j] * Hkv + kvh) * AT_KEYS;        // the (page, head) block's first row
                unsigned char* dst = (is_k ? k_tiles : v_tiles) + (size_t)s * KV_BYTES;
                at_expect_tx(full, KV_BYTES);
                for (int a = 0; a < ATOMS; ++a)
                    at_tma_2d(dst + (size_t)a * AT_KEYS * 128, is_k ? &map_k : &map_v, full, a * 64, row0);
                if (is_k) k_issued = j + 1; else v_issued = j + 1;
                return true;
            };
            ok = load(0, true);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) ok = load(j + 1, true);
                if (ok) ok = load(j, false);
            }
            if (!ok) {
                atomicExch(error, 1);
                // copies already issued still write shared memory: wait for them (bounded) before the block ends
                for (int j = max(0, k_issued - AT_KV_STAGES); j < k_issued; ++j) at_wait(&k_full[j % AT_KV_STAGES], (j / AT_KV_STAGES) & 1);
                for (int j = max(0, v_issued - AT_KV_STAGES); j < v_issued; ++j) at_wait(&v_full[j % AT_KV_STAGES], (j / AT_KV_STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = at_idesc(AT_ROWS, AT_KEYS, false);           // S [128 x 64] = Q [128 x HD] K[64 x HD]^T
            constexpr uint32_t idesc_o = at_idesc(AT_ROWS, HD, true);                  // O [128 x HD] += P [128 x 64] V [64 x HD]
            bool ok = at_wait(q_full, 0);
            // S runs two tiles ahead of P V: while the softmax warps work on one S buffer the tensor core fills the other.
            auto issue_s = [&](int j) -> bool {
                const int s = j % AT_KV_STAGES;
                if (!at_wait(&k_full[s], (j / AT_KV_STAGES) & 1)) return false;
                if (j >= 2 && !at_wait(&s_empty[j & 1], ((j >> 1) - 1) & 1)) return false;
                at_fence_after();
                const unsigned char* kt = k_tiles + (size_t)s * KV_BYTES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {                                    // 16 values of d per product
                    const uint64_t da = at_desc_kmajor(q_tile + (size_t)(k / 4) * AT_ROWS * 128) + 2 * (k % 4);
                    const uint64_t db = at_desc_kmajor(kt + (size_t)(k / 4) * AT_KEYS * 128) + 2 * (k % 4);
                    at_mma(tmem_s + (uint32_t)(j & 1) * 64, da, db, idesc_s, k > 0 ? 1u : 0u);
                }
                at_commit(&k_empty[s]);                                                // K of this tile is read
                at_commit(&s_full[j & 1]);
                return true;
            };
            if (ok) ok = issue_s(0);
            if (ok && n_tiles > 1) ok = issue_s(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % AT_KV_STAGES;
                ok = at_wait(&v_full[s], (j / AT_KV_STAGES) & 1) && at_wait(p_full, j & 1);   // V has landed; P is in shared memory
                if (!ok) break;
                at_fence_after();
                const unsigned char* vt = v_tiles + (size_t)s * KV_BYTES;
#pragma unroll
                for (int k = 0; k < AT_KEYS / 16; ++k) {                               // 16 keys per product
                    const uint64_t da = at_desc_kmajor(p_tile) + 2 * k;
                    const uint64_t db = at_desc_mnmajor(vt + (size_t)k * 16 * 128, AT_KEYS * 128);
                    at_mma(tmem_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                }
                at_commit(&v_empty[s]);                                                // V of this tile is read
                at_commit(o_full);
                if (j + 2 < n_tiles) ok = issue_s(j + 2);
            }
            if (!ok) {
                atomicExch(error, 2);
                at_commit(&s_full[0]);
                at_commit(&s_full[1]);
                at_commit(o_full);
            }
        }
    } else {
        const int lane_group = warp & 3;
        const int r = 32 * lane_group + lane;                                          // this thread's row = tensor-memory lane
        const int tok = q0 + r / G, head = kvh * G + r % G;
        const bool row_ok = r < tok_per_block * G && tok < n_new;                      // rows beyond the box hold nothing
        const int qp = row_ok ? p0 + tok : -1;
        const uint32_t lane_off = (uint32_t)(32 * lane_group) << 16;
        const float sl2 = scale * 1.4426950408889634f;
        float m_ref = -INFINITY, l = 0.f;                                              // reference maximum (raw score) and sum
        uint4* p_row = reinterpret_cast<uint4*>(p_tile + (size_t)r * 128);
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            ok = at_wait(&s_full[j & 1], (j >> 1) & 1);
            at_fence_after();
            if (!ok) { if (lane == 0) atomicExch(error, 3); break; }
            const int key0 = (tile_first + j) * AT_KEYS;
            uint32_t sv[2][32];
            at_ld32(tmem_s + (uint32_t)(j & 1) * 64 + lane_off, sv[0]);
            at_ld32(tmem_s + (uint32_t)(j & 1) * 64 + lane_off + 32, sv[1]);
            at_fence_before();                                                          // this S buffer may be filled again
            __syncwarp();
            if (lane == 0) at_arrive(&s_empty[j & 1]);
            // a tile that lies wholly inside what this row may see needs no mask
            const bool all_visible = key0 + AT_KEYS - 1 <= qp && key0 + AT_KEYS - 1 < len && (window <= 0 || key0 > qp - window);
            float mx = -INFINITY;
            if (all_visible) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[h][i]));
            } else {
                // this row sees the tile's keys [first, end): one subtraction and one unsigned comparison per key
                const int end = min(min(qp, len - 1) - key0 + 1, AT_KEYS);
                const int first = window > 0 ? max(qp - window + 1 - key0, 0) : 0;
                const unsigned span = end > first ? (unsigned)(end - first) : 0u;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const bool vis = (unsigned)(32 * h + i - first) < span;
                        const float sc = vis ? __uint_as_float(sv[h][i]) : -INFINITY;
                        sv[h][i] = __float_as_uint(sc);
                        mx = fmaxf(mx, sc);
                    }
            }
            // keep the old reference unless this tile's maximum is far above it
            const bool rescale = mx > m_ref + AT_RESCALE_LOG2 / sl2;
            const float m_new = rescale ? mx : m_ref;
            const float alpha = rescale ? at_exp2((m_ref - m_new) * sl2) : 1.f;       // m_ref = -inf gives 0
            const float base = m_new == -INFINITY ? 0.f : m_new * sl2;
            l *= alpha;
            m_ref = m_new;
            // the probabilities, packed to bfloat16, while the product before this one may still run
            uint32_t pk[2][16];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0v = at_exp2(__uint_as_float(sv[h][i]) * sl2 - base);
                    const float p1v = at_exp2(__uint_as_float(sv[h][i + 1]) * sl2 - base);
                    l += p0v + p1v;
                    __nv_bfloat162 v = __floats2bfloat162_rn(p0v, p1v);
                    pk[h][i / 2] = *reinterpret_cast<uint32_t*>(&v);
                }
            if (j > 0) {                                                               // the product before this one has read P and written O
                ok = at_wait(o_full, (j - 1) & 1);
                at_fence_after();
                if (!ok) { if (lane == 0) atomicExch(error, 4); break; }
                if (__any_sync(0xffffffffu, rescale)) {                                 // some row of this warp moves its reference: rescale O
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t ov[32];
                        at_ld32(tmem_o + lane_off + c, ov);
#pragma unroll
                        for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                        at_st32(tmem_o + lane_off + c, ov);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    p_row[(h * 4 + i) ^ (r & 7)] = make_uint4(pk[h][4 * i], pk[h][4 * i + 1], pk[h][4 * i + 2], pk[h][4 * i + 3]);
            at_fence_before();                                                          // O is rescaled (if at all); P is written
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) at_arrive(p_full);
        }
        if (ok) {
            ok = at_wait(o_full, (n_tiles - 1) & 1);
            at_fence_after();
            if (!ok && lane == 0) atomicExch(error, 5);
        }
        if (ok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(t0 + tok) * Hq + head) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                at_ld32(tmem_o + lane_off + c, ov);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t pk[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * u]) * inv, __uint_as_float(ov[i + 2 * u + 1]) * inv);
                            pk[u] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
    }
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------- host side
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtEncodeFn at_encode() {
    static AtEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AtEncodeFn>(p);
    }
    return fn;
}

template <int HD>
static int launch_attn_tc(const void* q, const void* k_pool, const void* v_pool, const int* page_table, const int* cu_seqlens,
                          const int* pos0, void* out, int B, int T, int max_new, int n_pages, int Hq, int Hkv, int table_width,
                          float scale, int window, int* error, cudaStream_t stream) {
    AtEncodeFn enc = at_encode();
    if (!enc) return qwb_fail(QWB_ERR_CUDA, "attn_tc_prefill: cuTensorMapEncodeTiled is not available from this driver");
    const int G = Hq / Hkv;
    CUtensorMap map_q, map_k, map_v;
    {   // q [T, Hq, HD]: boxes of [128 / G tokens][G heads][64 d]
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)Hq, (cuuint64_t)T};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)Hq * HD * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(AT_ROWS / G)};
        cuuint32_t elem[3] = {1, 1, 1};
        CUresult r = enc(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return qwb_fail(QWB_ERR_CUDA, "attn_tc_prefill: cuTensorMapEncodeTiled(q) failed with %d", (int)r);
    }
    const void* pools[2] = {k_pool, v_pool};
    CUtensorMap* maps[2] = {&map_k, &map_v};
    for (int i = 0; i < 2; ++i) {   // a pool [pages, Hkv, 64, HD] as rows of HD: boxes of [64 keys][64 d]
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)n_pages * Hkv * AT_KEYS};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, AT_KEYS};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = enc(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pools[i]), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return qwb_fail(QWB_ERR_CUDA, "attn_tc_prefill: cuTensorMapEncodeTiled(cache) failed with %d", (int)r);
    }
    const size_t smem = AtSmem<HD>::BYTES;
    cudaError_t e = cudaFuncSetAttribute(attn_tc_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_tc_prefill: %s", cudaGetErrorString(e));
    const int tok_per_block = AT_ROWS / G;
    dim3 grid(Hkv, (max_new + tok_per_block - 1) / tok_per_block, B);
    e = qwb_launch(attn_tc_prefill_kernel<HD>, grid, AT_THREADS, smem, stream, map_q, map_k, map_v, page_table, cu_seqlens, pos0,
                   (bf16*)out, Hq, Hkv, table_width, scale, window, G, error);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "attn_tc_prefill: launch failed: %s", cudaGetErrorString(e));
    return qwb_check_launch("attn_tc_prefill");
}

// bfloat16.  q [T, Hq, hd] with T the packed tokens of all B sequences; pools of n_pages pages; `error` as for qwb_gemm_tc.
extern "C" int qwb_attn_tc_prefill(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                                   const int* cu_seqlens, const int* pos0, void* out, int B, int T, int max_new, int n_pages,
                                   int Hq, int Hkv, int hd, int page_size, int table_width, float scale, int window, int* error,
                                   cudaStream_t stream) {
    if (B <= 0 || max_new <= 0 || T <= 0) return 0;
    if (hd != 64 && hd != 128) return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: head size %d is not 64 or 128", hd);
    if (page_size != AT_KEYS) return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: page size %d is not %d", page_size, AT_KEYS);
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: %d query heads are not a multiple of %d key/value heads", Hq, Hkv);
    const int G = Hq / Hkv;
    if (G > AT_ROWS / 2) return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: %d query heads per key/value head; this kernel takes up to %d", G, AT_ROWS / 2);
    if (B > 65535 || (max_new + AT_ROWS / G - 1) / (AT_ROWS / G) > 65535)
        return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: batch %d or %d new tokens of a sequence are more than the grid takes", B, max_new);
    if (!error) return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: an error word on the device is required");
    if ((uintptr_t)q % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 16)
        return qwb_fail(QWB_ERR_ARG, "attn_tc_prefill: operands must be 16-byte aligned");
    if (hd == 64) return launch_attn_tc<64>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, T, max_new, n_pages, Hq, Hkv, table_width, scale, window, error, stream);
    return launch_attn_tc<128>(q, k_pool, v_pool, page_table, cu_seqlens, pos0, out, B, T, max_new, n_pages, Hq, Hkv, table_width, scale, window, error, stream);
}
