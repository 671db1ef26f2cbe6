// Weight-streaming matrix product for up to 16 rows of bfloat16 x, fed by TMA through a ring in shared memory:
//     y[M,N] = x[M,K] W[N,K]^T (+ residual),  32-bit sums, y float;  or a = silu(gate) * up as bfloat16.
//
// A decode step reads every weight once, so a product's time is the time to stream W from HBM, and the loss is at its
// start and end: the first loads find nothing in flight, the last blocks drain.  This kernel is built around that:
//   * one block per SM, resident for the whole product (it walks over its tiles of 16 rows of W: tile b, b + blocks, ...);
//   * W arrives by TMA in boxes of 16 rows x 256 k (8 KB) that complete on a stage's mbarrier, into a ring of 16 stages:
//     the bytes in flight are the ring's 128 KB per SM whatever the warps are doing; rows beyond N and k beyond K arrive
//     as zeros;
//   * the kernel is launched with programmatic stream serialization: its blocks may start while the kernel before it is
//     still running, fill their rings (weights do not depend on that kernel) and only then wait for it
//     (griddepcontrol.wait).
// Stage i of a block's ring (counted over all its tiles) lies in slot i mod 16 and belongs to warp i mod 8, which asks
// for it, waits for it, multiplies with it and asks for the stage that comes into the slot next.  Two measurements
// decided that.  A thread starts TMA copies only so fast (about 0.15 us and 0.02 us a KB, whatever the box's shape;
// row-by-row bulk copies of 1 KB gave 3.1 TB/s, one producer thread with 8 KB boxes 3.7), so all eight warps ask.  And
// a wait names a phase by its parity only: a slot must always be awaited by the same warp, else a fast warp asks for the
// slot's next phase while the one before is still pending and is told "done" (seen as wrong sums whenever two launches
// overlapped).  The warps read W from shared memory into mma.m16n8k16 fragments (W is the 16-row operand, 8 rows of x the
// 8-column operand: y^T = W x^T; x comes through L1 and is asked for before the wait for W) and keep their sums over a
// whole tile in registers; at the tile's end the warps' sums meet in shared memory and are added in warp order.  Which
// warp takes which k depends on N, K and the number of SMs only, so a row's result depends neither on the batch nor on
// timing.  Every mbarrier wait is bounded: after a second the block raises *error, stops waiting and asking, and runs
// to its end.  (The reference's counterpart for few rows: ggml-cuda/mmvf.cu and mmf.cuh; it has no counterpart of the
// ring.)
//
// The split form (GR_EPI_SPLIT).  With whole tiles a matrix of 256 tiles keeps 148 SMs busy for two rounds of which the
// second is three quarters empty (4,096 rows: 86 % of the stream; 5,120 rows: 72 %).  In the split form every block takes
// an equal, contiguous share of all (tile, k) stages instead, so a tile may be cut between two or three blocks that
// follow one another.  Nobody waits for anybody: each block writes the sum over its piece of the tile into the piece's
// own plane of `y` ([pieces][M][N]; the piece of lowest k is plane 0), and the kernel that consumes the product - the
// norm that adds it onto the residual stream - adds a tile's planes in that order.  How many planes a tile has follows
// from N, K and the number of blocks alone (the host hands the consumer a table), so the result does not depend on timing.
#include "common.cuh"

#include <cuda.h>

#define GR_ROWS 16                    // rows of W per tile: the mma's 16-row operand
#define GR_WAIT_NS 1000000000ull       // a wait gives up after a second

#define GR_EPI_PLAIN 0                // y = product (+ residual)
#define GR_EPI_SWIGLU 1               // rows of W: for every 8 features their 8 gate rows, then their 8 up rows
#define GR_EPI_SPLIT 2                // equal shares of stages per block; y = [pieces][M][N], see above

__device__ __forceinline__ uint32_t gr_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gr_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gr_smem(bar)), "r"(count));
}
__device__ __forceinline__ void gr_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gr_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool gr_mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(gr_smem(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Once any wait of the block has run out, no thread of the block waits again: the block runs to its end
// on whatever lies in shared memory (its result is not valid, *error says so).
__device__ __forceinline__ uint64_t gr_now_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void gr_wait(uint64_t* bar, uint32_t parity, volatile int* failed, int* error, int code) {
    if (*failed) return;
    uint64_t start = 0;
    for (uint32_t i = 1;; ++i) {
        if (gr_mbar_try_wait(bar, parity)) return;
        if ((i & 1023u) == 0) {                              // the clock is read now and then, not at every poll
            const uint64_t now = gr_now_ns();
            if (!start) start = now;
            else if (now - start > GR_WAIT_NS) break;
        }
    }
    *failed = 1;
    if (error) atomicExch(error, code);
}
// One box of W, rows [row, row + 16) x k [k, k + 256): global -> shared, completing its 8 KB on the stage's mbarrier.
// k is a multiple of 256, so the copy starts on a 16-byte boundary as TMA demands.
__device__ __forceinline__ void gr_tma_box(void* dst, const CUtensorMap* map, uint64_t* bar, int k, int row) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(gr_smem(dst)), "l"(map), "r"(gr_smem(bar)), "r"(k), "r"(row) : "memory");
}
__device__ __forceinline__ void gr_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#define GR_BOX_K 256                  // k per TMA box (the most a box takes)
#define GR_BOX_BYTES (GR_ROWS * GR_BOX_K * 2)

template <int NT, int GR_KC, int GR_STAGES, int GR_WARPS>
struct GrSmem {
    static constexpr int STAGE_BYTES = GR_ROWS * GR_KC * 2;      // GR_KC / 256 boxes of [16 rows][256 k], one after the other
    static constexpr size_t PART_BYTES = (size_t)2 * GR_WARPS * NT * 4 * 32 * sizeof(float);    // two tiles' worth
    static constexpr size_t BYTES = 128 + (size_t)GR_STAGES * STAGE_BYTES + PART_BYTES + GR_STAGES * sizeof(uint64_t) + 16;   // 128: to align
};

// NT = number of 8-row tiles of x handled at once (M <= 8 * NT); GR_KC = k per stage; GR_STAGES = stages of the ring;
// GR_WARPS = warps (GR_STAGES is a multiple of it); SPW: see below (0: the general form).
template <int NT, int EPI, int GR_KC, int GR_STAGES, int GR_WARPS, int SPW>
__global__ void __launch_bounds__(GR_WARPS * 32)
gemm_ring_kernel(const bf16* x, const __grid_constant__ CUtensorMap map_w, const float* residual, float* y,
                 bf16* __restrict__ act, int M, int N, int K, int* error) {
    using Smem = GrSmem<NT, GR_KC, GR_STAGES, GR_WARPS>;
    constexpr int GR_STAGE_BYTES = Smem::STAGE_BYTES;
    extern __shared__ unsigned char gr_smem_unaligned[];
    unsigned char* stages = reinterpret_cast<unsigned char*>(((uintptr_t)gr_smem_unaligned + 127) & ~(uintptr_t)127);
    float* part = reinterpret_cast<float*>(stages + (size_t)GR_STAGES * GR_STAGE_BYTES);          // [2][warp][tile][c register][lane]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(part) + Smem::PART_BYTES);
    volatile int* failed = reinterpret_cast<volatile int*>(full_bar + GR_STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (N + GR_ROWS - 1) / GR_ROWS;
    const int n_stages = (K + GR_KC - 1) / GR_KC;           // stages per tile
    const int chunks = K >> 3;                               // 16-byte chunks per row of W and of x
    // the stages that pass through this block's ring: those of its tiles (tile b, b + blocks, ...), or, in the split form,
    // stages [begin, begin + total) of all the matrix's stages, counted tile by tile
    constexpr bool SPLIT = EPI == GR_EPI_SPLIT;
    const long long all_stages = (long long)n_tiles * n_stages;
    const int begin = SPLIT ? (int)(all_stages * blockIdx.x / gridDim.x) : 0;
    const int total = SPLIT ? (int)(all_stages * (blockIdx.x + 1) / gridDim.x) - begin
                            : (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x * n_stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GR_STAGES; ++s) gr_mbar_init(full_bar + s, 1);      // the arrival that announces the stage's bytes
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();                                 // the next kernel may start beside this one: it is built to fit

    // Stage i of the ring (counted over all of the block's tiles) lies in slot i mod GR_STAGES and belongs to warp
    // i mod GR_WARPS: the ring has a multiple of GR_WARPS slots, so a slot is always filled, awaited and read by the same
    // warp.  That matters twice.  A wait names a phase by its parity only, so whoever waits on a slot must have seen the
    // slot's phase before (a slot read by different warps in turn lets a fast warp ask for the next phase while the one
    // before is pending, and be told "done").  And a thread can start TMA copies only so fast (about 0.15 us and 0.02 us a
    // KB, measured), so one producer cannot feed an SM; here every warp asks for its own stages.
    auto request = [&](int i) {                              // lane 0: ask for stage i into its slot
        const int slot = i % GR_STAGES;
        const int tile = SPLIT ? (begin + i) / n_stages : blockIdx.x + (i / n_stages) * gridDim.x;
        const int k0 = (SPLIT ? (begin + i) % n_stages : i % n_stages) * GR_KC;
        const int boxes = min(GR_KC / GR_BOX_K, (K - k0 + GR_BOX_K - 1) / GR_BOX_K);          // none wholly beyond K
        gr_mbar_expect_tx(full_bar + slot, (uint32_t)boxes * GR_BOX_BYTES);
        for (int b = 0; b < boxes; ++b)
            gr_tma_box(stages + (size_t)slot * GR_STAGE_BYTES + (size_t)b * GR_BOX_BYTES, &map_w, full_bar + slot,
                       k0 + b * GR_BOX_K, tile * GR_ROWS);
    };
    // W does not depend on the kernel before this one: the ring fills before that kernel has ended
    if (lane == 0)
        for (int i = warp; i < GR_STAGES && i < total; i += GR_WARPS) request(i);
    pdl_wait();                                              // x (and the residual) come from the kernel before

    const int g = lane >> 2, t = lane & 3;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    constexpr int KB = GR_KC / 32;                           // blocks of 32 k per stage
    const uint4* xr[NT];
    bool x_ok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m = 8 * j + g;
        x_ok[j] = m < M;
        xr[j] = reinterpret_cast<const uint4*>(x + (size_t)min(m, M - 1) * K);
    }
    // SPW > 0: a tile has exactly SPW * GR_WARPS stages, so a warp meets the same k in every tile (stages kfix, kfix + 8, ...
    // of a tile, kfix = warp unless the block's share begins in the middle of a tile) and keeps its pieces of x in
    // registers for the whole product instead of asking L1 for them at every stage.
    // (With 1, 2 or 4 stages a tile the same holds with one stage a warp, kfix = warp modulo the stages, and a warp has a
    // stage only in every 8th, 4th or 2nd tile.)
    const int kfix = (begin + warp) % min(n_stages, GR_WARPS);
    uint4 xkeep[SPW > 0 ? SPW : 1][KB][NT];
    if (SPW > 0) {
#pragma unroll
        for (int q = 0; q < (SPW > 0 ? SPW : 1); ++q)
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int c = (kfix + q * GR_WARPS) * (GR_KC / 8) + kb * 4 + t;
                    xkeep[q][kb][j] = (c < chunks && x_ok[j]) ? __ldcg(xr[j] + c) : zero;
                }
    }
    // The block's pieces: stages [i_lo, i_lo + n_here) of its ring are stages [ks_lo, ks_lo + n_here) of one tile (a whole
    // tile unless the split form cuts it).
    int buf = 0;
    for (int i_lo = 0; i_lo < total; buf ^= 1) {
        const int tile = SPLIT ? (begin + i_lo) / n_stages : blockIdx.x + (i_lo / n_stages) * gridDim.x;
        const int ks_lo = SPLIT ? (begin + i_lo) % n_stages : 0;
        const int n_here = min(n_stages - ks_lo, total - i_lo);
        const int n0 = tile * GR_ROWS;
        float acc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        // the value that this thread's output of the tile is added onto: asked for now, used in the epilogue (asked for
        // there, every tile ended with a round trip to L2 during which the thread's warp asked for no new stage)
        static_assert(NT * 4 * 32 <= GR_WARPS * 32, "a thread has at most one output of a tile");
        float onto = 0.f;
        if (EPI == GR_EPI_PLAIN && !SPLIT && residual && threadIdx.x < NT * 4 * 32) {
            const int j = threadIdx.x >> 7, r = (threadIdx.x >> 5) & 3;
            const int n = n0 + (lane >> 2) + ((r & 2) ? 8 : 0), m = 8 * j + 2 * (lane & 3) + (r & 1);
            if (n < N && m < M) onto = __ldcg(residual + (size_t)m * N + n);
        }
        // one stage (i of the ring, ks of the tile): wait for its bytes, multiply, ask for the stage that comes into the slot next
        auto stage = [&](int i, int ks, const uint4 (&xv)[KB][NT]) {
            const int slot = i % GR_STAGES, use = i / GR_STAGES;
            const int c0 = ks * (GR_KC / 8);                 // the stage's first 16-byte chunk of a row
            gr_wait(full_bar + slot, use & 1, failed, error, 2);
            const unsigned char* st = stages + (size_t)slot * GR_STAGE_BYTES;
            // The slot is read, then the same warp asks for the stage that comes into it next (the fence orders the reads,
            // made through the generic proxy, before the copy's writes through the asynchronous one).  With two tiles of
            // rows the whole stage goes into registers first and the slot is handed back before the products, whose 32
            // instructions would else keep it out of flight (10 tiles a block: 36.8 -> 32.5 us); with one tile the loads
            // and products interleaved are faster (30.3 against 33.4 us).
            auto hand_back = [&]() {
                __syncwarp();
                if (lane == 0 && i + GR_STAGES < total && !*failed) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    request(i + GR_STAGES);
                }
            };
            if (NT >= 2 && SPW > 0) {                   // (with the rows of x loaded stage by stage as well: 22.6 against 22.0 us)
                uint4 lo[KB], hi[KB];
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const bool in = c0 + kb * 4 + t < chunks;
                    const unsigned char* box = st + (size_t)(kb / (GR_BOX_K / 32)) * GR_BOX_BYTES + (kb % (GR_BOX_K / 32)) * 64 + t * 16;
                    lo[kb] = in ? *reinterpret_cast<const uint4*>(box + (size_t)g * (GR_BOX_K * 2)) : zero;
                    hi[kb] = in ? *reinterpret_cast<const uint4*>(box + (size_t)(g + 8) * (GR_BOX_K * 2)) : zero;
                }
                hand_back();
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        gr_mma(acc[j], lo[kb].x, hi[kb].x, lo[kb].y, hi[kb].y, xv[kb][j].x, xv[kb][j].y);
                        gr_mma(acc[j], lo[kb].z, hi[kb].z, lo[kb].w, hi[kb].w, xv[kb][j].z, xv[kb][j].w);
                    }
            } else {
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const bool in = c0 + kb * 4 + t < chunks;
                    const unsigned char* box = st + (size_t)(kb / (GR_BOX_K / 32)) * GR_BOX_BYTES + (kb % (GR_BOX_K / 32)) * 64 + t * 16;
                    const uint4 lo = in ? *reinterpret_cast<const uint4*>(box + (size_t)g * (GR_BOX_K * 2)) : zero;
                    const uint4 hi = in ? *reinterpret_cast<const uint4*>(box + (size_t)(g + 8) * (GR_BOX_K * 2)) : zero;
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        gr_mma(acc[j], lo.x, hi.x, lo.y, hi.y, xv[kb][j].x, xv[kb][j].y);
                        gr_mma(acc[j], lo.z, hi.z, lo.w, hi.w, xv[kb][j].z, xv[kb][j].w);
                    }
                }
                hand_back();
            }
        };
        if (SPW > 0) {
#pragma unroll
            for (int q = 0; q < (SPW > 0 ? SPW : 1); ++q) {
                const int ks = kfix + q * GR_WARPS;          // stage ks of the tile is stage i_lo + ks - ks_lo of the ring
                const int i = i_lo + ks - ks_lo;
                if ((!SPLIT || (ks >= ks_lo && ks < ks_lo + n_here)) && (i % GR_WARPS == warp)) stage(i, ks, xkeep[q]);
            }
        } else {
            // a thread's 16 bytes are eight consecutive k of one row; W and x use the same renumbering of k inside a
            // block of 32, so no shuffle is needed (the sum over k does not care about the order).  The rows of x for a
            // stage are asked for one stage of the warp ahead (with one tile of rows; with two the registers do not
            // reach), by plain loads: through L1, which holds rows of up to about 5,000 values beside the ring.
            auto load_x = [&](int ks, uint4 (&xv)[KB][NT]) {
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const int c = ks * (GR_KC / 8) + kb * 4 + t;
                        xv[kb][j] = (c < chunks && x_ok[j]) ? xr[j][c] : zero;
                    }
            };
            const int i_first = i_lo + (warp - i_lo % GR_WARPS + GR_WARPS) % GR_WARPS;
            if (NT == 1) {
                uint4 xv[KB][NT], xn[KB][NT];
                if (i_first < i_lo + n_here) load_x(ks_lo + i_first - i_lo, xv);
                for (int i = i_first; i < i_lo + n_here; i += GR_WARPS) {
                    const bool more = i + GR_WARPS < i_lo + n_here;
                    if (more) load_x(ks_lo + i + GR_WARPS - i_lo, xn);
                    stage(i, ks_lo + i - i_lo, xv);
                    if (more) {
#pragma unroll
                        for (int kb = 0; kb < KB; ++kb) xv[kb][0] = xn[kb][0];
                    }
                }
            } else {
                for (int i = i_first; i < i_lo + n_here; i += GR_WARPS) {
                    uint4 xv[KB][NT];
                    load_x(ks_lo + i - i_lo, xv);
                    stage(i, ks_lo + i - i_lo, xv);
                }
            }
        }
        i_lo += n_here;
        float* mine = part + (size_t)buf * GR_WARPS * NT * 128;
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) mine[((warp * NT + j) * 4 + r) * 32 + lane] = acc[j][r];
        __syncthreads();
        // c0: (row g, col 2t), c1: (row g, col 2t+1), c2: (row g+8, col 2t), c3: (row g+8, col 2t+1);
        // rows are rows of W (outputs n), columns are rows of x (m).
        if (EPI == GR_EPI_PLAIN || SPLIT) {
            // split form: the plane of this piece = how many blocks before this one hold earlier pieces of the tile
            // (the tile's first stage lies in block ((first + 1) * blocks - 1) / all_stages)
            size_t plane = 0;
            if (SPLIT && ks_lo > 0)
                plane = (size_t)(blockIdx.x - (int)((((long long)tile * n_stages + 1) * gridDim.x - 1) / all_stages)) * M * N;
            for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += GR_WARPS * 32) {
                const int j = idx >> 7, r = (idx >> 5) & 3, ln = idx & 31;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < GR_WARPS; ++w) sum += mine[((w * NT + j) * 4 + r) * 32 + ln];
                const int n = n0 + (ln >> 2) + ((r & 2) ? 8 : 0), m = 8 * j + 2 * (ln & 3) + (r & 1);
                if (n < N && m < M) {
                    const size_t at = (size_t)m * N + n;
                    if (SPLIT) y[plane + at] = sum;
                    else y[at] = onto + sum;
                }
            }
        } else {                                             // rows g are gates, rows g + 8 the ups of the same features
            const int F = N >> 1, f0 = n0 >> 1;
            for (int idx = threadIdx.x; idx < NT * 2 * 32; idx += GR_WARPS * 32) {
                const int j = idx >> 6, r = (idx >> 5) & 1, ln = idx & 31;
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int w = 0; w < GR_WARPS; ++w) {
                    gate += mine[((w * NT + j) * 4 + r) * 32 + ln];
                    up += mine[((w * NT + j) * 4 + r + 2) * 32 + ln];
                }
                const int f = f0 + (ln >> 2), m = 8 * j + 2 * (ln & 3) + r;
                if (f < F && m < M) act[(size_t)m * F + f] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
            }
        }
    }
}

static int gr_sm_count() {
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    return n_sm;
}

typedef CUresult (*GrEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// W [rows, K] row-major bfloat16, moved in boxes of 16 rows x 256 k, as they lie (no swizzle); outside the matrix: zeros.
static int gr_make_map(CUtensorMap* map, const void* W, int rows, int K) {
    static GrEncodeTiledFn enc = nullptr;
    if (!enc) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            enc = reinterpret_cast<GrEncodeTiledFn>(p);
        if (!enc) return qwb_fail(QWB_ERR_CUDA, "gemm_ring: cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {GR_BOX_K, GR_ROWS};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(W), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qwb_fail(QWB_ERR_CUDA, "gemm_ring: cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

template <int NT, int EPI, int KC, int STAGES, int WARPS, int SPW>
static int launch_ring_as(const bf16* x, const bf16* W, const float* residual, float* y, bf16* act, int M, int N, int K,
                          int* error, cudaStream_t stream, int split_blocks) {
    static_assert(STAGES % WARPS == 0, "a slot of the ring must always go to the same warp");
    CUtensorMap map_w;
    if (int rc = gr_make_map(&map_w, W, N, K)) return rc;
    const size_t smem = GrSmem<NT, KC, STAGES, WARPS>::BYTES;
    static bool sized = false;
    if (!sized) {
        cudaError_t e = cudaFuncSetAttribute(gemm_ring_kernel<NT, EPI, KC, STAGES, WARPS, SPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "gemm_ring: %s", cudaGetErrorString(e));
        sized = true;
    }
    const int n_tiles = (N + GR_ROWS - 1) / GR_ROWS;
    int grid = n_tiles < gr_sm_count() ? n_tiles : gr_sm_count();              // one block per SM, each walks over its tiles
    if (EPI == GR_EPI_SPLIT) grid = split_blocks;                              // the caller's: the planes' table follows from it
    qwb_launch_early(gemm_ring_kernel<NT, EPI, KC, STAGES, WARPS, SPW>, grid, WARPS * 32, smem, stream, x, map_w, residual, y, act, M, N, K, error);
    return qwb_check_launch("gemm_ring");
}

// 16 stages of 16 rows x 256 k (one TMA box of 8 KB each): 128 KB in flight per SM, eight warps.  Measured against other
// rings on the products of a Qwen3-8B decode step (8 rows; us for q/k/v, o, gate/up, down, head): 8 stages 12.4, 8.7, 39.2,
// 21.4, 215; 16 stages 10.3, 7.5, 32.1, 18.2, 178; 24 stages 11.4, 8.0, 36.2, 18.8, 194 (the L1 that is left no longer
// holds the rows of x); 8 stages of 512 k 11.0, 7.8, 33.5, 18.8, 178; 12 stages with 6 or 12 warps 12.3-13.7, 8.6-9.4,
// 39.5-43.2, 19.5, 213-226.  With x kept in registers (rows of 4,096): 9.2, 6.7, 30.8 at 8 rows; at 16 rows 12.1, 9.2, 36.0
// and the head 197 against 13.3, 9.5, 42.0 and 233 without.
template <int NT, int EPI>
static int launch_ring(const bf16* x, const bf16* W, const float* residual, float* y, bf16* act, int M, int N, int K,
                       int* error, cudaStream_t stream, int split_blocks = 0) {
    // rows of 8 or 16 stages (up to 2,048 or 4,096 values), or of 1, 2 or 4: a warp meets the same one or two stages of k
    // in every tile that it has a stage of, and keeps its x
    const int n_stages = (K + 255) / 256;
    if (n_stages == 8 || n_stages == 4 || n_stages == 2 || n_stages == 1) return launch_ring_as<NT, EPI, 256, 16, 8, 1>(x, W, residual, y, act, M, N, K, error, stream, split_blocks);
    if (n_stages == 16) return launch_ring_as<NT, EPI, 256, 16, 8, 2>(x, W, residual, y, act, M, N, K, error, stream, split_blocks);
    return launch_ring_as<NT, EPI, 256, 16, 8, 0>(x, W, residual, y, act, M, N, K, error, stream, split_blocks);
}

static int check_ring(const void* x, const void* W, int M, int K) {
    if (K <= 0 || K % 8) return qwb_fail(QWB_ERR_ARG, "gemm_ring: inner size %d is not a multiple of 8", K);
    if (M > 16) return qwb_fail(QWB_ERR_ARG, "gemm_ring: %d rows; this kernel is for at most 16", M);
    if ((uintptr_t)x % 16 || (uintptr_t)W % 16) return qwb_fail(QWB_ERR_ARG, "gemm_ring: operands must be 16-byte aligned");
    return 0;
}

// error: one int on the device that a block sets when one of its bounded waits runs out (1: the producer waiting for a free
// stage, 2: a consumer waiting for a stage's bytes); the caller looks at it when it next synchronises.  May be null.
extern "C" int qwb_gemm_ring(const void* x, const void* W, const float* residual, float* y, int M, int N, int K, int* error,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (int rc = check_ring(x, W, M, K)) return rc;
    if (M <= 8) return launch_ring<1, GR_EPI_PLAIN>((const bf16*)x, (const bf16*)W, residual, y, nullptr, M, N, K, error, stream);
    return launch_ring<2, GR_EPI_PLAIN>((const bf16*)x, (const bf16*)W, residual, y, nullptr, M, N, K, error, stream);
}

// The split form: `planes` float [pieces][M][N], pieces = the most blocks that share a tile when `blocks` blocks take equal
// shares of the ceil(N / 16) * ceil(K / 256) stages (block b: stages [b * all / blocks, (b + 1) * all / blocks), counted
// tile by tile).  Plane p of a tile's columns holds the sum over the tile's p-th piece; planes that a tile does not have
// are not written.
extern "C" int qwb_gemm_ring_split(const void* x, const void* W, float* planes, int M, int N, int K, int blocks, int* error,
                                   cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (int rc = check_ring(x, W, M, K)) return rc;
    const long long all_stages = (long long)((N + GR_ROWS - 1) / GR_ROWS) * ((K + 255) / 256);
    if (blocks <= 0 || blocks > all_stages) return qwb_fail(QWB_ERR_ARG, "gemm_ring: %d blocks for %lld stages", blocks, all_stages);
    if (M <= 8) return launch_ring<1, GR_EPI_SPLIT>((const bf16*)x, (const bf16*)W, nullptr, planes, nullptr, M, N, K, error, stream, blocks);
    return launch_ring<2, GR_EPI_SPLIT>((const bf16*)x, (const bf16*)W, nullptr, planes, nullptr, M, N, K, error, stream, blocks);
}

// W [2 F, K]: for every 8 features their 8 gate rows, then their 8 up rows (F a multiple of 8).
// act bfloat16 [M, F] = silu(x gate^T) * (x up^T).
extern "C" int qwb_gemm_ring_swiglu(const void* x, const void* W, void* act, int M, int F, int K, int* error, cudaStream_t stream) {
    if (M <= 0 || F <= 0) return 0;
    if (F % 8) return qwb_fail(QWB_ERR_ARG, "gemm_ring: %d features are not a multiple of 8", F);
    if (int rc = check_ring(x, W, M, K)) return rc;
    if (M <= 8) return launch_ring<1, GR_EPI_SWIGLU>((const bf16*)x, (const bf16*)W, nullptr, nullptr, (bf16*)act, M, 2 * F, K, error, stream);
    return launch_ring<2, GR_EPI_SWIGLU>((const bf16*)x, (const bf16*)W, nullptr, nullptr, (bf16*)act, M, 2 * F, K, error, stream);
}
