// Matrix product on the fifth-generation tensor cores (tcgen05) for many rows of bfloat16 x:
//     y[M,N] = x[M,K] W[N,K]^T, 32-bit sums in tensor memory, with the epilogue fused:
//       EPI_STORE   y float                               (the q/k/v projection)
//       EPI_ADD     y += product, y float                 (o and down projections onto the residual stream)
//       EPI_SWIGLU  a = silu(gate) * up as bfloat16       (gate/up projection; W holds, for every 8 features, their 8 gate
//                                                          rows and then their 8 up rows)
//
// One block per SM walks over 128 x BN tiles of y (tile t, t + blocks, ...).  Six warps with fixed roles:
//   warp 0  one lane issues the TMA loads: per 64 columns of k a 128 x 64 tile of x and a BN x 64 tile of W, into a ring
//           of shared-memory stages in the 128-byte swizzle that the tensor core reads; each stage has a "full" mbarrier
//           that the loads complete and an "empty" mbarrier that the tensor core releases;
//   warp 1  allocates 2 x BN columns of tensor memory (two accumulators, so that one tile's epilogue runs under the next
//           tile's products); one lane issues four tcgen05.mma (128 x BN x 16) per stage straight from shared memory,
//           commits the stage's "empty" barrier after them and, after a tile's last stage, the accumulator's "full" barrier;
//   warps 2-5  wait for the accumulator, read it with tcgen05.ld (each warp its own 32 lanes = 32 rows of the tile), stage
//           it in shared memory and hand it to TMA: a store, or a reduce-add onto y for the residual sum.  A thread owns a
//           row, so the SwiGLU epilogue finds gate and up of one feature in the same thread.
// Rows and columns beyond M, N and K are zero-filled by the TMA loads and dropped by the TMA stores.  No wait is unbounded: each mbarrier
// wait gives up after a fixed number of polls, raises *error and lets the block run to its end, where outstanding loads are
// awaited (bounded) and the tensor memory is freed.  (The reference has only a library call here: cuBLAS above 16 rows,
// ggml-cuda/ggml-cuda.cu:1405-1617.)
#include "common.cuh"

#include <cuda.h>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_SPIN_LIMIT (1u << 22)
#define TC_STAGING_BYTES 4096      // one warp's staging tile of the epilogue: 32 rows of 128 bytes

#define EPI_STORE 0
#define EPI_ADD 1
#define EPI_SWIGLU 2

// ------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if the barrier did not flip within the poll limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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

// Shared-memory operand descriptor of a K-major tile whose rows are 64 bfloat16 = 128 bytes, in the 128-byte swizzle:
// start address / 16, leading offset 1 (unused for swizzled K-major), stride between groups of 8 rows = 1024 bytes,
// descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: D float (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1), both K-major (bits 15, 16 = 0),
// N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int BN> struct TcStages { static constexpr int value = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8); };

template <int BN>
struct TcSmem {
    static constexpr int STAGES = TcStages<BN>::value;
    static constexpr size_t A_BYTES = (size_t)TC_BM * TC_BK * 2, B_BYTES = (size_t)BN * TC_BK * 2;
    static constexpr size_t BYTES = 1024 + STAGES * (A_BYTES + B_BYTES) + 8 * TC_STAGING_BYTES + 512;   // 1024: to align
};

template <int BN, int EPI>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, int M, int N, int K, int* error) {
    constexpr int STAGES = TcSmem<BN>::STAGES;
    constexpr uint32_t A_BYTES = TcSmem<BN>::A_BYTES, B_BYTES = TcSmem<BN>::B_BYTES;
    constexpr int COLS_PER_TILE = EPI == EPI_SWIGLU ? BN / 2 : BN;     // output columns of one tile
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = tiles;
    unsigned char* b_tiles = tiles + STAGES * A_BYTES;
    unsigned char* staging = b_tiles + STAGES * B_BYTES;              // [4 warps][2][32 rows][128 bytes]
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + 4 * 2 * TC_STAGING_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_full = empty_bar + STAGES;                          // [2]: the tensor core has finished a tile
    uint64_t* acc_empty = acc_full + 2;                               // [2]: the epilogue has read a tile out
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    // The block walks over tiles first, first + gridDim.x, ...  Tiles are numbered with the row tile as the fast index:
    // blocks that run together share tiles of W, so W streams from HBM once and the (much smaller) x stays in L2.
    const int m_tiles = (M + TC_BM - 1) / TC_BM, n_tiles = (N + COLS_PER_TILE - 1) / COLS_PER_TILE;
    const int n_total = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 2 * BN);                     // two accumulators: one fills while the other drains
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_wait();                 // x comes from the kernel before this one
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                               // k blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * COLS_PER_TILE;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
                    tma_load_2d(a_tiles + (size_t)s * A_BYTES, &map_x, &full_bar[s], kb * TC_BK, m0);
                    // SwiGLU: COLS_PER_TILE features are BN rows of W, gate and up interleaved in eights
                    tma_load_2d(b_tiles + (size_t)s * B_BYTES, &map_w, &full_bar[s], kb * TC_BK, EPI == EPI_SWIGLU ? 2 * n0 : n0);
                }
            }
            if (!ok) {
                atomicExch(error, 1);
                // loads already issued still write shared memory: wait for them (bounded) before the block ends
                for (int j = max(0, it - STAGES); j < it; ++j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(TC_BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1);   // the epilogue is done with it
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_acc = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(&full_bar[s], (it / STAGES) & 1);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = make_smem_desc(a_tiles + (size_t)s * A_BYTES);
                    const uint64_t db = make_smem_desc(b_tiles + (size_t)s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)      // 16 columns of k = 32 bytes = 2 units of the start address
                        umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);               // arrives when these MMAs have read the stage
                }
                umma_commit(&acc_full[buf]);                  // arrives when every MMA issued so far is done
            }
            if (!ok) {
                atomicExch(error, 2);
                umma_commit(&acc_full[0]);                    // let the epilogue warps run out instead of timing out one by one
                umma_commit(&acc_full[1]);
            }
        }
    } else {
        // Each warp owns 32 rows.  Per chunk of output columns it moves its accumulator lanes into a staging tile in
        // shared memory (rows of 128 bytes, 16-byte pieces XOR-swizzled by the row so that neither these writes nor
        // the TMA unit meet bank conflicts) and one lane hands the tile to TMA: a store, or an add onto global memory
        // for the residual sum.  Two staging tiles per warp let the next chunk be prepared while the last one drains.
        const int lane_group = warp & 3;                      // a warp reads tensor-memory lanes [32 * (warp % 4), + 32)
        unsigned char* stage0 = staging + (size_t)lane_group * 2 * TC_STAGING_BYTES;
        constexpr int CHUNKS = EPI == EPI_SWIGLU ? BN / 2 / 64 : BN / 32;
        int local = 0, stores = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % m_tiles) * TC_BM, n0 = (tile / m_tiles) * COLS_PER_TILE;
            ok = mbar_wait(&acc_full[buf], (local >> 1) & 1);
            tc_fence_after();
            if (!ok) {
                if (lane == 0) atomicExch(error, 3);
                break;
            }
            const int row0 = m0 + 32 * lane_group;
            const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(32 * lane_group) << 16);
#pragma unroll 1
            for (int ch = 0; ch < CHUNKS; ++ch, ++stores) {
                unsigned char* st = stage0 + (size_t)(stores & 1) * TC_STAGING_BYTES;
                if (stores >= 2) {                            // the store that read this tile two chunks ago must be done
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
                uint4* my_row = reinterpret_cast<uint4*>(st + lane * 128);
                if (EPI == EPI_SWIGLU) {
                    // 64 features = 128 accumulator columns: per 16 columns 8 gates, then the 8 ups of the same features
#pragma unroll
                    for (int q = 0; q < 4; ++q) {             // 4 x 16 features -> 64 bfloat16 = one 128-byte row
                        uint32_t v[32];
                        tmem_ld32(taddr + ch * 128 + q * 32, v);
#pragma unroll
                        for (int grp = 0; grp < 2; ++grp) {
                            uint32_t pk[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float g0 = __uint_as_float(v[16 * grp + 2 * j]), g1 = __uint_as_float(v[16 * grp + 2 * j + 1]);
                                const float a0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(v[16 * grp + 8 + 2 * j]);
                                const float a1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(v[16 * grp + 8 + 2 * j + 1]);
                                __nv_bfloat162 r = __floats2bfloat162_rn(a0, a1);
                                pk[j] = *reinterpret_cast<uint32_t*>(&r);
                            }
                            my_row[(q * 2 + grp) ^ (lane & 7)] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    }
                } else {
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; i += 4) my_row[(i / 4) ^ (lane & 7)] = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                }
                if (ch == CHUNKS - 1) {                       // the accumulator is read out: the tensor core may have it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    const int col = n0 + ch * (EPI == EPI_SWIGLU ? 64 : 32);
                    if (EPI == EPI_ADD)
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_out), "r"(smem_u32(st)), "r"(col), "r"(row0) : "memory");
                    else
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_out), "r"(smem_u32(st)), "r"(col), "r"(row0) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory is read, global is written
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

// ------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// A [rows, cols] row-major matrix of bfloat16 (or float), moved in boxes of box_rows x 128 bytes in the 128-byte swizzle;
// reads outside the matrix give zero, writes outside are dropped.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows, const char* what, bool is_float = false) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return qwb_fail(QWB_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    const int elem_bytes = is_float ? 4 : 2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, is_float ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                     const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return qwb_fail(QWB_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
    return 0;
}

template <int BN, int EPI>
static int launch_tc(const void* x, const void* W, void* out, int M, int N, int K, int w_rows, int* error, cudaStream_t stream) {
    CUtensorMap map_x, map_w, map_out;
    if (int rc = make_map(&map_x, x, M, K, TC_BM, "x")) return rc;
    if (int rc = make_map(&map_w, W, w_rows, K, BN, "W")) return rc;
    if (int rc = make_map(&map_out, out, M, N, 32, "out", EPI != EPI_SWIGLU)) return rc;
    const size_t smem = TcSmem<BN>::BYTES;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "gemm_tc: %s", cudaGetErrorString(e));
    const int cols_per_block = EPI == EPI_SWIGLU ? BN / 2 : BN;
    const long long n_tiles = (long long)((M + TC_BM - 1) / TC_BM) * ((N + cols_per_block - 1) / cols_per_block);
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) n_sm = 148;
    }
    dim3 grid((unsigned)(n_tiles < n_sm ? n_tiles : n_sm));          // one block per SM, each walks over its tiles
    e = qwb_launch(gemm_tc_kernel<BN, EPI>, grid, TC_THREADS, smem, stream, map_x, map_w, map_out, M, N, K, error);
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "gemm_tc: launch failed: %s", cudaGetErrorString(e));
    return qwb_check_launch("gemm_tc");
}

// x [M, K] and W bfloat16, 16-byte aligned, K a multiple of 8.  `error` is one int on the device, 0 before the call; a
// value other than 0 afterwards means a wait inside the kernel gave up (the result is then not valid).
//   epilogue 0: W [N, K], out float [M, N]          1: the same, out += product
//   epilogue 2: W [2 N, K] (for every 8 features their 8 gate rows, then their 8 up rows), out bfloat16 [M, N] = silu(gate) * up
extern "C" int qwb_gemm_tc(const void* x, const void* W, void* out, int epilogue, int M, int N, int K, int tile_n, int* error,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8) return qwb_fail(QWB_ERR_ARG, "gemm_tc: inner size %d is not a multiple of 8", K);
    if (N % 8) return qwb_fail(QWB_ERR_ARG, "gemm_tc: %d output columns are not a multiple of 8", N);
    if ((uintptr_t)x % 16 || (uintptr_t)W % 16 || (uintptr_t)out % 16) return qwb_fail(QWB_ERR_ARG, "gemm_tc: operands must be 16-byte aligned");
    if (!error) return qwb_fail(QWB_ERR_ARG, "gemm_tc: an error word on the device is required");
    if (epilogue == EPI_SWIGLU) {
        if (tile_n == 128) return launch_tc<128, EPI_SWIGLU>(x, W, out, M, N, K, 2 * N, error, stream);
        if (tile_n == 256) return launch_tc<256, EPI_SWIGLU>(x, W, out, M, N, K, 2 * N, error, stream);
        return qwb_fail(QWB_ERR_ARG, "gemm_tc: tile width %d is not 128 or 256", tile_n);
    }
    if (epilogue != EPI_STORE && epilogue != EPI_ADD) return qwb_fail(QWB_ERR_ARG, "gemm_tc: unknown epilogue %d", epilogue);
#define TC_CASE(BN)                                                                                          \
    if (tile_n == BN)                                                                                        \
        return epilogue == EPI_STORE ? launch_tc<BN, EPI_STORE>(x, W, out, M, N, K, N, error, stream)        \
                                     : launch_tc<BN, EPI_ADD>(x, W, out, M, N, K, N, error, stream);
    TC_CASE(64) TC_CASE(128) TC_CASE(256)
#undef TC_CASE
    return qwb_fail(QWB_ERR_ARG, "gemm_tc: tile width %d is not 64, 128 or 256", tile_n);
}
