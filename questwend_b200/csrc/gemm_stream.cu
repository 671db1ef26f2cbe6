// Weight-streaming matrix product on the tensor cores, for up to 16 rows of bfloat16 x:
//     y[M,N] = x[M,K] W[N,K]^T (+ residual),  32-bit sums, y float.
// A decode step reads every weight once and does little arithmetic per byte, so the only
// goal is to keep HBM busy: each block owns 16 rows of W, its 8 or 16 warps split K between
// them, every thread pulls its part of W straight from global memory into registers with
// 16-byte loads that bypass L1 (W is used once; x stays cached), and feeds
// mma.m16n8k16 with W as the 16-row operand and 8 rows of x as the 8-column operand
// (y^T = W x^T).  A 16-byte load gives a thread eight consecutive k of one row; the
// instruction wants pairs (2t, 2t+1) and (2t+8, 2t+9).  The sum over k does not care about
// the order, so both operands use the same renumbering of k inside each block of 32 and
// no shuffle is needed.  The warps' partial sums meet in shared memory and are added in
// warp order; how K is split depends on N and K only, so a row's result depends neither on the
// batch nor on timing.
// With the SwiGLU epilogue W holds, for every 8 features, their 8 gate rows and then their 8 up
// rows: a block's 16 rows are the gates and ups of 8 features, one thread's accumulators hold a
// feature's gate (row g) and up (row g + 8), and the block writes a = silu(gate) * up as bfloat16.
// (The reference's counterpart for few rows: ggml-cuda/mmvf.cu and mmf.cuh.)
#include "common.cuh"

#define GS_ROWS 16

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = number of 8-row tiles of x handled at once (M <= 8 * NT).
template <int NT, int U, int GS_WARPS, bool SWIGLU>
__global__ void __launch_bounds__(GS_WARPS * 32)
gemm_stream_kernel(const bf16* x, const bf16* __restrict__ W, const float* residual, float* y,
                   bf16* __restrict__ act, int M, int N, int K) {
    __shared__ float part[GS_WARPS][NT][4][32];          // [warp][tile][c register][lane]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GS_ROWS;
    const int chunks = K >> 3;                            // 16-byte chunks per row
    const int blocks = (chunks + 3) >> 2;                 // blocks of 32 k
    const int per_warp = (blocks + GS_WARPS - 1) / GS_WARPS;
    const int kb0 = warp * per_warp, kb1 = min(blocks, kb0 + per_warp);

    const int r_lo = n0 + g, r_hi = n0 + g + 8;
    const uint4* w_lo = reinterpret_cast<const uint4*>(W + (size_t)min(r_lo, N - 1) * K);
    const uint4* w_hi = reinterpret_cast<const uint4*>(W + (size_t)min(r_hi, N - 1) * K);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // The weights do not depend on the kernel before this one: their first loads go out before the wait.
    uint4 lo[U], hi[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = (kb0 + u) * 4 + t;
        const bool in = kb0 + u < kb1 && c < chunks;
        lo[u] = in ? ld_stream16(w_lo + c) : zero;
        hi[u] = in ? ld_stream16(w_hi + c) : zero;
    }
    pdl_wait();
    pdl_launch_dependents();

    const uint4* xr[NT];
    bool x_ok[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int m = 8 * j + g;
        x_ok[j] = m < M;
        xr[j] = reinterpret_cast<const uint4*>(x + (size_t)min(m, M - 1) * K);
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    for (int kb = kb0; kb < kb1; kb += U) {
        uint4 nlo[U], nhi[U];                             // the next U blocks, in flight while these are used
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = (kb + U + u) * 4 + t;
            const bool in = kb + U + u < kb1 && c < chunks;
            nlo[u] = in ? ld_stream16(w_lo + c) : zero;
            nhi[u] = in ? ld_stream16(w_hi + c) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = (kb + u) * 4 + t;
            const bool in = kb + u < kb1 && c < chunks;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 xv = (in && x_ok[j]) ? __ldcg(xr[j] + c) : zero;
                mma_bf16_16816(acc[j], lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
                mma_bf16_16816(acc[j], lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) { lo[u] = nlo[u]; hi[u] = nhi[u]; }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) part[warp][j][r][lane] = acc[j][r];
    __syncthreads();

    // c0: (row g, col 2t), c1: (row g, col 2t+1), c2: (row g+8, col 2t), c3: (row g+8, col 2t+1);
    // rows are rows of W (outputs n), columns are rows of x (m).
    __shared__ float sums[SWIGLU ? NT : 1][4][32];       // SwiGLU: the block's sums, before gate meets up
    for (int idx = threadIdx.x; idx < NT * 4 * 32; idx += blockDim.x) {
        const int j = idx >> 7, r = (idx >> 5) & 3, ln = idx & 31;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < GS_WARPS; ++w) s += part[w][j][r][ln];
        if (SWIGLU) {
            sums[j][r][ln] = s;
        } else {
            const int gg = ln >> 2, tt = ln & 3;
            const int n = n0 + gg + ((r & 2) ? 8 : 0);
            const int m = 8 * j + 2 * tt + (r & 1);
            if (n < N && m < M) {
                const size_t at = (size_t)m * N + n;
                y[at] = residual ? residual[at] + s : s;
            }
        }
    }
    if (SWIGLU) {                                         // rows g are gates, rows g + 8 the ups of the same features
        __syncthreads();
        const int F = N >> 1, f0 = n0 >> 1;               // features in all; the block's first feature
        for (int idx = threadIdx.x; idx < NT * 2 * 32; idx += blockDim.x) {
            const int j = idx >> 6, r = (idx >> 5) & 1, ln = idx & 31;
            const float gate = sums[j][r][ln], up = sums[j][r + 2][ln];
            const int f = f0 + (ln >> 2), m = 8 * j + 2 * (ln & 3) + r;
            if (f < F && m < M) act[(size_t)m * F + f] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
    }
}

// u, w: blocks of 32 k that a warp keeps in flight, and warps per block of threads; 0, 0: chosen here.
template <bool SWIGLU>
static int launch_stream(const bf16* xp, const bf16* wp, const float* residual, float* y, bf16* act, int M, int N, int K,
                         int u, int w, cudaStream_t stream) {
    const int grid = (N + GS_ROWS - 1) / GS_ROWS;
    // How deep each warp prefetches (U blocks of 32 k) and how many warps split K, by what measured best at the sizes of
    // a Qwen3-8B decode step: long rows want deep prefetch; short rows with few blocks want more warps; else shallow.
    // (Other shapes have other optima, and for some the library wins: a caller that measures passes its choice.)
    if (u == 0 && w == 0) {
        if (K >= 8192) { u = 8; w = 8; }
        else if (N <= 4096) { u = 2; w = 16; }
        else { u = 2; w = 8; }
    }
#define GS_GO(NT, U, WARPS) qwb_launch_early(gemm_stream_kernel<NT, U, WARPS, SWIGLU>, grid, WARPS * 32, 0, stream, xp, wp, residual, y, act, M, N, K)
#define GS_PICK(NT)                                                  \
    do {                                                             \
        if (u == 2 && w == 8) GS_GO(NT, 2, 8);                       \
        else if (u == 4 && w == 8) GS_GO(NT, 4, 8);                  \
        else if (u == 8 && w == 8) GS_GO(NT, 8, 8);                  \
        else if (u == 2 && w == 16) GS_GO(NT, 2, 16);                \
        else if (u == 4 && w == 16) GS_GO(NT, 4, 16);                \
        else if (u == 2 && w == 32) GS_GO(NT, 2, 32);                \
        else return qwb_fail(QWB_ERR_ARG, "gemm_stream: no kernel with %d blocks in flight and %d warps", u, w);  \
    } while (0)
    if (M <= 8) GS_PICK(1);
    else GS_PICK(2);
#undef GS_PICK
#undef GS_GO
    return qwb_check_launch("gemm_stream");
}

static int check_stream(const void* x, const void* W, int M, int K) {
    if (K <= 0 || K % 8) return qwb_fail(QWB_ERR_ARG, "gemm_stream: inner size %d is not a multiple of 8", K);
    if (M > 16) return qwb_fail(QWB_ERR_ARG, "gemm_stream: %d rows; this kernel is for at most 16", M);
    if ((uintptr_t)x % 16 || (uintptr_t)W % 16) return qwb_fail(QWB_ERR_ARG, "gemm_stream: operands must be 16-byte aligned");
    return 0;
}

extern "C" int qwb_gemm_stream(const void* x, const void* W, const float* residual, float* y, int M, int N, int K,
                               int u, int w, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (int rc = check_stream(x, W, M, K)) return rc;
    return launch_stream<false>((const bf16*)x, (const bf16*)W, residual, y, nullptr, M, N, K, u, w, stream);
}

// W [2 F, K]: for every 8 features their 8 gate rows, then their 8 up rows (F a multiple of 8).
// act bfloat16 [M, F] = silu(x gate^T) * (x up^T).
extern "C" int qwb_gemm_stream_swiglu(const void* x, const void* W, void* act, int M, int F, int K, int u, int w,
                                      cudaStream_t stream) {
    if (M <= 0 || F <= 0) return 0;
    if (F % 8) return qwb_fail(QWB_ERR_ARG, "gemm_stream: %d features are not a multiple of 8", F);
    if (int rc = check_stream(x, W, M, K)) return rc;
    return launch_stream<true>((const bf16*)x, (const bf16*)W, nullptr, nullptr, (bf16*)act, M, 2 * F, K, u, w, stream);
}
