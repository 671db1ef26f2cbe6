// Shared helpers of the hand-written sm_100a kernels.  Every .cu file of this folder is
// one translation unit that becomes one shared library with a C ABI: launchers take raw
// device pointers and a stream, return 0 or an error code, and leave a message that
// qwb_last_error() returns.  Nothing here allocates device memory; callers pass buffers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstring>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define QWB_DT_F32 0
#define QWB_DT_BF16 1

#define QWB_ERR_ARG 1     // a size or option the kernel does not take
#define QWB_ERR_CUDA 2    // the launch itself failed

static thread_local char qwb_err_buf[512] = "";

static int qwb_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(qwb_err_buf, sizeof(qwb_err_buf), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char* qwb_last_error() { return qwb_err_buf; }

static int qwb_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return qwb_fail(QWB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return 0;
}

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  Every kernel of this library begins with pdl_wait() and can be
// launched with the programmatic-serialization attribute: the kernel may then be scheduled while
// its predecessor in the stream is still draining, and waits at pdl_wait() until the predecessor
// has finished and its writes are visible.  What a kernel does before pdl_wait() must not depend
// on the predecessor (weights may be prefetched, nothing may be written).  pdl_launch_dependents()
// lets the successor be scheduled early in the same way.  Without the attribute both instructions
// do nothing.  Giving the attribute to every kernel made a Qwen3-8B-sized decode step (batch 8)
// slower, 4.77 ms against 4.49 ms: the early blocks of the next kernel take room on the SMs from the
// running one.  So only kernels that gain from an early start get it (qwb_launch_early).  (The
// reference's CUDA back end has the same hooks, ggml-cuda/common.cuh:123-129.)
// A kernel that is launched early reads what its predecessor wrote with loads that are coherent at
// L2 (__ldcg, or plain loads through a pointer that is not __restrict__), never through the read-only
// path (__ldg, ld.global.nc): a block that was resident while the predecessor wrote has been seen to
// get the buffer's earlier contents from there after the wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// QWB200_PDL: unset or "some" = only the kernels that ask for it (qwb_launch_early: the weight-streaming
// product, whose first loads do not depend on the kernel before it); "all" = every kernel; "0" = none;
// a comma-separated list of kernel modules ("elementwise,rope_kv") = those too, for experiments.
#ifndef QWB_MODULE_NAME
#define QWB_MODULE_NAME ""
#endif
static int qwb_pdl_mode() {        // 0 none, 1 those that ask, 2 every kernel of this module
    static int mode = -1;
    if (mode < 0) {
        const char* e = getenv("QWB200_PDL");
        if (!e || !e[0] || !strcmp(e, "some")) mode = 1;
        else if (!strcmp(e, "all")) mode = 2;
        else if (!strcmp(e, "0") || !strcmp(e, "none")) mode = 0;
        else {
            mode = 1;
            const size_t n = strlen(QWB_MODULE_NAME);
            for (const char* p = e; n && (p = strstr(p, QWB_MODULE_NAME)); p += n)
                if ((p == e || p[-1] == ',') && (p[n] == 0 || p[n] == ',')) { mode = 2; break; }
        }
    }
    return mode;
}

template <typename... KArgs, typename... Args>
static cudaError_t qwb_launch_attr(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = early ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static cudaError_t qwb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return qwb_launch_attr(qwb_pdl_mode() == 2, kernel, grid, block, smem, stream, args...);
}

// For a kernel that has useful work before pdl_wait(): it may start while the kernel before it still runs.
template <typename... KArgs, typename... Args>
static cudaError_t qwb_launch_early(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return qwb_launch_attr(qwb_pdl_mode() >= 1, kernel, grid, block, smem, stream, args...);
}

// For the small kernels between two early-launched ones (a norm, the merge of attention's runs): launched early as well,
// with their trigger before their wait, they let the kernel after them start (and fill its ring) while the kernel before
// them still runs.  Measured on decode steps.  The norms: 4 % faster with one row, 1-2 % with 2 to 8 rows at the Qwen3-8B
// sizes, 0.7 % at 8 rows of the 32B sizes, nothing at 16: in steps of up to 16 rows.  The merge: nothing on its own at 8
// rows (attention's blocks and a ring do not fit into one SM's shared memory together), and with the norms 0.5 % slower
// there (5 % at the 32B sizes): in steps of up to 4 rows.  QWB200_CHAIN=<rows> sets another bound for both,
// QWB200_CHAIN_<module>=<rows> for one module's kernels, for experiments.
#define QWB_LINK_ROWS_NORM 16
#define QWB_LINK_ROWS_MERGE 4
static int qwb_link_max_rows(int by_default) {
    static int rows = -2;
    if (rows == -2) {
        char name[96];
        snprintf(name, sizeof(name), "QWB200_CHAIN_%s", QWB_MODULE_NAME);
        const char* e = getenv(name);
        if (!e || !e[0]) e = getenv("QWB200_CHAIN");
        rows = (e && e[0]) ? atoi(e) : -1;
    }
    return rows >= 0 ? rows : by_default;
}
template <typename... KArgs, typename... Args>
static cudaError_t qwb_launch_link(int rows, int max_rows, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return qwb_launch_attr(qwb_pdl_mode() == 2 || (qwb_pdl_mode() == 1 && rows <= qwb_link_max_rows(max_rows)), kernel, grid, block, smem, stream, args...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// 16-byte vectors of T: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 v;
    __device__ __forceinline__ void get(float* out) const { out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w; }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    uint4 v;
    __device__ __forceinline__ void get(float* out) const {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block in a fixed order (the same for every launch): warps first, then the
// warps' partial sums in index order.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += scratch[w];
    return total;
}
