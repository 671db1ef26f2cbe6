// qwb_attn_decode_noalloc: decode attention for callers that must not allocate.
//
// This entry point has no counterpart in kishida/questwend; it is an addition of this library.
//
// Who needs it.  qwb_attn_decode cuts each sequence's keys into runs and merges the runs'
// partial results, so it needs scratch memory, and its caller has to get that memory from
// somewhere.  Some callers cannot: code that runs between two steps of a latency-critical
// loop, where cudaMalloc would stall the whole device while it takes the allocator's locks;
// a host program that has handed all device memory to its own pool and has no pointer to
// spare; a plugin loaded into a process whose allocator it may not call.  For them the
// scratch lives inside this library, in a fixed array in device memory that is part of the
// loaded module.
//
// What it costs.  The array is QWB_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on
// which this library is loaded holds it from the first use of the library until the process
// exits, whether this entry point is ever called or not.
//
// Limits.  B * Hq * max_runs * (hd + 2) must not exceed QWB_NOALLOC_SCRATCH_FLOATS; a larger
// problem is refused with an error message (qwb_last_error), nothing is launched.  With 32
// heads of 128 a run takes 32 * 130 = 4,160 floats, so B * max_runs can be 1,008 at most: at
// the default run length of 256 keys that is 8 sequences of up to 126 runs = 32,256 keys, or
// 31 sequences of up to 32 runs = 8,192 keys (8 x 32,768 and 32 x 8,192 are just too many).
// max_runs must cover the longest sequence, max_runs >= ceil(longest / split_tokens): the
// lengths are on the device, so the launcher cannot check this; the kernels cut a longer
// sequence at max_runs runs rather than touch memory beyond the scratch.
//
// First call.  The first call on each device looks the array's device address up
// (cudaGetSymbolAddress, with that device current) and keeps it; that lookup is a
// synchronising runtime call, so make the first call on a device before any stream capture
// begins on it.  Later calls only launch kernels.  The function calls no cudaMalloc, no
// cudaFree and no library routine that allocates.  The kept address is not guarded by a
// lock: make a device's first call from one host thread, and let other threads call once it
// has returned.  The device that is current when the function is called decides which
// array is used, so `stream` must be a stream of the current device.
//
// Sharing.  All calls on a device use the same array.  Nothing in it has to start at zero
// (every value that is read was written earlier in the same call), so stale contents of an
// earlier call do no harm; but two calls that overlap on the GPU (different streams, or
// graphs replayed side by side) write the same memory and race.  Run them one after the
// other, or use qwb_attn_decode with scratch of your own.
//
// Arguments and result: those of qwb_attn_decode without `scratch`.
#pragma once

#include <cuda_runtime.h>

#define QWB_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int qwb_attn_decode_noalloc(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                            const int* seq_len, void* out, int dtype, int B, int Hq, int Hkv, int hd, int page_size,
                            int table_width, float scale, int window, int split_tokens, int max_runs,
                            cudaStream_t stream);

// The capacity of the built-in scratch, in floats.
long long qwb_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
