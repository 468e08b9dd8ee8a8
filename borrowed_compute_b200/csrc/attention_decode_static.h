// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts of this
// library that are not free to call an allocator at the moment they need attention:
//
//   - a program that took the whole GPU into an arena of its own at start-up, so that a
//     later cudaMalloc would simply fail;
//   - code that runs where allocation is forbidden or would stall everything, such as an
//     "enqueue" callback of an inference runtime's plug-in interface, or a latency-critical
//     loop in which the implicit device-wide synchronisation of cudaMalloc / cudaFree is not
//     acceptable;
//   - a binding from a language or process that has no handle on this library's usual
//     allocator (the Python face of this package borrows torch's).
//
// The ordinary entry point, bc_attention_decode_bf16, needs scratch memory from its caller
// when the cached positions are split across blocks.  This variant brings its own: a fixed
// array that lives in the library's device image.  The price is stated here:
//
//   - every GPU that loads the library holds BC_STATIC_SCRATCH_BYTES (about 4 MiB) until the
//     process exits, whether or not this function is ever called;
//   - a launch that would need more is refused with an error (code BC_ERR_LIMIT), never
//     truncated: rows * heads * n_splits * (head_dim + 2) floats may not exceed
//     BC_STATIC_SCRATCH_FLOATS, and rows * kv_heads counters may not exceed
//     BC_STATIC_SCRATCH_COUNTERS;
//   - all calls on one GPU share the one array, and it keeps whatever the last call left.
//     The function clears the counters it is about to use (on the given stream) and the
//     kernel overwrites every partial result before reading it, so calls that follow one
//     another on a stream are safe.  Two calls whose kernels may run at the same time on
//     one GPU (different streams, or different host threads on different streams) race on
//     the array and give wrong results: serialise them.
//
// The first call on each device looks the array's device address up (with that device
// current), and the first call for each head size on each device sets that kernel's
// shared-memory limit; neither allocates, but both are set-up work, so make a first call
// with the head size you will use before any stream capture begins.  After it, a call
// enqueues one memset and one kernel and nothing else.  The function never calls
// cudaMalloc, cudaFree or any routine that allocates, on the host or on the device.
#pragma once

#include <cuda_runtime.h>

#define BC_STATIC_SCRATCH_FLOATS (1 << 20)     // 4 MiB of partial results
#define BC_STATIC_SCRATCH_COUNTERS 4096        // one a (row, kv head)
#define BC_STATIC_SCRATCH_BYTES (BC_STATIC_SCRATCH_FLOATS * 4 + BC_STATIC_SCRATCH_COUNTERS * 4)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as bc_attention_decode_bf16 without the scratch pointers:
// q [rows, q_stride] bf16 with head h of row r at q + r * q_stride + h * head_dim; k_cache,
// v_cache [n_pages, kv_heads, 64, head_dim] bf16; page_table [slots, max_pages] int32;
// row_pos, row_slot [rows] int32 (a negative slot marks a padding row, whose output is
// zero); out [rows, heads * head_dim] bf16.  Returns 0, or an error code whose text
// bc_last_error() gives.
int bc_attention_decode_static_bf16(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* page_table,
                                    const int* row_pos, const int* row_slot, void* out, int rows, int heads, int kv_heads, int head_dim,
                                    int max_pages, int n_pages, int window, float scale, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
