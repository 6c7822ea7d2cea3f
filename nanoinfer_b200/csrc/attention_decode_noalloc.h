// ni_attention_decode_noalloc: split-K decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference engine.
//
// Who it is for.  Some programs that want to call this library's decode attention are not in a
// position to hand it scratch memory: a host application that gave its whole device-memory
// budget to its own cache pool at start-up and forbids allocations afterwards; a plug-in that
// runs under someone else's allocator and has no handle to it; a latency-critical decode loop
// that cannot afford cudaMalloc, which synchronises the whole device.  The regular entry point
// (ni_attention_decode) needs two scratch buffers from its caller: the per-split partial
// results and the arrival tickets.  This variant runs the same kernel with both buffers in
// arrays that are part of the library image itself (file-scope __device__ arrays, 256-byte
// aligned), so it calls no cudaMalloc, no cudaFree and no allocating library routine.  The
// caller still passes every input and the output.
//
// Limits.  The arrays have a fixed, modest size, and every GPU that loads the library holds
// them until the process exits:
//     partial results: NI_NOALLOC_MAX_PARTIAL_FLOATS floats (4 MiB)
//     tickets:         NI_NOALLOC_MAX_TICKETS ints          (16 KiB)
// A call needs n_items * n_q_heads * n_splits * (head_dim + 2) floats and
// n_items * n_kv_heads tickets.  A call that needs more is refused with
// NI_ERR_STATIC_SCRATCH_TOO_SMALL (-4) and launches nothing.
//
// Set-up.  The first call on each device looks up the device addresses of the arrays (with that
// device current) and keeps them; that first call should therefore be made before any stream
// capture begins.  In host code the arrays' names are only stand-ins, never addresses a kernel
// could use, which is why the look-up exists.
//
// Sharing.  All calls share the arrays, and the arrays keep what the last call left in them.
// Each call clears the tickets it is about to use (stream-ordered) before it launches; the
// partial results need no clearing, every slot is written before it is read.  Two calls that
// overlap on the GPU (different streams, or different host threads) race on the arrays and give
// wrong results: serialise them on one stream.
//
// Arguments are those of ni_attention_decode without `scratch` and `tickets`; the return value is
// 0, a negative NI_ERR_* code, or a positive cudaError_t.
#pragma once
#include <cuda_runtime.h>

#define NI_NOALLOC_MAX_PARTIAL_FLOATS (1 << 20)
#define NI_NOALLOC_MAX_TICKETS 4096
#define NI_ERR_STATIC_SCRATCH_TOO_SMALL (-4)

#ifdef __cplusplus
extern "C" {
#endif

int ni_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                const int* token_list, int n_items, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride,
                                int n_q_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                float scale, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
