// An entry point for callers that cannot allocate device memory.
//
// This has no counterpart in cosmonomic/pulsarlm; it is an addition of this library.
//
// Who needs it: code that drives the kernels from a place where cudaMalloc (or
// torch's allocator) may not be called: a plug-in running inside another
// framework's stream callback or memory-pool scope, a host thread that must never
// take the allocator's lock, a process whose device memory was handed out in full
// at start-up. Such a caller can own its inputs and outputs, but the split-key
// decode attention also needs a scratch area for the per-split partial results,
// and pl_attention_decode expects the caller to bring one.
//
// pl_attention_decode_static is pl_attention_decode with that scratch taken from an
// array built into the library: a file-scope `static __device__` array of
// PL_STATIC_SCRATCH_FLOATS floats (16 MiB). Every GPU on which the library is
// loaded holds that array until the process exits.
//
// Rules of use:
//  * The call allocates nothing: no cudaMalloc, cudaFree, or allocating library
//    routine. Inputs and outputs are the caller's.
//  * A call whose partials do not fit (tokens * heads * splits * (head_dim + 2)
//    floats > PL_STATIC_SCRATCH_FLOATS) is refused with an error; nothing is
//    launched. Use fewer splits, or fewer tokens per call.
//  * The first call on each device looks up the array's device address (with that
//    device current) and remembers it. Make that first call outside any stream
//    capture, and from one host thread: the remembered address is written without
//    a lock (two threads racing on the first call would both look it up and store
//    the same value, which is harmless but not guaranteed by the language).
//  * All calls share the one array, and it keeps what the last call left in it.
//    Nothing in it needs to start at zero: every partial a call reads was written
//    by that same call. But two calls that overlap on the GPU (different streams,
//    no ordering between them) race on it; order them, or give all but one of them
//    their own scratch through pl_attention_decode.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#define PL_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

extern "C" {

// Arguments as pl_attention_decode, without the scratch pointer. Returns 0, or a
// non-zero code with the reason in pl_last_error().
int pl_attention_decode_static(const void* q, int64_t q_row_stride, const void* k_pool, const void* v_pool,
                               int64_t page_stride, int64_t head_stride, int page_size, int n_pages,
                               const int32_t* table, int table_width, const int32_t* pos, const int32_t* entry,
                               void* out, int64_t out_row_stride, int n_tokens, int n_heads, int n_kv_heads,
                               int head_dim, int window, float scale, int n_splits, int32_t* status,
                               cudaStream_t stream);

// Floats of scratch the built-in array holds (PL_STATIC_SCRATCH_FLOATS).
int64_t pl_static_scratch_floats();
}
