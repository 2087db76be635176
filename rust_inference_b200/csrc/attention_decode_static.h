// ri_attention_decode_static: split-K decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in yudono/rust-inference; it exists for users of this
// library.  The regular entry point, ri_attention_decode, needs scratch memory for the
// partial results of its key splits and expects the caller to bring it.  Some callers cannot:
// code that runs where cudaMalloc is off limits (inside a region another framework's
// allocator or a stream capture owns, a real-time loop that must not touch the allocator,
// a plugin whose host forbids device allocations after start-up).  For them the scratch
// lives inside the library, in a fixed device array, and this function allocates nothing:
// no cudaMalloc, no cudaFree, no allocating library routine.
//
// Limits and rules:
//  * The array holds RI_DECODE_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads
//    the library carries it until the process exits.  A call needs
//    n_seqs * n_heads * n_splits * (head_dim + 2) floats; a larger call is refused with an
//    error message (ri_last_error), nothing is launched.
//  * The first call on a device looks up the array's device address and raises the kernel's
//    shared-memory limit (each once per device, with that device current; several devices in
//    one process each get their own).  Make that first call outside any stream capture.  Host
//    threads may make first calls at the same time: the per-device records are atomic.
//  * All calls share the one array, and it keeps what the last call left in it.  The kernel
//    writes every partial slot it later reads (empty splits included), so nothing has to be
//    cleared between calls.  Two calls that overlap on the GPU (different streams, no
//    ordering) race on the array: order them.
//  * Inputs, outputs and every other argument are exactly those of ri_attention_decode; the
//    caller still owns q, the cache, the page table, the index arrays and `out`.
#pragma once

#include <cuda_runtime.h>

#define RI_DECODE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

extern "C" int ri_attention_decode_static(const void* q, int q_ld, const void* kcache, const void* vcache,
                                          const int* page_table, int max_pages, const int* seq_slot,
                                          const int* seq_len, const int* cu_seqlens, void* out, int out_ld,
                                          int n_seqs, int n_heads, int n_kv_heads, int hd, int page_size,
                                          float scale, int window, int n_splits, cudaStream_t stream);
