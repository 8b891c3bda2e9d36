// lmsf_attention_decode_static: paged decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference (yinqiwen/lmsf); it is an addition of this
// library.
//
// Who it is for.  lmsf_attention_decode splits the keys of a request over several blocks and needs
// scratch memory for their partial results, which its caller has to provide.  Some callers cannot:
// a host program that handed all device memory to a pool of its own at start-up, a service loop
// that may not call cudaMalloc because the call synchronises the whole device, or a binding from
// another language that has this C ABI and no allocator behind it.  For them this variant keeps
// the scratch inside the library, in a static device array of kStaticScratchBytes (8 MiB) that
// every GPU holds from the moment it loads the library until the process ends.
//
// What it does.  The same kernels, the same arguments and the same results as
// lmsf_attention_decode, without the `scratch` argument.  It calls no cudaMalloc, cudaFree or other
// allocating routine.
//
// Limits and rules.
//   * 256 KiB of counters + n_seqs_total * n_q_heads * n_splits * (head_dim + 1) * 4 bytes must fit in 8 MiB; a larger
//     request is refused with LMSF_EBADARG and a message (lmsf_attention_mma_last_error()).
//   * The values of seq_ids must be below n_seqs_total; without seq_ids, n_served must not exceed it (the scratch
//     is indexed by the request's row).  The second is checked, the first cannot be on the host.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and sets the kernel's shared-memory limit.  Make that first call
//     outside any stream capture.
//   * All calls share the one array, and it keeps what the last call left in it.  The partial
//     results that a call reads were written by that same call.  The counters at the array's start
//     (one per request and group of heads: how many key splits have delivered) start as zeros, as static
//     storage does, and every call that completes leaves them zero again.  Two calls that overlap
//     on the GPU (different streams, no ordering between them) race on the array and give wrong
//     results; order them.
#pragma once
#include "common.cuh"

LMSF_API int lmsf_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* cache, long long page_stride, int block_size, int n_kv_heads,
                                          const int* block_table, int max_blocks, const int* seq_ids, int n_served,
                                          int n_seqs_total, const int* cu_q, const int* ctx_len, float scale,
                                          int window, int n_q_heads, int head_dim, int n_splits, void* stream);

// The size of the static scratch array in bytes.
LMSF_API long long lmsf_attention_decode_static_capacity();
