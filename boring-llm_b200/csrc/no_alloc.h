// An entry point for callers that cannot allocate device memory. It has no counterpart in the reference, whose
// single-sequence kernels take buffers that its own runtime grows and frees (src/model.br:1673-1681).
//
// Who needs it: code that runs where cudaMalloc is off limits. A plugin inside a host application that owns the
// device's memory budget, a real-time loop that may not take the allocator's lock, a process under a memory
// sandbox that only lets the loader map the library's image, or a thin C caller without PyTorch's caching
// allocator behind it. Such callers can still bring their inputs and outputs (those live in memory someone gave
// them); what they cannot supply is the working memory that the sliced decode attention needs for its partial
// results. Here that memory is a fixed array inside the library.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats (8 MiB). A call needs n * H * n_splits * (dh + 2) floats when
// n_splits > 1 and none for a single slice; e.g. 64 requests x 14 heads x 16 slices x head size 64 = 946,176.
#define BL_NO_ALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
// Counters for merging the slices, one per (request, group of up to 16 query heads that share a key/value head).
#define BL_NO_ALLOC_COUNTERS 16384

// Same computation, arguments and result as bl_attention_decode (tensor-core attention for requests with one new
// token each, their keys cut into n_splits slices that a second kernel merges), but without the scratch argument:
// partial results go to an array that is part of the library on each GPU. Calls no cudaMalloc, cudaFree or any
// allocating routine.
//
// - A call whose sizes need more than BL_NO_ALLOC_SCRATCH_FLOATS floats is refused (returns non-zero, the message
//   from bl_last_error() names the sizes); nothing is launched.
// - Every call asks the runtime for the array's device address (cudaGetSymbolAddress, for the device that is
//   current at the call): nothing is cached between calls, so calls from several host threads do not race on
//   any host-side state of this entry point, and an address from before a cudaDeviceReset is never reused. The
//   first look-up on a device may make the runtime load the library's image there; make that first call before
//   any stream capture begins on that device.
// - All calls on a device share the one array, and it keeps whatever the previous call left there. The partial
//   results need no clearing: every slot that the merge reads is written by the same call first. The counters
//   that tell the last-finishing block of a (request, head group) to merge must be zero when a call starts: they
//   are zero when the library is loaded, and each call puts them back to zero itself. Two calls that overlap on
//   the GPU (different streams, no ordering between them) race on both: order them.
int bl_attention_decode_no_alloc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                 const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                                 int n_splits, void* out, int H, int KV, int dh, int page_size, int window,
                                 float scale, void* stream);

#ifdef __cplusplus
}
#endif
