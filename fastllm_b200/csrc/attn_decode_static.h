// Paged decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library that cannot call
// cudaMalloc themselves: code running after a server has switched device allocation off for steady state,
// plug-ins that are handed tensors by another runtime and own no allocator, and callers inside a region where
// an allocation could synchronise the device or fragment a pool they do not control.
//
// fb_attn_decode_static does the same work as fb_attn_decode_plan + fb_attn_decode (same kernels) but takes
// NO scratch pointers: the work list, the per-page partial outputs and their
// (max, sum) pairs live in one file-scope device array inside the library.  The caller passes only the
// inputs (q, page pools, page table, sequence lengths) and the output.
//
// Limits (rejected with FB_STATIC_TOO_LARGE, nothing is launched):
//     B * max_pages                      <= FB_STATIC_MAX_ITEMS  (16384 work items)
//     B * Hkv * max_pages * (Hq / Hkv)   <= FB_STATIC_MAX_SLOTS  (16384 partial slots)
// The array is about 8.7 MB and every GPU that loads the library holds it until the process exits.
//
// First call on a device: resolves the array's device address (cudaGetSymbolAddress, with that device
// current) and sets kernel attributes.  Make that first call outside any stream capture.
//
// All calls on a device share the one array and it keeps the previous call's contents; nothing in it has to
// start at zero (every word is written before it is read within a call).  Two calls that overlap on the GPU
// (different streams, no dependency between them) race on it: serialise them.
//
// Preconditions on the caller's buffers (the regular entry point is more forgiving on the second):
//   * seq_lens[b] <= max_pages * 128 for every request.  A longer length is reported through the library's
//     error word (bad argument) and only the first max_pages pages are merged; the output row is then wrong.
//   * every page a request's table names holds FINITE values in all 128 rows, including the rows past the
//     request's length in its last page.  This entry loads whole pages; rows past the length get probability
//     zero, but 0 x NaN or 0 x Inf from a never-written tail would still poison the output row.  Pools that
//     come from a zero-filled allocation satisfy this; a pool of uninitialised memory does not.
//
// Calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define FB_STATIC_MAX_ITEMS 16384
#define FB_STATIC_MAX_SLOTS 16384
#define FB_STATIC_TOO_LARGE (-3)

// q, out: [B, Hq*128] 16-bit (dtype: 0 = fp16, 1 = bf16), row strides Hq*128 / ld_out elements.
// k_pool, v_pool: [num_slots, Hkv, 128]; page_table: int32 [B, max_pages] (row stride max_pages);
// seq_lens: int32 [B].  Returns 0, a cudaError_t, -1 (unsupported shape), -2 (tensor map), or FB_STATIC_TOO_LARGE.
int fb_attn_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out, int ld_out,
                          const int* page_table, const int* seq_lens, int B, int Hq, int Hkv, int D,
                          long long num_slots, int max_pages, float scale, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
