// Decode attention for callers that must not allocate.
//
// This entry point has no counterpart in RustingStudio/RustingStrata: there the caller
// always owns every buffer a kernel touches.  It exists for hosts that link this
// library into a process where device memory cannot be requested at the time of the
// call - a plug-in running inside another runtime's memory budget, a real-time loop
// that forbids allocator calls after start-up, a tool that runs under a fixed memory
// map - and that therefore cannot hand the split-KV attention kernel the workspace it
// normally takes as an argument.
//
// rs_attention_decode_noalloc computes exactly what the decode form of
// rs_attention_simt computes (one query token per listed sequence over its paged
// keys and values, cut into splits of `split_keys` keys whose partial results a
// second kernel merges), with the same arguments except that it takes no `partial`
// pointer.  The partial results live in an array that is part of the library image:
// RS_NOALLOC_MAX_FLOATS float32 values (8 MiB), resident on every GPU that loads the
// library for as long as the process lives.
//
// Rules for callers
//  * Limit: total_splits * n_q * (hd + 2) must not exceed RS_NOALLOC_MAX_FLOATS.  A
//    larger request is refused with RS_NOALLOC_TOO_LARGE before anything is launched;
//    rs_attention_decode_noalloc_error() then returns a sentence with both numbers.
//  * split_start lives in device memory, so the function cannot read it: it trusts
//    that split_start[i] + (splits of sequence i) never exceeds total_splits, and
//    checks total_splits against the limit.  Because the array is shared by every
//    caller and cannot be resized, the kernels guard it themselves: a partial result
//    whose slot lies beyond what the array holds for this shape is not written, the
//    sequence's output is left untouched and bit RS_STATUS_BAD_PLAN (16) is set in
//    *status.  Keep split_start[n_work] == total_splits.
//  * The first call on each device looks up the array's device address (one runtime
//    query, no allocation) and remembers it.  Make that first call outside any stream
//    capture, with the device you will launch on made current.
//  * The remembered address belongs to the device's current primary context.  After a
//    cudaDeviceReset the remembered value is stale and this entry point must not be
//    called again in that process (nothing here can notice the reset).
//  * All calls share the one array and it keeps whatever the last call left there.
//    The kernels write every slot they later read, so nothing has to be cleared
//    between calls; but two calls whose kernels can overlap on the GPU (different
//    streams without an ordering between them) would overwrite each other's partial
//    results.  Issue calls on one stream, or order them with events.
//  * The function calls no allocator: no cudaMalloc, cudaFree, cudaMallocAsync, and no
//    library routine that allocates.  Inputs and outputs remain the caller's.
//
// Returns 0 on success, a cudaError_t value for a failed runtime call or launch, or one
// of the negative codes below.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define RS_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)   /* 8 MiB of float32 partial results */
#define RS_NOALLOC_TOO_LARGE (-2)                 /* the request needs more scratch than the array holds */
#define RS_NOALLOC_BAD_ARGUMENT (-3)              /* a size or pointer the kernels cannot take */

int rs_attention_decode_noalloc(const void* q, long q_stride, void* out, long out_stride, int dt, const void* cache,
                                long page_stride, int num_pages, int page_size, const int* block_table,
                                int table_stride, const int* q_start, const int* kv_len, const int* work, int n_work,
                                int n_q, int n_kv, int hd, int window, float scale, int split_keys, int max_splits,
                                const int* split_start, int total_splits, int* status, void* stream);

/* The reason for the last non-zero return of rs_attention_decode_noalloc on this thread ("" if none). */
const char* rs_attention_decode_noalloc_error(void);

/* Capacity of the built-in array in float32 values (RS_NOALLOC_MAX_FLOATS of the loaded build). */
long rs_attention_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
