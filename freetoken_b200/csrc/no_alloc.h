// Paged attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference; it exists for users of this library whose
// code path cannot call cudaMalloc when a step runs:
//   * a host program that handed the whole device to its own pools at start-up (this engine does so
//     with its cache: memory_ratio of the GPU), where a later cudaMalloc can fail or wait for memory;
//   * a caller with a latency budget, for whom the device-wide synchronisation that cudaMalloc and
//     cudaFree imply in the middle of a step is not acceptable;
//   * a plain C (or ctypes) user of the shared object who has no tensor library to hand the kernel a
//     scratch buffer.
// ftk_paged_attention needs scratch for tiles whose key range is split (per split and query row: the
// running maximum, the running sum and the unnormalised output, all float32).  Here that scratch is a
// file-scope device array of FTK_STATIC_SCRATCH_BYTES inside the library, so the caller passes inputs
// and outputs only.  Every GPU that loads the library holds the array until the process exits.
//
// Rules of use:
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current) and keeps it; make that first call before any stream capture begins.
//   * A work list that needs more scratch than the array holds is refused with an error; nothing is
//     launched.  The need is slots x kv_heads x tile_rows x (head_dim + 2) floats, slots being the sum
//     of the split counts of the split tiles in the work list.
//   * All calls share the one array and it keeps the previous call's contents.  Nothing in it has to
//     start at zero: every entry that the merge step reads was written by a split of the same call.
//     Two calls that overlap on the GPU (different streams, or the same device from two threads) race
//     on it; keep calls on one stream or order them yourself.
//   * It calls no cudaMalloc, cudaFree or other allocating routine, of CUDA or of any tensor library.
#pragma once
#include <stdint.h>

#define FTK_STATIC_SCRATCH_BYTES (16u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as ftk_paged_attention without part_o, part_ml and n_slots.  Returns 0, or a
// non-zero status whose text ftk_last_error() gives.
int ftk_paged_attention_static_scratch(const void* q, const void* k_slab, const void* v_slab, int dtype,
                                       const int32_t* block_table, int bt_stride, const int32_t* seg_info,
                                       int n_segs, const int32_t* items_host_copy, const int32_t* items,
                                       int n_items, void* out, int n_q_heads, int n_kv_heads, int head_dim,
                                       int page_size, int num_pages, int tile_rows, float scale, int window,
                                       void* stream);

#ifdef __cplusplus
}
#endif
