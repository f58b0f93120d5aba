// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: its decode attention takes its scratch
// from buffers the engine allocated at start-up (src/gpu/dense.rs:116).  It exists for hosts
// that load this library into a process whose memory is already laid out and fixed: a runtime
// that has handed all device memory to its own pool, a plug-in called from inside another
// framework's captured region or real-time loop, or a harness that forbids cudaMalloc after
// start-up.  Such a caller can pass its inputs and outputs but has nowhere to get the float
// scratch that the split key range needs, and must not trigger an allocation to get it.
//
// The scratch therefore lives inside the library, in one array of LEB_NO_ALLOC_SCRATCH_FLOATS
// floats (4 MiB) in device memory.  Every GPU that loads the library holds that array until the
// process exits, whether or not this entry point is ever called.
//
// leb_attention_decode_static does what leb_attention_decode followed by leb_attention_merge do
// (one new row per sequence against the paged cache, bfloat16), with the same arguments except
// that it takes no scratch pointer.  It calls no cudaMalloc, cudaFree or any allocating routine.
//
//  * Every sequence brings one row: seq_qstart must be a permutation of 0..B-1 (the row of q and
//    out that sequence b uses).  A sequence whose seq_qstart is B or more is skipped, so the array
//    is never written past its end; a row that no sequence names keeps whatever the merge finds
//    in the array.
//  * Limit: rows * heads * n_splits * (head_dim + 2) must not exceed
//    LEB_NO_ALLOC_SCRATCH_FLOATS; beyond that the call fails with a message (leb_last_error)
//    and launches nothing.  With n_splits == 1 no scratch is used and there is no limit.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current).  Make that first call outside any stream
//    capture.
//  * All calls share the one array and it keeps what the last call left.  Nothing needs
//    clearing: every element the merge reads is written by the first stage of the same call.
//    Two calls that overlap on the GPU (different streams, no ordering between them) race on
//    the array; order them.
#pragma once
#include <cuda_runtime.h>

#define LEB_NO_ALLOC_SCRATCH_FLOATS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int leb_attention_decode_static(void* out, const void* q, const void* k_pool, const void* v_pool,
                                const int* block_table, int bt_width, const int* seq_slot,
                                const int* seq_pos0, const int* seq_qstart, const void* gate,
                                int gate_stride, int B, int nh, int nkv, int hd, int page_size,
                                int window, float scale, int n_splits, cudaStream_t st);

#ifdef __cplusplus
}
#endif
