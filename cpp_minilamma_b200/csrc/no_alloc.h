// Split decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference engine, whose every operation
// allocates its output and scratch with cudaMalloc (src/cuda_tensor.cc:85-95,
// src/cuda_attention.cu:246-249).
//
// Who needs it: a host program that hands the whole GPU to its own memory pool when it
// starts (an inference server, a game engine, a plugin host) leaves nothing for a library
// to cudaMalloc later, and a latency-bound loop cannot afford cudaMalloc anyway because it
// synchronises the device.  Such callers can pass inputs and outputs that they own, but the
// split decode kernel also needs room for the partial results of its context splits.
// Here that room is a fixed array inside the library itself.
//
// Limits and rules
//   * The scratch array holds MLL_NO_ALLOC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that
//     loads the library carries it until the process exits.  A call that needs more than
//     n_seqs * n_heads * n_splits * (head_dim + 2) <= MLL_NO_ALLOC_SCRATCH_FLOATS floats is
//     refused with an error message; nothing is launched.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress).  Make that first call outside any stream capture.
//   * All calls share the one array.  Nothing in it has to be cleared between calls - each
//     call writes every partial slot before its merge step reads it - but two calls whose
//     kernels overlap on the GPU (different streams, or graphs replayed concurrently) would
//     write the same slots and race.  Keep calls on one stream or order them with events.
//   * No cudaMalloc, cudaFree or allocating library routine is called, and nothing is
//     synchronised.
//
// Arguments are those of mll_attn_decode without the scratch pointer: q [n_seqs, n_heads *
// head_dim], the paged caches [pages, n_kv_heads, 64, head_dim], int32 seq_slot / seq_ctx
// [n_seqs], int32 block_table [slots, max_blocks], out [n_seqs, n_heads * head_dim];
// dtype 0 = float32, 1 = bfloat16.  Returns 0 on success; on refusal a negative code with
// the reason in mll_last_error().
#pragma once

#include <cuda_runtime.h>

#define MLL_NO_ALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int mll_attn_decode_no_alloc(
    const void* q, const void* k_cache, const void* v_cache, const int* seq_slot, const int* seq_ctx,
    const int* block_table, void* out, int dtype, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
    int max_blocks, int n_splits, int window, float scale, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
