// Decode attention on tensor cores (bfloat16): the entry points, and the kernels for head sizes that are
// multiples of 32.  The kernel itself is in attention_mma.cuh.
#include "attention_mma.cuh"

namespace mll {

static int launch_decode_mma_any(const DecodeMmaArgs& a, int head_dim, int n_seqs, bool fused, cudaStream_t stream) {
  switch (head_dim) {
    case 32: return launch_decode_mma_sized<32>(a, n_seqs, fused, stream);
    case 64: return launch_decode_mma_sized<64>(a, n_seqs, fused, stream);
    case 96: return launch_decode_mma_sized<96>(a, n_seqs, fused, stream);
    case 128: return launch_decode_mma_sized<128>(a, n_seqs, fused, stream);
    case 160: return launch_decode_mma_sized<160>(a, n_seqs, fused, stream);
    case 192: return launch_decode_mma_sized<192>(a, n_seqs, fused, stream);
    case 224: return launch_decode_mma_sized<224>(a, n_seqs, fused, stream);
    case 256: return launch_decode_mma_sized<256>(a, n_seqs, fused, stream);
    default: return launch_decode_mma_odd(a, head_dim, n_seqs, fused, stream);
  }
}

}  // namespace mll

MLL_API int mll_attn_decode_mma_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && head_dim >= 16 && head_dim <= 256 && head_dim % 16 == 0;
}

// Same contract as mll_attn_decode.  With n_splits > 1 and `counters` (int32, one per
// (sequence, kv head x head chunk), zero before the first launch; the kernel leaves them zero)
// the last block of each group merges the partial results; without counters the caller runs
// mll_attn_combine (scratch layout: partial outputs, then (max, sum) pairs).
MLL_API int mll_attn_decode_mma(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                                const int* seq_ctx, const int* block_table, float* scratch, void* out, int n_seqs,
                                int n_heads, int n_kv_heads, int head_dim, int max_blocks, int n_splits, int window,
                                float scale, int* counters,
                                cudaStream_t stream) {
  MLL_REQUIRE(mll_attn_decode_mma_supported(MLL_BF16, head_dim), "attention decode (mma): head_dim %d", head_dim);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention decode (mma): bad head counts");
  MLL_REQUIRE(n_seqs >= 0 && n_splits >= 1 && n_splits <= 65535, "attention decode (mma): bad batch or split count");
  MLL_REQUIRE(n_splits == 1 || scratch != nullptr, "attention decode (mma): %d splits need scratch memory", n_splits);
  if (n_seqs == 0) return 0;
  mll::DecodeMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                       seq_slot, seq_ctx, block_table, scratch,
                       scratch ? scratch + (size_t)n_seqs * n_heads * n_splits * head_dim : nullptr,
                       (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, n_splits, window, scale,
                       counters,
                       nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0};
  return mll::launch_decode_mma_any(a, head_dim, n_seqs, false, stream);
}

// The decode step's rotary encoding, cache write and attention in one launch: qkv [B, ld] holds
// the projection's output (q heads, then k heads, then v heads; no bias pending), row i
// belongs to sequence i, whose new token has position seq_ctx[i] - 1.  cos/sin: float32
// [max_pos, head_dim / 2] or null; write_kv = 0 for a layer that reads another layer's cache.
// Otherwise the contract of mll_attn_decode_mma.
MLL_API int mll_attn_decode_mma_fused(const void* qkv, int qkv_ld, const float* cos_table, const float* sin_table,
                                      int interleaved, int write_kv, void* k_cache, void* v_cache,
                                      const int* seq_slot, const int* seq_ctx, const int* block_table, float* scratch,
                                      void* out, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_blocks,
                                      int n_splits, int window, float scale, int* counters, cudaStream_t stream) {
  MLL_REQUIRE(mll_attn_decode_mma_supported(MLL_BF16, head_dim), "attention decode (fused): head_dim %d", head_dim);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention decode (fused): bad head counts");
  MLL_REQUIRE(n_seqs >= 0 && n_splits >= 1 && n_splits <= 65535, "attention decode (fused): bad batch or split count");
  MLL_REQUIRE(n_splits == 1 || scratch != nullptr, "attention decode (fused): %d splits need scratch memory", n_splits);
  MLL_REQUIRE(qkv_ld >= (n_heads + (write_kv ? 2 * n_kv_heads : 0)) * head_dim && qkv_ld % 2 == 0,
              "attention decode (fused): row stride %d shorter than the q/k/v columns", qkv_ld);
  MLL_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention decode (fused): one rotary table is missing");
  if (n_seqs == 0) return 0;
  mll::DecodeMmaArgs a{nullptr, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                       seq_slot, seq_ctx, block_table, scratch,
                       scratch ? scratch + (size_t)n_seqs * n_heads * n_splits * head_dim : nullptr,
                       (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, n_splits, window, scale,
                       counters,
                       (const __nv_bfloat16*)qkv, cos_table, sin_table,
                       write_kv ? (__nv_bfloat16*)k_cache : nullptr, write_kv ? (__nv_bfloat16*)v_cache : nullptr,
                       qkv_ld, interleaved};
  return mll::launch_decode_mma_any(a, head_dim, n_seqs, true, stream);
}
