// Rotary position encoding of q and k, optional projection bias, and the write of the
// rotated k and of v into the paged cache - one kernel per layer and step.
//
// Replaces RopeKernel / RopeNeoXKernel launched twice (src/cuda_ops.cu:254-299) plus
// two device-to-device copies per token (src/cuda_kvcache.cc:236-237).  The rotation is
//   (a, b) <- (a cos - b sin, a sin + b cos),   angle = position * frequency_i
// with pairs (2i, 2i+1) ("interleaved", the reference's Normal type) or (i, i + d/2)
// (its NeoX type), src/ops.cc:200-221.  cos and sin come from a float32 table that the
// host computes in double, so angles do not drift at large positions as the reference's
// float powf/cosf/sinf do.  The products are float32.
#include "common.cuh"

namespace mll {

struct RopeArgs {
  const void* qkv;          // [T, ld] activations: q heads, then k heads, then v heads
  const float* bias;        // optional [(Hq + 2 Hk) * d]
  const float* cos_table;   // [max_pos, d/2]
  const float* sin_table;
  const int* tok_pos;       // [T]
  const int* tok_seq;       // [T] index into seq_slot
  const int* seq_slot;      // [B]
  const int* block_table;   // [n_slots, max_blocks]
  void* q_out;              // [T, Hq * d]
  void* k_cache;            // [n_pages, Hk, PAGE, d] of this layer
  void* v_cache;
  int ld, n_heads, n_kv_heads, head_dim, max_blocks, interleaved, write_kv;
  Prefetch pf;
};

// grid (tokens, Hq + 2 Hk): one block per head of one token, one thread per pair, so that
// no thread waits for more than one round of loads.
template <typename T>
__global__ void rope_cache_kernel(RopeArgs a) {
  mll::pdl_begin();
  l2_prefetch_by_grid(a.pf);
  const int t = blockIdx.x;
  const int hb = blockIdx.y;  // q heads, then k heads, then v heads
  const int d = a.head_dim, half = d >> 1;
  const bool is_q = hb < a.n_heads;
  const bool is_k = !is_q && hb < a.n_heads + a.n_kv_heads;
  if (!is_q && !a.write_kv) return;
  const int pos = a.tok_pos[t];
  const T* row = (const T*)a.qkv + (size_t)t * a.ld + (size_t)hb * d;
  const float* bias = a.bias ? a.bias + (size_t)hb * d : nullptr;
  T* dst;
  if (is_q) {
    dst = (T*)a.q_out + (size_t)t * a.n_heads * d + (size_t)hb * d;
  } else {
    // where this token's k and v rows live
    const int slot = a.seq_slot[a.tok_seq[t]];
    const int page = a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE];
    const int head = is_k ? hb - a.n_heads : hb - a.n_heads - a.n_kv_heads;
    T* base = (T*)(is_k ? a.k_cache : a.v_cache);
    dst = base + (((size_t)page * a.n_kv_heads + head) * MLL_PAGE + pos % MLL_PAGE) * d;
  }
  const bool rotate = (is_q || is_k) && a.cos_table != nullptr;  // no table: positions are not encoded
  const float* cs = a.cos_table + (size_t)pos * half;
  const float* sn = a.sin_table + (size_t)pos * half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const bool split = (is_q || is_k) && !a.interleaved;
    const int e0 = split ? i : 2 * i;
    const int e1 = split ? i + half : 2 * i + 1;
    float x0 = to_float(row[e0]), x1 = to_float(row[e1]);
    if (bias) {
      x0 += bias[e0];
      x1 += bias[e1];
    }
    float y0 = x0, y1 = x1;
    if (rotate) {
      const float c = cs[i], s = sn[i];
      y0 = x0 * c - x1 * s;
      y1 = x0 * s + x1 * c;
    }
    dst[e0] = from_float<T>(y0);
    dst[e1] = from_float<T>(y1);
  }
}

}  // namespace mll

MLL_API int mll_rope_cache(const void* qkv, const float* bias, const float* cos_table,
                           const float* sin_table, const int* tok_pos, const int* tok_seq,
                           const int* seq_slot, const int* block_table, void* q_out, void* k_cache,
                           void* v_cache, int dtype, int n_tokens, int ld, int n_heads, int n_kv_heads,
                           int head_dim, int max_blocks, int interleaved, int write_kv,
                           const void* prefetch_ptr, long long prefetch_bytes, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0, "rope: bad sizes");
  MLL_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope: head_dim %d must be even", head_dim);
  MLL_REQUIRE(ld >= (n_heads + (write_kv ? 2 * n_kv_heads : 0)) * head_dim,
              "rope: row stride %d shorter than the q/k/v columns", ld);
  if (n_tokens == 0) return 0;
  mll::RopeArgs a{qkv, bias, cos_table, sin_table, tok_pos, tok_seq, seq_slot, block_table, q_out,
                  k_cache, v_cache, ld, n_heads, n_kv_heads, head_dim, max_blocks, interleaved, write_kv,
                  mll::Prefetch{prefetch_ptr, prefetch_ptr ? (unsigned long long)prefetch_bytes : 0ull}};
  const int half = head_dim / 2;
  const int threads = half >= 128 ? 128 : (half >= 64 ? 64 : 32);
  MLL_REQUIRE(n_heads + 2 * n_kv_heads <= 65535, "rope: too many heads for one launch");
  const dim3 grid(n_tokens, n_heads + (write_kv ? 2 * n_kv_heads : 0));
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::rope_cache_kernel<float>), grid, threads, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::rope_cache_kernel<__nv_bfloat16>), grid, threads, 0, stream, a);
  else
    MLL_REQUIRE(false, "rope: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
