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
};

template <typename T>
__global__ void rope_cache_kernel(RopeArgs a) {
  const int t = blockIdx.x;
  const int d = a.head_dim, half = d >> 1;
  const int pos = a.tok_pos[t];
  const T* row = (const T*)a.qkv + (size_t)t * a.ld;
  // no table: positions are not encoded and q, k pass through unrotated
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half : nullptr;

  // where this token's k and v rows live
  const int slot = a.seq_slot[a.tok_seq[t]];
  const int page = a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE];
  const int in_page = pos % MLL_PAGE;

  const int q_pairs = a.n_heads * half;
  const int k_pairs = a.write_kv ? a.n_kv_heads * half : 0;
  const int v_pairs = k_pairs;
  const int q_cols = a.n_heads * d, kv_cols = a.n_kv_heads * d;
  T* q_out = (T*)a.q_out + (size_t)t * q_cols;

  for (int w = threadIdx.x; w < q_pairs + k_pairs + v_pairs; w += blockDim.x) {
    if (w < q_pairs + k_pairs) {
      const bool is_q = w < q_pairs;
      const int p = is_q ? w : w - q_pairs;
      const int head = p / half, i = p % half;
      const int e0 = a.interleaved ? 2 * i : i;
      const int e1 = a.interleaved ? 2 * i + 1 : i + half;
      const int col = (is_q ? 0 : q_cols) + head * d;
      float x0 = to_float(row[col + e0]), x1 = to_float(row[col + e1]);
      if (a.bias) {
        x0 += a.bias[col + e0];
        x1 += a.bias[col + e1];
      }
      const float c = cs ? cs[i] : 1.f, s = cs ? sn[i] : 0.f;
      const float y0 = x0 * c - x1 * s, y1 = x0 * s + x1 * c;
      T* dst = is_q ? q_out + head * d
                    : (T*)a.k_cache + (((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * d;
      dst[e0] = from_float<T>(y0);
      dst[e1] = from_float<T>(y1);
    } else {
      const int p = w - q_pairs - k_pairs;
      const int head = p / half, i = p % half;
      const int col = q_cols + kv_cols + head * d;
      float x0 = to_float(row[col + 2 * i]), x1 = to_float(row[col + 2 * i + 1]);
      if (a.bias) {
        x0 += a.bias[col + 2 * i];
        x1 += a.bias[col + 2 * i + 1];
      }
      T* dst = (T*)a.v_cache + (((size_t)page * a.n_kv_heads + head) * MLL_PAGE + in_page) * d;
      dst[2 * i] = from_float<T>(x0);
      dst[2 * i + 1] = from_float<T>(x1);
    }
  }
}

}  // namespace mll

MLL_API int mll_rope_cache(const void* qkv, const float* bias, const float* cos_table,
                           const float* sin_table, const int* tok_pos, const int* tok_seq,
                           const int* seq_slot, const int* block_table, void* q_out, void* k_cache,
                           void* v_cache, int dtype, int n_tokens, int ld, int n_heads, int n_kv_heads,
                           int head_dim, int max_blocks, int interleaved, int write_kv,
                           cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_heads > 0 && n_kv_heads >= 0, "rope: bad sizes");
  MLL_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope: head_dim %d must be even", head_dim);
  MLL_REQUIRE(ld >= (n_heads + (write_kv ? 2 * n_kv_heads : 0)) * head_dim,
              "rope: row stride %d shorter than the q/k/v columns", ld);
  if (n_tokens == 0) return 0;
  mll::RopeArgs a{qkv, bias, cos_table, sin_table, tok_pos, tok_seq, seq_slot, block_table, q_out,
                  k_cache, v_cache, ld, n_heads, n_kv_heads, head_dim, max_blocks, interleaved, write_kv};
  const int work = (n_heads + 2 * n_kv_heads) * head_dim / 2;
  const int threads = work >= 2048 ? 256 : 128;
  if (dtype == MLL_F32)
    mll::rope_cache_kernel<float><<<n_tokens, threads, 0, stream>>>(a);
  else if (dtype == MLL_BF16)
    mll::rope_cache_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(a);
  else
    MLL_REQUIRE(false, "rope: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
