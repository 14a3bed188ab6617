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

// grid (tokens, Hq + 2 Hk): one block per head of one token, one thread per pair, so that
// no thread waits for more than one round of loads.
template <typename T>
__global__ void rope_cache_kernel(RopeArgs a) {
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

// bfloat16 with head_dim a multiple of 16: one thread per 16 elements of a head (8 pairs), moved as
// 16-byte words.  A step of thousands of tokens is bound by memory traffic, which scalar
// 2-byte accesses cannot saturate.  Same arithmetic, element by element, as the kernel above.
__device__ __forceinline__ void unpack8(const uint4& w, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 w;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return w;
}

__global__ void __launch_bounds__(256) rope_cache_vec_kernel(RopeArgs a, long long n_items) {
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= n_items) return;
  const int d = a.head_dim, half = d >> 1;
  const int chunks = d >> 4;                       // 16 elements each
  const int heads = a.n_heads + (a.write_kv ? 2 * a.n_kv_heads : 0);
  const int c = (int)(item % chunks);
  const int hb = (int)((item / chunks) % heads);
  const int t = (int)(item / ((long long)chunks * heads));
  const bool is_q = hb < a.n_heads;
  const bool is_k = !is_q && hb < a.n_heads + a.n_kv_heads;
  const int pos = a.tok_pos[t];
  const __nv_bfloat16* row = (const __nv_bfloat16*)a.qkv + (size_t)t * a.ld + (size_t)hb * d;
  const float* bias = a.bias ? a.bias + (size_t)hb * d : nullptr;
  __nv_bfloat16* dst;
  if (is_q) {
    dst = (__nv_bfloat16*)a.q_out + (size_t)t * a.n_heads * d + (size_t)hb * d;
  } else {
    const int slot = a.seq_slot[a.tok_seq[t]];
    const int page = a.block_table[(size_t)slot * a.max_blocks + pos / MLL_PAGE];
    const int head = is_k ? hb - a.n_heads : hb - a.n_heads - a.n_kv_heads;
    __nv_bfloat16* base = (__nv_bfloat16*)(is_k ? a.k_cache : a.v_cache);
    dst = base + (((size_t)page * a.n_kv_heads + head) * MLL_PAGE + pos % MLL_PAGE) * d;
  }
  const bool rotate = (is_q || is_k) && a.cos_table != nullptr;
  const bool split = rotate && !a.interleaved;
  // the two 8-element words of this thread: the halves' matching parts, or 16 neighbours
  const int e0 = split ? 8 * c : 16 * c;
  const int e1 = split ? half + 8 * c : 16 * c + 8;
  float x0[8], x1[8];
  unpack8(*reinterpret_cast<const uint4*>(row + e0), x0);
  unpack8(*reinterpret_cast<const uint4*>(row + e1), x1);
  if (bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x0[i] += bias[e0 + i];
      x1[i] += bias[e1 + i];
    }
  }
  if (rotate) {
    // pairs 8c .. 8c+7 of the head
    const float4* cs = reinterpret_cast<const float4*>(a.cos_table + (size_t)pos * half + 8 * c);
    const float4* sn = reinterpret_cast<const float4*>(a.sin_table + (size_t)pos * half + 8 * c);
    float cv[8], sv[8];
    *reinterpret_cast<float4*>(cv) = cs[0];
    *reinterpret_cast<float4*>(cv + 4) = cs[1];
    *reinterpret_cast<float4*>(sv) = sn[0];
    *reinterpret_cast<float4*>(sv + 4) = sn[1];
    if (split) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p = x0[i], q = x1[i];
        x0[i] = p * cv[i] - q * sv[i];
        x1[i] = p * sv[i] + q * cv[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float p = x0[2 * i], q = x0[2 * i + 1];
        x0[2 * i] = p * cv[i] - q * sv[i];
        x0[2 * i + 1] = p * sv[i] + q * cv[i];
        p = x1[2 * i], q = x1[2 * i + 1];
        x1[2 * i] = p * cv[4 + i] - q * sv[4 + i];
        x1[2 * i + 1] = p * sv[4 + i] + q * cv[4 + i];
      }
    }
  }
  *reinterpret_cast<uint4*>(dst + e0) = pack8(x0);
  *reinterpret_cast<uint4*>(dst + e1) = pack8(x1);
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
  const int half = head_dim / 2;
  const int threads = half >= 128 ? 128 : (half >= 64 ? 64 : 32);
  MLL_REQUIRE(n_heads + 2 * n_kv_heads <= 65535, "rope: too many heads for one launch");
  const dim3 grid(n_tokens, n_heads + (write_kv ? 2 * n_kv_heads : 0));
  const bool aligned16 = ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache |
                          (uintptr_t)cos_table | (uintptr_t)sin_table) % 16 == 0;
  if (dtype == MLL_BF16 && head_dim % 16 == 0 && ld % 8 == 0 && aligned16) {
    const long long items = (long long)n_tokens * grid.y * (head_dim / 16);
    MLL_REQUIRE((items + 255) / 256 <= 0x7fffffffLL, "rope: too many tokens for one launch");
    MLL_LAUNCH(mll::rope_cache_vec_kernel, (unsigned)((items + 255) / 256), 256, 0, stream, a, items);
  } else if (dtype == MLL_F32)
    MLL_LAUNCH((mll::rope_cache_kernel<float>), grid, threads, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::rope_cache_kernel<__nv_bfloat16>), grid, threads, 0, stream, a);
  else
    MLL_REQUIRE(false, "rope: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
