// Shared by the decode attention kernels (attention_mma.cu, attention_decode_tma.cu): their
// arguments, the tensor-core fragment helpers, the rule for the number of context splits and the
// merge of the splits by the block that finishes last.
#pragma once

#include "common.cuh"

namespace mll {

struct DecodeMmaArgs {
  const __nv_bfloat16* q;        // [B, Hq * d]
  const __nv_bfloat16* k_cache;  // [n_pages, Hk, PAGE, d]
  const __nv_bfloat16* v_cache;
  const int* seq_slot;
  const int* seq_ctx;
  const int* block_table;
  float* part_o;                 // [B, Hq, S, d]
  float* part_ml;                // [B, Hq, S, 2]
  __nv_bfloat16* out;            // [B, Hq * d]
  int n_heads, n_kv_heads, max_blocks, n_splits, window;
  float scale;
  int* counters;                 // optional [B, Hk x head chunks], zero between launches: the last split merges
  // fused variant: q, k and v of the step's token come straight from the projection's output;
  // the kernel rotates them and writes the new key and value row into the cache itself
  const __nv_bfloat16* qkv;      // [B, ld]: q heads, k heads, v heads
  const float* cos_table;        // [max_pos, d/2] or null (positions not encoded)
  const float* sin_table;
  __nv_bfloat16* k_write;        // the caches again, writable (null: this layer reads another layer's cache)
  __nv_bfloat16* v_write;
  int qkv_ld, interleaved;
  // optional [B]: the sequences in the order their blocks should start (the TMA kernel; longest contexts first
  // lets the short ones fill the end of the launch)
  const int* seq_order;
  // optional [work_pairs]: the launch as a list of (sequence, split) pairs in the order their blocks should start
  // (the TMA kernel without clusters; the grid's second index runs over it).  Entry: sequence | split << 16 |
  // splits of that sequence << 24, or -1 for an unused place.  A sequence then has the number of splits the
  // entry says (at most n_splits, which stays the stride of the partial results), long sequences more than
  // short ones.
  const int* work;
};

__device__ __forceinline__ float2 unpack_bf162(unsigned r) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r));
}
__device__ __forceinline__ unsigned pack_bf162(float x, float y) {
  __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // fewer source bytes than 16: the rest is written as zero
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// How many context splits a sequence with `pages` pages of keys uses out of the `offered` ones:
// at least one page per split; at most 16 splits until a split has 16 pages (1,024 keys) of its
// own, because the merge grows with the number of splits.  (The host uses the same rule to choose
// how many to offer: parts/attention.py.)
__host__ __device__ inline int decode_splits_for(int pages, int offered) {
  const int by_length = min(pages, max(16, pages / 16));
  return max(1, min(offered, by_length));
}

// Called by every thread of a block after it has written its split's partial result (float32
// output rows, running maximum and sum) for heads h0 .. h0 + ng - 1 of sequence b (item `item` of the
// sequence's `items_per_seq` kv heads x head chunks).  The block that
// arrives last for this (sequence, kv head, head chunk) merges the n_eff splits in use and writes
// the output; the others return.  smem_f: at least 16 * n_eff + 20 floats that the block no longer
// needs, its first word serving as a flag.  NTHREADS threads, all of which must call (it contains
// block-wide barriers).
template <int D, int NTHREADS>
__device__ __forceinline__ void merge_decode_splits(const DecodeMmaArgs& a, int b, int item, int items_per_seq, int h0,
                                                    int ng, int n_eff,
                                                    float* smem_f) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* is_last_word = reinterpret_cast<volatile int*>(smem_f);
  smem_f += 4;
  __threadfence();  // this block's partial results are visible before its arrival is counted
  __syncthreads();
  if (tid == 0) {
    int* counter = a.counters + (size_t)b * items_per_seq + item;
    const int arrived = atomicAdd(counter, 1);
    const int last = arrived == n_eff - 1;
    if (last) *counter = 0;  // ready for the next launch
    *is_last_word = last;
  }
  __syncthreads();
  if (!*is_last_word) return;
  __threadfence();
  // weights of the splits per head, once: w_s = exp(m_s - max m) (zero for an empty split)
  const int S = n_eff, stride = a.n_splits;  // splits in use; slots per head in the partial buffers
  float* w_s = smem_f;  // [ng][S] and [ng] sums, over the (finished) page ring
  float* l_s = w_s + 16 * S;
  for (int row = warp; row < ng; row += NTHREADS / 32) {
    const float* ml = a.part_ml + ((size_t)b * a.n_heads + h0 + row) * stride * 2;
    float m = -INFINITY;
    for (int sp = lane; sp < S; sp += 32) m = fmaxf(m, __ldcg(ml + 2 * sp));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    float l = 0.f;
    for (int sp = lane; sp < S; sp += 32) {
      const float ms = __ldcg(ml + 2 * sp);
      const float w = ms > -INFINITY ? __expf(ms - m) : 0.f;
      w_s[row * S + sp] = w;
      l += __ldcg(ml + 2 * sp + 1) * w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) l_s[row] = l;
  }
  __syncthreads();
  for (int idx = tid; idx < ng * D; idx += NTHREADS) {
    const int row = idx / D, col = idx % D;
    const size_t head = (size_t)b * a.n_heads + h0 + row;
    const float* po = a.part_o + head * stride * D + col;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    int sp = 0;
    for (; sp + 4 <= S; sp += 4) {  // four independent loads in flight
      const float v0 = __ldcg(po + (size_t)sp * D), v1 = __ldcg(po + (size_t)(sp + 1) * D);
      const float v2 = __ldcg(po + (size_t)(sp + 2) * D), v3 = __ldcg(po + (size_t)(sp + 3) * D);
      acc0 = fmaf(v0, w_s[row * S + sp], acc0);
      acc1 = fmaf(v1, w_s[row * S + sp + 1], acc1);
      acc2 = fmaf(v2, w_s[row * S + sp + 2], acc2);
      acc3 = fmaf(v3, w_s[row * S + sp + 3], acc3);
    }
    for (; sp < S; ++sp) acc0 = fmaf(__ldcg(po + (size_t)sp * D), w_s[row * S + sp], acc0);
    const float l = l_s[row];
    a.out[head * D + col] = __float2bfloat16_rn(l > 0.f ? ((acc0 + acc1) + (acc2 + acc3)) / l : 0.f);
  }
}

}  // namespace mll
