// Causal grouped-query attention over the paged cache: the general kernels.
//
// For query head h the kv head is h / (Hq / Hk); score_t = (q . k_t) * scale for every
// cached position t <= the query's own position (and, with a window w > 0, t > pos - w);
// p = softmax(score) with the maximum subtracted; out = sum_t p_t v_t - the reference's
// formula (src/forward.cc:265-298), which its CUDA path runs as ScoresKernel plus
// AttentionReduceKernel for one token of one sequence (src/cuda_attention.cu:77-163).
//
// Here the keys and values are read through a block table (pages of MLL_PAGE positions),
// the softmax is computed online in float32, and two kernels cover the two phases:
//   * decode: one query token per sequence, the context split over `n_splits` blocks per
//     (sequence, kv head) whose partial results a second kernel merges;
//   * prefill: tiles of 64 query tokens per (sequence, head), flash style.
// Both take any head_dim that is a multiple of 16 up to 256 and any head/group count, in
// float32 or bfloat16 storage.  They are SIMT kernels: the reference arithmetic in a
// parallel order, meant to be right for every size.
#include "common.cuh"

namespace mll {

struct AttnArgs {
  const void* q;           // [T, Hq * d]
  const void* k_cache;     // [n_pages, Hk, PAGE, d] of this layer
  const void* v_cache;
  const int* seq_slot;     // [B]
  const int* seq_ctx;      // [B] cached length including this step's tokens
  const int* seq_qstart;   // [B] first token row of the sequence in q (prefill)
  const int* seq_qlen;     // [B] number of query tokens of the sequence (prefill)
  const int* tile_seq;     // [n_tiles] (prefill)
  const int* tile_row0;    // [n_tiles] first query row of the tile within its sequence
  const int* block_table;  // [n_slots, max_blocks]
  float* part_o;           // [B, Hq, S, d] unnormalised partial outputs (decode)
  float* part_ml;          // [B, Hq, S, 2] running maximum and sum (decode)
  void* out;               // [T, Hq * d]
  int n_heads, n_kv_heads, head_dim, max_blocks, n_splits, window, heads_per_block;
  float scale;
};

template <typename T>
struct Vec16;  // 16 bytes of T
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
};

// ---------------------------------------------------------------------------------- //
// decode                                                                             //
// ---------------------------------------------------------------------------------- //
// grid (B, Hk * head_chunks, n_splits), 128 threads.  A block owns up to
// `heads_per_block` query heads of one kv head and a contiguous range of pages.
template <typename T, int NACC>
__global__ void __launch_bounds__(128)
attn_decode_kernel(AttnArgs a, int two_stage) {
  constexpr int PAD = 16 / sizeof(T);
  constexpr int VN = Vec16<T>::N;
  const int d = a.head_dim;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + a.heads_per_block - 1) / a.heads_per_block;
  const int b = blockIdx.x;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int split = blockIdx.z;
  const int g0 = chunk * a.heads_per_block;
  const int ng = min(a.heads_per_block, group - g0);  // heads of this block
  const int h0 = kvh * group + g0;                    // first query head
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int ctx = a.seq_ctx[b];
  const int first_key = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int pages_total = (ctx + MLL_PAGE - 1) / MLL_PAGE;
  const int first_page = first_key / MLL_PAGE;
  const int per_split = (pages_total - first_page + a.n_splits - 1) / a.n_splits;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(pages_total, p_begin + per_split);
  const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_blocks;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* q_s = reinterpret_cast<float*>(smem_raw);            // [hpb][d]
  float* s_s = q_s + a.heads_per_block * d;                   // [hpb][PAGE]
  float* m_s = s_s + a.heads_per_block * MLL_PAGE;            // [hpb]
  float* l_s = m_s + a.heads_per_block;
  float* alpha_s = l_s + a.heads_per_block;
  // 16-byte aligned start of the tiles
  size_t off = (size_t)((alpha_s + a.heads_per_block) - q_s) * sizeof(float);
  off = (off + 15) & ~(size_t)15;
  const int k_stride = d + PAD;  // elements
  const size_t k_tile = (size_t)MLL_PAGE * k_stride, v_tile = (size_t)MLL_PAGE * d;
  T* k_s = reinterpret_cast<T*>(smem_raw + off);
  T* v_s = k_s + (two_stage ? 2 : 1) * k_tile;

  const T* qrow = (const T*)a.q + (size_t)b * a.n_heads * d + (size_t)h0 * d;
  for (int i = tid; i < ng * d; i += 128) q_s[i] = to_float(qrow[i]);
  for (int i = tid; i < ng; i += 128) {
    m_s[i] = -INFINITY;
    l_s[i] = 0.f;
  }
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;

  const int cpr = d / VN;  // 16-byte chunks per row
  auto load_tiles = [&](int page_index, int stage) {
    const int page = table[page_index];
    const T* kg = (const T*)a.k_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * d;
    const T* vg = (const T*)a.v_cache + ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * d;
    T* kd = k_s + stage * k_tile;
    T* vd = v_s + stage * v_tile;
    for (int c = tid; c < MLL_PAGE * cpr; c += 128) {
      const int r = c / cpr, cc = c % cpr;
      cp_async16(kd + (size_t)r * k_stride + cc * VN, kg + (size_t)r * d + cc * VN);
      cp_async16(vd + (size_t)r * d + cc * VN, vg + (size_t)r * d + cc * VN);
    }
  };

  if (p_begin < p_end) {
    load_tiles(p_begin, 0);
    cp_async_commit();
  }
  for (int p = p_begin, it = 0; p < p_end; ++p, ++it) {
    const int cur = two_stage ? (it & 1) : 0;
    if (two_stage && p + 1 < p_end) {
      load_tiles(p + 1, cur ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    const T* kt = k_s + cur * k_tile;
    const T* vt = v_s + cur * v_tile;
    const int jlo = max(0, first_key - p * MLL_PAGE);
    const int jhi = min(MLL_PAGE, ctx - p * MLL_PAGE);

    // scores of (head, key) pairs
    for (int idx = tid; idx < ng * MLL_PAGE; idx += 128) {
      const int g = idx / MLL_PAGE, j = idx % MLL_PAGE;
      float s = -INFINITY;
      if (j >= jlo && j < jhi) {
        const T* kr = kt + (size_t)j * k_stride;
        const float* qg = q_s + g * d;
        float dot = 0.f;
        for (int e = 0; e < d; e += VN) {
          float kv[VN];
          Vec16<T>::load(kr + e, kv);
#pragma unroll
          for (int u = 0; u < VN; ++u) dot = fmaf(qg[e + u], kv[u], dot);
        }
        s = dot * a.scale;
      }
      s_s[idx] = s;
    }
    __syncthreads();

    // online softmax, one warp per head
    for (int g = warp; g < ng; g += 4) {
      const float v0 = s_s[g * MLL_PAGE + lane], v1 = s_s[g * MLL_PAGE + lane + 32];
      const float tile_max = warp_max(fmaxf(v0, v1));
      const float m_old = m_s[g];
      const float m_new = fmaxf(m_old, tile_max);
      float p0 = 0.f, p1 = 0.f, alpha = 1.f;
      if (m_new > -INFINITY) {
        alpha = expf(m_old - m_new);
        p0 = expf(v0 - m_new);
        p1 = expf(v1 - m_new);
      }
      s_s[g * MLL_PAGE + lane] = p0;
      s_s[g * MLL_PAGE + lane + 32] = p1;
      const float psum = warp_sum(p0 + p1);
      if (lane == 0) {
        l_s[g] = l_s[g] * alpha + psum;
        m_s[g] = m_new;
        alpha_s[g] = alpha;
      }
    }
    __syncthreads();

    // out += p . V
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int o = tid + 128 * i;
      if (o < ng * d) {
        const int g = o / d, e = o % d;
        float v = acc[i] * alpha_s[g];
        const float* pg = s_s + g * MLL_PAGE;
        for (int j = jlo; j < jhi; ++j) v = fmaf(pg[j], to_float(vt[(size_t)j * d + e]), v);
        acc[i] = v;
      }
    }
    __syncthreads();
    if (!two_stage && p + 1 < p_end) {
      load_tiles(p + 1, 0);
      cp_async_commit();
    }
  }

  if (a.n_splits == 1) {
    T* out = (T*)a.out + (size_t)b * a.n_heads * d + (size_t)h0 * d;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int o = tid + 128 * i;
      if (o < ng * d) {
        const float l = l_s[o / d];
        out[o] = from_float<T>(l > 0.f ? acc[i] / l : 0.f);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int o = tid + 128 * i;
      if (o < ng * d) {
        const int g = o / d, e = o % d;
        a.part_o[(((size_t)b * a.n_heads + h0 + g) * a.n_splits + split) * d + e] = acc[i];
      }
    }
    for (int g = tid; g < ng; g += 128) {
      float* ml = a.part_ml + (((size_t)b * a.n_heads + h0 + g) * a.n_splits + split) * 2;
      ml[0] = m_s[g];
      ml[1] = l_s[g];
    }
  }
}

// grid (B * Hq), merges the splits of one (sequence, head) in a fixed order.
template <typename T>
__global__ void attn_combine_kernel(AttnArgs a) {
  const int bh = blockIdx.x;
  const int d = a.head_dim, S = a.n_splits;
  const float* ml = a.part_ml + (size_t)bh * S * 2;
  float m = -INFINITY;
  for (int s = 0; s < S; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < S; ++s)
    if (ml[2 * s] > -INFINITY) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < S; ++s)
      if (ml[2 * s] > -INFINITY)
        o += a.part_o[((size_t)bh * S + s) * d + e] * expf(ml[2 * s] - m);
    ((T*)a.out)[(size_t)bh * d + e] = from_float<T>(o * inv);
  }
}

// ---------------------------------------------------------------------------------- //
// prefill                                                                            //
// ---------------------------------------------------------------------------------- //
// grid (n_tiles, Hq), 256 threads as 16 x 16: thread (ty, tx) owns query rows
// 4 ty .. 4 ty + 3, key columns tx + 16 jj and output columns tx + 16 i (i < DT).
// Tiles are kept in shared memory as float32 whatever the storage type.
template <typename T, int DT>
__global__ void __launch_bounds__(256)
attn_prefill_kernel(AttnArgs a) {
  constexpr int BM = 64, BN = MLL_PAGE;
  const int d = a.head_dim;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int seq = a.tile_seq[blockIdx.x], row0 = a.tile_row0[blockIdx.x];
  const int h = blockIdx.y;
  const int kvh = h / (a.n_heads / a.n_kv_heads);
  const int ctx = a.seq_ctx[seq], qlen = a.seq_qlen[seq];
  const int rows = min(BM, qlen - row0);
  const int pos0 = ctx - qlen + row0;  // position of the tile's first query
  const int* table = a.block_table + (size_t)a.seq_slot[seq] * a.max_blocks;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int qk_stride = d + 4;
  float* q_s = reinterpret_cast<float*>(smem_raw);  // [BM][d + 4]
  float* k_s = q_s + BM * qk_stride;                // [BN][d + 4]
  float* v_s = k_s + BN * qk_stride;                // [BN][d]
  float* p_s = v_s + BN * d;                        // [BM][BN + 1]

  const int groups = d / 4;  // 4-element groups per row
  {
    const T* qg = (const T*)a.q + ((size_t)a.seq_qstart[seq] + row0) * a.n_heads * d + (size_t)h * d;
    for (int idx = tid; idx < BM * groups; idx += 256) {
      const int r = idx / groups, c = (idx % groups) * 4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < rows) {
        const T* src = qg + (size_t)r * a.n_heads * d + c;
        v = make_float4(to_float(src[0]), to_float(src[1]), to_float(src[2]), to_float(src[3]));
      }
      *reinterpret_cast<float4*>(q_s + r * qk_stride + c) = v;
    }
  }

  float acc[4][DT];
  float m_run[4], l_run[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DT; ++i) acc[r][i] = 0.f;
  }

  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int last_key = pos0 + rows - 1;
  for (int p = first_key / BN; p <= last_key / BN; ++p) {
    __syncthreads();  // previous tile fully consumed (and q_s written, first time)
    {
      const int page = table[p];
      const T* kg = (const T*)a.k_cache + ((size_t)page * a.n_kv_heads + kvh) * BN * d;
      const T* vg = (const T*)a.v_cache + ((size_t)page * a.n_kv_heads + kvh) * BN * d;
      for (int idx = tid; idx < BN * groups; idx += 256) {
        const int r = idx / groups, c = (idx % groups) * 4;
        float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
        if (p * BN + r < ctx) {  // rows past the cached length hold no data
          const T* ks = kg + (size_t)r * d + c;
          const T* vs = vg + (size_t)r * d + c;
          kv = make_float4(to_float(ks[0]), to_float(ks[1]), to_float(ks[2]), to_float(ks[3]));
          vv = make_float4(to_float(vs[0]), to_float(vs[1]), to_float(vs[2]), to_float(vs[3]));
        }
        *reinterpret_cast<float4*>(k_s + r * qk_stride + c) = kv;
        *reinterpret_cast<float4*>(v_s + r * d + c) = vv;
      }
    }
    __syncthreads();

    // S = Q K^T for this thread's 4 x 4 sub-tile
    float s[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[r][j] = 0.f;
    for (int e = 0; e < d; e += 4) {
      float4 qv[4], kv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) qv[r] = *reinterpret_cast<const float4*>(q_s + (ty * 4 + r) * qk_stride + e);
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = *reinterpret_cast<const float4*>(k_s + (tx + 16 * j) * qk_stride + e);
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[r][j] = fmaf(qv[r].x, kv[j].x, s[r][j]);
          s[r][j] = fmaf(qv[r].y, kv[j].y, s[r][j]);
          s[r][j] = fmaf(qv[r].z, kv[j].z, s[r][j]);
          s[r][j] = fmaf(qv[r].w, kv[j].w, s[r][j]);
        }
    }

    // mask, online softmax per row (the 16 lanes with equal ty share a row)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = ty * 4 + r;
      const int qpos = pos0 + row;
      float row_max = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kpos = p * BN + tx + 16 * j;
        const bool ok = row < rows && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
        s[r][j] = ok ? s[r][j] * a.scale : -INFINITY;
        row_max = fmaxf(row_max, s[r][j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
      const float m_new = fmaxf(m_run[r], row_max);
      float alpha = 1.f, row_sum = 0.f;
      if (m_new > -INFINITY) {
        alpha = expf(m_run[r] - m_new);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[r][j] = expf(s[r][j] - m_new);
          row_sum += s[r][j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[r][j] = 0.f;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) row_sum += __shfl_xor_sync(0xffffffffu, row_sum, o);
      l_run[r] = l_run[r] * alpha + row_sum;
      m_run[r] = m_new;
#pragma unroll
      for (int i = 0; i < DT; ++i) acc[r][i] *= alpha;
#pragma unroll
      for (int j = 0; j < 4; ++j) p_s[row * (BN + 1) + tx + 16 * j] = s[r][j];
    }
    __syncthreads();

    // O += P V
    for (int j = 0; j < BN; ++j) {
      float pv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) pv[r] = p_s[(ty * 4 + r) * (BN + 1) + j];
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        const int c = tx + 16 * i;
        if (c < d) {
          const float v = v_s[j * d + c];
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[r][i] = fmaf(pv[r], v, acc[r][i]);
        }
      }
    }
  }

  T* out = (T*)a.out + ((size_t)a.seq_qstart[seq] + row0) * a.n_heads * d + (size_t)h * d;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = ty * 4 + r;
    if (row < rows) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        const int c = tx + 16 * i;
        if (c < d) out[(size_t)row * a.n_heads * d + c] = from_float<T>(acc[r][i] * inv);
      }
    }
  }
}

template <typename T, int NACC>
int launch_decode(const AttnArgs& a, int n_seqs, int chunks, size_t smem, int two_stage, cudaStream_t stream) {
  auto kernel = attn_decode_kernel<T, NACC>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("attention decode: cannot reserve %zu bytes of shared memory: %s", smem,
                    cudaGetErrorString(err));
      return (int)err;
    }
  }
  dim3 grid(n_seqs, a.n_kv_heads * chunks, a.n_splits);
  MLL_LAUNCH((kernel), grid, 128, smem, stream, a, two_stage);
  MLL_LAUNCH_CHECK();
  return 0;
}

template <typename T>
int decode_dispatch(AttnArgs a, int n_seqs, cudaStream_t stream) {
  const int d = a.head_dim, group = a.n_heads / a.n_kv_heads;
  int hpb = 2048 / d;  // at most 16 accumulators per thread
  if (hpb > group) hpb = group;
  a.heads_per_block = hpb;
  const int chunks = (group + hpb - 1) / hpb;
  const int need = (hpb * d + 127) / 128;
  const size_t head_bytes = ((size_t)hpb * (d + MLL_PAGE + 3) * sizeof(float) + 15) & ~(size_t)15;
  const size_t stage_bytes = (size_t)MLL_PAGE * ((d + 16 / sizeof(T)) + d) * sizeof(T);
  const size_t limit = 200 * 1024;
  int two_stage = head_bytes + 2 * stage_bytes <= limit ? 1 : 0;
  const size_t smem = head_bytes + (two_stage ? 2 : 1) * stage_bytes;
  if (smem > limit) {
    mll_set_error("attention decode: head_dim %d with %d heads per block needs %zu bytes of shared memory",
                  d, hpb, smem);
    return -1;
  }
  int rc;
  if (need <= 1) rc = launch_decode<T, 1>(a, n_seqs, chunks, smem, two_stage, stream);
  else if (need <= 2) rc = launch_decode<T, 2>(a, n_seqs, chunks, smem, two_stage, stream);
  else if (need <= 4) rc = launch_decode<T, 4>(a, n_seqs, chunks, smem, two_stage, stream);
  else if (need <= 8) rc = launch_decode<T, 8>(a, n_seqs, chunks, smem, two_stage, stream);
  else rc = launch_decode<T, 16>(a, n_seqs, chunks, smem, two_stage, stream);
  if (rc != 0) return rc;
  if (a.n_splits > 1) {
    MLL_LAUNCH((attn_combine_kernel<T>), n_seqs * a.n_heads, 128, 0, stream, a);
    MLL_LAUNCH_CHECK();
  }
  return 0;
}

template <typename T, int DT>
int launch_prefill(const AttnArgs& a, int n_tiles, cudaStream_t stream) {
  const int d = a.head_dim;
  const size_t smem = ((size_t)2 * 64 * (d + 4) + (size_t)64 * d + (size_t)64 * 65) * sizeof(float);
  auto kernel = attn_prefill_kernel<T, DT>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("attention prefill: cannot reserve %zu bytes of shared memory: %s", smem,
                    cudaGetErrorString(err));
      return (int)err;
    }
  }
  dim3 grid(n_tiles, a.n_heads);
  MLL_LAUNCH((kernel), grid, 256, smem, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

template <typename T>
int prefill_dispatch(const AttnArgs& a, int n_tiles, cudaStream_t stream) {
  if (a.head_dim <= 64) return launch_prefill<T, 4>(a, n_tiles, stream);
  if (a.head_dim <= 128) return launch_prefill<T, 8>(a, n_tiles, stream);
  return launch_prefill<T, 16>(a, n_tiles, stream);
}

static int check_common(const AttnArgs& a, const char* what) {
  MLL_REQUIRE(a.head_dim >= 16 && a.head_dim <= 256 && a.head_dim % 16 == 0,
              "%s: head_dim %d is not a multiple of 16 in [16, 256]", what, a.head_dim);
  MLL_REQUIRE(a.n_heads > 0 && a.n_kv_heads > 0 && a.n_heads % a.n_kv_heads == 0,
              "%s: %d heads are not a multiple of %d kv heads", what, a.n_heads, a.n_kv_heads);
  MLL_REQUIRE(a.window >= 0, "%s: negative window", what);
  return 0;
}

}  // namespace mll

// Scratch floats the decode kernel needs for `n_splits` > 1: partial outputs then (m, l).
MLL_API long long mll_attn_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
  return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

MLL_API int mll_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                            const int* seq_ctx, const int* block_table, float* scratch, void* out,
                            int dtype, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                            int max_blocks, int n_splits, int window, float scale, cudaStream_t stream) {
  mll::AttnArgs a{};
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache; a.seq_slot = seq_slot; a.seq_ctx = seq_ctx;
  a.block_table = block_table; a.out = out;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.max_blocks = max_blocks;
  a.n_splits = n_splits; a.window = window; a.scale = scale;
  if (mll::check_common(a, "attention decode") != 0) return -1;
  MLL_REQUIRE(n_seqs >= 0 && n_splits >= 1 && n_splits <= 65535, "attention decode: bad batch or split count");
  MLL_REQUIRE(n_splits == 1 || scratch != nullptr, "attention decode: %d splits need scratch memory", n_splits);
  if (n_seqs == 0) return 0;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)n_seqs * n_heads * n_splits * head_dim : nullptr;
  if (dtype == MLL_F32) return mll::decode_dispatch<float>(a, n_seqs, stream);
  if (dtype == MLL_BF16) return mll::decode_dispatch<__nv_bfloat16>(a, n_seqs, stream);
  MLL_REQUIRE(false, "attention decode: unknown dtype %d", dtype);
  return -1;
}

// Merges the partial results of a split decode (scratch layout as written by the decode kernels).
MLL_API int mll_attn_combine(float* scratch, void* out, int dtype, int n_seqs, int n_heads, int head_dim,
                             int n_splits, cudaStream_t stream) {
  MLL_REQUIRE(n_seqs >= 0 && n_heads > 0 && head_dim > 0 && n_splits >= 1, "attention combine: bad sizes");
  if (n_seqs == 0) return 0;
  mll::AttnArgs a{};
  a.part_o = scratch;
  a.part_ml = scratch + (size_t)n_seqs * n_heads * n_splits * head_dim;
  a.out = out;
  a.n_heads = n_heads; a.head_dim = head_dim; a.n_splits = n_splits;
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::attn_combine_kernel<float>), n_seqs * n_heads, 128, 0, stream, a);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::attn_combine_kernel<__nv_bfloat16>), n_seqs * n_heads, 128, 0, stream, a);
  else
    MLL_REQUIRE(false, "attention combine: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                             const int* seq_ctx, const int* seq_qstart, const int* seq_qlen,
                             const int* tile_seq, const int* tile_row0, const int* block_table, void* out,
                             int dtype, int n_tiles, int n_heads, int n_kv_heads, int head_dim,
                             int max_blocks, int window, float scale, cudaStream_t stream) {
  mll::AttnArgs a{};
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache; a.seq_slot = seq_slot; a.seq_ctx = seq_ctx;
  a.seq_qstart = seq_qstart; a.seq_qlen = seq_qlen; a.tile_seq = tile_seq; a.tile_row0 = tile_row0;
  a.block_table = block_table; a.out = out;
  a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.max_blocks = max_blocks;
  a.n_splits = 1; a.window = window; a.scale = scale;
  if (mll::check_common(a, "attention prefill") != 0) return -1;
  MLL_REQUIRE(n_tiles >= 0, "attention prefill: negative tile count");
  if (n_tiles == 0) return 0;
  if (dtype == MLL_F32) return mll::prefill_dispatch<float>(a, n_tiles, stream);
  if (dtype == MLL_BF16) return mll::prefill_dispatch<__nv_bfloat16>(a, n_tiles, stream);
  MLL_REQUIRE(false, "attention prefill: unknown dtype %d", dtype);
  return -1;
}

// ---------------------------------------------------------------------------------- //
// decode without allocation (declared and explained in no_alloc.h)                    //
// ---------------------------------------------------------------------------------- //
#include <mutex>

#include "no_alloc.h"

// Partial results of the context splits live here instead of in caller-provided scratch.
// In host code this name is only a handle for the runtime; the device address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_no_alloc_scratch[MLL_NO_ALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_no_alloc_address[kMaxDevices] = {};
std::mutex g_no_alloc_lock;

// Device address of the scratch array on the current device, looked up once per device.
int no_alloc_scratch(float** address) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    mll_set_error("attention decode (no alloc): cudaGetDevice failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  if (device < 0 || device >= kMaxDevices) {
    mll_set_error("attention decode (no alloc): device %d is beyond the %d devices this table holds", device, kMaxDevices);
    return -1;
  }
  std::lock_guard<std::mutex> guard(g_no_alloc_lock);
  if (g_no_alloc_address[device] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      mll_set_error("attention decode (no alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
      return err != cudaSuccess ? (int)err : -1;
    }
    g_no_alloc_address[device] = static_cast<float*>(ptr);
  }
  *address = g_no_alloc_address[device];
  return 0;
}
}  // namespace

MLL_API int mll_attn_decode_no_alloc(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                                     const int* seq_ctx, const int* block_table, void* out, int dtype, int n_seqs,
                                     int n_heads, int n_kv_heads, int head_dim, int max_blocks, int n_splits,
                                     int window, float scale, cudaStream_t stream) {
  MLL_REQUIRE(n_seqs >= 0 && n_heads > 0 && head_dim > 0 && n_splits >= 1,
              "attention decode (no alloc): bad sizes seqs=%d heads=%d head_dim=%d splits=%d", n_seqs, n_heads,
              head_dim, n_splits);
  const long long need = mll_attn_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits);
  MLL_REQUIRE(need <= (long long)MLL_NO_ALLOC_SCRATCH_FLOATS,
              "attention decode (no alloc): %d sequences x %d heads x %d splits x (head_dim %d + 2) = %lld floats of "
              "scratch exceed the built-in %d; use fewer splits or the entry point that takes scratch from the caller",
              n_seqs, n_heads, n_splits, head_dim, need, MLL_NO_ALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  const int rc = no_alloc_scratch(&scratch);
  if (rc != 0) return rc;
  return mll_attn_decode(q, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch, out, dtype, n_seqs, n_heads,
                         n_kv_heads, head_dim, max_blocks, n_splits, window, scale, stream);
}
