// Decode attention on tensor cores (bfloat16, head_dim 64 / 128 / 256).
//
// One block of four warps per (sequence, kv head [, chunk of 16 query heads], split of the
// context).  The block walks its pages together: key and value pages arrive in shared
// memory through a cp.async pipeline; every warp scores the query heads against its 16 of
// the page's 64 keys (mma.sync m16n8k16, heads padded to the 16 rows of the tile), the warps
// exchange row maxima and sums through shared memory (online softmax in float32), the
// probabilities go to shared memory as bfloat16, and every warp multiplies them with its
// quarter of the value columns.  The arithmetic is that of the general kernel in
// attention.cu (the reference's src/forward.cc:265-298); only the order of the sums differs.
// The output format (direct, or partial results + (max, sum) per split for the combine
// kernel) is the same as the general kernel's, which remains the path for other head sizes
// and for float32.
#include "attention_decode.cuh"
#include "common.cuh"

namespace mll {

template <int D, int STAGES>
struct DecodeMmaSmem {
  static constexpr int STRIDE = D + 8;                       // bf16 elements per key row (16 bytes of padding)
  static constexpr int TILE = MLL_PAGE * STRIDE;             // elements of one K or V page
  static constexpr int P_STRIDE = MLL_PAGE + 8;
  static constexpr size_t BYTES = (size_t)STAGES * 2 * TILE * 2 + 16 * P_STRIDE * 2 + 2 * 4 * 16 * sizeof(float);
};

// grid (B, Hk * head_chunks, n_splits); 128 threads.  FUSED: the rotary encoding and the cache
// write of the step's token happen here instead of in a kernel of their own (one launch less
// per layer): every block rotates its query heads in registers; the block whose pages include
// the sequence's last one rotates the new key, puts it and the new value into its shared-memory
// copy of that page and into the cache.
template <int D, int STAGES, bool FUSED>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(DecodeMmaArgs a) {
  using L = DecodeMmaSmem<D, STAGES>;
  constexpr int KSTEPS = D / 16;       // k-steps of the score product
  constexpr int NT_OUT = D / 32;       // value n-tiles (8 columns) per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);         // [STAGES][2][PAGE][STRIDE]
  __nv_bfloat16* p_s = kv_s + (size_t)STAGES * 2 * L::TILE;                 // [16][P_STRIDE]
  float* wmax = reinterpret_cast<float*>(p_s + 16 * L::P_STRIDE);           // [4][16]
  float* wsum = wmax + 4 * 16;                                              // [4][16]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + 15) / 16;
  const int b = blockIdx.x;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int split = blockIdx.z;
  const int ng = min(16, group - chunk * 16);
  const int h0 = kvh * group + chunk * 16;

  const int ctx = a.seq_ctx[b];
  const int first_key = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int pages_total = (ctx + MLL_PAGE - 1) / MLL_PAGE;
  const int first_page = first_key / MLL_PAGE;
  // The launch offers n_splits blocks per (sequence, kv head); a sequence uses as many of them as
  // its own length pays for (the rest leave at once), so one captured launch serves short and
  // long contexts alike.  Without arrival counters a separate kernel merges all n_splits.
  const int n_eff = a.counters ? decode_splits_for(pages_total - first_page, a.n_splits) : a.n_splits;
  if (split >= n_eff) return;
  const int per_split = (pages_total - first_page + n_eff - 1) / n_eff;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(pages_total, p_begin + per_split);
  const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_blocks;

  // The block's page numbers, fetched ahead into a ring of 256 entries: a lookup in global
  // memory right before each page's copies would put one more memory latency into every iteration.
  __shared__ int page_ids[256];
  for (int j = tid; j < min(p_end - p_begin, 256); j += 128) page_ids[j] = table[p_begin + j];
  __syncthreads();

  constexpr int CPR = D / 8;  // 16-byte chunks per key row
  auto load_page = [&](int page_index, int stage) {
    const int page = page_ids[(page_index - p_begin) & 255];
    const size_t base = ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * D;
    __nv_bfloat16* kd = kv_s + (size_t)stage * 2 * L::TILE;
    __nv_bfloat16* vd = kd + L::TILE;
    const int valid_rows = ctx - page_index * MLL_PAGE;  // rows past the sequence hold no data
    for (int c = tid; c < MLL_PAGE * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      cp_async16(kd + r * L::STRIDE + cc * 8, a.k_cache + base + (size_t)r * D + cc * 8);
      cp_async16_zfill(vd + r * L::STRIDE + cc * 8, a.v_cache + base + (size_t)r * D + cc * 8, r < valid_rows);
    }
  };

  float o[NT_OUT][4];
#pragma unroll
  for (int n = 0; n < NT_OUT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8

  const int n_pages = max(0, p_end - p_begin);
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_pages) load_page(p_begin + s, s);
    cp_async_commit();
  }
  // FUSED: the block whose pages include the sequence's last one fetches the new key pair and
  // value pair of its kv head now (one pair per thread), long before the page comes up
  const bool owns_new_row = FUSED && a.k_write != nullptr && ctx > 0 && p_begin <= pages_total - 1 &&
                            pages_total - 1 < p_end;
  __nv_bfloat16 new_k0 = __float2bfloat16_rn(0.f), new_k1 = new_k0;
  unsigned new_v = 0;
  if (owns_new_row && tid < D / 2) {
    const __nv_bfloat16* k_in = a.qkv + (size_t)b * a.qkv_ld + (size_t)(a.n_heads + kvh) * D;
    const __nv_bfloat16* v_in = k_in + (size_t)a.n_kv_heads * D;
    const int e0 = a.interleaved ? 2 * tid : tid, e1 = a.interleaved ? 2 * tid + 1 : tid + D / 2;
    const float x0 = __bfloat162float(k_in[e0]), x1 = __bfloat162float(k_in[e1]);
    new_v = *reinterpret_cast<const unsigned*>(v_in + 2 * tid);
    float y0 = x0, y1 = x1;
    if (a.cos_table != nullptr) {
      const float c = a.cos_table[(size_t)(ctx - 1) * (D / 2) + tid], sv = a.sin_table[(size_t)(ctx - 1) * (D / 2) + tid];
      y0 = x0 * c - x1 * sv;
      y1 = x0 * sv + x1 * c;
    }
    new_k0 = __float2bfloat16_rn(y0);
    new_k1 = __float2bfloat16_rn(y1);
  }

  // the first pages are on their way: the queries' latency hides behind theirs
  // query fragments (A operand), rows = heads of this chunk, zero beyond ng
  unsigned qf[KSTEPS][4];
  {
    const __nv_bfloat16* q0 = FUSED ? a.qkv + (size_t)b * a.qkv_ld + (size_t)h0 * D
                                    : a.q + ((size_t)b * a.n_heads + h0) * D;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int col = ks * 16 + 2 * t;
      qf[ks][0] = g < ng ? *reinterpret_cast<const unsigned*>(q0 + (size_t)g * D + col) : 0u;
      qf[ks][1] = g + 8 < ng ? *reinterpret_cast<const unsigned*>(q0 + (size_t)(g + 8) * D + col) : 0u;
      qf[ks][2] = g < ng ? *reinterpret_cast<const unsigned*>(q0 + (size_t)g * D + col + 8) : 0u;
      qf[ks][3] = g + 8 < ng ? *reinterpret_cast<const unsigned*>(q0 + (size_t)(g + 8) * D + col + 8) : 0u;
    }
    if (FUSED && a.cos_table != nullptr && ctx > 0) {
      // the token's position is ctx - 1 for every head; registers [2j] and [2j + 1] hold rows g and
      // g + 8 at columns col + 8 j, col + 8 j + 1
      const float* cs = a.cos_table + (size_t)(ctx - 1) * (D / 2);
      const float* sn = a.sin_table + (size_t)(ctx - 1) * (D / 2);
      if (a.interleaved) {  // pairs (2i, 2i + 1): both halves of a pair sit in one register
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int pair = ks * 8 + t + 4 * j;
            const float c = cs[pair], sv = sn[pair];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float2 x = unpack_bf162(qf[ks][2 * j + r]);
              qf[ks][2 * j + r] = pack_bf162(x.x * c - x.y * sv, x.x * sv + x.y * c);
            }
          }
      } else {  // pairs (i, i + d/2): the partner sits in the same place of k-step ks + KSTEPS / 2
#pragma unroll
        for (int ks = 0; ks < KSTEPS / 2; ++ks)
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int i0 = ks * 16 + 2 * t + 8 * j;
            const float c0 = cs[i0], s0 = sn[i0], c1 = cs[i0 + 1], s1 = sn[i0 + 1];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const float2 lo = unpack_bf162(qf[ks][2 * j + r]), hi = unpack_bf162(qf[ks + KSTEPS / 2][2 * j + r]);
              qf[ks][2 * j + r] = pack_bf162(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
              qf[ks + KSTEPS / 2][2 * j + r] = pack_bf162(lo.x * s0 + hi.x * c0, lo.y * s1 + hi.y * c1);
            }
          }
      }
    }
  }

  for (int it = 0; it < n_pages; ++it) {
    const int p = p_begin + it;
    cp_async_wait<STAGES - 2>();  // page `it` has landed (one group per iteration, committed even when empty)
    __syncthreads();              // ... for every thread's copies; and all warps are done with page it - 1
    if (it + STAGES - 1 < n_pages) load_page(p + STAGES - 1, (it + STAGES - 1) % STAGES);
    cp_async_commit();
    if ((it & 127) == 0 && it > 0) {  // entries it + 128 .. it + 255 take the places of pages long done
      const int j = it + 128 + tid;
      if (j < n_pages) page_ids[j & 255] = table[p_begin + j];
    }

    const __nv_bfloat16* kt = kv_s + (size_t)(it % STAGES) * 2 * L::TILE;
    const __nv_bfloat16* vt = kt + L::TILE;
    if (FUSED && owns_new_row && p == pages_total - 1) {
      // the step's token lies in this page: its key (rotated) and value replace whatever the cache held
      const int row = (ctx - 1) % MLL_PAGE;
      if (tid < D / 2) {
        __nv_bfloat16* k_row = kv_s + (size_t)(it % STAGES) * 2 * L::TILE + row * L::STRIDE;
        __nv_bfloat16* v_row = k_row + L::TILE;
        const size_t cache_row = (((size_t)page_ids[it & 255] * a.n_kv_heads + kvh) * MLL_PAGE + row) * D;
        const int e0 = a.interleaved ? 2 * tid : tid, e1 = a.interleaved ? 2 * tid + 1 : tid + D / 2;
        k_row[e0] = new_k0;
        k_row[e1] = new_k1;
        a.k_write[cache_row + e0] = new_k0;
        a.k_write[cache_row + e1] = new_k1;
        *reinterpret_cast<unsigned*>(v_row + 2 * tid) = new_v;
        *reinterpret_cast<unsigned*>(a.v_write + cache_row + 2 * tid) = new_v;
      }
      __syncthreads();
    }

    // scores of the 16 heads against this warp's 16 keys: two n-tiles of 8 keys
    float s_acc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      // matrices: (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
      unsigned kb[4];
      const int key = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int dim = ks * 16 + (((lane >> 3) & 1) << 3);
      ldmatrix_x4(kb, kt + key * L::STRIDE + dim);
      mma_16816(s_acc[0], qf[ks], kb[0], kb[1]);
      mma_16816(s_acc[1], qf[ks], kb[2], kb[3]);
    }
    // scale, mask, row maxima over this warp's keys
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kpos = p * MLL_PAGE + warp * 16 + n * 8 + 2 * t + (i & 1);
        const bool ok = kpos < ctx && kpos >= first_key;
        const float v = ok ? s_acc[n][i] * a.scale : -INFINITY;
        s_acc[n][i] = v;
        tile_max[i >> 1] = fmaxf(tile_max[i >> 1], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    }
    if (t == 0) {
      wmax[warp * 16 + g] = tile_max[0];
      wmax[warp * 16 + g + 8] = tile_max[1];
    }
    __syncthreads();
    float alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      const float m_tile = fmaxf(fmaxf(wmax[row], wmax[16 + row]), fmaxf(wmax[32 + row], wmax[48 + row]));
      const float m_new = fmaxf(m_run[r], m_tile);
      alpha[r] = m_new > -INFINITY ? __expf(m_run[r] - m_new) : 1.f;
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float pv = m_new > -INFINITY ? __expf(s_acc[n][2 * r + i] - m_new) : 0.f;
          s_acc[n][2 * r + i] = pv;
          row_sum[r] += pv;
        }
      m_run[r] = m_new;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int col = warp * 16 + n * 8 + 2 * t;
      *reinterpret_cast<__nv_bfloat162*>(p_s + g * L::P_STRIDE + col) = __floats2bfloat162_rn(s_acc[n][0], s_acc[n][1]);
      *reinterpret_cast<__nv_bfloat162*>(p_s + (g + 8) * L::P_STRIDE + col) =
          __floats2bfloat162_rn(s_acc[n][2], s_acc[n][3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
      row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    if (t == 0) {
      wsum[warp * 16 + g] = row_sum[0];
      wsum[warp * 16 + g + 8] = row_sum[1];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      l_run[r] = l_run[r] * alpha[r] + ((wsum[row] + wsum[16 + row]) + (wsum[32 + row] + wsum[48 + row]));
    }
    // out[:, this warp's columns] = alpha * out + P[16 x 64] . V[64 x columns]
#pragma unroll
    for (int n = 0; n < NT_OUT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }
#pragma unroll
    for (int ks = 0; ks < MLL_PAGE / 16; ++ks) {
      unsigned pa[4];
      // matrices: (rows 0-7, keys 0-7), (rows 8-15, keys 0-7), (rows 0-7, keys 8-15), (rows 8-15, keys 8-15)
      ldmatrix_x4(pa, p_s + ((lane & 7) + (((lane >> 3) & 1) << 3)) * L::P_STRIDE + ks * 16 + ((lane >> 4) << 3));
#pragma unroll
      for (int n = 0; n < NT_OUT; n += 2) {
        // transposed 8x8 tiles of V: (keys 0-7, cols n), (keys 8-15, cols n), (keys 0-7, cols n+1), (keys 8-15, cols n+1)
        unsigned vb[4];
        const int key = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int col = warp * (D / 4) + (n + (lane >> 4)) * 8;
        ldmatrix_x4_trans(vb, vt + key * L::STRIDE + col);
        mma_16816(o[n], pa, vb[0], vb[1]);
        if (n + 1 < NT_OUT) mma_16816(o[n + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

  // rows g and g + 8 of the tile are heads h0 + g and h0 + g + 8; this thread holds columns
  // warp * D/4 + n * 8 + 2 t + {0, 1}
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (row >= ng) continue;
    const size_t head = (size_t)b * a.n_heads + h0 + row;
    if (n_eff == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
      for (int n = 0; n < NT_OUT; ++n) {
        const int col = warp * (D / 4) + n * 8 + 2 * t;
        *reinterpret_cast<__nv_bfloat162*>(a.out + head * D + col) =
            __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
      }
    } else {
      float* po = a.part_o + (head * a.n_splits + split) * D;
#pragma unroll
      for (int n = 0; n < NT_OUT; ++n) {
        const int col = warp * (D / 4) + n * 8 + 2 * t;
        *reinterpret_cast<float2*>(po + col) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
      }
      if (warp == 0 && t == 0) {
        float* ml = a.part_ml + (head * a.n_splits + split) * 2;
        ml[0] = m_run[r];
        ml[1] = l_run[r];
      }
    }
  }
  if (n_eff == 1 || a.counters == nullptr) return;

  merge_decode_splits<D, 128>(a, b, blockIdx.y, gridDim.y, h0, ng, n_eff, reinterpret_cast<float*>(smem_raw));
}

template <int D, int STAGES, bool FUSED>
int launch_decode_mma(const DecodeMmaArgs& a, int n_seqs, cudaStream_t stream) {
  const size_t smem = DecodeMmaSmem<D, STAGES>::BYTES;
  auto kernel = attn_decode_mma_kernel<D, STAGES, FUSED>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("attention decode (mma): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  const int group = a.n_heads / a.n_kv_heads;
  dim3 grid(n_seqs, a.n_kv_heads * ((group + 15) / 16), a.n_splits);
  MLL_LAUNCH((kernel), grid, 128, smem, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}


// ---------------------------------------------------------------------------------- //
// prefill                                                                            //
// ---------------------------------------------------------------------------------- //
struct PrefillMmaArgs {
  const __nv_bfloat16* q;        // [T, Hq * d]
  const __nv_bfloat16* k_cache;  // [n_pages, Hk, PAGE, d]
  const __nv_bfloat16* v_cache;
  const int* seq_slot;
  const int* seq_ctx;
  const int* seq_qstart;
  const int* seq_qlen;
  const int* tile_seq;
  const int* tile_row0;
  const int* block_table;
  __nv_bfloat16* out;            // [T, Hq * d]
  int n_heads, n_kv_heads, max_blocks, window;
  float scale_log2;              // scale * log2(e): the softmax runs in base 2
};

template <int D>
struct PrefillMmaSmem {
  static constexpr int STRIDE = D + 8;
  static constexpr int TILE = 64 * STRIDE;  // elements of the Q tile or of one K or V page
  static constexpr size_t BYTES = (size_t)(2 * 2) * TILE * 2;  // two stages of (K, V); Q passes through stage 1
};

// Flash-style attention for tiles of 64 query tokens: grid (n_tiles, Hq), four warps, each
// warp owns 16 query rows.  Per key page: S = Q K^T (tensor cores), online softmax in
// registers (float32, base 2), P re-used from the accumulator registers as the A operand of
// O += P V.  Pages arrive through a two-stage cp.async ring shared by the four warps.
template <int D>
__global__ void __launch_bounds__(128, 3)
attn_prefill_mma_kernel(PrefillMmaArgs a) {
  using L = PrefillMmaSmem<D>;
  constexpr int KSTEPS = D / 16;
  constexpr int NT_OUT = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2 stages][K, V][64][STRIDE]
  __nv_bfloat16* q_s = kv_s + 2 * L::TILE;  // the query tile lands in stage 1 and moves to registers before page 1

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int seq = a.tile_seq[blockIdx.x], row0 = a.tile_row0[blockIdx.x];
  const int h = blockIdx.y;
  const int kvh = h / (a.n_heads / a.n_kv_heads);
  const int ctx = a.seq_ctx[seq], qlen = a.seq_qlen[seq];
  const int rows = min(64, qlen - row0);
  const int pos0 = ctx - qlen + row0;
  const int* table = a.block_table + (size_t)a.seq_slot[seq] * a.max_blocks;
  constexpr int CPR = D / 8;

  {  // the query tile; rows past the sequence's tokens are zero
    const __nv_bfloat16* qg = a.q + ((size_t)a.seq_qstart[seq] + row0) * a.n_heads * D + (size_t)h * D;
    for (int c = tid; c < 64 * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      cp_async16_zfill(q_s + r * L::STRIDE + cc * 8, qg + (size_t)min(r, rows - 1) * a.n_heads * D + cc * 8, r < rows);
    }
  }
  auto load_page = [&](int page_index, int stage) {
    const int page = table[page_index];
    const size_t base = ((size_t)page * a.n_kv_heads + kvh) * MLL_PAGE * D;
    __nv_bfloat16* kd = kv_s + (size_t)stage * 2 * L::TILE;
    __nv_bfloat16* vd = kd + L::TILE;
    const int valid_rows = ctx - page_index * MLL_PAGE;
    for (int c = tid; c < MLL_PAGE * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      cp_async16(kd + r * L::STRIDE + cc * 8, a.k_cache + base + (size_t)r * D + cc * 8);
      cp_async16_zfill(vd + r * L::STRIDE + cc * 8, a.v_cache + base + (size_t)r * D + cc * 8, r < valid_rows);
    }
  };

  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int p_first = first_key / MLL_PAGE, p_last = (pos0 + rows - 1) / MLL_PAGE;
  load_page(p_first, 0);
  cp_async_commit();

  unsigned qf[KSTEPS][4];
  float o[NT_OUT][4];
#pragma unroll
  for (int n = 0; n < NT_OUT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows warp * 16 + g and + 8

  for (int p = p_first; p <= p_last; ++p) {
    const int stage = (p - p_first) & 1;
    cp_async_wait<0>();
    __syncthreads();  // page p (and, the first time, Q) landed; every warp is done with page p - 1
    if (p == p_first) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(qf[ks], q_s + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * L::STRIDE + ks * 16 +
                                ((lane >> 4) << 3));
      __syncthreads();  // every warp holds its query fragments: stage 1 may be overwritten
    }
    if (p < p_last) load_page(p + 1, stage ^ 1);
    cp_async_commit();
    const __nv_bfloat16* kt = kv_s + (size_t)stage * 2 * L::TILE;
    const __nv_bfloat16* vt = kt + L::TILE;

    // S = Q K^T: 16 rows x 64 keys per warp
    float s_acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int n = 0; n < 8; n += 2) {
        unsigned kb[4];  // (keys n*8.., dims 0-7), (same keys, dims 8-15), (keys (n+1)*8.., dims 0-7), (.., dims 8-15)
        const int key = n * 8 + (lane & 7) + ((lane >> 4) << 3);
        const int dim = ks * 16 + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(kb, kt + key * L::STRIDE + dim);
        mma_16816(s_acc[n], qf[ks], kb[0], kb[1]);
        mma_16816(s_acc[n + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // scale; mask where the page meets the diagonal, the window's edge or the tile's end
    const bool needs_mask = (p * MLL_PAGE + MLL_PAGE - 1 > pos0 + warp * 16) || a.window > 0 || rows < 64;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = s_acc[n][i] * a.scale_log2;
        if (needs_mask) {
          const int row = warp * 16 + g + ((i >> 1) << 3);
          const int qpos = pos0 + row;
          const int kpos = p * MLL_PAGE + n * 8 + 2 * t + (i & 1);
          const bool ok = row < rows && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
          v = ok ? v : -INFINITY;
        }
        s_acc[n][i] = v;
      }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) mx = fmaxf(mx, fmaxf(s_acc[n][2 * r], s_acc[n][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float base = m_new > -INFINITY ? m_new : 0.f;  // a fully masked row stays at zero weight
      alpha[r] = exp2f(m_run[r] - base);
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const float p0 = exp2f(s_acc[n][2 * r] - base), p1 = exp2f(s_acc[n][2 * r + 1] - base);
        s_acc[n][2 * r] = p0;
        s_acc[n][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[r] = l_run[r] * alpha[r] + sum;
      m_run[r] = m_new;
    }
#pragma unroll
    for (int n = 0; n < NT_OUT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }
    // O += P V; the accumulator registers of two neighbouring key tiles are one A fragment
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      unsigned pa[4];
      __nv_bfloat162 t0 = __floats2bfloat162_rn(s_acc[2 * ks][0], s_acc[2 * ks][1]);
      __nv_bfloat162 t1 = __floats2bfloat162_rn(s_acc[2 * ks][2], s_acc[2 * ks][3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(s_acc[2 * ks + 1][0], s_acc[2 * ks + 1][1]);
      __nv_bfloat162 t3 = __floats2bfloat162_rn(s_acc[2 * ks + 1][2], s_acc[2 * ks + 1][3]);
      pa[0] = *reinterpret_cast<unsigned*>(&t0);
      pa[1] = *reinterpret_cast<unsigned*>(&t1);
      pa[2] = *reinterpret_cast<unsigned*>(&t2);
      pa[3] = *reinterpret_cast<unsigned*>(&t3);
#pragma unroll
      for (int n = 0; n < NT_OUT; n += 2) {
        unsigned vb[4];  // transposed: (keys 0-7, cols n), (keys 8-15, cols n), (keys 0-7, cols n+1), (keys 8-15, cols n+1)
        const int key = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int col = (n + (lane >> 4)) * 8;
        ldmatrix_x4_trans(vb, vt + key * L::STRIDE + col);
        mma_16816(o[n], pa, vb[0], vb[1]);
        mma_16816(o[n + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= rows) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* dst = a.out + ((size_t)a.seq_qstart[seq] + row0 + row) * a.n_heads * D + (size_t)h * D;
#pragma unroll
    for (int n = 0; n < NT_OUT; ++n)
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + 2 * t) =
          __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

template <int D>
int launch_prefill_mma(const PrefillMmaArgs& a, int n_tiles, cudaStream_t stream) {
  const size_t smem = PrefillMmaSmem<D>::BYTES;
  auto kernel = attn_prefill_mma_kernel<D>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("attention prefill (mma): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  MLL_LAUNCH((kernel), dim3(n_tiles, a.n_heads), 128, smem, stream, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

MLL_API int mll_attn_decode_mma_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && (head_dim == 64 || head_dim == 128 || head_dim == 256);
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
  if (head_dim == 64) return mll::launch_decode_mma<64, 3, false>(a, n_seqs, stream);
  if (head_dim == 128) return mll::launch_decode_mma<128, 3, false>(a, n_seqs, stream);
  return mll::launch_decode_mma<256, 2, false>(a, n_seqs, stream);
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
  if (head_dim == 64) return mll::launch_decode_mma<64, 3, true>(a, n_seqs, stream);
  if (head_dim == 128) return mll::launch_decode_mma<128, 3, true>(a, n_seqs, stream);
  return mll::launch_decode_mma<256, 2, true>(a, n_seqs, stream);
}

MLL_API int mll_attn_prefill_mma_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && (head_dim == 64 || head_dim == 128);
}

// Same contract as mll_attn_prefill (bfloat16, head_dim 64 or 128).
MLL_API int mll_attn_prefill_mma(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                                 const int* seq_ctx, const int* seq_qstart, const int* seq_qlen, const int* tile_seq,
                                 const int* tile_row0, const int* block_table, void* out, int n_tiles, int n_heads,
                                 int n_kv_heads, int head_dim, int max_blocks, int window, float scale,
                                 cudaStream_t stream) {
  MLL_REQUIRE(mll_attn_prefill_mma_supported(MLL_BF16, head_dim), "attention prefill (mma): head_dim %d", head_dim);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention prefill (mma): bad head counts");
  MLL_REQUIRE(n_tiles >= 0 && n_heads <= 65535, "attention prefill (mma): bad tile or head count");
  if (n_tiles == 0) return 0;
  mll::PrefillMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                        seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0, block_table,
                        (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, window, scale * 1.4426950408889634f};
  if (head_dim == 64) return mll::launch_prefill_mma<64>(a, n_tiles, stream);
  return mll::launch_prefill_mma<128>(a, n_tiles, stream);
}
