// Decode attention on tensor cores (bfloat16, head sizes 16 .. 256 in steps of 16): the kernel template.
// attention_mma.cu instantiates the head sizes that are multiples of 32, attention_mma_odd.cu the others
// (two files so that they compile side by side).
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
// kernel) is the same as the general kernel's, which remains the path for float32.
#pragma once

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
  constexpr int NT_ALL = D / 8;                // value n-tiles (8 columns) of a head
  constexpr int NT_OUT = (NT_ALL + 3) / 4;     // ... per warp: warp w owns tiles w NT_OUT .. (w + 1) NT_OUT - 1 that exist
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
      } else {
        // pairs (i, i + d/2).  The head's lower half is KSTEPS groups of 8 columns; group grp lies in registers
        // [2j], [2j + 1] of k-step ks with grp = 2 ks + j, its partner is group grp + KSTEPS.
#pragma unroll
        for (int grp = 0; grp < KSTEPS; ++grp) {
          const int ks = grp >> 1, j = grp & 1, ks2 = (grp + KSTEPS) >> 1, j2 = (grp + KSTEPS) & 1;
          const int i0 = grp * 8 + 2 * t;
          const float c0 = cs[i0], s0 = sn[i0], c1 = cs[i0 + 1], s1 = sn[i0 + 1];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float2 lo = unpack_bf162(qf[ks][2 * j + r]), hi = unpack_bf162(qf[ks2][2 * j2 + r]);
            qf[ks][2 * j + r] = pack_bf162(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
            qf[ks2][2 * j2 + r] = pack_bf162(lo.x * s0 + hi.x * c0, lo.y * s1 + hi.y * c1);
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
        const int tile = warp * NT_OUT + n + (lane >> 4);  // a tile past the head's columns is read as tile 0 and not used
        ldmatrix_x4_trans(vb, vt + key * L::STRIDE + (tile < NT_ALL ? tile : 0) * 8);
        if (warp * NT_OUT + n < NT_ALL) mma_16816(o[n], pa, vb[0], vb[1]);
        if (n + 1 < NT_OUT && warp * NT_OUT + n + 1 < NT_ALL) mma_16816(o[n + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

  // rows g and g + 8 of the tile are heads h0 + g and h0 + g + 8; this thread holds columns
  // (warp NT_OUT + n) * 8 + 2 t + {0, 1}
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (row >= ng) continue;
    const size_t head = (size_t)b * a.n_heads + h0 + row;
    if (n_eff == 1) {
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
      for (int n = 0; n < NT_OUT; ++n) {
        const int col = (warp * NT_OUT + n) * 8 + 2 * t;
        if (col < D)
          *reinterpret_cast<__nv_bfloat162*>(a.out + head * D + col) =
              __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
      }
    } else {
      float* po = a.part_o + (head * a.n_splits + split) * D;
#pragma unroll
      for (int n = 0; n < NT_OUT; ++n) {
        const int col = (warp * NT_OUT + n) * 8 + 2 * t;
        if (col < D) *reinterpret_cast<float2*>(po + col) = make_float2(o[n][2 * r], o[n][2 * r + 1]);
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

// Ring stages by head size: three while two blocks still fit a multiprocessor.
template <int D>
constexpr int decode_mma_stages() { return D <= 128 ? 3 : 2; }

template <int D>
int launch_decode_mma_sized(const DecodeMmaArgs& a, int n_seqs, bool fused, cudaStream_t stream) {
  return fused ? launch_decode_mma<D, decode_mma_stages<D>(), true>(a, n_seqs, stream)
               : launch_decode_mma<D, decode_mma_stages<D>(), false>(a, n_seqs, stream);
}

// head sizes 16, 48, 80, ..., 240 (attention_mma_odd.cu)
int launch_decode_mma_odd(const DecodeMmaArgs& a, int head_dim, int n_seqs, bool fused, cudaStream_t stream);

}  // namespace mll
