// Prefill attention on tensor cores by mma.sync (bfloat16, head sizes 16 .. 256 in steps of 16): the path for the
// head sizes that the tcgen05 kernel (attention_tc5.cu: 64 and 128) does not take.
#include "attention_decode.cuh"
#include "common.cuh"

namespace mll {

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
__global__ void __launch_bounds__(128, (D <= 128 ? 3 : D <= 192 ? 2 : 1))
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

MLL_API int mll_attn_prefill_mma_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && head_dim >= 16 && head_dim <= 256 && head_dim % 16 == 0;
}

// Same contract as mll_attn_prefill (bfloat16, head sizes 16 .. 256 in steps of 16).
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
  switch (head_dim) {
    case 16: return mll::launch_prefill_mma<16>(a, n_tiles, stream);
    case 32: return mll::launch_prefill_mma<32>(a, n_tiles, stream);
    case 48: return mll::launch_prefill_mma<48>(a, n_tiles, stream);
    case 64: return mll::launch_prefill_mma<64>(a, n_tiles, stream);
    case 80: return mll::launch_prefill_mma<80>(a, n_tiles, stream);
    case 96: return mll::launch_prefill_mma<96>(a, n_tiles, stream);
    case 112: return mll::launch_prefill_mma<112>(a, n_tiles, stream);
    case 128: return mll::launch_prefill_mma<128>(a, n_tiles, stream);
    case 144: return mll::launch_prefill_mma<144>(a, n_tiles, stream);
    case 160: return mll::launch_prefill_mma<160>(a, n_tiles, stream);
    case 176: return mll::launch_prefill_mma<176>(a, n_tiles, stream);
    case 192: return mll::launch_prefill_mma<192>(a, n_tiles, stream);
    case 208: return mll::launch_prefill_mma<208>(a, n_tiles, stream);
    case 224: return mll::launch_prefill_mma<224>(a, n_tiles, stream);
    case 240: return mll::launch_prefill_mma<240>(a, n_tiles, stream);
    case 256: return mll::launch_prefill_mma<256>(a, n_tiles, stream);
    default: return -1;  // not reached: checked above
  }
}
