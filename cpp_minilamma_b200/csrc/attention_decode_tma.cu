// Decode attention (one query token per sequence) over the paged cache, bfloat16, head_dim 64 or
// 128: pages arrive by TMA, and the four compute warps of a block never meet inside the page loop.
//
// One block per (sequence, kv head [, chunk of 16 query heads], split of the context):
//   * warp 4, one thread: producer.  Per page it loads the keys and the values of the block's kv
//     head ([64 positions x 64 dims] boxes, 128-byte swizzle) into a ring of three stages guarded
//     by full/empty mbarriers; page numbers are looked up one page ahead.
//   * warps 0-3: warp w owns keys 16 w .. 16 w + 15 of EVERY page.  It scores the (up to 16)
//     query heads against its 16 keys (mma.sync m16n8k16, fragments by ldmatrix from the swizzled
//     tile), keeps a running maximum and sum of its own (online softmax, float32), uses the
//     probabilities straight from the accumulator registers as the A operand, and accumulates
//     its own [16 heads x head_dim] output over its 16 value rows.  Nothing is exchanged between
//     warps per page: no block-wide barrier, no probabilities through shared memory; each warp
//     reads only its quarter of a page.
//   * after the last page the four partial results (maximum, sum, output) are merged through
//     shared memory, once.  With 2 to 16 context splits the blocks of a (sequence, kv head, chunk) form a
//     thread-block cluster: after a cluster barrier every split reads its share of all splits' results
//     through distributed shared memory and writes that share of the output.  With more splits (or
//     cluster_merge off) the block writes its partial result to global memory and the block that arrives
//     last merges the splits (attention_decode.cuh).
// The fused variant also rotates q in registers and the step's new key, and writes the new key
// and value row into the cache and into the block's copy of the last page, as the mma.sync
// kernel's fused variant does (attention_mma.cu).  Rows of the last page beyond the context are
// masked (keys) and zeroed in shared memory (values): the cache may hold anything there.
//
// Every mbarrier wait is bounded; a wait that runs out raises an error flag (read through
// mll_take_device_error) and makes the block's later waits return at once; the block then
// stores nothing.  The cluster barriers are reached by every block of a cluster on every path (blocks
// without work and blocks that gave up included).  No load uses cluster multicast.
//
// Arithmetic: that of the general kernel in attention.cu (the reference's src/forward.cc:265-298);
// only the order of the sums differs.
#include <cooperative_groups.h>
#include <cuda.h>

#include "attention_decode.cuh"
#include "tensor_map.h"

namespace cg = cooperative_groups;

__device__ int mll_attn_decode_tma_error_flag = 0;

namespace mll {

constexpr int DT_STAGES = 3;
constexpr int DT_THREADS = 160;  // four compute warps and the producer warp
constexpr long long DT_WAIT_CLOCKS = 2ll << 30;

template <int D>
struct DecodeTmaSmem {
  static constexpr int BOXES = D / 64;
  static constexpr int BOX_BYTES = MLL_PAGE * 128;      // [64 rows x 128 bytes]
  static constexpr int HALF = BOXES * BOX_BYTES;        // one page's keys (or values)
  static constexpr int STAGE = 2 * HALF;
  static constexpr int RING = DT_STAGES * STAGE;        // 96 KB for head_dim 128: two blocks per multiprocessor
  static constexpr int MERGE_FLOATS = 4 * (16 * D + 32);  // the warps' partial results, over the ring once it is drained
  static_assert(MERGE_FLOATS * 4 + (16 * D + 32) * 4 <= RING, "the merge buffers must fit into the ring");
  static constexpr int BAR_OFF = RING;                  // full[S], empty[S]
  static constexpr size_t BYTES = (size_t)RING + 64;
};

__device__ __forceinline__ unsigned dt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
// One try: the hardware parks the thread until the phase completes or a time limit of its own runs out (a spin
// on test_wait would spend the multiprocessor's issue slots, which the other block's warps can use).
__device__ __forceinline__ bool dt_mbar_try(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void dt_mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
  if (*abort_flag) return;
  if (dt_mbar_try(bar, parity)) return;
  const long long began = clock64();
  while (clock64() - began < DT_WAIT_CLOCKS) {  // about a second: a load that has not come by then never will
    if (dt_mbar_try(bar, parity) || *abort_flag) return;
  }
  *abort_flag = 1;
  atomicExch(&mll_attn_decode_tma_error_flag, 1);
}
__device__ __forceinline__ void dt_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// Byte offset of 16-byte chunk `chunk` (8 bfloat16) of row `row` in a K or V half: the half is
// D / 64 boxes of [64 rows x 128 bytes], and the 128-byte swizzle xors the chunk index within
// the box with the row's low three bits.
__device__ __forceinline__ unsigned dt_chunk_offset(int row, int chunk) {
  return (unsigned)((chunk >> 3) * (MLL_PAGE * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
__device__ __forceinline__ float dt_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void dt_ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dt_ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// The step's new key (rotated) and value of kv head `kvh` of sequence b, one pair of each per thread (tid < D / 2).
template <int D>
__device__ __forceinline__ void dt_fetch_new_row(const DecodeMmaArgs& a, int b, int kvh, int ctx, int tid,
                                                 __nv_bfloat16& new_k0, __nv_bfloat16& new_k1, unsigned& new_v) {
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

// The query fragments (A operand of the score product) of heads h0 .. h0 + ng - 1 of sequence b: rows = heads,
// zero beyond ng; the fused variant rotates them (the token's position is ctx - 1).
template <int D, bool FUSED>
__device__ __forceinline__ void dt_load_query(const DecodeMmaArgs& a, int b, int h0, int ng, int ctx, int g, int t,
                                              unsigned (&qf)[D / 16][4]) {
  constexpr int KSTEPS = D / 16;
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

// One page (64 keys, in the ring stage at `stage`) for one compute warp: the warp's 16 keys against the (up to
// 16) query heads, its running maximum and sum, and its [16 heads x head_dim] output.  p: the page's number in
// the sequence.  On the sequence's last page the fused variant first puts the step's new key and value into the
// stage and into the cache (the block that owns that page; the four compute warps meet once for it), and rows
// beyond the context are masked (keys) and zeroed (values).
template <int D, bool FUSED>
__device__ __forceinline__ void dt_page_step(const DecodeMmaArgs& a, unsigned char* stage, int p, int ctx, int first_key,
                                             int pages_total, bool owns_new_row, const int* table, int kvh,
                                             __nv_bfloat16 new_k0, __nv_bfloat16 new_k1, unsigned new_v,
                                             const unsigned (&qf)[D / 16][4], float (&o)[D / 8][4], float (&m_run)[2],
                                             float (&l_run)[2]) {
  constexpr int KSTEPS = D / 16, NT = D / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t = lane & 3;
  const unsigned kt = dt_smem(stage), vt = kt + DecodeTmaSmem<D>::HALF;
  if (p == pages_total - 1) {
    if (FUSED && owns_new_row) {
      // the step's token lies in this page: its key (rotated) and value replace whatever the cache held
      const int row = (ctx - 1) % MLL_PAGE;
      if (tid < D / 2) {
        const size_t cache_row = (((size_t)table[p] * a.n_kv_heads + kvh) * MLL_PAGE + row) * D;
        const int e0 = a.interleaved ? 2 * tid : tid, e1 = a.interleaved ? 2 * tid + 1 : tid + D / 2;
        unsigned char* k_half = stage;
        unsigned char* v_half = k_half + DecodeTmaSmem<D>::HALF;
        *reinterpret_cast<__nv_bfloat16*>(k_half + dt_chunk_offset(row, e0 >> 3) + (e0 & 7) * 2) = new_k0;
        *reinterpret_cast<__nv_bfloat16*>(k_half + dt_chunk_offset(row, e1 >> 3) + (e1 & 7) * 2) = new_k1;
        a.k_write[cache_row + e0] = new_k0;
        a.k_write[cache_row + e1] = new_k1;
        *reinterpret_cast<unsigned*>(v_half + dt_chunk_offset(row, (2 * tid) >> 3) + ((2 * tid) & 7) * 2) = new_v;
        *reinterpret_cast<unsigned*>(a.v_write + cache_row + 2 * tid) = new_v;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the compute warps only; once per block
    }
    const int valid = ctx - p * MLL_PAGE;  // positions of this page that the sequence has
    if (valid < MLL_PAGE) {                // the rest of the page may hold anything: zero this warp's value rows
      unsigned char* v_half = stage + DecodeTmaSmem<D>::HALF;
      for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
        const int row = warp * 16 + idx / (D / 8), ch = idx % (D / 8);
        if (row >= valid) *reinterpret_cast<uint4*>(v_half + dt_chunk_offset(row, ch)) = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
    }
  }

  // Where this lane's ldmatrix rows lie in the swizzled tiles.  Chunk c of row r is stored at chunk c ^ (r & 7); the
  // chunk a lane reads is an even number known at compile time plus one bit of the lane, so the lane's part is
  // worked out once and the rest is one XOR with a constant (the tiles are 1,024-byte aligned).
  const int k_row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
  const unsigned k_lane = kt + k_row * 128 + (((((lane >> 3) & 1) ^ k_row) & 7) << 4);
  const int v_row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
  const unsigned v_lane = vt + v_row * 128 + ((((lane >> 4) ^ v_row) & 7) << 4);

  // scores of the 16 heads against this warp's 16 keys: two n-tiles of 8 keys; where registers allow (head_dim 64)
  // even and odd k-steps go to accumulators of their own, which halves the chains of dependent MMAs
  float s_acc[2][4], s_odd[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) s_acc[n][i] = s_odd[n][i] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    // matrices: (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
    unsigned kb[4];
    dt_ldmatrix_x4(kb, (k_lane ^ (unsigned)(((ks * 2) & 7) << 4)) + (ks >> 2) * DecodeTmaSmem<D>::BOX_BYTES);
    if (D == 64 && (ks & 1)) {
      mma_16816(s_odd[0], qf[ks], kb[0], kb[1]);
      mma_16816(s_odd[1], qf[ks], kb[2], kb[3]);
    } else {
      mma_16816(s_acc[0], qf[ks], kb[0], kb[1]);
      mma_16816(s_acc[1], qf[ks], kb[2], kb[3]);
    }
  }
  // scale, mask (only a sequence's first and last page have keys to mask), the warp's row maxima
  const bool edge = (p + 1) * MLL_PAGE > ctx || p * MLL_PAGE < first_key;
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int n = 0; n < 2; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = (s_acc[n][i] + s_odd[n][i]) * a.scale;
      if (edge) {
        const int kpos = p * MLL_PAGE + warp * 16 + n * 8 + 2 * t + (i & 1);
        if (!(kpos < ctx && kpos >= first_key)) v = -INFINITY;
      }
      s_acc[n][i] = v;
      tile_max[i >> 1] = fmaxf(tile_max[i >> 1], v);
    }
  // exp(x - m) = 2^(x log2(e) - m log2(e)): one FMA and one ex2 per score.  A masked score is -inf and gives 0;
  // while a row has seen no key at all its maximum is -inf, and 0 stands in for it so that nothing becomes NaN.
  constexpr float LOG2E = 1.4426950408889634f;
  float alpha[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
    tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
    const float m_new = fmaxf(m_run[r], tile_max[r]);
    const float base = m_new > -INFINITY ? m_new * LOG2E : 0.f;
    alpha[r] = m_new > -INFINITY ? dt_exp2((m_run[r] - m_new) * LOG2E) : 1.f;  // exactly 1 while the maximum stands
    float sum = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float pv = dt_exp2(fmaf(s_acc[n][2 * r + i], LOG2E, -base));
        s_acc[n][2 * r + i] = pv;
        sum += pv;
      }
    l_run[r] = l_run[r] * alpha[r] + sum;  // this thread's share of the row; the quad is summed after the loop
    m_run[r] = m_new;
  }
  // the probabilities as the A fragment of a 16-key step: (row g, keys 2t..), (row g + 8, keys 2t..),
  // (row g, keys 8 + 2t..), (row g + 8, keys 8 + 2t..)
  unsigned pa[4];
  pa[0] = pack_bf162(s_acc[0][0], s_acc[0][1]);
  pa[1] = pack_bf162(s_acc[0][2], s_acc[0][3]);
  pa[2] = pack_bf162(s_acc[1][0], s_acc[1][1]);
  pa[3] = pack_bf162(s_acc[1][2], s_acc[1][3]);
  // out = alpha * out + P[16 x 16] . V[this warp's 16 keys x head_dim]; after a sequence's first pages the maxima
  // rarely move, and a warp none of whose rows moved leaves its output as it is
  if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }
  }
#pragma unroll
  for (int n = 0; n < NT; n += 2) {
    // transposed 8x8 tiles of V: (keys 0-7, cols n), (keys 8-15, cols n), (keys 0-7, cols n+1), (keys 8-15, cols n+1)
    unsigned vb[4];
    dt_ldmatrix_x4_trans(vb, (v_lane ^ (unsigned)((n & 7) << 4)) + (n >> 3) * DecodeTmaSmem<D>::BOX_BYTES);
    mma_16816(o[n], pa, vb[0], vb[1]);
    mma_16816(o[n + 1], pa, vb[2], vb[3]);
  }
}

// grid (Hk * head_chunks, B, n_splits); 160 threads.
template <int D, bool FUSED, bool CLUSTER>
__global__ void __launch_bounds__(DT_THREADS, 2)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                       DecodeMmaArgs a) {
  using L = DecodeTmaSmem<D>;
  constexpr int KSTEPS = D / 16;  // k-steps of the score product
  constexpr int NT = D / 8;       // output n-tiles (8 columns) per warp: every warp holds all columns
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem_raw + L::BAR_OFF);
  // no static shared memory in this kernel: it would sit before the ring and could move it off its boundary
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * DT_STAGES);
  const unsigned ring = dt_smem(smem_raw);
  const unsigned full = dt_smem(bars), empty = dt_smem(bars + DT_STAGES);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.n_heads / a.n_kv_heads;
  const int chunks = (group + 15) / 16;
  // sequences are the slower grid index, so blocks start in the order of `seq_order` (longest contexts first);
  // with a work list the slower index runs over its (sequence, split) pairs instead
  const int entry = !CLUSTER && a.work != nullptr ? a.work[blockIdx.y] : 0;
  if (entry < 0) return;  // an unused place of the list (the same for the whole block)
  const bool listed = !CLUSTER && a.work != nullptr;
  const int b = listed ? (entry & 0xffff) : a.seq_order != nullptr ? a.seq_order[blockIdx.y] : blockIdx.y;
  const int item = blockIdx.x;  // kv head x head chunk
  const int kvh = item / chunks, chunk = item % chunks;
  const int split = listed ? ((entry >> 16) & 0xff) : blockIdx.z;
  const int ng = min(16, group - chunk * 16);
  const int h0 = kvh * group + chunk * 16;

  const int ctx = a.seq_ctx[b];
  const int first_key = a.window > 0 ? max(0, ctx - a.window) : 0;
  const int pages_total = (ctx + MLL_PAGE - 1) / MLL_PAGE;
  const int first_page = first_key / MLL_PAGE;
  // a sequence uses as many of the offered splits as its own length pays for (attention_decode.cuh)
  // ... or as many as its entry of the work list says
  const int n_eff = listed ? min(entry >> 24, max(1, pages_total - first_page))
                           : decode_splits_for(pages_total - first_page, a.n_splits);
  const bool misplaced = (ring & 1023u) != 0;  // cannot hold swizzled tiles: report, and do no work (uniform for the block)
  if (misplaced && tid == 0) atomicExch(&mll_attn_decode_tma_error_flag, 2);
  // splits beyond the sequence's own count have no work; in a cluster they still meet the others at its barriers
  const bool active = split < n_eff && !misplaced;
  if (!CLUSTER && !active) return;
  // where the block's result lies once its four warps are merged (over the drained ring)
  float* part = reinterpret_cast<float*>(smem_raw);       // [4 warps][16 rows][D], then [4][16] maxima, [4][16] sums
  float* part_m = part + 4 * 16 * D;
  float* part_l = part_m + 4 * 16;
  float* merged = part_l + 4 * 16;                        // [16][D], then [16] maxima, [16] sums
  float* merged_m = merged + 16 * D;
  float* merged_l = merged_m + 16;
  bool failed = true;
  if (active) {
    const int per_split = (pages_total - first_page + n_eff - 1) / n_eff;
    const int p_begin = first_page + split * per_split;
    const int p_end = min(pages_total, p_begin + per_split);
    const int n_pages = max(0, p_end - p_begin);
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_blocks;

    if (tid == 0) {
      for (int s = 0; s < DT_STAGES; ++s) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full + 8 * s), "r"(1u));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty + 8 * s), "r"(4u));  // one arrival per compute warp
      }
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float o[NT][4];
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows g and g + 8, this warp's keys only

    if (warp == 4) {
      // ---- producer ---------------------------------------------------------------------------- //
      if (lane == 0 && n_pages > 0) {
        int page = table[p_begin];
        for (int it = 0; it < n_pages; ++it) {
          const int st = it % DT_STAGES;
          dt_mbar_wait(empty + 8 * st, ((it / DT_STAGES) & 1) ^ 1, abort_flag);  // the stage's previous use (none in the first round)
          if (*abort_flag) break;
          const int row = (page * a.n_kv_heads + kvh) * MLL_PAGE;
          if (it + 1 < n_pages) page = table[p_begin + it + 1];  // looked up while this page's loads fly
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full + 8 * st), "r"((unsigned)L::STAGE)
                       : "memory");
          const unsigned dst = ring + st * L::STAGE;
#pragma unroll
          for (int bx = 0; bx < L::BOXES; ++bx) {
            dt_tma_load_2d(dst + bx * L::BOX_BYTES, &kmap, bx * 64, row, full + 8 * st);
            dt_tma_load_2d(dst + L::HALF + bx * L::BOX_BYTES, &vmap, bx * 64, row, full + 8 * st);
          }
        }
      }
    } else {
      // ---- compute warps ----------------------------------------------------------------------- //
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

      // FUSED: the block whose pages include the sequence's last one fetches the new key pair and
      // value pair of its kv head now (one pair per thread), long before the page comes up
      const bool owns_new_row = FUSED && a.k_write != nullptr && ctx > 0 && p_begin <= pages_total - 1 &&
                                pages_total - 1 < p_end;
      __nv_bfloat16 new_k0 = __float2bfloat16_rn(0.f), new_k1 = new_k0;
      unsigned new_v = 0;
      if (owns_new_row && tid < D / 2) dt_fetch_new_row<D>(a, b, kvh, ctx, tid, new_k0, new_k1, new_v);

      unsigned qf[KSTEPS][4];
      dt_load_query<D, FUSED>(a, b, h0, ng, ctx, g, t, qf);

      for (int it = 0; it < n_pages; ++it) {
        const int p = p_begin + it;
        const int st = it % DT_STAGES;
        dt_mbar_wait(full + 8 * st, (it / DT_STAGES) & 1, abort_flag);
        dt_page_step<D, FUSED>(a, smem_raw + st * L::STAGE, p, ctx, first_key, pages_total, owns_new_row, table, kvh,
                               new_k0, new_k1, new_v, qf, o, m_run, l_run);
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty + 8 * st) : "memory");
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      }
    }

    // ---- the four warps' partial results, merged through the drained ring --------------------- //
    __syncthreads();  // every page has been consumed: the ring is free
    if (warp < 4) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int col = n * 8 + 2 * t;
        *reinterpret_cast<float2*>(part + ((size_t)warp * 16 + g) * D + col) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(part + ((size_t)warp * 16 + g + 8) * D + col) = make_float2(o[n][2], o[n][3]);
      }
      if (t == 0) {
        part_m[warp * 16 + g] = m_run[0];
        part_m[warp * 16 + g + 8] = m_run[1];
        part_l[warp * 16 + g] = l_run[0];
        part_l[warp * 16 + g + 8] = l_run[1];
      }
    }
    __syncthreads();
    failed = *abort_flag != 0;
    for (int idx = tid; idx < ng * D; idx += DT_THREADS) {
      const int row = idx / D, col = idx % D;
      const float m0 = part_m[row], m1 = part_m[16 + row], m2 = part_m[32 + row], m3 = part_m[48 + row];
      const float m = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      const float w0 = m0 > -INFINITY ? __expf(m0 - m) : 0.f, w1 = m1 > -INFINITY ? __expf(m1 - m) : 0.f;
      const float w2 = m2 > -INFINITY ? __expf(m2 - m) : 0.f, w3 = m3 > -INFINITY ? __expf(m3 - m) : 0.f;
      const float l = (part_l[row] * w0 + part_l[16 + row] * w1) + (part_l[32 + row] * w2 + part_l[48 + row] * w3);
      const float v = (part[(size_t)row * D + col] * w0 + part[((size_t)16 + row) * D + col] * w1) +
                      (part[((size_t)32 + row) * D + col] * w2 + part[((size_t)48 + row) * D + col] * w3);
      merged[(size_t)row * D + col] = v;
      if (col == 0) {
        merged_m[row] = m;
        merged_l[row] = l;
      }
    }
    __syncthreads();
  }
  if (CLUSTER) {
    // The splits of one (sequence, kv head, head chunk) are the blocks of one cluster: their results meet in
    // distributed shared memory instead of global memory, an arrival counter and a second pass by the last
    // block (about 3 us less on a 10-16 us launch).  Every block of the cluster comes here, with or without work.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every block's merged result is in its shared memory
    if (active && !failed) {
      const int share = (ng * D + n_eff - 1) / n_eff;  // split number `split` writes outputs [split * share, + share)
      for (int idx = split * share + tid; idx < min(ng * D, (split + 1) * share); idx += DT_THREADS) {
        const int row = idx / D, col = idx % D;
        float m = -INFINITY;
        for (int sp = 0; sp < n_eff; ++sp) m = fmaxf(m, *cluster.map_shared_rank(merged_m + row, sp));
        float l = 0.f, v = 0.f;
        for (int sp = 0; sp < n_eff; ++sp) {  // in split order: the same sum on every run
          const float ms = *cluster.map_shared_rank(merged_m + row, sp);
          const float w = ms > -INFINITY ? __expf(ms - m) : 0.f;
          l = fmaf(*cluster.map_shared_rank(merged_l + row, sp), w, l);
          v = fmaf(*cluster.map_shared_rank(merged + (size_t)row * D + col, sp), w, v);
        }
        a.out[((size_t)b * a.n_heads + h0 + row) * D + col] = __float2bfloat16_rn(l > 0.f ? v / l : 0.f);
      }
    }
    cluster.sync();  // nobody leaves while another block may still read its shared memory
    return;
  }
  if (failed) return;
  for (int idx = tid; idx < ng * D; idx += DT_THREADS) {
    const int row = idx / D, col = idx % D;
    const size_t head = (size_t)b * a.n_heads + h0 + row;
    if (n_eff == 1) {
      const float l = merged_l[row];
      a.out[head * D + col] = __float2bfloat16_rn(l > 0.f ? merged[(size_t)row * D + col] / l : 0.f);
    } else {
      a.part_o[(head * a.n_splits + split) * D + col] = merged[(size_t)row * D + col];
      if (col == 0) {
        float* ml = a.part_ml + (head * a.n_splits + split) * 2;
        ml[0] = merged_m[row];
        ml[1] = merged_l[row];
      }
    }
  }
  if (n_eff == 1) return;
  merge_decode_splits<D, DT_THREADS>(a, b, item, gridDim.x, h0, ng, n_eff, merged_l + 16);
}

// cluster: the splits of a group are the blocks of one thread-block cluster and merge through distributed
// shared memory (n_splits 2 .. 16); otherwise through global memory and arrival counters.
template <int D, bool FUSED, bool CLUSTER>
int launch_decode_tma_as(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeMmaArgs& a, int n_seqs,
                         cudaStream_t stream) {
  const size_t smem = DecodeTmaSmem<D>::BYTES;
  auto kernel = attn_decode_tma_kernel<D, FUSED, CLUSTER>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err == cudaSuccess && CLUSTER && a.n_splits > 8)
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (err != cudaSuccess) {
    mll_set_error("attention decode (tma): cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  const int group = a.n_heads / a.n_kv_heads;
  cudaLaunchConfig_t config = {};
  // with a work list: one block per (item, pair); n_seqs is then the length of the list
  config.gridDim = dim3(a.n_kv_heads * ((group + 15) / 16), n_seqs, !CLUSTER && a.work != nullptr ? 1 : a.n_splits);
  config.blockDim = dim3(DT_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  if (CLUSTER) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = a.n_splits;
    config.attrs = attr;
    config.numAttrs = 1;
  }
  err = cudaLaunchKernelEx(&config, kernel, kmap, vmap, a);
  if (err != cudaSuccess) {
    mll_set_error("attention decode (tma): launch failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  return 0;
}

// How many clusters of `n_splits` of these blocks the device holds at once (0: such a cluster cannot be
// launched); asked once per kernel and size.
template <int D, bool FUSED>
int decode_clusters_resident(int n_splits) {
  static int known[17] = {0};  // 0 unknown, -1 none, else the count
  if (n_splits < 2 || n_splits > 16) return 0;
  if (known[n_splits] == 0) {
    auto kernel = attn_decode_tma_kernel<D, FUSED, true>;
    const size_t smem = DecodeTmaSmem<D>::BYTES;
    int clusters = 0;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err == cudaSuccess && n_splits > 8)
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err == cudaSuccess) {
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(1, 1, n_splits);
      config.blockDim = dim3(DT_THREADS);
      config.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = n_splits;
      config.attrs = attr;
      config.numAttrs = 1;
      err = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
    }
    if (err != cudaSuccess) cudaGetLastError();  // not an error of the caller's: the other merge is used
    known[n_splits] = (err == cudaSuccess && clusters >= 1) ? clusters : -1;
  }
  return max(known[n_splits], 0);
}

template <int D, bool FUSED>
int launch_decode_tma(const CUtensorMap& kmap, const CUtensorMap& vmap, const DecodeMmaArgs& a, int n_seqs,
                      int cluster_merge, cudaStream_t stream) {
  if (cluster_merge && a.work == nullptr && decode_clusters_resident<D, FUSED>(a.n_splits) >= 1)
    return launch_decode_tma_as<D, FUSED, true>(kmap, vmap, a, n_seqs, stream);
  return launch_decode_tma_as<D, FUSED, false>(kmap, vmap, a, n_seqs, stream);
}

}  // namespace mll

// The device address of this file's error flag (nullptr if it cannot be had); device_error.cu reads,
// clears and hands it to the sampling kernels.
extern "C" int* mll_attn_decode_tma_error_address() {
  int* address = nullptr;
  if (cudaGetSymbolAddress((void**)&address, mll_attn_decode_tma_error_flag) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return address;
}

MLL_API int mll_attn_decode_tma_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && (head_dim == 64 || head_dim == 128);
}

// Clusters of `n_splits` blocks of the (fused) kernel for this head size that the device holds at once; 0 if
// such a cluster cannot be launched or the head size is not taken.
MLL_API int mll_attn_decode_tma_resident_clusters(int head_dim, int fused, int n_splits) {
  if (head_dim == 64)
    return fused ? mll::decode_clusters_resident<64, true>(n_splits) : mll::decode_clusters_resident<64, false>(n_splits);
  if (head_dim == 128)
    return fused ? mll::decode_clusters_resident<128, true>(n_splits) : mll::decode_clusters_resident<128, false>(n_splits);
  return 0;
}

// One query token per sequence over the paged cache (bfloat16, head_dim 64 or 128).  Either q [B, Hq d]
// (already rotated) or, for the fused variant, qkv [B, qkv_ld] with the rotary tables as in
// mll_attn_decode_mma_fused (then q is ignored).  n_pages: pages of k_cache and v_cache.  With
// n_splits > 1, scratch and counters (int32, one per (sequence, kv head x head chunk), zero
// before the first launch; left zero) are required: the last block of a group merges the splits.
// cluster_merge != 0: with 2 to 16 splits the blocks of a group form a thread-block cluster and merge
// through distributed shared memory instead (scratch and counters stay untouched).  seq_order: optional
// permutation of 0 .. n_seqs - 1; the blocks of sequence seq_order[0] start first (give the longest first).
// work: optional list of work_pairs (sequence, split) entries (attention_decode.cuh) that replaces the grid over
// sequences and splits, so that sequences of one launch have different numbers of splits; n_splits is then the
// most any sequence has, and no cluster is formed.
MLL_API int mll_attn_decode_tma(const void* q, const void* qkv, int qkv_ld, const float* cos_table,
                                const float* sin_table, int interleaved, int write_kv, void* k_cache, void* v_cache,
                                long long n_pages, const int* seq_slot, const int* seq_ctx, const int* block_table,
                                float* scratch, void* out, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                int max_blocks, int n_splits, int window, float scale, int* counters,
                                int cluster_merge, const int* seq_order, const int* work, int work_pairs,
                                cudaStream_t stream) {
  MLL_REQUIRE(mll_attn_decode_tma_supported(MLL_BF16, head_dim), "attention decode (tma): head_dim %d", head_dim);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention decode (tma): bad head counts");
  MLL_REQUIRE(n_seqs >= 0 && n_splits >= 1 && n_splits <= 65535, "attention decode (tma): bad batch or split count");
  MLL_REQUIRE(work == nullptr || (work_pairs >= n_seqs && work_pairs <= 65535 && n_seqs <= 65535 && n_splits <= 127),
              "attention decode (tma): a work list of %d pairs for %d sequences and up to %d splits", work_pairs, n_seqs, n_splits);
  MLL_REQUIRE(n_splits == 1 || (scratch != nullptr && counters != nullptr),
              "attention decode (tma): %d splits need scratch memory and arrival counters", n_splits);
  MLL_REQUIRE(q != nullptr || qkv != nullptr, "attention decode (tma): neither q nor qkv");
  MLL_REQUIRE(qkv == nullptr || (qkv_ld >= (n_heads + (write_kv ? 2 * n_kv_heads : 0)) * head_dim && qkv_ld % 2 == 0),
              "attention decode (tma): row stride %d shorter than the q/k/v columns", qkv_ld);
  MLL_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention decode (tma): one rotary table is missing");
  MLL_REQUIRE(n_pages > 0 && n_pages * n_kv_heads * MLL_PAGE < (1ll << 31),
              "attention decode (tma): %lld pages are more than the row coordinate holds", n_pages);
  MLL_REQUIRE(((uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0, "attention decode (tma): caches must be 16-byte aligned");
  if (n_seqs == 0) return 0;
  CUtensorMap kmap, vmap;
  if (mll::tensor_map_bf16(k_cache, n_pages * n_kv_heads * MLL_PAGE, head_dim, MLL_PAGE, &kmap) != 0) return -1;
  if (mll::tensor_map_bf16(v_cache, n_pages * n_kv_heads * MLL_PAGE, head_dim, MLL_PAGE, &vmap) != 0) return -1;
  const bool fused = qkv != nullptr;
  mll::DecodeMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                       seq_slot, seq_ctx, block_table, scratch,
                       scratch ? scratch + (size_t)n_seqs * n_heads * n_splits * head_dim : nullptr,
                       (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, n_splits, window, scale, counters,
                       (const __nv_bfloat16*)qkv, fused ? cos_table : nullptr, fused ? sin_table : nullptr,
                       fused && write_kv ? (__nv_bfloat16*)k_cache : nullptr,
                       fused && write_kv ? (__nv_bfloat16*)v_cache : nullptr, qkv_ld, interleaved, seq_order, work};
  const int rows = work != nullptr ? work_pairs : n_seqs;  // the grid's second index
  if (head_dim == 64)
    return fused ? mll::launch_decode_tma<64, true>(kmap, vmap, a, rows, cluster_merge, stream)
                 : mll::launch_decode_tma<64, false>(kmap, vmap, a, rows, cluster_merge, stream);
  return fused ? mll::launch_decode_tma<128, true>(kmap, vmap, a, rows, cluster_merge, stream)
               : mll::launch_decode_tma<128, false>(kmap, vmap, a, rows, cluster_merge, stream);
}
