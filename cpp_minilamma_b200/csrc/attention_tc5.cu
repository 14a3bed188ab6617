// Causal attention of many query tokens over the paged cache on the fifth-generation tensor
// cores: TMA -> shared memory -> tcgen05.mma -> tensor memory (bfloat16, head_dim 64 or 128).
//
// One block of four warps owns 128 query rows of one head; thread i owns row i, which is
// lane i of tensor memory, so the softmax needs no exchange between threads:
//   * thread 0 loads the query tile once and the key and value pages (64 positions each)
//     through a two-stage ring of TMA boxes with the 128-byte swizzle, and issues the MMAs;
//   * S = Q K^T: M = 128 rows, N = 64 keys, both operands K-major, accumulator in one of two
//     64-column buffers of tensor memory, so that the product of the next page runs while
//     the threads work on this one;
//   * each thread reads its row of S (tcgen05.ld), masks it where the page meets the
//     diagonal, the window's edge or the end of the tile, keeps the running maximum and sum
//     in float32 (base 2) and writes P as bfloat16 into a K-major swizzled tile;
//   * O_page = P V: A = P from shared memory, B = the value page as it lies in the cache
//     ([position][dim], that is MN-major), accumulator in 64 or 128 further columns; each
//     thread folds it into its float32 output row: o = o * alpha + O_page.
// Two blocks fit a multiprocessor (112 KB of shared memory, 256 columns of tensor memory
// each): one block's MMAs run under the other's softmax.  Rows of the last page beyond the
// context are zeroed in shared memory (P is zero there, but the cache may hold anything).
//
// Every mbarrier wait is bounded; a wait that runs out raises an error flag (read through
// mll_take_device_error), the block agrees on it at its next barrier, stores nothing, frees its
// tensor memory and exits.  No load uses cluster multicast.
//
// The reference computes attention with one thread block per head and one pass per token
// (src/cuda_attention.cu:19-120); formulas as in src/ops.cc:223-290.
#include <cuda.h>

#include "common.cuh"
#include "tensor_map.h"

__device__ int mll_attn_tc5_error_flag = 0;

namespace mll {

constexpr int A_ROWS = 128;  // query rows per block (the MMA's M)
constexpr unsigned A_SPIN_LIMIT = 4u << 20;

struct PrefillTc5Args {
  const int* seq_slot;
  const int* seq_ctx;
  const int* seq_qstart;
  const int* seq_qlen;
  const int* tile_seq;   // tiles of 64 rows; this kernel works on those that start a multiple of 128
  const int* tile_row0;
  const int* block_table;
  __nv_bfloat16* out;    // [T, Hq * d]
  int n_heads, n_kv_heads, max_blocks, window;
  float scale_log2;
};

__device__ __forceinline__ unsigned a_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void a_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void a_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool a_mbar_test(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool a_mbar_wait(unsigned bar, unsigned parity) {
  for (unsigned spin = 0; spin < A_SPIN_LIMIT; ++spin) {
    if (a_mbar_test(bar, parity)) return true;
    if (spin > 256) __nanosleep(32);
  }
  atomicExch(&mll_attn_tc5_error_flag, 1);
  return false;
}
__device__ __forceinline__ void a_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Shared-memory matrix descriptors, 128-byte swizzle, descriptor version 1.  Rows are 128
// bytes (64 bfloat16), groups of 8 rows are 1024 bytes apart (stride byte offset).
//   K-major (Q, K, P): a row is one M or N index, its 64 elements run along K; the leading
//   byte offset is not used.  Steps of K = 16 advance the address by 32 bytes.
//   MN-major (V): a row is one K index (a position), its 64 elements run along N (the head
//   dimension); the next 64 of N lie one box further (leading byte offset).  Steps of K = 16
//   advance the address by 16 rows.
__device__ __forceinline__ unsigned long long a_desc(unsigned addr, unsigned leading_bytes) {
  return (unsigned long long)((addr >> 4) & 0x3FFFu) | ((unsigned long long)((leading_bytes >> 4) & 0x3FFFu) << 16) |
         ((unsigned long long)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: float32 accumulator, bfloat16 A and B, A K-major.
__host__ __device__ constexpr unsigned a_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void a_umma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                       unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void a_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void a_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void a_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// generic-proxy writes to shared memory become visible to the tensor cores and TMA
__device__ __forceinline__ void a_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 32 consecutive float32 columns of this thread's lane
__device__ __forceinline__ void a_tmem_ld32(unsigned addr, float* v) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(addr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float a_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct PrefillTc5Smem {
  static constexpr int Q_BYTES = A_ROWS * D * 2;       // D / 64 boxes of [128 rows x 128 bytes]
  static constexpr int KV_BYTES = MLL_PAGE * D * 2;    // D / 64 boxes of [64 rows x 128 bytes]
  static constexpr int P_BYTES = A_ROWS * MLL_PAGE * 2;
  static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + 2 * KV_BYTES, P_OFF = V_OFF + 2 * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  // Two blocks per multiprocessor: 2 x (BYTES + 1 KB that the system keeps per block) must stay
  // within 227 KB, which leaves no room for alignment slack: the kernel checks that its dynamic
  // shared memory starts on a 1024-byte boundary (the swizzle's period) and refuses otherwise.
  // Never three blocks: their tensor memory would not fit.
  static constexpr size_t USED = (size_t)BAR_OFF + 128;
  static constexpr size_t BYTES = USED > 80 * 1024 ? USED : 80 * 1024;
  static constexpr int TMEM_COLS = 256;                // S: 2 x 64, O: up to 128
  static constexpr int O_COL = 128;
};

template <int D>
__global__ void __launch_bounds__(A_ROWS, 2)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap, PrefillTc5Args a) {
  using L = PrefillTc5Smem<D>;
  constexpr int DB = D / 64;  // 64-column boxes per row of Q, K or V
  mll::pdl_begin();
  // later tiles of a sequence see more keys: they go first, so that the short ones fill the tail
  const int tile = (gridDim.x - 1 - blockIdx.x) / a.n_heads;   // all heads of a tile are neighbours
  const int row0 = a.tile_row0[tile];
  if (row0 % A_ROWS != 0) return;  // the second half of a 128-row tile

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = smem_raw;
  if (a_smem(base) & 1023u) {  // cannot hold swizzled tiles: report and leave (uniform for the block)
    if (threadIdx.x == 0) atomicExch(&mll_attn_tc5_error_flag, 2);
    return;
  }
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + L::BAR_OFF);
  // barriers: 0 query, 1-2 keys of stage 0/1, 3-4 values, 5-6 S buffers, 7 O
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 8);
  const unsigned q_s = a_smem(base + L::Q_OFF), k_s = a_smem(base + L::K_OFF), v_s = a_smem(base + L::V_OFF);
  const unsigned p_s = a_smem(base + L::P_OFF);
  const unsigned bar_q = a_smem(bars), bar_k = a_smem(bars + 1), bar_v = a_smem(bars + 3), bar_s = a_smem(bars + 5);
  const unsigned bar_o = a_smem(bars + 7);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int seq = a.tile_seq[tile];
  const int h = blockIdx.x % a.n_heads;
  const int kvh = h / (a.n_heads / a.n_kv_heads);
  const int ctx = a.seq_ctx[seq], qlen = a.seq_qlen[seq], qstart = a.seq_qstart[seq];
  const int rows = min(A_ROWS, qlen - row0);
  const int pos0 = ctx - qlen + row0;
  const int* table = a.block_table + (size_t)a.seq_slot[seq] * a.max_blocks;
  const int first_key = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int p_first = first_key / MLL_PAGE, p_last = (pos0 + rows - 1) / MLL_PAGE;
  const int n_pages = p_last - p_first + 1;

  if (tid == 0) {
    for (int i = 0; i < 8; ++i) a_mbar_init(a_smem(bars + i), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(a_smem(tmem_slot)),
                 "r"((unsigned)L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  a_fence_before();
  __syncthreads();
  a_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_row = tmem_base + ((unsigned)(warp * 32) << 16);

  auto load_page = [&](int i, int page) {  // thread 0: keys and values of the block's i-th page into stage i % 2
    const int st = i & 1;
    const int row = (page * a.n_kv_heads + kvh) * MLL_PAGE;
    a_mbar_expect_tx(bar_k + 8 * st, L::KV_BYTES);
    a_mbar_expect_tx(bar_v + 8 * st, L::KV_BYTES);
#pragma unroll
    for (int b = 0; b < DB; ++b) {
      a_tma_load_2d(k_s + st * L::KV_BYTES + b * (MLL_PAGE * 128), &kmap, b * 64, row, bar_k + 8 * st);
      a_tma_load_2d(v_s + st * L::KV_BYTES + b * (MLL_PAGE * 128), &vmap, b * 64, row, bar_v + 8 * st);
    }
  };
  auto issue_s = [&](int i) {  // thread 0: S[i % 2] = Q K_i^T
    constexpr unsigned idesc = a_idesc(A_ROWS, MLL_PAGE, false);
    const unsigned kt = k_s + (i & 1) * L::KV_BYTES;
#pragma unroll
    for (int b = 0; b < DB; ++b)
#pragma unroll
      for (int k = 0; k < 4; ++k)
        a_umma(tmem_base + (i & 1) * MLL_PAGE, a_desc(q_s + b * (A_ROWS * 128) + k * 32, 16),
               a_desc(kt + b * (MLL_PAGE * 128) + k * 32, 16), idesc, (b > 0 || k > 0) ? 1u : 0u);
    a_commit(bar_s + 8 * (i & 1));
  };

  bool ok = true;
  int next_page = 0;
  if (tid == 0) {
    a_mbar_expect_tx(bar_q, L::Q_BYTES);
#pragma unroll
    for (int b = 0; b < DB; ++b) a_tma_load_2d(q_s + b * (A_ROWS * 128), &qmap, h * D + b * 64, qstart + row0, bar_q);
    load_page(0, table[p_first]);
    if (n_pages > 1) load_page(1, table[p_first + 1]);
    if (n_pages > 2) next_page = table[p_first + 2];  // looked up one iteration before its loads are issued
    ok = a_mbar_wait(bar_q, 0) && a_mbar_wait(bar_k, 0);
    a_fence_after();
    if (ok) issue_s(0);
  }

  float o[D];
#pragma unroll
  for (int c = 0; c < D; ++c) o[c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int qpos = pos0 + tid;
  bool failed = false;

  for (int i = 0; i < n_pages; ++i) {
    const int st = i & 1;
    ok = a_mbar_wait(bar_s + 8 * st, (i >> 1) & 1) && ok;
    a_fence_after();
    if (tid == 0 && i + 1 < n_pages) {  // the next page's product runs under this page's softmax
      ok = a_mbar_wait(bar_k + 8 * (st ^ 1), ((i + 1) >> 1) & 1) && ok;
      a_fence_after();
      if (ok) issue_s(i + 1);
    }
    __syncwarp();

    float s[MLL_PAGE];
    a_tmem_ld32(tmem_row + st * MLL_PAGE, s);
    a_tmem_ld32(tmem_row + st * MLL_PAGE + 32, s + 32);
    const int k0 = (p_first + i) * MLL_PAGE;
    const bool needs_mask = (k0 + MLL_PAGE - 1 > pos0) || a.window > 0 || rows < A_ROWS;
    if (needs_mask) {
#pragma unroll
      for (int c = 0; c < MLL_PAGE; ++c) {
        const int kpos = k0 + c;
        const bool keep = tid < rows && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
        s[c] = keep ? s[c] : -INFINITY;
      }
    }
    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains instead of one
#pragma unroll
    for (int c = 0; c < MLL_PAGE; c += 4) {
      mx4[0] = fmaxf(mx4[0], s[c]);
      mx4[1] = fmaxf(mx4[1], s[c + 1]);
      mx4[2] = fmaxf(mx4[2], s[c + 2]);
      mx4[3] = fmaxf(mx4[3], s[c + 3]);
    }
    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
    const float m_new = fmaxf(m_run, mx * a.scale_log2);
    const float shift = m_new > -INFINITY ? m_new : 0.f;  // a fully masked row stays at zero weight
    const float alpha = a_exp2(m_run - shift);
    float sum4[4] = {0.f, 0.f, 0.f, 0.f};
    unsigned packed[MLL_PAGE / 2];
#pragma unroll
    for (int c = 0; c < MLL_PAGE; c += 2) {
      const float p0 = a_exp2(fmaf(s[c], a.scale_log2, -shift)), p1 = a_exp2(fmaf(s[c + 1], a.scale_log2, -shift));
      sum4[(c >> 1) & 3] += p0 + p1;
      __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
      packed[c >> 1] = *reinterpret_cast<unsigned*>(&pair);
    }
    l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
    m_run = m_new;
    {  // row tid of P: eight 16-byte chunks, chunk index xor (row % 8)
      const unsigned row_addr = p_s + (tid >> 3) * 1024 + (tid & 7) * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + ((c ^ (tid & 7)) << 4)),
                     "r"(packed[4 * c]), "r"(packed[4 * c + 1]), "r"(packed[4 * c + 2]), "r"(packed[4 * c + 3])
                     : "memory");
    }
    const int valid = ctx - k0;  // positions of this page that the sequence has
    if (valid < MLL_PAGE) {      // only the sequence's last page: the rest of it may hold anything
      ok = a_mbar_wait(bar_v + 8 * st, (i >> 1) & 1) && ok;
      unsigned char* vt = base + L::V_OFF + st * L::KV_BYTES;
      const int n_chunks = (MLL_PAGE - valid) * 8;  // 16-byte chunks per box
      for (int b = 0; b < DB; ++b)
        for (int c = tid; c < n_chunks; c += A_ROWS)
          *reinterpret_cast<uint4*>(vt + b * (MLL_PAGE * 128) + valid * 128 + c * 16) = make_uint4(0, 0, 0, 0);
    }
    a_fence_async_smem();
    a_fence_before();
    failed = __syncthreads_or(!ok);
    if (failed) break;
    if (tid == 0) {
      ok = a_mbar_wait(bar_v + 8 * st, (i >> 1) & 1);
      a_fence_after();
      if (ok) {
        constexpr unsigned idesc = a_idesc(A_ROWS, D, true);
        const unsigned vt = v_s + st * L::KV_BYTES;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          a_umma(tmem_base + L::O_COL, a_desc(p_s + k * 32, 16), a_desc(vt + k * (16 * 128), MLL_PAGE * 128), idesc,
                 k > 0 ? 1u : 0u);
        a_commit(bar_o);
      }
    }
    __syncwarp();
    ok = a_mbar_wait(bar_o, i & 1) && ok;
    a_fence_after();
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      float t[32];
      a_tmem_ld32(tmem_row + L::O_COL + c, t);
#pragma unroll
      for (int j = 0; j < 32; ++j) o[c + j] = fmaf(o[c + j], alpha, t[j]);
    }
    if (tid == 0 && ok && i + 2 < n_pages) {  // both products of page i are complete
      load_page(i + 2, next_page);
      if (i + 3 < n_pages) next_page = table[p_first + i + 3];
    }
    __syncwarp();
  }
  a_fence_before();
  if (!failed) failed = __syncthreads_or(!ok);

  if (!failed && tid < rows) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* dst = a.out + ((size_t)qstart + row0 + tid) * a.n_heads * D + (size_t)h * D;
#pragma unroll
    for (int c = 0; c < D; c += 8) {
      uint4 w;
      __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) hp[j] = __floats2bfloat162_rn(o[c + 2 * j] * inv, o[c + 2 * j + 1] * inv);
      *reinterpret_cast<uint4*>(dst + c) = w;
    }
  }
  if (failed) {  // loads may still be in flight: give them time before the shared memory is given up
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 0) {
    a_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)L::TMEM_COLS));
  }
}

template <int D>
int launch_prefill_tc5(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                       const PrefillTc5Args& a, int n_tiles, cudaStream_t stream) {
  const size_t smem = PrefillTc5Smem<D>::BYTES;
  auto kernel = attn_prefill_tc5_kernel<D>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("attention prefill (tcgen05): cannot reserve %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(err));
    return (int)err;
  }
  MLL_LAUNCH((kernel), dim3((unsigned)(n_tiles * a.n_heads)), A_ROWS, smem, stream, qmap, kmap, vmap, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

// Used by mll_take_device_error(): this file's flag, read and cleared.
extern "C" int mll_attn_tc5_take_error() {
  int flag = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&flag, mll_attn_tc5_error_flag, sizeof(int)) != cudaSuccess) return -1;
  if (flag) cudaMemcpyToSymbol(mll_attn_tc5_error_flag, &zero, sizeof(int));
  return flag;
}

MLL_API int mll_attn_prefill_tc5_supported(int dtype, int head_dim) {
  return dtype == MLL_BF16 && (head_dim == 64 || head_dim == 128);
}

// Same contract as mll_attn_prefill (bfloat16, head_dim 64 or 128); n_tokens is the number of
// rows of q and out, n_pages the number of pages of k_cache and v_cache.
MLL_API int mll_attn_prefill_tc5(const void* q, const void* k_cache, const void* v_cache, const int* seq_slot,
                                 const int* seq_ctx, const int* seq_qstart, const int* seq_qlen, const int* tile_seq,
                                 const int* tile_row0, const int* block_table, void* out, int n_tokens,
                                 long long n_pages, int n_tiles, int n_heads, int n_kv_heads, int head_dim,
                                 int max_blocks, int window, float scale, cudaStream_t stream) {
  MLL_REQUIRE(mll_attn_prefill_tc5_supported(MLL_BF16, head_dim), "attention prefill (tcgen05): head_dim %d", head_dim);
  MLL_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attention prefill (tcgen05): bad head counts");
  MLL_REQUIRE(n_tiles >= 0 && n_tokens >= 0 && (long long)n_tiles * n_heads < (1ll << 31),
              "attention prefill (tcgen05): bad tile or head count");
  MLL_REQUIRE(n_pages > 0 && n_pages * n_kv_heads * MLL_PAGE < (1ll << 31),
              "attention prefill (tcgen05): %lld pages are more than the row coordinate holds", n_pages);
  MLL_REQUIRE(((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 == 0,
              "attention prefill (tcgen05): operands must be 16-byte aligned");
  if (n_tiles == 0 || n_tokens == 0) return 0;
  CUtensorMap qmap, kmap, vmap;
  if (mll::tensor_map_bf16(q, n_tokens, (long long)n_heads * head_dim, mll::A_ROWS, &qmap) != 0) return -1;
  if (mll::tensor_map_bf16(k_cache, n_pages * n_kv_heads * MLL_PAGE, head_dim, MLL_PAGE, &kmap) != 0) return -1;
  if (mll::tensor_map_bf16(v_cache, n_pages * n_kv_heads * MLL_PAGE, head_dim, MLL_PAGE, &vmap) != 0) return -1;
  mll::PrefillTc5Args a{seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0, block_table,
                        (__nv_bfloat16*)out, n_heads, n_kv_heads, max_blocks, window, scale * 1.4426950408889634f};
  if (head_dim == 64) return mll::launch_prefill_tc5<64>(qmap, kmap, vmap, a, n_tiles, stream);
  return mll::launch_prefill_tc5<128>(qmap, kmap, vmap, a, n_tiles, stream);
}
