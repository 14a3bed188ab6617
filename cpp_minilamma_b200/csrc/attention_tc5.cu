// Causal attention of many query tokens over the paged cache on the fifth-generation tensor
// cores: TMA -> shared memory -> tcgen05.mma -> tensor memory (bfloat16, head_dim 64 or 128).
//
// One block owns 128 query rows of one head.  Its warps:
//   * warps 0-3, the softmax: thread i owns query row i, which is lane i of tensor memory, so the
//     softmax needs no exchange between threads.  Per page of 64 keys a thread reads its row of S
//     (tcgen05.ld), masks it where the page meets the diagonal, the window's edge or the end of the
//     tile, keeps the running maximum and sum in float32 (base 2), and writes P back over the first
//     half of the S columns as packed bfloat16 (tcgen05.st);
//   * warp 4, one thread: TMA loads with the 128-byte swizzle - the query tile once, then the key and
//     the value pages (64 positions each) into a ring of two stages (three at head size 64) guarded by
//     full / empty mbarriers;
//   * warp 5, one thread: S = Q K^T (M = 128 rows, N = 64 keys, both operands K-major) into one of two
//     64-column buffers of tensor memory (three at head size 64, where O takes half the columns); S_i is issued
//     as soon as page i's keys are there and the buffer's last user, the P V of two (three) pages before, is
//     done, so it runs under the softmax of the pages between.  The warp also
//     allocates and frees the block's 256 columns;
//   * warp 6, one thread: O += P_i V_i, with P as the tensor-memory A operand and the value page as it lies
//     in the cache ([position][dim], MN-major) as B; O stays in tensor memory (64 or 128 further columns).
//     The two products have a thread each because a tcgen05.mma is accepted only when the tensor pipe has
//     room and a wait costs about a hundred clocks even when it is over: one thread for both sent a page's
//     twelve MMAs out one behind the other with its waits in between, 2,300 clocks a page of which the tensor
//     cores worked 640, and the softmax warps waited (742 us for 8,192 tokens; 535 us with two threads).
// O and P are scaled by a maximum that follows the row's true maximum only in steps of 2^8: O in
// tensor memory is rescaled when a row's maximum has grown by more than that, which is rare, and
// O / l does not depend on the scale, so the result is exact all the same.  Two blocks fit a
// multiprocessor (80 KB of shared memory, 256 columns of tensor memory each): one block's MMAs run
// under the other's softmax.  Rows of the last page beyond the context are zeroed in shared memory
// (P is zero there, but the cache may hold anything).  Tiles come as a list of (sequence, first row)
// entries, walked from the back (the caller puts the tiles that read the most keys last); an entry
// whose first row is no multiple of 128 (a list made for 64-row tiles) makes its block return at
// once - at a price: launched only to return, such blocks took the place of working ones for
// microseconds each, 72 instead of 47 us for a 2,048-token prompt, so the caller passes a list of
// 128-row tiles.
//
// Every mbarrier wait is bounded; a wait that runs out raises an error flag (read through
// mll_take_device_error), makes the block's later waits return at once, the block stores nothing,
// frees its tensor memory and exits.  Every warp-wide tensor-memory instruction sits in warp-uniform
// control flow.  No load uses cluster multicast.
//
// The reference computes attention for one query token per call with two kernels, scores into a
// buffer and then softmax and values in a second pass (src/cuda_attention.cu:77-163); the formulas
// are those of its CPU path (src/forward.cc:265-298).
#include <cuda.h>

#include "common.cuh"
#include "tensor_map.h"

__device__ int mll_attn_tc5_error_flag = 0;

namespace mll {

constexpr int A_ROWS = 128;  // query rows per block (the MMA's M)
constexpr long long A_WAIT_CLOCKS = 2ll << 30;  // clocks a wait may take (about a second)

struct PrefillTc5Args {
  const int* seq_slot;
  const int* seq_ctx;
  const int* seq_qstart;
  const int* seq_qlen;
  const int* tile_seq;   // tiles of 128 rows (entries that do not start a multiple of 128 are skipped)
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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool a_mbar_wait(unsigned bar, unsigned parity) {
  if (a_mbar_test(bar, parity)) return true;
  const long long began = clock64();
  while (clock64() - began < A_WAIT_CLOCKS) {
    if (a_mbar_test(bar, parity)) return true;
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
// 64 consecutive float32 columns of this thread's lane with one wait: both loads are in flight together
__device__ __forceinline__ void a_tmem_ld64(unsigned addr, float* v) {
  unsigned r[64];
#pragma unroll
  for (int half = 0; half < 2; ++half)
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[32 * half + 0]), "=r"(r[32 * half + 1]), "=r"(r[32 * half + 2]), "=r"(r[32 * half + 3]),
          "=r"(r[32 * half + 4]), "=r"(r[32 * half + 5]), "=r"(r[32 * half + 6]), "=r"(r[32 * half + 7]),
          "=r"(r[32 * half + 8]), "=r"(r[32 * half + 9]), "=r"(r[32 * half + 10]), "=r"(r[32 * half + 11]),
          "=r"(r[32 * half + 12]), "=r"(r[32 * half + 13]), "=r"(r[32 * half + 14]), "=r"(r[32 * half + 15]),
          "=r"(r[32 * half + 16]), "=r"(r[32 * half + 17]), "=r"(r[32 * half + 18]), "=r"(r[32 * half + 19]),
          "=r"(r[32 * half + 20]), "=r"(r[32 * half + 21]), "=r"(r[32 * half + 22]), "=r"(r[32 * half + 23]),
          "=r"(r[32 * half + 24]), "=r"(r[32 * half + 25]), "=r"(r[32 * half + 26]), "=r"(r[32 * half + 27]),
          "=r"(r[32 * half + 28]), "=r"(r[32 * half + 29]), "=r"(r[32 * half + 30]), "=r"(r[32 * half + 31])
        : "r"(addr + 32 * half));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// Two float32 values in one 64-bit register and the arithmetic that works on both at once (sm_100): the
// softmax is bound by the instructions it issues and by the special-function unit (16 exponentials per
// clock and multiprocessor), not by the tensor cores.
typedef unsigned long long a_f32x2;
__device__ __forceinline__ a_f32x2 a_pack2(float lo, float hi) {
  a_f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void a_unpack2(a_f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ a_f32x2 a_fma2(a_f32x2 a, a_f32x2 b, a_f32x2 c) {
  a_f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ a_f32x2 a_add2(a_f32x2 a, a_f32x2 b) {
  a_f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float a_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for both halves of x on the FMA pipe: x = n + f with n = round(x) (the magic-number add leaves n in the
// low mantissa bits of t), 2^f on [-0.5, 0.5] by a cubic whose relative error is below 7.5e-5 (P is rounded to
// 8 bits of mantissa afterwards, and the same values go into the row's sum), and n added to the exponent bits.
// x is clamped at -126 (a masked score is -infinity; 2^-126 is nothing against a row's largest term, which is 1
// or more).  Every other pair of exponentials goes this way, the rest to the special-function unit, so that
// both run side by side.
__device__ __forceinline__ void a_exp2_pair_fma(a_f32x2 x, float& p0, float& p1) {
  float x0, x1;
  a_unpack2(x, x0, x1);
  x = a_pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const a_f32x2 magic = a_pack2(12582912.f, 12582912.f), minus_magic = a_pack2(-12582912.f, -12582912.f);
  const a_f32x2 t = a_add2(x, magic);
  const a_f32x2 n = a_add2(t, minus_magic);
  const a_f32x2 f = a_fma2(n, a_pack2(-1.f, -1.f), x);
  a_f32x2 p = a_fma2(f, a_pack2(0.055171654f, 0.055171654f), a_pack2(0.24261113f, 0.24261113f));
  p = a_fma2(p, f, a_pack2(0.69326097f, 0.69326097f));
  p = a_fma2(p, f, a_pack2(0.99992806f, 0.99992806f));
  float t0, t1, q0, q1;
  a_unpack2(t, t0, t1);
  a_unpack2(p, q0, q1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// 32 consecutive 32-bit columns of this thread's lane, written from registers
__device__ __forceinline__ void a_tmem_st32(unsigned addr, const unsigned* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void a_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] . B[smem]: the A operand (M = 128 rows in the 128 lanes, 16 bfloat16 of K
// packed in 8 columns) comes from tensor memory
__device__ __forceinline__ void a_umma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long desc_b, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void a_mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Warps 0-3: one query row per thread; warp 4: TMA loads; warp 5: the S MMAs; warp 6: the P V MMAs; warp 7 only
// fills the second warpgroup.  Eight warps put two warps of every block on each of the multiprocessor's four
// schedulers, so a new block fits as soon as one of the two resident blocks leaves.  With six warps of 168
// registers it did not: the schedulers' register files held exactly three such warps each, a block put two
// warps on two of the schedulers and one on the others, and the next block's warps mostly fell on the wrong
// ones - the freed place stayed empty until the other block had ended as well (a 2,048-token prompt: 62 us,
// of which the longest block ran 47).  The block is launched with 128 registers per thread; the softmax
// warpgroup then takes 168 (setmaxnreg) and the other warpgroup gives back all but 40.
//
// Tried and taken out again: blocks of two tiles (the same rows of two heads that share a kv head: eight softmax
// warps, one block a multiprocessor, all 512 columns of tensor memory, a four-stage key/value ring, each page
// loaded once for both tiles).  877 against 1,027 TFLOP/s at 8,192 tokens: what bounds the kernel is the chain
// softmax -> P V -> S -> softmax of each S buffer (3,500 clocks for two pages, a quarter of it hand-overs), and
// two blocks of one tile have the same number of chains but two threads for each product.
constexpr int A_SOFTMAX_REGS = 168, A_OTHER_REGS = 40;
constexpr float A_RESCALE_STEP = 8.f;  // the output is rescaled only when a row's maximum grows by more than 2^8

template <int D>
struct PrefillTc5Smem {
  static constexpr int THREADS = 256;
  static constexpr int KV_STAGES = D == 64 ? 3 : 2;   // as many key/value stages as S buffers (80 KB a block either way)
  static constexpr int Q_BYTES = A_ROWS * D * 2;       // D / 64 boxes of [128 rows x 128 bytes]
  static constexpr int KV_BYTES = MLL_PAGE * D * 2;    // D / 64 boxes of [64 rows x 128 bytes]
  static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + KV_STAGES * KV_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * KV_BYTES;
  // Two blocks per multiprocessor (their tensor memory: 2 x 256 columns); never three: the request
  // is padded above a third of the shared memory.  The kernel checks that its dynamic shared
  // memory starts on a 1024-byte boundary (the swizzle's period) and refuses otherwise.
  static constexpr size_t USED = (size_t)BAR_OFF + 512;
  static constexpr size_t BYTES = USED < 80 * 1024 ? 80 * 1024 : USED;
  // Tensor memory, 256 columns a block: S / P buffers of 64 columns, then O (D columns).  Head size 128 leaves room
  // for two S buffers, head size 64 for three: the chain softmax -> P V -> S -> softmax that bounds a block's pace
  // then runs over three pages instead of two.
  static constexpr int S_BUFS = D == 64 ? 3 : 2;
  static constexpr int TMEM_COLS = 256;
  static constexpr int O_COL = S_BUFS * MLL_PAGE;
  static_assert(O_COL + D <= TMEM_COLS, "S buffers and O must fit the block's columns");
  // barrier slots: the queries; keys and values full / empty per ring stage; per S buffer: S full, P ready,
  // P V done
  static constexpr int AB_Q = 0, AB_K_FULL = 1, AB_V_FULL = AB_K_FULL + KV_STAGES, AB_K_EMPTY = AB_V_FULL + KV_STAGES,
                       AB_V_EMPTY = AB_K_EMPTY + KV_STAGES, AB_S_FULL = AB_V_EMPTY + KV_STAGES,
                       AB_P_READY = AB_S_FULL + S_BUFS, AB_PV_DONE = AB_P_READY + S_BUFS,
                       AB_COUNT = AB_PV_DONE + S_BUFS;
  static_assert(AB_COUNT * 8 + 16 <= 512, "the barriers must fit behind the tiles");
};

template <int D>
__global__ void __launch_bounds__(PrefillTc5Smem<D>::THREADS, 2)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap, PrefillTc5Args a) {
  using L = PrefillTc5Smem<D>;
  constexpr int DB = D / 64;  // 64-column boxes per row of Q, K or V
  constexpr int KS = L::KV_STAGES, SB = L::S_BUFS;
  constexpr int LOAD_WARP = 4, MMA_WARP = 5, PV_WARP = 6;
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
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + L::AB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + L::AB_COUNT) + 1;
  const unsigned q_s = a_smem(base + L::Q_OFF), k_s = a_smem(base + L::K_OFF), v_s = a_smem(base + L::V_OFF);
  auto bar = [&](int slot, int index) { return a_smem(bars + slot + index); };
  // a wait that gives up makes every later wait of the block return at once
  auto wait = [&](unsigned barrier, unsigned parity) {
    if (*abort_flag) return;
    if (!a_mbar_wait(barrier, parity)) *abort_flag = 1;
  };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
    for (int i = 0; i < L::AB_COUNT; ++i)
      a_mbar_init(a_smem(bars + i), (i >= L::AB_P_READY && i < L::AB_PV_DONE) ? 4 : 1);  // P ready: one arrival a softmax warp
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(a_smem(tmem_slot)),
                 "r"((unsigned)L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  a_fence_before();
  __syncthreads();
  a_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(A_OTHER_REGS));
  if (warp == LOAD_WARP) {
    // ---- loads: the query tile once, then key and value pages into the ring ----------------- //
    if (lane == 0) {
      a_mbar_expect_tx(bar(L::AB_Q, 0), L::Q_BYTES);
#pragma unroll
      for (int b = 0; b < DB; ++b)
        a_tma_load_2d(q_s + b * (A_ROWS * 128), &qmap, h * D + b * 64, qstart + row0, bar(L::AB_Q, 0));
      int page = table[p_first];
      for (int i = 0; i < n_pages && !*abort_flag; ++i) {
        const int st = i % KS;
        const unsigned parity = ((i / KS) & 1) ^ 1;  // the stage's previous use (none in the first round)
        const int row = (page * a.n_kv_heads + kvh) * MLL_PAGE;
        if (i + 1 < n_pages) page = table[p_first + i + 1];  // looked up while this page's loads fly
        wait(bar(L::AB_K_EMPTY, st), parity);
        a_mbar_expect_tx(bar(L::AB_K_FULL, st), L::KV_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          a_tma_load_2d(k_s + st * L::KV_BYTES + b * (MLL_PAGE * 128), &kmap, b * 64, row, bar(L::AB_K_FULL, st));
        wait(bar(L::AB_V_EMPTY, st), parity);
        a_mbar_expect_tx(bar(L::AB_V_FULL, st), L::KV_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          a_tma_load_2d(v_s + st * L::KV_BYTES + b * (MLL_PAGE * 128), &vmap, b * 64, row, bar(L::AB_V_FULL, st));
      }
    }
  } else if (warp == MMA_WARP) {
    // ---- S = Q K^T, one thread.  S_i goes into buffer i % SB, which held P_{i-SB}: it waits for that page's P V.
    if (lane == 0) {
      constexpr unsigned idesc_s = a_idesc(A_ROWS, MLL_PAGE, false);
      // The descriptors are built once; a step inside a tile only adds to the address field (16-byte units, 14
      // bits: the tiles lie in the first 256 KB of shared memory, so the sum cannot carry out of it).  Built
      // anew for every instruction they cost this thread some twenty dependent instructions per MMA.
      const unsigned long long q_desc = a_desc(q_s, 16);
      unsigned long long k_desc[KS];
#pragma unroll
      for (int s = 0; s < KS; ++s) k_desc[s] = a_desc(k_s + s * L::KV_BYTES, 16);
      wait(bar(L::AB_Q, 0), 0);
      for (int i = 0; i < n_pages && !*abort_flag; ++i) {
        const int sb = i % SB, st = i % KS;
        unsigned long long kd = k_desc[0];
#pragma unroll
        for (int s = 1; s < KS; ++s)
          if (st == s) kd = k_desc[s];
        wait(bar(L::AB_K_FULL, st), (i / KS) & 1);
        if (i >= SB) wait(bar(L::AB_PV_DONE, sb), ((i - SB) / SB) & 1);  // the buffer's P, of page i - SB, has been read
        a_fence_after();
        if (*abort_flag) break;
        const unsigned d = tmem_base + sb * MLL_PAGE;
#pragma unroll
        for (int b = 0; b < DB; ++b)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            a_umma(d, q_desc + (unsigned long long)((b * (A_ROWS * 128) + k * 32) >> 4),
                   kd + (unsigned long long)((b * (MLL_PAGE * 128) + k * 32) >> 4), idesc_s, (b > 0 || k > 0) ? 1u : 0u);
        a_commit(bar(L::AB_S_FULL, sb));
        a_commit(bar(L::AB_K_EMPTY, st));
      }
    }
  } else if (warp == PV_WARP) {
    // ---- O += P V, a thread of its own: with one thread for both products a page's MMAs went out one behind
    // the other (75 clocks apiece for S, 135 for P V, and a hundred for every wait, even one that is over),
    // 2,400 to 3,000 clocks a page of which the tensor cores worked 640, and the softmax warps waited
    if (lane == 0) {
      constexpr unsigned idesc_o = a_idesc(A_ROWS, D, true);
      unsigned long long v_desc[KS];
#pragma unroll
      for (int s = 0; s < KS; ++s) v_desc[s] = a_desc(v_s + s * L::KV_BYTES, MLL_PAGE * 128);
      for (int i = 0; i < n_pages && !*abort_flag; ++i) {
        const int sb = i % SB, st = i % KS;
        unsigned long long vd = v_desc[0];
#pragma unroll
        for (int s = 1; s < KS; ++s)
          if (st == s) vd = v_desc[s];
        wait(bar(L::AB_V_FULL, st), (i / KS) & 1);
        wait(bar(L::AB_P_READY, sb), (i / SB) & 1);
        a_fence_after();
        if (*abort_flag) break;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // P: 16 keys = 8 packed columns per step
          a_umma_ts(tmem_base + L::O_COL, tmem_base + sb * MLL_PAGE + k * 8, vd + (unsigned long long)((k * (16 * 128)) >> 4),
                    idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        a_commit(bar(L::AB_PV_DONE, sb));
        a_commit(bar(L::AB_V_EMPTY, st));
      }
    }
  } else if (warp < 4) {
    // ---- softmax: thread r owns query row r = lane r of tensor memory ------------------------- //
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(A_SOFTMAX_REGS));
    const int r = tid;
    const unsigned tmem_row = tmem_base + ((unsigned)(warp * 32) << 16);
    const int qpos = pos0 + r;
    float m_used = -INFINITY, l_run = 0.f;  // the maximum that P and O are scaled by; the sum
    for (int i = 0; i < n_pages; ++i) {
      const int sb = i % SB, st = i % KS;
      wait(bar(L::AB_S_FULL, sb), (i / SB) & 1);
      a_fence_after();
      float s[MLL_PAGE];
      a_tmem_ld64(tmem_row + sb * MLL_PAGE, s);
      const int k0 = (p_first + i) * MLL_PAGE;
      const bool needs_mask = (k0 + MLL_PAGE - 1 > pos0) || a.window > 0 || rows < A_ROWS;
      if (needs_mask) {
#pragma unroll
        for (int c = 0; c < MLL_PAGE; ++c) {
          const int kpos = k0 + c;
          const bool keep = r < rows && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
          s[c] = keep ? s[c] : -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < MLL_PAGE; c += 8) {  // three-input maxima: half the instructions
        mx4[0] = a_max3(mx4[0], s[c], s[c + 1]);
        mx4[1] = a_max3(mx4[1], s[c + 2], s[c + 3]);
        mx4[2] = a_max3(mx4[2], s[c + 4], s[c + 5]);
        mx4[3] = a_max3(mx4[3], s[c + 6], s[c + 7]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;
      // P and O stay scaled by m_used while the row's maximum is within 2^8 of it: exact all the
      // same (O / l does not depend on the scale), and O in tensor memory is touched only rarely
      const bool moved = mx > m_used + A_RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY);
      if (i > 0 && __any_sync(0xffffffffu, moved)) {
        const float alpha = moved ? a_exp2(m_used - mx) : 1.f;
        wait(bar(L::AB_PV_DONE, (i - 1) % SB), ((i - 1) / SB) & 1);  // O holds every page before this one
        a_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          float o[32];
          a_tmem_ld32(tmem_row + L::O_COL + c, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= alpha;
          a_tmem_st32(tmem_row + L::O_COL + c, reinterpret_cast<const unsigned*>(o));
        }
        l_run *= alpha;
      }
      if (moved) m_used = mx;
      const float shift = m_used > -INFINITY ? m_used : 0.f;  // a fully masked row stays at zero weight
      // p = 2^(s * scale - shift), two columns per instruction; the pairs alternate between the special-function
      // unit and the FMA pipe
      const a_f32x2 scale2 = a_pack2(a.scale_log2, a.scale_log2), shift2 = a_pack2(-shift, -shift);
      a_f32x2 sum2[2] = {a_pack2(0.f, 0.f), a_pack2(0.f, 0.f)};
      unsigned packed[MLL_PAGE / 2];
#pragma unroll
      for (int c = 0; c < MLL_PAGE; c += 2) {
        const a_f32x2 x = a_fma2(a_pack2(s[c], s[c + 1]), scale2, shift2);
        float p0, p1;
        if ((c >> 1) & 1) {
          a_exp2_pair_fma(x, p0, p1);
        } else {
          float x0, x1;
          a_unpack2(x, x0, x1);
          p0 = a_exp2(x0);
          p1 = a_exp2(x1);
        }
        sum2[(c >> 2) & 1] = a_add2(sum2[(c >> 2) & 1], a_pack2(p0, p1));
        __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
        packed[c >> 1] = *reinterpret_cast<unsigned*>(&pair);
      }
      {
        float s0, s1, s2, s3;
        a_unpack2(sum2[0], s0, s1);
        a_unpack2(sum2[1], s2, s3);
        l_run += (s0 + s1) + (s2 + s3);
      }
      a_tmem_st32(tmem_row + sb * MLL_PAGE, packed);  // P over the first half of S
      const int valid = ctx - k0;  // positions of this page that the sequence has
      if (valid < MLL_PAGE) {      // only the sequence's last page: the rest of it may hold anything
        wait(bar(L::AB_V_FULL, st), (i / KS) & 1);
        unsigned char* vt = base + L::V_OFF + st * L::KV_BYTES;
        const int n_chunks = (MLL_PAGE - valid) * 8;  // 16-byte chunks per box
        for (int b = 0; b < DB; ++b)
          for (int c = r; c < n_chunks; c += A_ROWS)
            *reinterpret_cast<uint4*>(vt + b * (MLL_PAGE * 128) + valid * 128 + c * 16) = make_uint4(0, 0, 0, 0);
        a_fence_async_smem();
      }
      a_tmem_wait_st();
      a_fence_before();
      __syncwarp();  // one arrival a warp: 128 arrivals on one barrier are 128 shared-memory atomics in a row
      if (lane == 0) a_mbar_arrive(bar(L::AB_P_READY, sb));
    }
    // the output row: O / l
    wait(bar(L::AB_PV_DONE, (n_pages - 1) % SB), ((n_pages - 1) / SB) & 1);
    a_fence_after();
    {
      // tcgen05.ld is a warp-wide instruction: every thread of the warp reads its lane, and only the
      // threads that own a row of the sequence store
      const bool store = !*abort_flag && r < rows;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = a.out + ((size_t)qstart + row0 + (store ? r : 0)) * a.n_heads * D + (size_t)h * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        float o[32];
        a_tmem_ld32(tmem_row + L::O_COL + c, o);
        if (store) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e) hp[e] = __floats2bfloat162_rn(o[j + 2 * e] * inv, o[j + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(dst + c + j) = w;
          }
        }
      }
    }
  }

  a_fence_before();
  __syncthreads();
  if (*abort_flag && tid == 0) {  // loads may still be in flight: give them time before the shared memory goes
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == MMA_WARP) {
    a_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)L::TMEM_COLS));
  }
}

template <int D>
int launch_prefill_tc5(const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                       const PrefillTc5Args& a, int n_tiles, cudaStream_t stream) {
  using L = PrefillTc5Smem<D>;
  const size_t smem = L::BYTES;
  auto kernel = attn_prefill_tc5_kernel<D>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("attention prefill (tcgen05): cannot reserve %zu bytes of shared memory: %s", smem,
                  cudaGetErrorString(err));
    return (int)err;
  }
  MLL_LAUNCH((kernel), dim3((unsigned)(n_tiles * a.n_heads)), L::THREADS, smem, stream, qmap, kmap, vmap, a);
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

// The device address of this file's error flag (nullptr if it cannot be had); device_error.cu reads,
// clears and hands it to the sampling kernels.
extern "C" int* mll_attn_tc5_error_address() {
  int* address = nullptr;
  if (cudaGetSymbolAddress((void**)&address, mll_attn_tc5_error_flag) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return address;
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
