// y[M, N] = x[M, K] . W[N, K]^T for at most 64 rows: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
// The fifth-generation tensor cores read both operands straight from shared memory and keep
// the accumulator in tensor memory, so the block needs no fragment loads at all:
//   * warps 4 and 6, one thread each: TMA producers for the even and the odd k-blocks.  Per
//     k-block of 64 a producer loads a [128 weight rows x 64] box and the [16..64 activation
//     rows x 64] box (128-byte swizzle, K-major) into a ring of stages guarded by full/empty
//     mbarriers;
//   * warps 5 and 7, one thread each: issue four tcgen05.mma (M = 128 weight rows, N = batch
//     rows padded to 16/32/64, K = 16) per stage from shared-memory descriptors, each into an
//     accumulator of its own, and release the stage with tcgen05.commit; warp 5 allocates and
//     frees the block's TMEM columns.  (One thread issuing every box or every MMA of a block
//     caps the block's stream; two of each measured 1 % of a decode step.);
//   * warps 0-3: after the last commits they read the two 128 x N float32 accumulators from
//     TMEM (tcgen05.ld, one row per thread) and add them into shared memory, batch row by batch
//     row ([m][weight row]: neighbouring threads write neighbouring words).
// "Swap-AB": the weights are the M operand, the batch is N, so a decode step with 1..64
// sequences fills the 128-row MMA.  K is split over the blocks of a cluster; every block of the
// cluster then owns a share of the batch rows, sums the partial tiles of all blocks for them in
// rank order through distributed shared memory (reproducible) and runs the epilogue on them:
// bias, SwiGLU on gate/up rows interleaved in blocks of 8, bfloat16 or float32 output, or the
// residual epilogue (add to the float32 residual stream, write the new stream times the next norm's
// weight with partial sums of squares per 16 columns).  Rows and columns outside the matrices are
// zero-filled by TMA, so any N, any M <= 64 and any K % 8 == 0 are taken.  No load uses cluster multicast.
//
// The ring has an even number of stages for every batch width.  The two producers (and the two MMA
// issuers) take the even and the odd k-blocks; with an even number of stages a stage is always
// refilled by the producer that filled it before, which has seen that stage's previous phase
// complete, so it can never wait on a barrier that is two phases behind (a parity wait cannot tell
// those apart).  An earlier 32-column variant had five stages; that flaw was found by reading.
//
// Every mbarrier wait is bounded; on a timeout the thread raises an error flag (read with
// mll_take_device_error) and leaves its loop, the block still reaches its barriers, frees its TMEM and exits.
//
// The reference calls cublasSgemm with rows = 1 for every linear (src/cuda_matmul.cc:181-186).
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
#include "tensor_map.h"

namespace cg = cooperative_groups;

// raised by a bounded wait that ran out; read and cleared through mll_take_device_error()
__device__ int mll_tc5_error_flag = 0;

namespace mll {

enum : int { CEPI_BF16 = 0, CEPI_F32 = 1, CEPI_SWIGLU = 2, CEPI_RESID = 3 };
constexpr int C_ROWS = 128;     // weight rows per block (the MMA's M)
constexpr int C_KB = 64;        // k elements per stage: one 128-byte swizzle span
constexpr int C_THREADS = 256;  // 4 epilogue warps, then producer A, MMA A, producer B, MMA B (even / odd k-blocks)
constexpr long long C_WAIT_CLOCKS = 2ll << 30;  // clocks a wait may take

struct Tc5Args {
  const float* bias;
  void* out;
  int M, N, K, epilogue, blocks_per_rank;
  RowNormIn in;  // x still lacks its norm's factor (sumsq null: it does not)
  float* resid;         // CEPI_RESID: float32 residual [M, N], updated in place
  const float* next_w;  // CEPI_RESID: weight [N] of the norm that follows
  float* out_sumsq;     // CEPI_RESID: [M, out_stride], entry [m][j] = sum of resid[m]^2 over columns 16 j .. 16 j + 15
  int out_stride;
};

__device__ __forceinline__ unsigned c_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void c_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void c_mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool c_mbar_test(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool c_mbar_wait(unsigned bar, unsigned parity) {
  // each try parks the thread until the phase completes or a time limit of the hardware's own runs out (a spin
  // on test_wait spends issue slots that the other warps of the multiprocessor can use); about a second in all
  if (c_mbar_test(bar, parity)) return true;
  const long long began = clock64();
  while (clock64() - began < C_WAIT_CLOCKS) {
    if (c_mbar_test(bar, parity)) return true;
  }
  atomicExch(&mll_tc5_error_flag, 1);
  return false;
}
__device__ __forceinline__ void c_tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16)
// with the 128-byte swizzle: groups of 8 rows are 1024 bytes apart (stride byte offset), the
// leading byte offset is not used by swizzled K-major layouts, descriptor version 1,
// layout type 2 (SWIZZLE_128B).  `addr` is the shared-memory byte address of the first row,
// advanced by 32 bytes per K = 16 step inside the swizzle span.
__device__ __forceinline__ unsigned long long umma_desc_sw128(unsigned addr) {
  return (unsigned long long)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((unsigned long long)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: float32 accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr unsigned umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

template <int NB>  // batch columns of the MMA: 16, 32 or 64
struct Tc5Smem {
  static constexpr int W_BYTES = C_ROWS * C_KB * 2;  // 16384
  static constexpr int X_BYTES = NB * C_KB * 2;      // 2048 .. 8192
  static constexpr int STAGE = W_BYTES + X_BYTES;    // a multiple of 1024
  static constexpr int STAGES = NB <= 16 ? 6 : 4;  // even (see the header); 80 to 108 KB of ring: two blocks per multiprocessor
  static constexpr int RED_FLOATS = C_ROWS * NB;
  static constexpr int TMEM_COLS = 2 * NB < 32 ? 32 : 2 * NB;  // one accumulator per MMA issuer
  // the float32 tile that the epilogue works on reuses the ring once the last MMA is done
  static constexpr int RING = STAGES * STAGE > RED_FLOATS * 4 ? STAGES * STAGE : RED_FLOATS * 4;
  static constexpr size_t BYTES = 1024 + (size_t)RING + 128 + NB * 4;  // ring, barriers and tensor-memory slot, row factors
};

template <int NB, bool CLUSTER>
__global__ void __launch_bounds__(C_THREADS)
linear_tc5_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, Tc5Args a) {
  using L = Tc5Smem<NB>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(base);  // [NB][128], over the ring: written only after the last MMA
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(base + L::RING);  // full[S], empty[S], done
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * L::STAGES + 1);
  float* row_factor = reinterpret_cast<float*>(base + L::RING + 128);  // [NB]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int rank = 0, ranks = 1;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    rank = (int)cluster.block_rank();
    ranks = (int)cluster.num_blocks();
  }
  const int tile = blockIdx.x / ranks;
  const int n0 = tile * C_ROWS;
  // the batch rows whose sums and epilogue this block owns
  const int m_begin = rank * (NB / ranks), m_end = min(a.M, m_begin + NB / ranks);
  const int k_blocks = (a.K + C_KB - 1) / C_KB;
  const int first = rank * a.blocks_per_rank;
  const int count = max(0, min(k_blocks, first + a.blocks_per_rank) - first);
  const unsigned done_bar = c_smem(bars + 2 * L::STAGES);

  if (tid == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      c_mbar_init(c_smem(bars + s), 1);             // full: the producer's expect_tx arrival
      c_mbar_init(c_smem(bars + L::STAGES + s), 1);  // empty: one tcgen05.commit per use
    }
    c_mbar_init(done_bar, 2);  // both MMA issuers commit to it
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {  // this warp allocates and frees the block's tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(c_smem(tmem_slot)),
                 "r"((unsigned)L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  // Two producers and two MMA issuers share the k-blocks (even / odd): one thread that issues every
  // TMA box, or every MMA, of a block caps the block's stream well below what the ring allows.
  if (warp == 4 || warp == 6) {
    if (lane == 0) {
      const int mine = warp == 4 ? 0 : 1;
      // the ring's first round needs no free-stage wait; its weight boxes go out before the
      // (small, L2-resident) activation boxes, so that the HBM requests start as early as possible
      const int primed = min(count, L::STAGES);
      for (int i = mine; i < primed; i += 2) {
        const unsigned full = c_smem(bars + i);
        c_mbar_expect_tx(full, L::STAGE);
        c_tma_load_2d(c_smem(base + (size_t)i * L::STAGE), &wmap, (first + i) * C_KB, n0, full);
      }
      for (int i = mine; i < primed; i += 2)
        c_tma_load_2d(c_smem(base + (size_t)i * L::STAGE) + L::W_BYTES, &xmap, (first + i) * C_KB, 0, c_smem(bars + i));
      for (int i = primed + ((primed & 1) != mine ? 1 : 0); i < count; i += 2) {
        const int s = i % L::STAGES;
        if (!c_mbar_wait(c_smem(bars + L::STAGES + s), ((i / L::STAGES) & 1) ^ 1)) break;
        const unsigned full = c_smem(bars + s);
        const unsigned dst = c_smem(base + (size_t)s * L::STAGE);
        c_mbar_expect_tx(full, L::STAGE);
        c_tma_load_2d(dst, &wmap, (first + i) * C_KB, n0, full);
        c_tma_load_2d(dst + L::W_BYTES, &xmap, (first + i) * C_KB, 0, full);
      }
    }
  } else if (warp == 5 || warp == 7) {
    if (lane == 0) {
      const int mine = warp == 5 ? 0 : 1;
      constexpr unsigned idesc = umma_idesc_bf16(C_ROWS, NB);
      for (int i = mine; i < count; i += 2) {
        const int s = i % L::STAGES;
        if (!c_mbar_wait(c_smem(bars + s), (i / L::STAGES) & 1)) break;
        tc_fence_after();
        const unsigned wt = c_smem(base + (size_t)s * L::STAGE);
        const unsigned xt = wt + L::W_BYTES;
#pragma unroll
        for (int k = 0; k < C_KB / 16; ++k)
          umma_bf16(tmem_base + mine * NB, umma_desc_sw128(wt + k * 32), umma_desc_sw128(xt + k * 32), idesc,
                    (i > mine || k > 0) ? 1u : 0u);
        umma_commit(c_smem(bars + L::STAGES + s));  // the stage is free once these MMAs have read it
      }
      umma_commit(done_bar);  // arrives when every MMA issued above is complete
    }
  }

  // epilogue warps: accumulator row (weight row) = TMEM lane, one row per thread
  if (warp < 4) {
    if (a.in.sumsq) {  // while the products run: the norm factors of this block's rows, for the epilogue
      for (int m = m_begin + warp; m < m_end; m += 8) {  // rows m and m + 4, their loads in flight together
        const bool second = m + 4 < m_end;
        float f0, f1;
        row_norm_factors2(a.in.sumsq + (size_t)m * a.in.stride, a.in.sumsq + (size_t)(m + 4) * a.in.stride, second,
                          a.in.partials, a.K, a.in.eps, lane, f0, f1);
        if (lane == 0) {
          row_factor[m] = f0;
          if (second) row_factor[m + 4] = f1;
        }
      }
    }
    const bool ok = c_mbar_wait(done_bar, 0);
    tc_fence_after();
    float* row = red + warp * 32 + lane;  // this weight row's column of the [NB][128] tile
    if (ok && count > 0) {
#pragma unroll
      for (int c = 0; c < NB; c += 16) {
        unsigned v[16], w[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)c));
        asm volatile(  // the odd k-blocks' accumulator (left unwritten when the block has a single k-block)
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
              "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15])
            : "r"(tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(NB + c)));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j)
          row[(c + j) * C_ROWS] = __uint_as_float(v[j]) + (count > 1 ? __uint_as_float(w[j]) : 0.f);
      }
    } else {
#pragma unroll
      for (int c = 0; c < NB; ++c) row[c * C_ROWS] = 0.f;  // no k-block for this rank (or a timeout)
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {  // every read of the accumulator is done
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)L::TMEM_COLS));
  }
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every block's partial tile is complete and visible
    for (int i = m_begin * C_ROWS + tid; i < m_end * C_ROWS; i += C_THREADS) {
      float part[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) part[r] = r < ranks ? *cluster.map_shared_rank(red + i, r) : 0.f;  // loads in flight together
      float sum = part[0];
#pragma unroll
      for (int r = 1; r < 8; ++r) sum += part[r];  // rank order: the same result on every run
      red[i] = sum;  // the peers read other batch rows of this block's tile, never these
    }
    __syncthreads();
  }

  // red[m][row] is y[m][n0 + row]; neighbouring threads take neighbouring weight rows
  const int span = max(0, m_end - m_begin);
  if (a.epilogue == CEPI_SWIGLU) {
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    const int half = a.N >> 1;
    for (int i = tid; i < span * (C_ROWS / 2); i += C_THREADS) {
      const int m = m_begin + i / (C_ROWS / 2), j = i % (C_ROWS / 2);
      const int row = (j >> 3) * 16 + (j & 7);  // gate row; its up row is 8 further
      if (n0 + row + 8 < a.N) {
        const float f = a.in.sumsq ? row_factor[m] : 1.f;
        const float gate = red[m * C_ROWS + row] * f, up = red[m * C_ROWS + row + 8] * f;
        out[(size_t)m * half + (n0 >> 1) + j] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      }
    }
  } else if (a.epilogue == CEPI_RESID) {
    // whole warps run the loop (its bound is a multiple of 32): 16 consecutive lanes hold 16 consecutive columns
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    for (int i = tid; i < span * C_ROWS; i += C_THREADS) {
      const int m = m_begin + i / C_ROWS, row = i % C_ROWS;
      float now = 0.f;
      if (n0 + row < a.N) {
        float v = red[m * C_ROWS + row];
        if (a.in.sumsq) v *= row_factor[m];
        if (a.bias) v += a.bias[n0 + row];
        const size_t at = (size_t)m * a.N + n0 + row;
        now = a.resid[at] + v;
        a.resid[at] = now;
        out[at] = __float2bfloat16_rn(now * a.next_w[n0 + row]);
      }
      float sq = now * now;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if ((row & 15) == 0 && n0 + row < a.N) a.out_sumsq[(size_t)m * a.out_stride + ((n0 + row) >> 4)] = sq;
    }
  } else {
    for (int i = tid; i < span * C_ROWS; i += C_THREADS) {
      const int m = m_begin + i / C_ROWS, row = i % C_ROWS;
      if (n0 + row < a.N) {
        float v = red[m * C_ROWS + row];
        if (a.in.sumsq) v *= row_factor[m];
        if (a.bias) v += a.bias[n0 + row];
        if (a.epilogue == CEPI_F32)
          ((float*)a.out)[(size_t)m * a.N + n0 + row] = v;
        else
          ((__nv_bfloat16*)a.out)[(size_t)m * a.N + n0 + row] = __float2bfloat16_rn(v);
      }
    }
  }
  if (CLUSTER) cg::this_cluster().sync();  // the peers have read this block's tile: its shared memory may go
  if (*(volatile int*)&mll_tc5_error_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
}

template <int NB>
int launch_linear_tc5(const CUtensorMap& wmap, const CUtensorMap& xmap, const Tc5Args& a, int tiles, int ranks,
                      cudaStream_t stream) {
  const size_t smem = Tc5Smem<NB>::BYTES;
  cudaError_t err;
  if (ranks > 1)
    err = cudaFuncSetAttribute(linear_tc5_kernel<NB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  else
    err = cudaFuncSetAttribute(linear_tc5_kernel<NB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("linear_tc5: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(tiles * ranks);
  config.blockDim = dim3(C_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  config.attrs = attr;
  config.numAttrs = 0;
  if (ranks > 1) {
    attr[config.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[config.numAttrs].val.clusterDim.x = ranks;
    attr[config.numAttrs].val.clusterDim.y = 1;
    attr[config.numAttrs].val.clusterDim.z = 1;
    ++config.numAttrs;
    err = cudaLaunchKernelEx(&config, linear_tc5_kernel<NB, true>, wmap, xmap, a);
  } else {
    err = cudaLaunchKernelEx(&config, linear_tc5_kernel<NB, false>, wmap, xmap, a);
  }
  if (err != cudaSuccess) {
    mll_set_error("linear_tc5: launch failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  return 0;
}

}  // namespace mll

// The device address of this file's error flag (nullptr if it cannot be had); device_error.cu reads,
// clears and hands it to the sampling kernels.
extern "C" int* mll_linear_tc5_error_address() {
  int* address = nullptr;
  if (cudaGetSymbolAddress((void**)&address, mll_tc5_error_flag) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return address;
}

// Up to 64 rows: 16, 32 or 64 batch columns per MMA, chosen by the row count.
MLL_API int mll_linear_tc5_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > 64 || N < 1 || K < 8 || K % 8 != 0) return 0;
  if (epilogue == mll::CEPI_SWIGLU && N % 16 != 0) return 0;
  return 1;
}

// Same contract as mll_linear_small_fused (epilogue 3, the residual epilogue, included, here for up to 64
// rows).  ranks: cluster size along K (1, 2, 4 or 8), 0 = choose.
MLL_API int mll_linear_tc5_fused(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                                 int epilogue, int ranks, const float* in_sumsq, int in_partials, int in_stride,
                                 float in_eps, float* resid, const float* next_w, float* out_sumsq, int out_stride,
                                 cudaStream_t stream) {
  MLL_REQUIRE(!in_sumsq || (in_partials >= 1 && in_stride >= in_partials && in_eps >= 0.f),
              "linear_tc5: partial sums: %d of stride %d", in_partials, in_stride);
  MLL_REQUIRE(epilogue >= 0 && epilogue <= 3, "linear_tc5: unknown epilogue %d", epilogue);
  MLL_REQUIRE(mll_linear_tc5_supported(M, N, K, epilogue == mll::CEPI_RESID ? 0 : epilogue),
              "linear_tc5: unsupported sizes M=%d N=%d K=%d", M, N, K);
  MLL_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear_tc5: operands must be 16-byte aligned");
  MLL_REQUIRE(epilogue != mll::CEPI_SWIGLU || bias == nullptr, "linear_tc5: the SwiGLU epilogue takes no bias");
  if (epilogue == mll::CEPI_RESID)
    MLL_REQUIRE(resid && next_w && out_sumsq && out_stride >= (N + 15) / 16,
                "linear_tc5: the residual epilogue needs resid, next_w and out_sumsq with stride >= %d", (N + 15) / 16);
  const int tiles = (N + mll::C_ROWS - 1) / mll::C_ROWS;
  const int k_blocks = (K + mll::C_KB - 1) / mll::C_KB;
  if (ranks <= 0) {
    // split K while all blocks can be resident together (2 per multiprocessor)
    // and each keeps >= 8 k-blocks
    const int resident = mll_sm_count() * 2;
    ranks = 1;
    while (ranks < 8 && tiles * ranks * 2 <= resident && k_blocks / (ranks * 2) >= 8) ranks *= 2;
  }
  MLL_REQUIRE(ranks == 1 || ranks == 2 || ranks == 4 || ranks == 8, "linear_tc5: cluster size %d", ranks);
  const int nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap wmap, xmap;
  if (mll::tensor_map_bf16(w, N, K, mll::C_ROWS, &wmap) != 0) return -1;
  if (mll::tensor_map_bf16(x, M, K, nb, &xmap) != 0) return -1;
  mll::Tc5Args a{bias, out, M, N, K, epilogue, (k_blocks + ranks - 1) / ranks,
                 mll::RowNormIn{in_sumsq, in_partials, in_stride, in_eps}, resid, next_w, out_sumsq, out_stride};
  if (nb == 16) return mll::launch_linear_tc5<16>(wmap, xmap, a, tiles, ranks, stream);
  if (nb == 32) return mll::launch_linear_tc5<32>(wmap, xmap, a, tiles, ranks, stream);
  return mll::launch_linear_tc5<64>(wmap, xmap, a, tiles, ranks, stream);
}

MLL_API int mll_linear_tc5(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                           int epilogue, int ranks, cudaStream_t stream) {
  MLL_REQUIRE(epilogue != mll::CEPI_RESID, "linear_tc5: the residual epilogue needs mll_linear_tc5_fused");
  return mll_linear_tc5_fused(x, w, bias, out, M, N, K, epilogue, ranks, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr, 0,
                              stream);
}
