// y[M, N] = x[M, K] . W[N, K]^T for a handful of rows (decode): a weight-streaming kernel.
//
// With M <= 64 the product is bound by reading W once from HBM.  The weights are the A
// operand of mma.sync.m16n8k16 (16 weight rows per warp tile), the activations the B
// operand (8 batch rows per n-tile): "swap-AB".  Every thread loads 16 contiguous bytes of a
// weight row straight from global memory into its fragment registers - the k order inside
// a 32-element chunk is permuted the same way for both operands, which a dot product does
// not mind - so nothing is staged in shared memory and each warp streams on its own.
// K is split over the warps of a block and over the blocks of a thread-block cluster; the
// partial 16 x M tiles are summed in a fixed order through (distributed) shared memory, so
// the result is reproducible, and the epilogue (bias, SwiGLU, bfloat16 or float32 output)
// runs once on the full sum.
//
// Two optional fusions with the RMS norm around the product (the reference keeps them apart:
// src/forward.cc:385-414 adds, normalises and multiplies in separate calls):
//   * the rows may arrive not yet normalised (RowNormIn): the result is multiplied by the row's factor;
//   * epilogue EPI_RESID adds the result to the float32 residual stream, and writes the new row times the
//     next norm's weight, in bfloat16, with the tile's share of the row's sum of squares.
//
// The reference calls cublasSgemm with rows = 1 for every linear (src/cuda_matmul.cc:181-186).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace mll {

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_RESID = 3 };

struct LinearArgs {
  const __nv_bfloat16* x;  // [M, K]
  const __nv_bfloat16* w;  // [N, K]
  const float* bias;       // optional [N]
  void* out;               // [M, N] (EPI_SWIGLU: [M, N / 2])
  int M, N, K, epilogue, chunks_per_warp;
  RowNormIn in;            // x still lacks its norm's factor
  float* resid;            // EPI_RESID: float32 residual [M, N], updated in place
  const float* next_w;     // EPI_RESID: weight [N] of the norm that follows
  float* out_sumsq;        // EPI_RESID: [M, out_stride], entry [m][tile] = sum over the tile's columns of resid^2
  int out_stride;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_keep(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// grid: (row tiles * cluster size); block: LS_WARPS warps.  NT: n-tiles of 8 batch rows.
// LS_UNROLL: 32-element chunks in flight per warp; LS_WARPS: warps per block (K is split over them);
// OCC: resident warps per multiprocessor that the register allocation aims at (0: the compiler's choice).
// Without it the compiler's own occupancy guess decides how many of the loads stay in flight, and an
// unrelated edit of the epilogue moved that guess (o of the 8B shape: 8.7 -> 11.9 us); 16 gives the
// loop 128 registers, 24 gives it 80.
template <int NT, bool CLUSTER, int LS_UNROLL, int LS_WARPS, int OCC>
__global__ void __launch_bounds__(LS_WARPS * 32, OCC / LS_WARPS)
linear_small_kernel(LinearArgs a) {
  __shared__ float red[LS_WARPS][16][8 * NT];
  __shared__ float row_factor[8 * NT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  int rank = 0, ranks = 1;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    rank = (int)cluster.block_rank();
    ranks = (int)cluster.num_blocks();
  }
  const int tile = blockIdx.x / ranks;
  const int n0 = tile * 16;
  const int chunks = a.K >> 5;
  const int first = (rank * LS_WARPS + warp) * a.chunks_per_warp;
  const int last = min(chunks, first + a.chunks_per_warp);

  const int row_a = min(n0 + g, a.N - 1), row_b = min(n0 + g + 8, a.N - 1);  // clamped: extra rows are never stored
  const __nv_bfloat16* wa = a.w + (size_t)row_a * a.K + t * 8;
  const __nv_bfloat16* wb = a.w + (size_t)row_b * a.K + t * 8;
  const __nv_bfloat16* xr[NT];
  bool x_ok[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int m = n * 8 + g;
    x_ok[n] = m < a.M;
    xr[n] = a.x + (size_t)(x_ok[n] ? m : 0) * a.K + t * 8;
  }

  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

  // At most 16 rows and 8 warps: warp m works out the norm factors of rows m and m + 8 now, before its loop.  The partial sums lie
  // in the L2 cache, so this is one cache latency (0.5 us); the warp first asks the L2 cache for the weights of its
  // first round of loads, which come from HBM and take longer, so nothing is lost.  (That request alone, without
  // a factor to wait for, helps products of many tiles and long rows by up to 1 us and costs the short one-wave
  // ones as much: it is made only here.)  Worked out after the loop, as
  // the wider cases still do, the factor cost every block that latency at its end, with nothing to hide it: with
  // the 1,792 blocks of a 28672-row gate/up product 5 us of 43 at 8 rows.
  constexpr bool EARLY_FACTORS = NT <= 2 && LS_WARPS == 8;  // at most 16 rows: warp m has rows m and m + 8
  const bool early = EARLY_FACTORS && a.in.sumsq != nullptr && rank == 0;
  if (early && warp < a.M) {
#pragma unroll
    for (int u = 0; u < LS_UNROLL; ++u)
      if (first + u < last) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wa + (size_t)(first + u) * 32));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wb + (size_t)(first + u) * 32));
      }
    if (NT == 1) {
      const float f = row_norm_factor<32>(a.in.sumsq + (size_t)warp * a.in.stride, a.in.partials, a.K, a.in.eps, lane,
                                          0xffffffffu);
      if (lane == 0) row_factor[warp] = f;
    } else {
      const bool second = warp + LS_WARPS < a.M;
      float f0, f1;
      row_norm_factors2(a.in.sumsq + (size_t)warp * a.in.stride, a.in.sumsq + (size_t)(warp + LS_WARPS) * a.in.stride,
                        second, a.in.partials, a.K, a.in.eps, lane, f0, f1);
      if (lane == 0) {
        row_factor[warp] = f0;
        if (second) row_factor[warp + LS_WARPS] = f1;
      }
    }
  }

  // The residual epilogue of the 8-warp variants has one element per thread (16 weight rows x up to 16 batch rows):
  // the thread asks for its residual value and the next norm's weight now, so that the block's end does not wait
  // a memory latency for them.
  constexpr bool EARLY_RESID = NT <= 2 && LS_WARPS == 8;
  float resid_early = 0.f, next_w_early = 0.f;
  if (EARLY_RESID && a.epilogue == EPI_RESID && rank == 0 && threadIdx.x < 16 * 8 * NT) {
    const int m = threadIdx.x >> 4, r = threadIdx.x & 15;
    if (m < a.M && n0 + r < a.N) {
      resid_early = a.resid[(size_t)m * a.N + n0 + r];
      next_w_early = a.next_w[n0 + r];
    }
  }

  int c = first;
  for (; c + LS_UNROLL <= last; c += LS_UNROLL) {
    uint4 fa[LS_UNROLL], fb[LS_UNROLL];
#pragma unroll
    for (int u = 0; u < LS_UNROLL; ++u) {
      fa[u] = ldg_stream(wa + (size_t)(c + u) * 32);
      fb[u] = ldg_stream(wb + (size_t)(c + u) * 32);
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      uint4 fx[LS_UNROLL];
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u)
        fx[u] = x_ok[n] ? ldg_keep(xr[n] + (size_t)(c + u) * 32) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < LS_UNROLL; ++u) {
        mma_bf16(acc[n], fa[u].x, fb[u].x, fa[u].y, fb[u].y, fx[u].x, fx[u].y);
        mma_bf16(acc[n], fa[u].z, fb[u].z, fa[u].w, fb[u].w, fx[u].z, fx[u].w);
      }
    }
  }
  for (; c < last; ++c) {
    const uint4 ta = ldg_stream(wa + (size_t)c * 32), tb = ldg_stream(wb + (size_t)c * 32);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const uint4 fx = x_ok[n] ? ldg_keep(xr[n] + (size_t)c * 32) : make_uint4(0u, 0u, 0u, 0u);
      mma_bf16(acc[n], ta.x, tb.x, ta.y, tb.y, fx.x, fx.y);
      mma_bf16(acc[n], ta.z, tb.z, ta.w, tb.w, fx.z, fx.w);
    }
  }

  // this warp's 16 x (8 NT) partial tile: rows g and g + 8, batch columns n * 8 + 2 t + {0, 1}
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    red[warp][g][n * 8 + 2 * t] = acc[n][0];
    red[warp][g][n * 8 + 2 * t + 1] = acc[n][1];
    red[warp][g + 8][n * 8 + 2 * t] = acc[n][2];
    red[warp][g + 8][n * 8 + 2 * t + 1] = acc[n][3];
  }
  __syncthreads();
  // sum the warps into red[0], in warp order
  for (int i = threadIdx.x; i < 16 * 8 * NT; i += LS_WARPS * 32) {
    float* cell = &red[0][0][0] + i;
    float s = cell[0];
#pragma unroll
    for (int w = 1; w < LS_WARPS; ++w) s += cell[w * 16 * 8 * NT];
    cell[0] = s;
  }
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every block's red[0] is complete and visible
    if (rank == 0) {
      for (int i = threadIdx.x; i < 16 * 8 * NT; i += LS_WARPS * 32) {
        float* cell = &red[0][0][0] + i;
        float s = cell[0];
        for (int r = 1; r < ranks; ++r) s += *cluster.map_shared_rank(cell, r);
        cell[0] = s;
      }
    }
    cluster.sync();  // rank 0 has read its peers' shared memory; they may leave
    if (rank != 0) return;
  }
  if (a.in.sumsq) {
    // the rows' norm factors, from partial sums that lie in the L2 cache: plain loads here, at the end, cost
    // 0.6 us (q/k/v of the 8B shape); fetching them into shared memory during the main loop cost 1.5 us,
    // through the share of the L1 cache that the buffer takes from the activations
    if (early) {  // done before the loop
    } else if (NT == 1) {  // at most 8 rows: one per warp of the 8-warp variants (the two-row form cost them 0.4 us)
      for (int m = warp; m < a.M; m += LS_WARPS) {
        const float f = row_norm_factor<32>(a.in.sumsq + (size_t)m * a.in.stride, a.in.partials, a.K, a.in.eps, lane,
                                            0xffffffffu);
        if (lane == 0) row_factor[m] = f;
      }
    } else {
      for (int m = warp; m < a.M; m += 2 * LS_WARPS) {  // rows m and m + LS_WARPS, their loads in flight together
        const bool second = m + LS_WARPS < a.M;
        float f0, f1;
        row_norm_factors2(a.in.sumsq + (size_t)m * a.in.stride, a.in.sumsq + (size_t)(m + LS_WARPS) * a.in.stride,
                          second, a.in.partials, a.K, a.in.eps, lane, f0, f1);
        if (lane == 0) {
          row_factor[m] = f0;
          if (second) row_factor[m + LS_WARPS] = f1;
        }
      }
    }
  }
  __syncthreads();

  // epilogue on the full sums: element (row, m) of the tile is y[m][n0 + row]
  if (a.epilogue == EPI_SWIGLU) {
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    const int half = a.N >> 1;
    for (int i = threadIdx.x; i < 8 * 8 * NT; i += LS_WARPS * 32) {
      const int m = i >> 3, r = i & 7;
      if (m < a.M && n0 + r + 8 < a.N) {
        const float f = a.in.sumsq ? row_factor[m] : 1.f;
        const float gate = red[0][r][m] * f, up = red[0][r + 8][m] * f;
        out[(size_t)m * half + (n0 >> 1) + r] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      }
    }
  } else if (a.epilogue == EPI_RESID) {
    // whole warps run the loop (its bound is a multiple of 32): 16 consecutive lanes hold one row's tile
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += LS_WARPS * 32) {
      const int m = i >> 4, r = i & 15;
      float now = 0.f;
      if (m < a.M && n0 + r < a.N) {
        float v = red[0][r][m];
        if (a.in.sumsq) v *= row_factor[m];
        if (a.bias) v += a.bias[n0 + r];
        const size_t at = (size_t)m * a.N + n0 + r;
        now = (EARLY_RESID ? resid_early : a.resid[at]) + v;  // EARLY_RESID: i is threadIdx.x, one round of this loop
        a.resid[at] = now;
        out[at] = __float2bfloat16_rn(now * (EARLY_RESID ? next_w_early : a.next_w[n0 + r]));
      }
      float sq = now * now;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      if (r == 0 && m < a.M) a.out_sumsq[(size_t)m * a.out_stride + tile] = sq;
    }
  } else {
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += LS_WARPS * 32) {
      const int m = i >> 4, r = i & 15;
      if (m < a.M && n0 + r < a.N) {
        float v = red[0][r][m];
        if (a.in.sumsq) v *= row_factor[m];
        if (a.bias) v += a.bias[n0 + r];
        if (a.epilogue == EPI_F32)
          ((float*)a.out)[(size_t)m * a.N + n0 + r] = v;
        else
          ((__nv_bfloat16*)a.out)[(size_t)m * a.N + n0 + r] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <int NT, int U, int LS_WARPS, int OCC>
int launch_linear_small(const LinearArgs& a, int tiles, int ranks, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(tiles * ranks);
  config.blockDim = dim3(LS_WARPS * 32);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  cudaError_t err;
  config.attrs = attr;
  config.numAttrs = 0;
  if (ranks > 1) {
    attr[config.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[config.numAttrs].val.clusterDim.x = ranks;
    attr[config.numAttrs].val.clusterDim.y = 1;
    attr[config.numAttrs].val.clusterDim.z = 1;
    ++config.numAttrs;
    err = cudaLaunchKernelEx(&config, linear_small_kernel<NT, true, U, LS_WARPS, OCC>, a);
  } else {
    err = cudaLaunchKernelEx(&config, linear_small_kernel<NT, false, U, LS_WARPS, OCC>, a);
  }
  if (err != cudaSuccess) {
    mll_set_error("linear_small: launch failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  return 0;
}

}  // namespace mll

// Whether mll_linear_small takes this problem (the caller uses the library GEMM otherwise).
MLL_API int mll_linear_small_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > 64 || N < 16 || K < 32 || K % 32 != 0) return 0;
  if (epilogue == mll::EPI_SWIGLU && N % 16 != 0) return 0;
  return 1;
}

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; bias: optional float32 [N];
// out: bfloat16 [M, N] (epilogue 0), float32 [M, N] (1), or bfloat16 [M, N / 2] = silu(gate) * up
// with gate and up rows of w interleaved in blocks of 8 (2).  ranks: cluster size along K
// (1, 2, 4 or 8), 0 = choose.
// in_sumsq (optional, float32 [M, in_stride], in_partials of each row used): x lacks its RMS norm's
// factor 1 / sqrt(sum / K + in_eps), which the result is multiplied by.
// Epilogue 3 (at most 16 rows): resid (float32 [M, N]) += result; out (bfloat16 [M, N]) = resid * next_w;
// out_sumsq (float32 [M, out_stride], out_stride >= ceil(N / 16)): entry [m][j] = sum of resid[m]^2 over
// columns 16 j .. 16 j + 15.
MLL_API int mll_linear_small_fused(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                                   int epilogue, int ranks, const float* in_sumsq, int in_partials, int in_stride,
                                   float in_eps, float* resid, const float* next_w, float* out_sumsq, int out_stride,
                                   cudaStream_t stream) {
  MLL_REQUIRE(epilogue >= 0 && epilogue <= 3, "linear_small: unknown epilogue %d", epilogue);
  MLL_REQUIRE(mll_linear_small_supported(M, N, K, epilogue == mll::EPI_RESID ? 0 : epilogue),
              "linear_small: unsupported sizes M=%d N=%d K=%d", M, N, K);
  MLL_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear_small: operands must be 16-byte aligned");
  MLL_REQUIRE(epilogue != mll::EPI_SWIGLU || bias == nullptr, "linear_small: the SwiGLU epilogue takes no bias");
  if (in_sumsq) {
    MLL_REQUIRE(in_partials >= 1 && in_stride >= in_partials, "linear_small: partial sums: %d of stride %d",
                in_partials, in_stride);
    MLL_REQUIRE(in_eps >= 0.f, "linear_small: eps must be non-negative");
  }
  if (epilogue == mll::EPI_RESID) {
    MLL_REQUIRE(M <= 16, "linear_small: the residual epilogue takes at most 16 rows, got %d", M);
    MLL_REQUIRE(resid && next_w && out_sumsq && out_stride >= (N + 15) / 16,
                "linear_small: the residual epilogue needs resid, next_w and out_sumsq with stride >= %d", (N + 15) / 16);
  }
  const int tiles = (N + 15) / 16;
  const int chunks = K / 32;
  // The variant (8B shapes, CUDA-graph timings at 8 / 16 rows, us; ideal = bytes / 6.65 TB/s):
  //   * K of 2048 or more, at most 16 rows: 8 warps per block.  All tiles in one wave of the 128-register
  //     kernel (2 blocks per multiprocessor): that one, 8 chunks in flight per warp (o 7.8 / 8.5, ideal 5.0;
  //     down 21.6 / 24.1, ideal 17.7); more tiles: the 80-register kernel with 4 chunks in flight, 3 blocks per
  //     multiprocessor (q/k/v 10.0-10.6 / 11.6-12.4, ideal 7.6).  Both without k-ranks at these sizes.
  //   * otherwise 4 warps and the compiler's register choice.
  const bool wide = chunks >= 64 && M <= 16;
  const bool one_wave = tiles <= mll_sm_count() * 2;
  const int warps = wide ? 8 : 4;
  if (ranks <= 0) {
    // split K while every block still fits on the machine at once and a warp keeps at least 4 chunks
    const int resident = mll_sm_count() * (wide ? (one_wave ? 2 : 3) : 10);
    ranks = 1;
    while (ranks < 8 && tiles * ranks * 2 <= resident && chunks / (warps * ranks * 2) >= 4) ranks *= 2;
  }
  MLL_REQUIRE(ranks == 1 || ranks == 2 || ranks == 4 || ranks == 8, "linear_small: cluster size %d", ranks);
  mll::LinearArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, out, M, N, K, epilogue, 0,
                    mll::RowNormIn{in_sumsq, in_partials, in_stride, in_eps}, resid, next_w, out_sumsq, out_stride};
  const int splits = warps * ranks;
  a.chunks_per_warp = (chunks + splits - 1) / splits;
  if (M <= 8) {
    if (wide && one_wave) return mll::launch_linear_small<1, 8, 8, 16>(a, tiles, ranks, stream);
    if (wide) return mll::launch_linear_small<1, 4, 8, 24>(a, tiles, ranks, stream);
    return mll::launch_linear_small<1, 4, 4, 0>(a, tiles, ranks, stream);
  }
  if (M <= 16) {
    if (wide && one_wave) return mll::launch_linear_small<2, 8, 8, 16>(a, tiles, ranks, stream);
    if (wide) return mll::launch_linear_small<2, 4, 8, 24>(a, tiles, ranks, stream);
    return mll::launch_linear_small<2, 4, 4, 0>(a, tiles, ranks, stream);
  }
  if (M <= 32) return mll::launch_linear_small<4, 2, 4, 0>(a, tiles, ranks, stream);
  return mll::launch_linear_small<8, 2, 4, 0>(a, tiles, ranks, stream);
}

MLL_API int mll_linear_small(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                             int epilogue, int ranks, cudaStream_t stream) {
  MLL_REQUIRE(epilogue != mll::EPI_RESID, "linear_small: the residual epilogue needs mll_linear_small_fused");
  return mll_linear_small_fused(x, w, bias, out, M, N, K, epilogue, ranks, nullptr, 0, 0, 0.f, nullptr, nullptr,
                                nullptr, 0, stream);
}
