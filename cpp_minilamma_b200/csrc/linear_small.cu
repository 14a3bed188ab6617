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
// The reference calls cublasSgemm with rows = 1 for every linear (src/cuda_matmul.cc:181-186).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace mll {

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

struct LinearArgs {
  const __nv_bfloat16* x;  // [M, K]
  const __nv_bfloat16* w;  // [N, K]
  const float* bias;       // optional [N]
  void* out;               // [M, N] (EPI_SWIGLU: [M, N / 2])
  int M, N, K, epilogue, chunks_per_warp;
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


// grid: (row tiles * cluster size); block: 128 threads.  NT: n-tiles of 8 batch rows.
// LS_UNROLL: 32-element chunks in flight per warp; LS_WARPS: warps per block (K is split over them)
template <int NT, bool CLUSTER, int LS_UNROLL, int LS_WARPS>
__global__ void __launch_bounds__(LS_WARPS * 32)
linear_small_kernel(LinearArgs a) {
  __shared__ float red[LS_WARPS][16][8 * NT];
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
  __syncthreads();

  // epilogue on the full sums: element (row, m) of the tile is y[m][n0 + row]
  if (a.epilogue == EPI_SWIGLU) {
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    const int half = a.N >> 1;
    for (int i = threadIdx.x; i < 8 * 8 * NT; i += LS_WARPS * 32) {
      const int m = i >> 3, r = i & 7;
      if (m < a.M && n0 + r + 8 < a.N) {
        const float gate = red[0][r][m], up = red[0][r + 8][m];
        out[(size_t)m * half + (n0 >> 1) + r] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      }
    }
  } else {
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += LS_WARPS * 32) {
      const int m = i >> 4, r = i & 15;
      if (m < a.M && n0 + r < a.N) {
        float v = red[0][r][m];
        if (a.bias) v += a.bias[n0 + r];
        if (a.epilogue == EPI_F32)
          ((float*)a.out)[(size_t)m * a.N + n0 + r] = v;
        else
          ((__nv_bfloat16*)a.out)[(size_t)m * a.N + n0 + r] = __float2bfloat16_rn(v);
      }
    }
  }
}

template <int NT, int U, int LS_WARPS>
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
    err = cudaLaunchKernelEx(&config, linear_small_kernel<NT, true, U, LS_WARPS>, a);
  } else {
    err = cudaLaunchKernelEx(&config, linear_small_kernel<NT, false, U, LS_WARPS>, a);
  }
  if (err != cudaSuccess) {
    mll_set_error("linear_small: launch failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  return 0;
}

}  // namespace mll

// tuning knob for experiments: chunks in flight per warp for M <= 16 (2 only up to 8 rows, 4 or 8)
extern "C" __attribute__((visibility("default"))) int mll_linear_small_unroll = 4;
// tuning knob for experiments: warps per block for M <= 16 (4 or 8)
extern "C" __attribute__((visibility("default"))) int mll_linear_small_warps = 4;

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
MLL_API int mll_linear_small(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                             int epilogue, int ranks,
                             cudaStream_t stream) {
  MLL_REQUIRE(mll_linear_small_supported(M, N, K, epilogue), "linear_small: unsupported sizes M=%d N=%d K=%d", M, N, K);
  MLL_REQUIRE(epilogue >= 0 && epilogue <= 2, "linear_small: unknown epilogue %d", epilogue);
  MLL_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear_small: operands must be 16-byte aligned");
  MLL_REQUIRE(epilogue != mll::EPI_SWIGLU || bias == nullptr, "linear_small: the SwiGLU epilogue takes no bias");
  const int tiles = (N + 15) / 16;
  const int chunks = K / 32;
  // With the knobs at their defaults the variant is chosen here (8B shape, 8 rows, CUDA-graph timing):
  //   * two k-ranks of every tile fit on the machine at the 8-fold unrolled kernel's occupancy (128
  //     registers: 4 blocks per multiprocessor): that kernel, twice the loads in flight per warp and
  //     half the trips (o 8.7 against 9.2 us, down 22.0 against 24.4);
  //   * more tiles than that (q/k/v): 8 warps per block, 8-fold unrolled, no k-ranks (11.0 against 12.6 us).
  const bool knobs_default = mll_linear_small_warps == 4 && mll_linear_small_unroll == 4 && ranks <= 0;
  const bool defaults = knobs_default && M <= 8;
  const bool deep = defaults && tiles * 2 <= 148 * 4 && chunks / (4 * 2) >= 8;
  //   * 9 to 16 rows (two batch tiles): 8 warps per block, no k-ranks, 8-fold unrolled when one wave of
  //     that kernel takes all tiles (o 8.7, down 23.3, q/k/v 11.8 us at 16 rows; library 9.8 / 23.5 / 12.5).
  const bool two_tiles = knobs_default && M > 8 && M <= 16 && chunks >= 64;
  const int warps = (mll_linear_small_warps == 8 && M <= 16) || (defaults && !deep && chunks >= 64) || two_tiles ? 8 : 4;
  const bool wide_unroll = mll_linear_small_unroll == 8 || (two_tiles && tiles <= 148 * 2);
  if (deep) ranks = 2;
  if (two_tiles) ranks = 1;
  if (ranks <= 0) {
    // split K while every block still fits on the machine at once and a warp keeps at least 4 chunks
    const int resident = 148 * (warps == 8 ? 5 : 10);
    ranks = 1;
    while (ranks < 8 && tiles * ranks * 2 <= resident && chunks / (warps * ranks * 2) >= 4) ranks *= 2;
  }
  MLL_REQUIRE(ranks == 1 || ranks == 2 || ranks == 4 || ranks == 8, "linear_small: cluster size %d", ranks);
  mll::LinearArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, out, M, N, K, epilogue, 0};
  const int splits = warps * ranks;
  a.chunks_per_warp = (chunks + splits - 1) / splits;
  if (M <= 8) {
    if (warps == 8 && (mll_linear_small_unroll == 8 || defaults)) return mll::launch_linear_small<1, 8, 8>(a, tiles, ranks, stream);
    if (warps == 8) return mll::launch_linear_small<1, 4, 8>(a, tiles, ranks, stream);
    if (mll_linear_small_unroll == 2) return mll::launch_linear_small<1, 2, 4>(a, tiles, ranks, stream);
    if (mll_linear_small_unroll == 8 || deep) return mll::launch_linear_small<1, 8, 4>(a, tiles, ranks, stream);
    return mll::launch_linear_small<1, 4, 4>(a, tiles, ranks, stream);
  }
  if (M <= 16) {
    if (warps == 8 && wide_unroll) return mll::launch_linear_small<2, 8, 8>(a, tiles, ranks, stream);
    if (warps == 8) return mll::launch_linear_small<2, 4, 8>(a, tiles, ranks, stream);
    if (mll_linear_small_unroll == 8) return mll::launch_linear_small<2, 8, 4>(a, tiles, ranks, stream);
    return mll::launch_linear_small<2, 4, 4>(a, tiles, ranks, stream);
  }
  if (M <= 32) return mll::launch_linear_small<4, 2, 4>(a, tiles, ranks, stream);
  return mll::launch_linear_small<8, 2, 4>(a, tiles, ranks, stream);
}
