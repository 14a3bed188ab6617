// y[M, N] = x[M, K] . W[N, K]^T for at most 64 rows (decode), weights streamed by TMA.
//
// A decode-time product is bound by reading W once from HBM, so what counts is how many
// bytes a multiprocessor keeps in flight.  Here a producer thread issues
// cp.async.bulk.tensor (TMA) loads of [64 weight rows x 64 k] boxes (8 KB, 128-byte
// swizzle) and of the matching [8..64 activation rows x 64 k] box into a ring of shared
// memory stages guarded by full/empty mbarriers; four consumer warps read their fragments
// with ldmatrix from the swizzled boxes and run mma.sync.m16n8k16 with the weights as the
// A operand ("swap-AB": 16 weight rows per warp, 8 batch rows per n-tile).  No register
// holds a load in flight, so a block of 160 threads keeps its whole ring (3 stages, 27 KB)
// outstanding and seven blocks fit on a multiprocessor.
//
// K is split over the blocks of a thread-block cluster; the partial tiles are summed in
// rank order through distributed shared memory (reproducible), and the epilogue - bias,
// SwiGLU on interleaved gate/up rows, bfloat16 or float32 output - runs once on the sum.
// Rows or columns beyond the matrix are zero-filled by the TMA unit, so any N, any M <= 64
// and any K that is a multiple of 8 are taken.  No load uses cluster multicast.
//
// Every mbarrier wait is bounded: on a timeout the thread raises the library's error flag
// (mll_error_flag) and leaves its loop; the block still reaches its barriers and exits.
//
// The reference calls cublasSgemm with rows = 1 for every linear (src/cuda_matmul.cc:181-186).
#include <cooperative_groups.h>
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tensor_map.h"

namespace cg = cooperative_groups;

__device__ int mll_device_error_flag = 0;

namespace mll {

enum : int { TEPI_BF16 = 0, TEPI_F32 = 1, TEPI_SWIGLU = 2 };
constexpr int T_ROWS = 64;     // weight rows per block
constexpr int T_KB = 64;       // k elements per stage (128 bytes: one swizzle span)
constexpr int T_STAGES = 3;
constexpr int T_THREADS = 160; // four consumer warps and one producer warp
constexpr long long T_WAIT_CLOCKS = 2ll << 30;  // clocks a wait may take

struct TmaLinearArgs {
  const float* bias;  // optional [N]
  void* out;          // [M, N] (SwiGLU: [M, N / 2])
  int M, N, K, epilogue, blocks_per_rank;
  RowNormIn in;       // x still lacks its norm's factor (sumsq null: it does not)
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
// Bounded wait; false (and the error flag raised) when the phase never completes.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
  // each try parks the thread until the phase completes or a time limit of the hardware's own runs out (a spin
  // on test_wait spends issue slots and power while the block waits for memory); about a second in all
  if (mbar_test(bar, parity)) return true;
  const long long began = clock64();
  while (clock64() - began < T_WAIT_CLOCKS) {
    if (mbar_test(bar, parity)) return true;
  }
  atomicExch(&mll_device_error_flag, 1);
  return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_tma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT>
struct TmaSmem {
  static constexpr int W_BYTES = T_ROWS * T_KB * 2;       // 8192
  static constexpr int X_BYTES = 8 * NT * T_KB * 2;       // 1024 per n-tile
  static constexpr int STAGE = W_BYTES + X_BYTES;         // a multiple of 1024
  static constexpr int RED_FLOATS = T_ROWS * 8 * NT;
  static constexpr size_t BYTES = 1024 /* alignment slack */ + (size_t)T_STAGES * STAGE + RED_FLOATS * 4 + 64 + 8 * NT * 4;
};

// grid: row tiles * cluster size; block: 160 threads.
template <int NT, bool CLUSTER>
__global__ void __launch_bounds__(T_THREADS)
linear_tma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, TmaLinearArgs a) {
  using L = TmaSmem<NT>;
  extern __shared__ unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: stages start on 1024-byte boundaries
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* red = reinterpret_cast<float*>(base + (size_t)T_STAGES * L::STAGE);          // [64][8 NT]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(red + L::RED_FLOATS);  // full[S], empty[S]
  float* row_factor = reinterpret_cast<float*>(bars + 8);                                 // [8 NT]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int rank = 0, ranks = 1;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    rank = (int)cluster.block_rank();
    ranks = (int)cluster.num_blocks();
  }
  const int tile = blockIdx.x / ranks;
  const int n0 = tile * T_ROWS;
  const int k_blocks = (a.K + T_KB - 1) / T_KB;
  const int first = rank * a.blocks_per_rank;
  const int count = max(0, min(k_blocks, first + a.blocks_per_rank) - first);

  if (tid == 0) {
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(smem_u32(bars + s), 1);             // full: the producer's expect_tx arrival
      mbar_init(smem_u32(bars + T_STAGES + s), 4);  // empty: one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

  if (warp == 4) {
    if (lane == 0) {
      // the ring's first round needs no free-stage wait; all its weight boxes go out before the
      // (small, L2-resident) activation boxes, so that the HBM requests start as early as possible
      const int primed = min(count, T_STAGES);
      for (int i = 0; i < primed; ++i) {
        const unsigned full = smem_u32(bars + i);
        mbar_expect_tx(full, L::STAGE);
        tma_load_2d(smem_u32(base + (size_t)i * L::STAGE), &wmap, (first + i) * T_KB, n0, full);
      }
      for (int i = 0; i < primed; ++i)
        tma_load_2d(smem_u32(base + (size_t)i * L::STAGE) + L::W_BYTES, &xmap, (first + i) * T_KB, 0,
                    smem_u32(bars + i));
      for (int i = primed; i < count; ++i) {
        const int s = i % T_STAGES;
        if (!mbar_wait(smem_u32(bars + T_STAGES + s), ((i / T_STAGES) & 1) ^ 1)) break;
        const unsigned full = smem_u32(bars + s);
        const unsigned dst = smem_u32(base + (size_t)s * L::STAGE);
        mbar_expect_tx(full, L::STAGE);
        tma_load_2d(dst, &wmap, (first + i) * T_KB, n0, full);
        tma_load_2d(dst + L::W_BYTES, &xmap, (first + i) * T_KB, 0, full);
      }
    }
  } else {
    // consumer warp: weight rows warp * 16 .. + 15 of the tile
    const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);  // ldmatrix row of this lane (A)
    const unsigned a_row_off = row * 128;
    const unsigned a_xor = row & 7;
    const unsigned a_hi = lane >> 4;  // second 16-byte chunk of the k-step
    const unsigned x_chunk = lane >> 3;  // B: chunks 2 ks + {0, 1} and 2 (ks + 1) + {0, 1}
    if (a.in.sumsq && rank == 0) {
      // the first stage is a memory latency away: time for the rows' norm factors, which the epilogue needs
      for (int m = warp; m < a.M; m += 8) {  // rows m and m + 4, their loads in flight together
        const bool second = m + 4 < a.M;
        float f0, f1;
        row_norm_factors2(a.in.sumsq + (size_t)m * a.in.stride, a.in.sumsq + (size_t)(m + 4) * a.in.stride, second,
                          a.in.partials, a.K, a.in.eps, lane, f0, f1);
        if (lane == 0) {
          row_factor[m] = f0;
          if (second) row_factor[m + 4] = f1;
        }
      }
    }
    for (int i = 0; i < count; ++i) {
      const int s = i % T_STAGES;
      if (!mbar_wait(smem_u32(bars + s), (i / T_STAGES) & 1)) break;
      const unsigned wt = smem_u32(base + (size_t)s * L::STAGE);
      const unsigned xt = wt + L::W_BYTES;
#pragma unroll
      for (int ks = 0; ks < T_KB / 16; ks += 2) {
        unsigned fa0[4], fa1[4];
        ldsm_x4(fa0, wt + a_row_off + (((2 * ks + a_hi) ^ a_xor) << 4));
        ldsm_x4(fa1, wt + a_row_off + (((2 * ks + 2 + a_hi) ^ a_xor) << 4));
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          unsigned fx[4];
          const unsigned xr = n * 8 + (lane & 7);
          ldsm_x4(fx, xt + xr * 128 + (((2 * ks + x_chunk) ^ (xr & 7)) << 4));
          mma_tma(acc[n], fa0, fx[0], fx[1]);
          mma_tma(acc[n], fa1, fx[2], fx[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bars + T_STAGES + s));
    }
    // this warp's 16 x (8 NT) partial tile
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      float* r0 = red + (warp * 16 + g) * 8 * NT + n * 8 + 2 * t;
      float* r1 = red + (warp * 16 + g + 8) * 8 * NT + n * 8 + 2 * t;
      r0[0] = acc[n][0];
      r0[1] = acc[n][1];
      r1[0] = acc[n][2];
      r1[1] = acc[n][3];
    }
  }
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every block's partial tile is complete and visible
    if (rank == 0) {
      for (int i = tid; i < L::RED_FLOATS; i += T_THREADS) {
        float s = red[i];
        for (int r = 1; r < ranks; ++r) s += *cluster.map_shared_rank(red + i, r);
        red[i] = s;
      }
    }
    cluster.sync();  // rank 0 has read its peers' shared memory; they may leave
    if (rank != 0) return;
  }
  __syncthreads();

  // epilogue on the full sums: red[row][m] is y[m][n0 + row]
  constexpr int COLS = 8 * NT;
  if (a.epilogue == TEPI_SWIGLU) {
    __nv_bfloat16* out = (__nv_bfloat16*)a.out;
    const int half = a.N >> 1;
    for (int i = tid; i < (T_ROWS / 2) * COLS; i += T_THREADS) {
      const int m = i / (T_ROWS / 2), j = i % (T_ROWS / 2);  // j: output column within the tile's 32
      const int row = (j >> 3) * 16 + (j & 7);               // gate row; its up row is 8 further
      if (m < a.M && n0 + row + 8 < a.N) {
        const float f = a.in.sumsq ? row_factor[m] : 1.f;
        const float gate = red[row * COLS + m] * f, up = red[(row + 8) * COLS + m] * f;
        out[(size_t)m * half + (n0 >> 1) + j] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
      }
    }
  } else {
    for (int i = tid; i < T_ROWS * COLS; i += T_THREADS) {
      const int m = i / T_ROWS, row = i % T_ROWS;
      if (m < a.M && n0 + row < a.N) {
        float v = red[row * COLS + m];
        if (a.in.sumsq) v *= row_factor[m];
        if (a.bias) v += a.bias[n0 + row];
        if (a.epilogue == TEPI_F32)
          ((float*)a.out)[(size_t)m * a.N + n0 + row] = v;
        else
          ((__nv_bfloat16*)a.out)[(size_t)m * a.N + n0 + row] = __float2bfloat16_rn(v);
      }
    }
  }
  // after a timeout copies may still be in flight towards this block's shared memory: give them time
  if (*(volatile int*)&mll_device_error_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
}

// ---- tensor maps ------------------------------------------------------------------ //
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
        status == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows * 1315423911LL + k.cols) << 1) ^ k.box_rows;
  }
};

int tensor_map_bf16(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex lock;
  std::lock_guard<std::mutex> guard(lock);
  const MapKey key{ptr, rows, cols, box_rows};
  auto hit = cache.find(key);
  if (hit != cache.end()) {
    *out = hit->second;
    return 0;
  }
  EncodeTiledFn encode = encode_fn();
  if (!encode) {
    mll_set_error("linear_tma: the driver does not provide cuTensorMapEncodeTiled");
    return -1;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)T_KB, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    mll_set_error("linear_tma: cuTensorMapEncodeTiled failed with code %d for a [%lld, %lld] matrix", (int)rc, rows, cols);
    return -1;
  }
  if (cache.size() > 4096) cache.clear();
  cache[key] = map;
  *out = map;
  return 0;
}

template <int NT>
int launch_linear_tma(const CUtensorMap& wmap, const CUtensorMap& xmap, const TmaLinearArgs& a, int tiles, int ranks,
                      cudaStream_t stream) {
  const size_t smem = TmaSmem<NT>::BYTES;
  cudaError_t err;
  if (ranks > 1)
    err = cudaFuncSetAttribute(linear_tma_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  else
    err = cudaFuncSetAttribute(linear_tma_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (err != cudaSuccess) {
    mll_set_error("linear_tma: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    return (int)err;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(tiles * ranks);
  config.blockDim = dim3(T_THREADS);
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
    err = cudaLaunchKernelEx(&config, linear_tma_kernel<NT, true>, wmap, xmap, a);
  } else {
    err = cudaLaunchKernelEx(&config, linear_tma_kernel<NT, false>, wmap, xmap, a);
  }
  if (err != cudaSuccess) {
    mll_set_error("linear_tma: launch failed: %s", cudaGetErrorString(err));
    return (int)err;
  }
  return 0;
}

}  // namespace mll

// The device address of this file's error flag (nullptr if it cannot be had); device_error.cu reads,
// clears and hands it to the sampling kernels.
extern "C" int* mll_linear_tma_error_address() {
  int* address = nullptr;
  if (cudaGetSymbolAddress((void**)&address, mll_device_error_flag) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return address;
}

MLL_API int mll_linear_tma_supported(int M, int N, int K, int epilogue) {
  if (M < 1 || M > 64 || N < 1 || K < 8 || K % 8 != 0) return 0;
  if (epilogue == mll::TEPI_SWIGLU && N % 16 != 0) return 0;
  return 1;
}

// x: bfloat16 [M, K]; w: bfloat16 [N, K]; bias: optional float32 [N]; out and epilogue as in
// mll_linear_small.  ranks: cluster size along K (1, 2, 4 or 8), 0 = choose.  in_sumsq, in_partials,
// in_stride, in_eps: as in mll_linear_small_fused (x lacks its RMS norm's factor), or null.
MLL_API int mll_linear_tma_fused(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                                 int epilogue, int ranks, const float* in_sumsq, int in_partials, int in_stride,
                                 float in_eps, cudaStream_t stream) {
  MLL_REQUIRE(!in_sumsq || (in_partials >= 1 && in_stride >= in_partials && in_eps >= 0.f),
              "linear_tma: partial sums: %d of stride %d", in_partials, in_stride);
  MLL_REQUIRE(mll_linear_tma_supported(M, N, K, epilogue), "linear_tma: unsupported sizes M=%d N=%d K=%d", M, N, K);
  MLL_REQUIRE(epilogue >= 0 && epilogue <= 2, "linear_tma: unknown epilogue %d", epilogue);
  MLL_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0), "linear_tma: operands must be 16-byte aligned");
  MLL_REQUIRE(epilogue != mll::TEPI_SWIGLU || bias == nullptr, "linear_tma: the SwiGLU epilogue takes no bias");
  const int tiles = (N + mll::T_ROWS - 1) / mll::T_ROWS;
  const int k_blocks = (K + mll::T_KB - 1) / mll::T_KB;
  if (ranks <= 0) {
    // As many blocks as can be resident together (7 per multiprocessor), each with at least 32 k-blocks (2,048
    // columns) once every multiprocessor has a block, 8 before that.  (With 8 everywhere the 16384 x 2048 gate/up
    // product of a 2,048-wide model got clusters of 4 with 512 columns a block: 20.5 us in a graph against 15.0
    // without any split; 28672 x 4096 keeps its clusters of 2: 41.3 against 42.5 us.)
    ranks = 1;
    while (ranks < 8 && tiles * ranks * 2 <= mll_sm_count() * 7 &&
           k_blocks / (ranks * 2) >= (tiles * ranks * 2 <= mll_sm_count() ? 8 : 32))
      ranks *= 2;
  }
  MLL_REQUIRE(ranks == 1 || ranks == 2 || ranks == 4 || ranks == 8, "linear_tma: cluster size %d", ranks);
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  CUtensorMap wmap, xmap;
  if (mll::tensor_map_bf16(w, N, K, mll::T_ROWS, &wmap) != 0) return -1;
  if (mll::tensor_map_bf16(x, M, K, 8 * nt, &xmap) != 0) return -1;
  mll::TmaLinearArgs a{bias, out, M, N, K, epilogue, (k_blocks + ranks - 1) / ranks,
                       mll::RowNormIn{in_sumsq, in_partials, in_stride, in_eps}};
  if (nt == 1) return mll::launch_linear_tma<1>(wmap, xmap, a, tiles, ranks, stream);
  if (nt == 2) return mll::launch_linear_tma<2>(wmap, xmap, a, tiles, ranks, stream);
  if (nt == 4) return mll::launch_linear_tma<4>(wmap, xmap, a, tiles, ranks, stream);
  return mll::launch_linear_tma<8>(wmap, xmap, a, tiles, ranks, stream);
}

MLL_API int mll_linear_tma(const void* x, const void* w, const float* bias, void* out, int M, int N, int K,
                           int epilogue, int ranks, cudaStream_t stream) {
  return mll_linear_tma_fused(x, w, bias, out, M, N, K, epilogue, ranks, nullptr, 0, 0, 0.f, stream);
}
