// Shared device helpers of the kernel library (sm_100a).
//
// Every exported entry point is `extern "C"`, takes raw device pointers, sizes and
// a stream, validates its arguments on the host and returns 0 on success.  A refused
// argument returns a negative code and leaves a message for mll_last_error(); a CUDA
// launch error returns the positive cudaError_t.  Nothing here allocates memory or
// synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MLL_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python binding
enum : int { MLL_F32 = 0, MLL_BF16 = 1 };

// number of cache positions in one page
#define MLL_PAGE 64

void mll_set_error(const char* fmt, ...);

#define MLL_REQUIRE(cond, ...)        \
  do {                                \
    if (!(cond)) {                    \
      mll_set_error(__VA_ARGS__);     \
      return -1;                      \
    }                                 \
  } while (0)

// Launches `kernel` on `stream`; the outcome is picked up by MLL_LAUNCH_CHECK.
#define MLL_LAUNCH(kernel, grid, block, smem, stream, ...) \
  mll_launch_status = mll::launch_kernel(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, ##__VA_ARGS__)

#define MLL_LAUNCH_CHECK()                          \
  do {                                              \
    cudaError_t err__ = mll_launch_status;          \
    mll_launch_status = cudaSuccess;                \
    if (err__ == cudaSuccess) err__ = cudaGetLastError(); \
    if (err__ != cudaSuccess) {                     \
      mll_set_error("%s:%d launch failed: %s", __FILE__, __LINE__, cudaGetErrorString(err__)); \
      return (int)err__;                            \
    }                                               \
  } while (0)

extern thread_local cudaError_t mll_launch_status;

// Multiprocessors of the current device (asked once per device; the kernels size their grids by it).
int mll_sm_count();

namespace mll {

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed reduction tree (same result on every run).
// `scratch` holds at least 32 floats; every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < nwarps) ? scratch[lane] : 0.f;
  total = warp_sum(total);
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = (lane < nwarps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

// 16-byte asynchronous copy global -> shared (both 16-byte aligned)
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Rows whose RMS norm is still to be applied.  The kernel that added to the residual stream wrote, for
// every row m, `partials` sums of squares over column tiles at sumsq[m * stride + p] and the row itself
// multiplied by the norm's weight; a product over such rows multiplies its result by
// 1 / sqrt(sum_p sumsq[m][p] / width + eps), which is what the norm would have put into the row.
struct RowNormIn {
  const float* sumsq;  // null: the rows are taken as they are
  int partials, stride;
  float eps;
};

// That factor for one row, computed by LANES consecutive lanes of a warp (LANES 16 or 32; `sub` is the
// lane's index among them, `mask` names them) in a fixed order; every one of them gets the result.
template <int LANES>
__device__ __forceinline__ float row_norm_factor(const float* row_partials, int partials, int width, float eps,
                                                 int sub, unsigned mask) {
  float s = 0.f;
  for (int p0 = sub; p0 < partials; p0 += 8 * LANES) {
    float v[8];  // eight loads in flight: the sum below must not wait for one load after the other
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = p0 + i * LANES < partials ? row_partials[p0 + i * LANES] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += v[i];
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) s += __shfl_xor_sync(mask, s, o);
  return 1.f / sqrtf(s / (float)width + eps);
}

// The same for two rows at once (the second only if `second`): their loads are in flight together, so that
// a warp with two rows to do pays one memory latency, and each sum is formed as above.
__device__ __forceinline__ void row_norm_factors2(const float* row_a, const float* row_b, bool second, int partials,
                                                  int width, float eps, int lane, float& fa, float& fb) {
  float sa = 0.f, sb = 0.f;
  for (int p0 = lane; p0 < partials; p0 += 8 * 32) {
    float va[8], vb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool in = p0 + i * 32 < partials;
      va[i] = in ? row_a[p0 + i * 32] : 0.f;
      vb[i] = in && second ? row_b[p0 + i * 32] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sa += va[i];
      sb += vb[i];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sa += __shfl_xor_sync(0xffffffffu, sa, o);
    sb += __shfl_xor_sync(0xffffffffu, sb, o);
  }
  fa = 1.f / sqrtf(sa / (float)width + eps);
  fb = 1.f / sqrtf(sb / (float)width + eps);
}

}  // namespace mll
