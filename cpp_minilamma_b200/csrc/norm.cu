// RMSNorm fused with the residual add, and the gathered variant for the final norm.
//
//   x[t, :] += delta[t, :]            (float32 residual stream, updated in place)
//   out[t, i] = x[t, i] * w[i] / sqrt(mean_j(x[t, j]^2) + eps)
//
// The formula is the reference's (src/ops.cc:95-110; eps inside the root).  Its GPU
// version sums squares with float atomics (src/cuda_ops.cu:151-164), which is not
// reproducible; here every row is reduced by one block with a fixed tree, in float32.
#include "common.cuh"

namespace mll {

// One block per output row.  The row (after the add) is kept in shared memory between
// the two passes.  `rows` (optional) selects which rows of x are normalised: output row
// r reads x row rows[r]; the residual add is then not written back to x.
template <typename DeltaT, typename OutT>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta,
                                   const float* __restrict__ weight, OutT* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float row_buf[];
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      v += to_float(dr[i]);
      if (!rows) xr[i] = v;
    }
    row_buf[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.f / sqrtf(ss / (float)width + eps);
  OutT* o = out + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    o[i] = from_float<OutT>(row_buf[i] * scale * weight[i]);
}

template <typename DeltaT, typename OutT>
int launch_add_rmsnorm(float* x, const void* delta, const float* weight, void* out, const int* rows,
                       int n_rows, int width, float eps, cudaStream_t stream) {
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  const size_t smem = (size_t)width * sizeof(float);
  auto kernel = add_rmsnorm_kernel<DeltaT, OutT>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) {
      mll_set_error("rmsnorm: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
      return (int)err;
    }
  }
  kernel<<<n_rows, threads, smem, stream>>>(x, (const DeltaT*)delta, weight, (OutT*)out, rows, width, eps);
  MLL_LAUNCH_CHECK();
  return 0;
}

}  // namespace mll

// x: float32 [*, width] residual stream; delta: optional [*, width] of `act_dtype`;
// weight: float32 [width]; out: [n_rows, width] of `act_dtype`; rows: optional int32
// [n_rows] gather list.
MLL_API int mll_add_rmsnorm(float* x, const void* delta, const float* weight, void* out,
                            const int* rows, int act_dtype, int n_rows, int width, float eps,
                            cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
  MLL_REQUIRE(width <= 50 * 1024, "rmsnorm: width %d exceeds the 51200 floats one block can hold", width);
  MLL_REQUIRE(eps >= 0.f, "rmsnorm: eps must be non-negative");
  if (n_rows == 0) return 0;
  if (act_dtype == MLL_F32)
    return mll::launch_add_rmsnorm<float, float>(x, delta, weight, out, rows, n_rows, width, eps, stream);
  if (act_dtype == MLL_BF16)
    return mll::launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, delta, weight, out, rows, n_rows,
                                                                 width, eps, stream);
  MLL_REQUIRE(false, "rmsnorm: unknown dtype %d", act_dtype);
  return -1;
}
