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

// Rows whose width is a multiple of 4 and at most 4 * NV * blockDim: every thread keeps
// its share of the row in registers and issues all its loads before the first use, so the
// kernel costs one memory latency instead of one per loop trip (decode has very few rows).
template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename DeltaT, typename OutT, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ x, const DeltaT* __restrict__ delta,
                       const float* __restrict__ weight, OutT* __restrict__ out,
                       const int* __restrict__ rows, int width, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + (size_t)src * width;
  const DeltaT* dr = delta ? delta + (size_t)src * width : nullptr;
  const int groups = width >> 2;
  float4 v[NV], w[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) {
      v[k] = load4<float>(xr + 4 * g);
      w[k] = load4<float>(weight + 4 * g);
    }
  }
  if (dr) {
    float4 dl[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) dl[k] = load4<DeltaT>(dr + 4 * g);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int g = threadIdx.x + k * 256;
      if (g < groups) {
        v[k].x += dl[k].x; v[k].y += dl[k].y; v[k].z += dl[k].z; v[k].w += dl[k].w;
        if (!rows) store4(xr + 4 * g, v[k]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.f / sqrtf(ss / (float)width + eps);
  OutT* o = out + (size_t)r * width;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int g = threadIdx.x + k * 256;
    if (g < groups)
      store4(o + 4 * g, make_float4(v[k].x * scale * w[k].x, v[k].y * scale * w[k].y, v[k].z * scale * w[k].z,
                                    v[k].w * scale * w[k].w));
  }
}

template <typename DeltaT, typename OutT>
int launch_add_rmsnorm(float* x, const void* delta, const float* weight, void* out, const int* rows,
                       int n_rows, int width, float eps, cudaStream_t stream) {
  const bool aligned = width % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                       ((uintptr_t)out % 8 == 0) && (!delta || (uintptr_t)delta % 8 == 0);
  if (aligned && width <= 4 * 256 * 8) {
    const int groups = width / 4;
    if (groups <= 256 * 2)
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 2>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight,
                 (OutT*)out, rows, width, eps);
    else if (groups <= 256 * 4)
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 4>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight,
                 (OutT*)out, rows, width, eps);
    else
      MLL_LAUNCH((add_rmsnorm_vec_kernel<DeltaT, OutT, 8>), n_rows, 256, 0, stream, x, (const DeltaT*)delta, weight,
                 (OutT*)out, rows, width, eps);
    MLL_LAUNCH_CHECK();
    return 0;
  }
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
  MLL_LAUNCH((kernel), n_rows, threads, smem, stream, x, (const DeltaT*)delta, weight, (OutT*)out, rows, width, eps);
  MLL_LAUNCH_CHECK();
  return 0;
}

// Finishes a norm whose rows were left without their factor (RowNormIn), for a product that cannot do
// it itself: out[m, i] = values[m, i] * factor(m).  One block per row.
__global__ void apply_row_norm_kernel(const __nv_bfloat16* __restrict__ values, RowNormIn in,
                                      __nv_bfloat16* __restrict__ out, int width) {
  __shared__ float factor;
  const int m = blockIdx.x;
  if (threadIdx.x < 32) {
    const float f = row_norm_factor<32>(in.sumsq + (size_t)m * in.stride, in.partials, width, in.eps, threadIdx.x,
                                        0xffffffffu);
    if (threadIdx.x == 0) factor = f;
  }
  __syncthreads();
  const float f = factor;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[(size_t)m * width + i] = __float2bfloat16_rn(__bfloat162float(values[(size_t)m * width + i]) * f);
}

}  // namespace mll

// values, out: bfloat16 [n_rows, width]; sumsq: float32 [n_rows, stride] with `partials` sums of squares
// per row; out = values / sqrt(sum / width + eps).
MLL_API int mll_apply_row_norm(const void* values, const float* sumsq, int partials, int stride, float eps, void* out,
                               int n_rows, int width, cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0 && partials >= 1 && stride >= partials && eps >= 0.f,
              "apply_row_norm: bad sizes rows=%d width=%d partials=%d stride=%d", n_rows, width, partials, stride);
  if (n_rows == 0) return 0;
  MLL_LAUNCH((mll::apply_row_norm_kernel), n_rows, 256, 0, stream, (const __nv_bfloat16*)values,
             mll::RowNormIn{sumsq, partials, stride, eps}, (__nv_bfloat16*)out, width);
  MLL_LAUNCH_CHECK();
  return 0;
}

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
