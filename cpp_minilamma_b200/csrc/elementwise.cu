// Embedding gather, dtype casts and the SwiGLU activation.
//
// Replaces the reference's EmbeddingKernel, SiluKernel and ElementWiseMulKernel
// (src/cuda_ops.cu:165-192) with batched kernels; SiLU and the product are one pass.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void mll_set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

MLL_API const char* mll_last_error() { return g_error; }

thread_local cudaError_t mll_launch_status = cudaSuccess;

// Identifies the build; the Python side checks it after loading the library.
MLL_API int mll_abi_version() { return 27; }

// Cache positions per page, for the Python side to check against its own constant.
MLL_API int mll_page() { return MLL_PAGE; }

int mll_sm_count() {
  constexpr int kMaxDevices = 64;
  static int known[kMaxDevices] = {0};
  int device = 0, count = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    cudaGetLastError();
    device = 0;
  }
  if (known[device] == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1) {
      cudaGetLastError();
      count = 148;  // a B200, the device this library is written for
    }
    known[device] = count;
  }
  return known[device];
}

MLL_API int mll_multiprocessor_count() { return mll_sm_count(); }

namespace mll {

// x[t, :] = float(table[token[t], :]); the residual stream is float32.
template <typename TableT>
__global__ void embedding_kernel(const int* __restrict__ tokens, const TableT* __restrict__ table,
                                 float* __restrict__ x, int width) {
  const int t = blockIdx.x;
  const TableT* row = table + (size_t)tokens[t] * width;
  float* out = x + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = to_float(row[i]);
}

// the same for a bfloat16 table whose rows are multiples of 8 elements: 16-byte loads, one per thread and pass
__global__ void embedding_bf16_vec8_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                           float* __restrict__ x, int width) {
  const int t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)tokens[t] * width);
  float4* out = reinterpret_cast<float4*>(x + (size_t)t * width);
  for (int i = threadIdx.x; i < (width >> 3); i += blockDim.x) {
    const uint4 raw = row[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    const float2 c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
    out[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    out[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
  }
}

template <typename In, typename Out>
__global__ void cast_kernel(const In* __restrict__ in, Out* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = from_float<Out>(to_float(in[i]));
}

// out[t, i] = silu(gate) * up.  `gu` rows hold gate and up either as two halves
// ([gate(0..I) | up(0..I)], block == 0) or interleaved in blocks of `block` columns
// ([gate(0..b) | up(0..b) | gate(b..2b) | ...]); I is a multiple of `block` then.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int tokens,
                              int inter, int block) {
  const size_t total = (size_t)tokens * inter;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const int t = (int)(idx / inter), i = (int)(idx % inter);
    const T* row = gu + (size_t)t * 2 * inter;
    float g, u;
    if (block == 0) {
      g = to_float(row[i]);
      u = to_float(row[inter + i]);
    } else {
      const int b = i / block, r = i % block;
      g = to_float(row[(size_t)b * 2 * block + r]);
      u = to_float(row[(size_t)b * 2 * block + block + r]);
    }
    const float act = g / (1.f + expf(-g));
    out[idx] = from_float<T>(act * u);
  }
}

// The same over groups of 8 consecutive outputs (inter % 8 == 0, block 0 or 8): 16- or
// 32-byte loads of a gate group and its up group, one vector store.
template <typename T>
struct Pack8;
template <>
struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};
template <>
struct Pack8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// silu(g) * u.  The float32 path keeps the accurate exponential and division; a bfloat16 result
// is rounded to 8 bits anyway, so it takes the fast ones (a prefill step spends a tenth of its
// non-GEMM time here, and the accurate forms make the kernel compute-bound).
template <typename T>
__device__ __forceinline__ float silu_mul(float g, float u);
template <>
__device__ __forceinline__ float silu_mul<float>(float g, float u) { return g / (1.f + expf(-g)) * u; }
template <>
__device__ __forceinline__ float silu_mul<__nv_bfloat16>(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

template <typename T>
__global__ void swiglu_vec8_kernel(const T* __restrict__ gu, T* __restrict__ out, int tokens, int inter, int block) {
  const int groups = inter >> 3;
  const size_t total = (size_t)tokens * groups;
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) {
    const int t = (int)(idx / groups), b = (int)(idx % groups);
    const T* row = gu + (size_t)t * 2 * inter;
    const T* gp = block ? row + (size_t)b * 16 : row + (size_t)b * 8;
    const T* up = block ? gp + 8 : row + inter + (size_t)b * 8;
    float g[8], u[8], r[8];
    Pack8<T>::load(gp, g);
    Pack8<T>::load(up, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = silu_mul<T>(g[i], u[i]);
    Pack8<T>::store(out + (size_t)t * inter + (size_t)b * 8, r);
  }
}

// x[t, i] += bias[i] (bias float32, sum in float32)
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, size_t total, int width) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < total; idx += stride) x[idx] = from_float<T>(to_float(x[idx]) + bias[idx % width]);
}

// As swiglu_vec8_kernel (bfloat16, gate and up interleaved in blocks of 8), for rows of gate/up that still lack their
// RMS norm's factor (the product ran on x * w_norm): both are multiplied by the row's factor first.  One row per
// blockIdx.y; warp 0 computes the factor from the row's partial sums of squares.
__global__ void swiglu_rows_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter,
                                   int block, RowNormIn in, int width) {
  __shared__ float factor;
  const int m = blockIdx.y;
  if (threadIdx.x < 32) {
    const float f = row_norm_factor<32>(in.sumsq + (size_t)m * in.stride, in.partials, width, in.eps, threadIdx.x,
                                        0xffffffffu);
    if (threadIdx.x == 0) factor = f;
  }
  __syncthreads();
  const float f = factor;
  const int groups = inter >> 3;
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= groups) return;
  const __nv_bfloat16* row = gu + (size_t)m * 2 * inter;
  const __nv_bfloat16* gp = block ? row + (size_t)b * 16 : row + (size_t)b * 8;
  const __nv_bfloat16* up = block ? gp + 8 : row + inter + (size_t)b * 8;
  float g[8], u[8], r[8];
  Pack8<__nv_bfloat16>::load(gp, g);
  Pack8<__nv_bfloat16>::load(up, u);
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = silu_mul<__nv_bfloat16>(g[i] * f, u[i] * f);
  Pack8<__nv_bfloat16>::store(out + (size_t)m * inter + (size_t)b * 8, r);
}

// table[staged[r][0]][:] = staged[r][1 : 1 + width] for r < n_rows: rows of a block table that changed on
// the host, brought over inside the step's index buffer.
__global__ void scatter_rows_kernel(int* __restrict__ table, const int* __restrict__ staged, int width, int table_rows) {
  const int* row = staged + (size_t)blockIdx.x * (width + 1);
  const int target = row[0];
  if (target < 0 || target >= table_rows) return;
  for (int i = threadIdx.x; i < width; i += blockDim.x) table[(size_t)target * width + i] = row[1 + i];
}

// dst[i] = src[index[i]] for i < n; an index outside [0, n_src) gives 0.
__global__ void gather_int32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ index, int n,
                                    int n_src) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int at = index[i];
  dst[i] = at >= 0 && at < n_src ? src[at] : 0;
}

}  // namespace mll

// dst: int32 [n]; src: int32 [n_src]; index: int32 [n].  dst and src must not overlap.
MLL_API int mll_gather_int32(int* dst, const int* src, const int* index, int n, int n_src, cudaStream_t stream) {
  MLL_REQUIRE(n >= 0 && n_src > 0, "gather_int32: bad sizes n=%d n_src=%d", n, n_src);
  if (n == 0) return 0;
  MLL_LAUNCH((mll::gather_int32_kernel), (n + 127) / 128, 128, 0, stream, dst, src, index, n, n_src);
  MLL_LAUNCH_CHECK();
  return 0;
}

// table: int32 [table_rows, width]; staged: int32 [n_rows, 1 + width], column 0 the row of `table` to replace.
MLL_API int mll_scatter_rows(int* table, const int* staged, int n_rows, int width, int table_rows, cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0 && table_rows > 0, "scatter_rows: bad sizes rows=%d width=%d", n_rows, width);
  if (n_rows == 0) return 0;
  MLL_LAUNCH((mll::scatter_rows_kernel), n_rows, width >= 128 ? 128 : 32, 0, stream, table, staged, width, table_rows);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_add_bias(void* x, const float* bias, int dtype, int n_rows, int width, cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && width > 0, "add_bias: bad sizes rows=%d width=%d", n_rows, width);
  if (n_rows == 0) return 0;
  const size_t total = (size_t)n_rows * width;
  long long blocks = (long long)((total + 255) / 256);
  if (blocks > mll_sm_count() * 16) blocks = mll_sm_count() * 16;
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::add_bias_kernel<float>), (int)blocks, 256, 0, stream, (float*)x, bias, total, width);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::add_bias_kernel<__nv_bfloat16>), (int)blocks, 256, 0, stream, (__nv_bfloat16*)x, bias, total, width);
  else
    MLL_REQUIRE(false, "add_bias: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_embedding(const int* tokens, const void* table, int table_dtype, float* x,
                          int n_tokens, int width, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && width > 0, "embedding: bad sizes tokens=%d width=%d", n_tokens, width);
  if (n_tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == MLL_F32)
    MLL_LAUNCH((mll::embedding_kernel<float>), n_tokens, threads, 0, stream, tokens, (const float*)table, x, width);
  else if (table_dtype == MLL_BF16 && width % 8 == 0 && ((uintptr_t)table % 16 == 0) && ((uintptr_t)x % 16 == 0))
    MLL_LAUNCH((mll::embedding_bf16_vec8_kernel), n_tokens, width >= 2048 ? 256 : 64, 0, stream, tokens,
               (const __nv_bfloat16*)table, x, width);
  else if (table_dtype == MLL_BF16)
    MLL_LAUNCH((mll::embedding_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, tokens, (const __nv_bfloat16*)table, x, width);
  else
    MLL_REQUIRE(false, "embedding: unknown table dtype %d", table_dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                     cudaStream_t stream) {
  MLL_REQUIRE(n >= 0, "cast: negative size");
  if (n == 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > mll_sm_count() * 16) blocks = mll_sm_count() * 16;
  if (in_dtype == MLL_F32 && out_dtype == MLL_BF16)
    MLL_LAUNCH((mll::cast_kernel<float, __nv_bfloat16>), (int)blocks, threads, 0, stream, (const float*)in, (__nv_bfloat16*)out, (size_t)n);
  else if (in_dtype == MLL_BF16 && out_dtype == MLL_F32)
    MLL_LAUNCH((mll::cast_kernel<__nv_bfloat16, float>), (int)blocks, threads, 0, stream, (const __nv_bfloat16*)in, (float*)out, (size_t)n);
  else
    MLL_REQUIRE(false, "cast: unsupported dtype pair %d -> %d", in_dtype, out_dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}

// bfloat16 gu [n_tokens, 2 inter] (halves: block 0; blocks of 8: block 8) computed from rows that lack their RMS
// norm's factor 1 / sqrt(sum_p sumsq[m][p] / width + eps): out = silu(gate f) * (up f).
MLL_API int mll_swiglu_rows(const void* gu, void* out, int n_tokens, int inter, int block, const float* sumsq, int partials,
                            int stride, float eps, int width, cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && n_tokens <= 65535 && inter > 0 && inter % 8 == 0 && (block == 0 || block == 8),
              "swiglu_rows: bad sizes tokens=%d inter=%d block=%d", n_tokens, inter, block);
  MLL_REQUIRE(sumsq && partials >= 1 && stride >= partials && eps >= 0.f && width > 0,
              "swiglu_rows: partial sums: %d of stride %d", partials, stride);
  MLL_REQUIRE(((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0), "swiglu_rows: operands must be 16-byte aligned");
  if (n_tokens == 0) return 0;
  const int groups = inter / 8;
  MLL_LAUNCH((mll::swiglu_rows_kernel), dim3((groups + 255) / 256, n_tokens), 256, 0, stream, (const __nv_bfloat16*)gu,
             (__nv_bfloat16*)out, inter, block, mll::RowNormIn{sumsq, partials, stride, eps}, width);
  MLL_LAUNCH_CHECK();
  return 0;
}

MLL_API int mll_swiglu(const void* gu, void* out, int dtype, int n_tokens, int inter, int block,
                       cudaStream_t stream) {
  MLL_REQUIRE(n_tokens >= 0 && inter > 0, "swiglu: bad sizes tokens=%d inter=%d", n_tokens, inter);
  MLL_REQUIRE(block >= 0 && (block == 0 || inter % block == 0),
              "swiglu: intermediate size %d is not a multiple of the interleave block %d", inter, block);
  if (n_tokens == 0) return 0;
  const int threads = 256;
  const bool vec = inter % 8 == 0 && (block == 0 || block == 8) && ((uintptr_t)gu % 16 == 0) &&
                   ((uintptr_t)out % 16 == 0);
  if (vec) {
    long long groups = ((long long)n_tokens * (inter / 8) + threads - 1) / threads;
    if (groups > mll_sm_count() * 32) groups = mll_sm_count() * 32;
    if (dtype == MLL_F32)
      MLL_LAUNCH((mll::swiglu_vec8_kernel<float>), (int)groups, threads, 0, stream, (const float*)gu, (float*)out, n_tokens,
                                                                       inter, block);
    else if (dtype == MLL_BF16)
      MLL_LAUNCH((mll::swiglu_vec8_kernel<__nv_bfloat16>), (int)groups, threads, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens, inter, block);
    else
      MLL_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
    MLL_LAUNCH_CHECK();
    return 0;
  }
  long long blocks = ((long long)n_tokens * inter + threads - 1) / threads;
  if (blocks > mll_sm_count() * 32) blocks = mll_sm_count() * 32;
  if (dtype == MLL_F32)
    MLL_LAUNCH((mll::swiglu_kernel<float>), (int)blocks, threads, 0, stream, (const float*)gu, (float*)out, n_tokens, inter, block);
  else if (dtype == MLL_BF16)
    MLL_LAUNCH((mll::swiglu_kernel<__nv_bfloat16>), (int)blocks, threads, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n_tokens, inter, block);
  else
    MLL_REQUIRE(false, "swiglu: unknown dtype %d", dtype);
  MLL_LAUNCH_CHECK();
  return 0;
}
