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

// Launches `kernel` on `stream`; with programmatic dependent launch switched on
// (mll_set_pdl) the launch may begin while the previous kernel of the stream is still
// draining: every kernel of this library calls pdl_wait() before it touches anything that
// an earlier kernel wrote or still reads.  The outcome is picked up by MLL_LAUNCH_CHECK.
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
extern int mll_pdl_enabled;

namespace mll {

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  if (mll_pdl_enabled) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// Programmatic dependent launch: let the next kernel of the stream start its prologue now,
// and wait until everything earlier kernels wrote is complete and visible.  Both are
// no-ops for a kernel that was launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Start of a short kernel: nothing to overlap, so it lets the next kernel launch right away
// and waits for its own inputs.  Longer kernels call pdl_launch_dependents() after their main
// loop instead, so that the next kernel's prologue overlaps their tail and not their body.
__device__ __forceinline__ void pdl_begin() {
  pdl_launch_dependents();
  pdl_wait();
}
__device__ __forceinline__ void pdl_begin_long() { pdl_wait(); }

// A range of global memory (weights that a later kernel of the step will stream) that the
// blocks of a latency-bound kernel ask the L2 cache to fetch while they do their own work.
// Decode steps alternate kernels that wait on latencies with kernels that wait on HBM; the
// hints keep HBM busy during the former.  ptr is 16-byte aligned, bytes a multiple of 16.
struct Prefetch {
  const void* ptr;
  unsigned long long bytes;
};

// Called by one thread per block: block `block` of `blocks` requests every blocks-th 16 KB chunk.
__device__ __forceinline__ void l2_prefetch_chunks(const Prefetch& pf, unsigned block, unsigned blocks) {
  constexpr unsigned long long kChunk = 16384;
  const unsigned long long chunks = (pf.bytes + kChunk - 1) / kChunk;
  for (unsigned long long c = block; c < chunks; c += blocks) {
    const unsigned long long off = c * kChunk;
    const unsigned size = (unsigned)(pf.bytes - off < kChunk ? pf.bytes - off : kChunk);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"((const char*)pf.ptr + off), "r"(size) : "memory");
  }
}
__device__ __forceinline__ void l2_prefetch_by_grid(const Prefetch& pf) {
  if (pf.bytes == 0 || threadIdx.x != 0 || threadIdx.y != 0 || threadIdx.z != 0) return;
  const unsigned blocks = gridDim.x * gridDim.y * gridDim.z;
  const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  l2_prefetch_chunks(pf, block, blocks);
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

}  // namespace mll
