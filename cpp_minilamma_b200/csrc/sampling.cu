// Sampling on the device: greedy, temperature and top-k, one block per logits row.
//
// Rules of the reference's CPU sampler (src/sampler.cc):
//   * greedy returns the first index of the maximum (:31-41);
//   * temperature sampling draws u in [0, 1), weights w_i = exp((l_i - max) / T) and
//     returns the first candidate whose cumulative w / sum reaches u, else the last (:42-79);
//   * top-k keeps the k largest logits and walks them in descending order (:110-134);
//     equal logits are ordered by lower id here (the reference leaves that open).
// The reference draws u from std::mt19937; here u is a pure function of
// (seed, request, step) - three chained splitmix64 rounds - so that a request's tokens do
// not depend on its place in a batch.  Non-finite logits (:10-19) set bit 0 of status[row].
// The sampling kernel is the last kernel of a step, and its status words are what the host reads with
// the tokens: the block of row 0 therefore also reads and clears the error flags of the kernels that
// can give up (device_error.h) and passes them on in bits 8-11 of status[0].
#include <cooperative_groups.h>

#include "common.cuh"
#include "device_error.h"

namespace cg = cooperative_groups;

namespace mll {

__device__ __forceinline__ int take_error_bits(const MllDeviceErrorWords& errors) {
  int bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (errors.word[i] != nullptr && *(volatile int*)errors.word[i] != 0) {
      atomicExch(errors.word[i], 0);
      bits |= 0x100 << i;
    }
  return bits;
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ float uniform01(unsigned long long seed, int request, int step) {
  unsigned long long z = mix64(seed);
  z = mix64(z ^ (unsigned long long)(long long)request);
  z = mix64(z ^ (unsigned long long)(long long)step);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // larger value wins; equal values: lower index wins
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

constexpr int SAMPLE_THREADS = 1024;

// Exclusive prefix sum over one value per thread (fixed order); returns the exclusive
// prefix and stores the block total in *total.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_exclusive_scan(float v, float* scratch, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float w = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0.f;
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    scratch[lane] = wi - w;  // exclusive prefix of the warp totals
    if (lane == 31) scratch[32] = wi;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

__device__ __forceinline__ int block_min_int(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int r = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = min(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ tokens, int* __restrict__ status,
              MllDeviceErrorWords errors) {
  __shared__ Best warp_best[32];
  __shared__ int bad;
  const float* row = logits + (size_t)blockIdx.x * vocab;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  Best best{-INFINITY, 0x7fffffff};
  bool nonfinite = false;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) nonfinite = true;
    if (v > best.v) best = Best{v, i};
  }
  if (nonfinite) bad = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? warp_best[threadIdx.x] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (threadIdx.x == 0) {
      tokens[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
      status[blockIdx.x] = bad | (blockIdx.x == 0 ? take_error_bits(errors) : 0);
    }
  }
}

// Greedy over a large vocabulary: the eight blocks of a thread-block cluster share one row, each scans an
// eighth of it with 16-byte loads (four in flight per thread), and block 0 picks among the eight
// candidates through distributed shared memory.  One block per row reads its 128,256 logits one
// 4-byte load after the other: 48 us for eight rows, a fixed cost of every decode step; this takes 4 us.
constexpr int ARGMAX_CLUSTER = 8;
constexpr int ARGMAX_THREADS = 512;

__global__ void __cluster_dims__(ARGMAX_CLUSTER, 1, 1) __launch_bounds__(ARGMAX_THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ tokens, int* __restrict__ status,
                      MllDeviceErrorWords errors) {
  __shared__ Best warp_best[ARGMAX_THREADS / 32];
  __shared__ int warp_bad[ARGMAX_THREADS / 32];
  __shared__ Best block_best;
  __shared__ int block_bad;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int row_index = blockIdx.y;
  const float* row = logits + (size_t)row_index * vocab;
  const int per = ((vocab + ARGMAX_CLUSTER * 4 - 1) / (ARGMAX_CLUSTER * 4)) * 4;  // a multiple of four
  const int begin = min(vocab, rank * per), end = min(vocab, begin + per);
  Best best{-INFINITY, 0x7fffffff};
  bool nonfinite = false;
  auto take = [&](float v, int i) {
    if (!isfinite(v)) nonfinite = true;
    if (v > best.v) best = Best{v, i};  // indices rise within a thread: the first of equal values stays
  };
  if (vocab % 4 == 0 && ((uintptr_t)logits & 15) == 0) {
    const float4* p = reinterpret_cast<const float4*>(row + begin);
    const int n4 = (end - begin) >> 2;
    int i = threadIdx.x;
    for (; i + 3 * ARGMAX_THREADS < n4; i += 4 * ARGMAX_THREADS) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = p[i + u * ARGMAX_THREADS];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int at = begin + 4 * (i + u * ARGMAX_THREADS);
        take(v[u].x, at);
        take(v[u].y, at + 1);
        take(v[u].z, at + 2);
        take(v[u].w, at + 3);
      }
    }
    for (; i < n4; i += ARGMAX_THREADS) {
      const float4 v = p[i];
      const int at = begin + 4 * i;
      take(v.x, at);
      take(v.y, at + 1);
      take(v.z, at + 2);
      take(v.w, at + 3);
    }
  } else {
    for (int i = begin + threadIdx.x; i < end; i += ARGMAX_THREADS) take(row[i], i);
  }
  int bad = __any_sync(0xffffffffu, nonfinite) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if ((threadIdx.x & 31) == 0) {
    warp_best[threadIdx.x >> 5] = best;
    warp_bad[threadIdx.x >> 5] = bad;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const bool in = threadIdx.x < ARGMAX_THREADS / 32;
    best = in ? warp_best[threadIdx.x] : Best{-INFINITY, 0x7fffffff};
    bad = __any_sync(0xffffffffu, in && warp_bad[threadIdx.x] != 0) ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (threadIdx.x == 0) {
      block_best = best;
      block_bad = bad;
    }
  }
  cluster.sync();  // every block's candidate is in its shared memory
  if (rank == 0 && threadIdx.x < 32) {
    const bool in = threadIdx.x < ARGMAX_CLUSTER;
    best = in ? *cluster.map_shared_rank(&block_best, threadIdx.x) : Best{-INFINITY, 0x7fffffff};
    bad = __any_sync(0xffffffffu, in && *cluster.map_shared_rank(&block_bad, in ? threadIdx.x : 0) != 0) ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (threadIdx.x == 0) {
      tokens[row_index] = best.i == 0x7fffffff ? 0 : best.i;
      status[row_index] = bad | (row_index == 0 ? take_error_bits(errors) : 0);
    }
  }
  cluster.sync();  // block 0 has read its peers' shared memory
}

// Temperature sampling over the whole vocabulary, candidates in id order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_temperature_kernel(const float* __restrict__ logits, int vocab, float temperature,
                          unsigned long long seed, const int* __restrict__ request,
                          const int* __restrict__ step, int* __restrict__ tokens, int* __restrict__ status,
                          MllDeviceErrorWords errors) {
  __shared__ float fscratch[33];
  __shared__ int iscratch[32];
  __shared__ int bad;
  const float* row = logits + (size_t)blockIdx.x * vocab;
  const int tid = threadIdx.x;
  if (tid == 0) bad = 0;
  float mx = -INFINITY;
  bool nonfinite = false;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) nonfinite = true;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, fscratch);
  if (nonfinite) bad = 1;
  // each thread owns a contiguous chunk so that prefix sums follow the id order
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
  const float inv_t = 1.f / temperature;
  float mine = 0.f;
  for (int i = begin; i < end; ++i) mine += expf((row[i] - mx) * inv_t);
  float total;
  const float before = block_exclusive_scan(mine, fscratch, &total);
  const float u = uniform01(seed, request[blockIdx.x], step[blockIdx.x]);
  const float threshold = u * total;
  const int owner = block_min_int((end > begin && threshold <= before + mine) ? tid : 0x7fffffff, iscratch);
  if (owner == 0x7fffffff) {
    if (tid == 0) tokens[blockIdx.x] = vocab - 1;
  } else if (tid == owner) {
    float cum = before;
    int pick = end - 1;
    for (int i = begin; i < end; ++i) {
      cum += expf((row[i] - mx) * inv_t);
      if (threshold <= cum) {
        pick = i;
        break;
      }
    }
    tokens[blockIdx.x] = pick;
  }
  __syncthreads();
  if (tid == 0) status[blockIdx.x] = bad | (blockIdx.x == 0 ? take_error_bits(errors) : 0);
}

__device__ __forceinline__ unsigned order_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Top-k (k <= 1024) then temperature sampling over the kept candidates in descending order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_top_k_kernel(const float* __restrict__ logits, int vocab, int top_k, float temperature,
                    unsigned long long seed, const int* __restrict__ request, const int* __restrict__ step,
                    int* __restrict__ tokens, int* __restrict__ status, MllDeviceErrorWords errors) {
  __shared__ unsigned long long cand[SAMPLE_THREADS];
  __shared__ int hist[256];
  __shared__ float fscratch[33];
  __shared__ int iscratch[32];
  __shared__ unsigned sel_prefix;
  __shared__ int sel_remaining, bad;
  const float* row = logits + (size_t)blockIdx.x * vocab;
  const int tid = threadIdx.x;
  if (tid == 0) {
    sel_prefix = 0;
    sel_remaining = top_k;
    bad = 0;
  }
  cand[tid] = 0ull;
  __syncthreads();

  // radix select of the k-th largest key, 8 bits at a time from the top
  bool nonfinite = false;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = sel_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (pass == 0 && !isfinite(v)) nonfinite = true;
      const unsigned k = order_key(v);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int remaining = sel_remaining, bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= remaining) break;
        remaining -= hist[bin];
      }
      sel_prefix = prefix | ((unsigned)bin << shift);
      sel_remaining = remaining;
    }
    __syncthreads();
  }
  if (nonfinite) bad = 1;
  const unsigned kth = sel_prefix;       // key of the k-th largest logit
  const int need_equal = sel_remaining;  // how many logits equal to it are kept (lowest ids)

  // gather: contiguous chunks per thread keep the id order
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
  int n_greater = 0, n_equal = 0;
  for (int i = begin; i < end; ++i) {
    const unsigned k = order_key(row[i]);
    n_greater += k > kth;
    n_equal += k == kth;
  }
  // integer scans through the float helper would lose exactness; scan as ints
  auto scan_int = [&](int v, int* total) {
    const int lane = tid & 31, warp = tid >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    __syncthreads();
    if (lane == 31) iscratch[warp] = incl;
    __syncthreads();
    int base = 0, sum = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      if (w < warp) base += iscratch[w];
      sum += iscratch[w];
    }
    *total = sum;
    return base + incl - v;
  };
  int total_greater, total_equal;
  int pos_g = scan_int(n_greater, &total_greater);
  int pos_e = scan_int(n_equal, &total_equal);
  for (int i = begin; i < end; ++i) {
    const unsigned k = order_key(row[i]);
    const unsigned long long packed = ((unsigned long long)k << 32) | (unsigned)(0xffffffffu - (unsigned)i);
    if (k > kth) {
      cand[pos_g++] = packed;
    } else if (k == kth) {
      if (pos_e < need_equal) cand[total_greater + pos_e] = packed;
      ++pos_e;
    }
  }
  __syncthreads();

  // bitonic sort, descending; unused entries are 0 and sink to the end
  for (int size = 2; size <= SAMPLE_THREADS; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int partner = tid ^ stride;
      if (partner > tid) {
        const unsigned long long x = cand[tid], y = cand[partner];
        const bool descending = (tid & size) == 0;
        if (descending ? x < y : x > y) {
          cand[tid] = y;
          cand[partner] = x;
        }
      }
      __syncthreads();
    }
  }

  const int kept = top_k;  // == total_greater + need_equal
  const float mx = key_value((unsigned)(cand[0] >> 32));
  const float inv_t = 1.f / temperature;
  const float w = tid < kept ? expf((key_value((unsigned)(cand[tid] >> 32)) - mx) * inv_t) : 0.f;
  float total;
  const float before = block_exclusive_scan(w, fscratch, &total);
  const float u = uniform01(seed, request[blockIdx.x], step[blockIdx.x]);
  const float threshold = u * total;
  const int pick = block_min_int((tid < kept && threshold <= before + w) ? tid : 0x7fffffff, iscratch);
  if (tid == 0) {
    const int at = pick == 0x7fffffff ? kept - 1 : pick;
    tokens[blockIdx.x] = (int)(0xffffffffu - (unsigned)(cand[at] & 0xffffffffull));
    status[blockIdx.x] = bad | (blockIdx.x == 0 ? take_error_bits(errors) : 0);
  }
}

}  // namespace mll

// logits: float32 [n_rows, vocab]; tokens, status: int32 [n_rows].
MLL_API int mll_argmax(const float* logits, int n_rows, int vocab, int* tokens, int* status,
                       cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && vocab > 0, "argmax: bad sizes rows=%d vocab=%d", n_rows, vocab);
  if (n_rows == 0) return 0;
  MllDeviceErrorWords errors;
  mll_device_error_words(&errors);  // all null if they cannot be had: the kernel then passes nothing on
  if (vocab >= 8192 && n_rows <= 65535)
    MLL_LAUNCH((mll::argmax_cluster_kernel), dim3(mll::ARGMAX_CLUSTER, n_rows), mll::ARGMAX_THREADS, 0, stream, logits, vocab,
               tokens, status, errors);
  else
    MLL_LAUNCH((mll::argmax_kernel), n_rows, mll::SAMPLE_THREADS, 0, stream, logits, vocab, tokens, status, errors);
  MLL_LAUNCH_CHECK();
  return 0;
}

// temperature > 0; top_k == 0 samples from the whole vocabulary, 2 <= top_k <= 1024 from the
// k largest logits.  request/step: int32 [n_rows] random-number counters.
MLL_API int mll_sample(const float* logits, int n_rows, int vocab, float temperature, int top_k,
                       unsigned long long seed, const int* request, const int* step, int* tokens,
                       int* status, cudaStream_t stream) {
  MLL_REQUIRE(n_rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
  MLL_REQUIRE(temperature > 0.f && isfinite(temperature), "sample: temperature must be finite and > 0");
  MLL_REQUIRE(top_k >= 0, "sample: top_k must be >= 0");
  if (top_k > vocab) top_k = vocab;
  MLL_REQUIRE(top_k <= mll::SAMPLE_THREADS,
              "sample: top_k %d above the supported maximum of %d", top_k, mll::SAMPLE_THREADS);
  if (n_rows == 0) return 0;
  MllDeviceErrorWords errors;
  mll_device_error_words(&errors);
  if (top_k == 0)
    MLL_LAUNCH((mll::sample_temperature_kernel), n_rows, mll::SAMPLE_THREADS, 0, stream, logits, vocab, temperature, seed, request, step, tokens, status, errors);
  else
    MLL_LAUNCH((mll::sample_top_k_kernel), n_rows, mll::SAMPLE_THREADS, 0, stream, logits, vocab, top_k, temperature, seed, request, step, tokens, status, errors);
  MLL_LAUNCH_CHECK();
  return 0;
}
