// Sampling on the device: greedy, temperature and top-k, one block per logits row, or a cluster of eight for a
// large vocabulary.
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


// ---------------------------------------------------------------------------------------------------- //
// Sampling over a large vocabulary: the eight blocks of a thread-block cluster share one row.  Every
// thread keeps VPT consecutive logits of the row in registers (block r the r-th eighth, thread t of it
// the t-th run of VPT), so the row is read from memory once, and whatever runs over the candidates in
// id order (the cumulative weights, the lowest ids among equal logits) is a scan over threads and then
// over blocks.  One block per row (above) reads its 128,256 logits several times with 4-byte or
// scattered loads: 60 us (temperature) and 190 us (top-k) a decode step at eight rows; these take a tenth.
// ---------------------------------------------------------------------------------------------------- //
constexpr int SC_CLUSTER = 8;
constexpr int SC_THREADS = 512;

__device__ __forceinline__ int block_exclusive_scan_int(int v, int* scratch, int* total) {
  // scratch: 33 ints; fixed order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    scratch[lane] = wi - w;
    if (lane == 31) scratch[32] = wi;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

// The thread's VPT logits of row `row` (ids first .. first + VPT - 1, those at or beyond `end` read as -inf);
// returns whether one of them is not finite.
template <int VPT>
__device__ __forceinline__ bool load_run(const float* __restrict__ row, int first, int end, bool vector_ok, float (&v)[VPT]) {
  bool nonfinite = false;
  if (vector_ok && first + VPT <= end) {
#pragma unroll
    for (int j = 0; j < VPT; j += 4) {
      const float4 x = *reinterpret_cast<const float4*>(row + first + j);
      v[j] = x.x;
      v[j + 1] = x.y;
      v[j + 2] = x.z;
      v[j + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < VPT; ++j) v[j] = first + j < end ? row[first + j] : -INFINITY;
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (first + j < end && !isfinite(v[j])) nonfinite = true;
  return nonfinite;
}

// How a row is cut: block `rank` takes ids [begin, end), a multiple of four of them.
__device__ __forceinline__ void cluster_slice(int vocab, int rank, int& begin, int& end) {
  const int per = ((vocab + SC_CLUSTER * 4 - 1) / (SC_CLUSTER * 4)) * 4;
  begin = min(vocab, rank * per);
  end = min(vocab, begin + per);
}

// Temperature sampling over the whole vocabulary, candidates in id order (the rule of sample_temperature_kernel).
// Every block takes its weights relative to its own maximum; after one cluster barrier each block knows all
// eight (maximum, sum) pairs and with them the row's maximum, the total and the sum before its own share.  The
// thread whose run holds the threshold reports its token to block 0 (the lowest id wins), which writes it out
// after the second barrier.
template <int VPT>
__global__ void __cluster_dims__(SC_CLUSTER, 1, 1) __launch_bounds__(SC_THREADS, (VPT <= 32 ? 2 : 1))
sample_temperature_cluster_kernel(const float* __restrict__ logits, int vocab, float temperature,
                                  unsigned long long seed, const int* __restrict__ request,
                                  const int* __restrict__ step, int* __restrict__ tokens, int* __restrict__ status,
                                  MllDeviceErrorWords errors) {
  __shared__ float fscratch[33];
  __shared__ int iscratch[32];
  __shared__ float blk_max, blk_total;
  __shared__ int cl_pick, cl_bad;  // block 0's are the cluster's
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int row_index = blockIdx.y, tid = threadIdx.x;
  const float* row = logits + (size_t)row_index * vocab;
  int begin, end;
  cluster_slice(vocab, rank, begin, end);
  const int first = begin + tid * VPT;
  float v[VPT];
  const bool nonfinite = load_run<VPT>(row, first, end, vocab % 4 == 0 && ((uintptr_t)logits & 15) == 0, v);
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < VPT; ++j) mx = fmaxf(mx, v[j]);
  mx = block_max(mx, fscratch);
  const int any_bad = __syncthreads_or(nonfinite ? 1 : 0);
  const float inv_t = 1.f / temperature;
  float mine = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    v[j] = (first + j < end && v[j] > -INFINITY) ? expf((v[j] - mx) * inv_t) : 0.f;  // the weights, from here on
    mine += v[j];
  }
  float total;
  const float before = block_exclusive_scan(mine, fscratch, &total);
  if (tid == 0) {
    blk_max = mx;
    blk_total = total;
    cl_pick = 0x7fffffff;
    cl_bad = 0;
  }
  cluster.sync();  // every block's maximum and sum stand
  float row_max = -INFINITY;
#pragma unroll
  for (int r = 0; r < SC_CLUSTER; ++r) row_max = fmaxf(row_max, *cluster.map_shared_rank(&blk_max, r));
  float base = 0.f, grand = 0.f, scale = 0.f;
#pragma unroll
  for (int r = 0; r < SC_CLUSTER; ++r) {
    const float m = *cluster.map_shared_rank(&blk_max, r);
    const float f = m > -INFINITY ? expf((m - row_max) * inv_t) : 0.f;  // block r's weights relative to the row's maximum
    const float t = *cluster.map_shared_rank(&blk_total, r) * f;
    if (r < rank) base += t;
    if (r == rank) scale = f;
    grand += t;
  }
  const float u = uniform01(seed, request[row_index], step[row_index]);
  const float threshold = u * grand;
  const int owner = block_min_int((first < end && threshold <= base + (before + mine) * scale) ? tid : 0x7fffffff, iscratch);
  if (tid == owner) {
    float cum = base + before * scale;
    int pick = min(end, first + VPT) - 1;
    bool found = false;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      cum += v[j] * scale;
      if (!found && first + j < end && threshold <= cum) {
        pick = first + j;
        found = true;
      }
    }
    atomicMin(cluster.map_shared_rank(&cl_pick, 0), pick);  // ids rise with the rank: the first block that holds it wins
  }
  if (tid == 0 && any_bad) atomicOr(cluster.map_shared_rank(&cl_bad, 0), 1);
  cluster.sync();  // the candidates and flags are in block 0's shared memory
  if (rank == 0 && tid == 0) {
    tokens[row_index] = cl_pick == 0x7fffffff ? vocab - 1 : cl_pick;
    status[row_index] = cl_bad | (row_index == 0 ? take_error_bits(errors) : 0);
  }
}

constexpr int SC_BITS0 = 11, SC_BITS1 = 11, SC_BITS2 = 10;  // radix digits of the three selection passes
constexpr int SC_BINS = 1 << SC_BITS0;
constexpr int SC_CAND = 1024;

// Top-k (k <= 1024) then temperature sampling over the kept candidates in descending order, equal logits by
// lower id (the rule of sample_top_k_kernel).  The k-th largest key is narrowed down by a radix selection over the
// registers, 11, 11 and 10 bits at a time; after each pass every block sums the eight histograms through
// distributed shared memory and finds the digit for itself (two histogram buffers in turn, so one cluster barrier
// a pass).  As soon as no more than 1,024 keys are left at or above the digit's lower bound - with a few dozen
// kept out of 128,256 that is after the first pass - they all go to block 0, which sorts them and draws among the
// first k.  Only when more than 1,024 keys tie with the k-th does the exact rule need the counts of every block.
template <int VPT>
__global__ void __cluster_dims__(SC_CLUSTER, 1, 1) __launch_bounds__(SC_THREADS, (VPT <= 32 ? 2 : 1))
sample_top_k_cluster_kernel(const float* __restrict__ logits, int vocab, int top_k, float temperature,
                            unsigned long long seed, const int* __restrict__ request, const int* __restrict__ step,
                            int* __restrict__ tokens, int* __restrict__ status, MllDeviceErrorWords errors) {
  __shared__ unsigned long long cand[SC_CAND];  // used in block 0
  __shared__ int hist[2][SC_BINS];
  __shared__ float fscratch[33];
  __shared__ int iscratch[33];
  __shared__ unsigned sel_prefix;
  __shared__ int sel_remaining, sel_at_or_above;
  __shared__ int blk_greater, blk_equal;
  __shared__ int cl_count, cl_bad;              // block 0's are the cluster's
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int row_index = blockIdx.y, tid = threadIdx.x;
  const float* row = logits + (size_t)row_index * vocab;
  int begin, end;
  cluster_slice(vocab, rank, begin, end);
  const int first = begin + tid * VPT;
  unsigned key[VPT];
  int any_bad;
  {
    float v[VPT];
    const bool nonfinite = load_run<VPT>(row, first, end, vocab % 4 == 0 && ((uintptr_t)logits & 15) == 0, v);
#pragma unroll
    for (int j = 0; j < VPT; ++j) key[j] = order_key(v[j]);
    any_bad = __syncthreads_or(nonfinite ? 1 : 0);
  }
  for (int i = tid; i < SC_CAND; i += SC_THREADS) cand[i] = 0ull;
  if (tid == 0) {
    cl_count = 0;
    cl_bad = 0;
  }
  unsigned prefix = 0;       // the digits of the k-th key found so far
  int remaining = top_k;     // its rank among the keys that share them
  int at_or_above = vocab;   // keys at or above the lower bound that the digits give
  int passes = 0;
  for (; passes < 3 && at_or_above > SC_CAND; ++passes) {
    const int bits = passes == 0 ? SC_BITS0 : passes == 1 ? SC_BITS1 : SC_BITS2;
    const int shift = passes == 0 ? SC_BITS1 + SC_BITS2 : passes == 1 ? SC_BITS2 : 0;
    const int bins = 1 << bits;
    const unsigned mask = passes == 0 ? 0u : (0xffffffffu << (shift + bits));
    int* mine_hist = hist[passes & 1];  // the peers read pass p's buffer before they arrive at pass p + 1's barrier
    for (int i = tid; i < bins; i += SC_THREADS) mine_hist[i] = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < VPT; ++j)
      if (first + j < end && (key[j] & mask) == prefix) atomicAdd(&mine_hist[(key[j] >> shift) & (unsigned)(bins - 1)], 1);
    cluster.sync();  // every block's histogram stands (block-wide barrier included)
    // thread t sums bins[bins - 1 - per t - i], i < per, over the blocks: a scan over the threads then counts from the top
    const int per = bins / SC_THREADS;
    int c[SC_BINS / SC_THREADS];
    int mine = 0;
#pragma unroll
    for (int i = 0; i < SC_BINS / SC_THREADS; ++i) {
      c[i] = 0;
      if (i < per) {
        const int bin = bins - 1 - (tid * per + i);
#pragma unroll
        for (int r = 0; r < SC_CLUSTER; ++r) c[i] += cluster.map_shared_rank(mine_hist, r)[bin];
      }
      mine += c[i];
    }
    int total;
    int above = block_exclusive_scan_int(mine, iscratch, &total);
    if (above < remaining && remaining <= above + mine) {  // exactly one thread: the k-th key falls into its bins
#pragma unroll
      for (int i = 0; i < SC_BINS / SC_THREADS; ++i) {
        if (i < per && above < remaining) {
          const int bin = bins - 1 - (tid * per + i);
          if (remaining <= above + c[i]) {
            sel_prefix = prefix | ((unsigned)bin << shift);
            sel_remaining = remaining - above;
            sel_at_or_above = (top_k - remaining) + above + c[i];
            above = remaining;  // done
          } else {
            above += c[i];
          }
        }
      }
    }
    __syncthreads();
    prefix = sel_prefix;
    remaining = sel_remaining;
    at_or_above = sel_at_or_above;
  }
  unsigned long long* out = cluster.map_shared_rank(cand, 0);
  int n_cand;
  if (at_or_above <= SC_CAND) {
    // every key at or above the lower bound: the order in which they arrive does not matter, block 0 sorts them
    n_cand = at_or_above;
    int n = 0;
#pragma unroll
    for (int j = 0; j < VPT; ++j) n += first + j < end && key[j] >= prefix;
    if (n > 0) {
      int at = atomicAdd(cluster.map_shared_rank(&cl_count, 0), n);
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (first + j < end && key[j] >= prefix)
          out[at++] = ((unsigned long long)key[j] << 32) | (unsigned)(0xffffffffu - (unsigned)(first + j));
    }
  } else {
    // more than 1,024 keys equal to the k-th (all three passes are done: prefix is that key): the greater ones
    // and, of the equal ones, those with the lowest ids
    n_cand = top_k;
    const unsigned kth = prefix;
    const int need_equal = remaining;
    int n_greater = 0, n_equal = 0;
#pragma unroll
    for (int j = 0; j < VPT; ++j)
      if (first + j < end) {
        n_greater += key[j] > kth;
        n_equal += key[j] == kth;
      }
    int total_g, total_e;
    int pos_g = block_exclusive_scan_int(n_greater, iscratch, &total_g);
    int pos_e = block_exclusive_scan_int(n_equal, iscratch, &total_e);
    if (tid == 0) {
      blk_greater = total_g;
      blk_equal = total_e;
    }
    cluster.sync();  // every block's counts stand (the branch is the same for the whole cluster)
    int all_greater = 0;
#pragma unroll
    for (int r = 0; r < SC_CLUSTER; ++r) {
      const int g = *cluster.map_shared_rank(&blk_greater, r), e = *cluster.map_shared_rank(&blk_equal, r);
      if (r < rank) {
        pos_g += g;
        pos_e += e;
      }
      all_greater += g;
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j)
      if (first + j < end) {
        const unsigned long long packed = ((unsigned long long)key[j] << 32) | (unsigned)(0xffffffffu - (unsigned)(first + j));
        if (key[j] > kth) {
          out[pos_g++] = packed;
        } else if (key[j] == kth) {
          if (pos_e < need_equal) out[all_greater + pos_e] = packed;
          ++pos_e;
        }
      }
  }
  if (tid == 0 && any_bad) atomicOr(cluster.map_shared_rank(&cl_bad, 0), 1);
  cluster.sync();  // the candidates are in block 0's shared memory; the peers are done
  if (rank != 0) return;

  // bitonic sort of the first `width` entries, descending; unused entries are 0 and sink to the end
  int width = 2;
  while (width < n_cand) width <<= 1;
  for (int size = 2; size <= width; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < width; i += SC_THREADS) {
        const int partner = i ^ stride;
        if (partner > i) {
          const unsigned long long x = cand[i], y = cand[partner];
          const bool descending = (i & size) == 0;
          if (descending ? x < y : x > y) {
            cand[i] = y;
            cand[partner] = x;
          }
        }
      }
      __syncthreads();
    }
  }
  const int kept = top_k;  // the first k of the sorted candidates
  const float mx = key_value((unsigned)(cand[0] >> 32));
  const float inv_t = 1.f / temperature;
  // thread t holds entries 2 t and 2 t + 1 of the sorted list
  const float w0 = 2 * tid < kept ? expf((key_value((unsigned)(cand[2 * tid] >> 32)) - mx) * inv_t) : 0.f;
  const float w1 = 2 * tid + 1 < kept ? expf((key_value((unsigned)(cand[2 * tid + 1] >> 32)) - mx) * inv_t) : 0.f;
  float total;
  const float before = block_exclusive_scan(w0 + w1, fscratch, &total);
  const float u = uniform01(seed, request[row_index], step[row_index]);
  const float threshold = u * total;
  int mine = 0x7fffffff;
  if (2 * tid < kept && threshold <= before + w0) mine = 2 * tid;
  else if (2 * tid + 1 < kept && threshold <= before + w0 + w1) mine = 2 * tid + 1;
  const int pick = block_min_int(mine, iscratch);
  if (tid == 0) {
    const int at = pick == 0x7fffffff ? kept - 1 : pick;
    tokens[row_index] = (int)(0xffffffffu - (unsigned)(cand[at] & 0xffffffffull));
    status[row_index] = cl_bad | (row_index == 0 ? take_error_bits(errors) : 0);
  }
}

// Logits a thread of the cluster kernels keeps for a vocabulary (16, 32 or 64: a block's share of the row, a
// multiple of four, spread over its threads), or 0 where the one-block kernels run (small or huge vocabularies).
inline int sample_cluster_run(int vocab) {
  if (vocab < 8192) return 0;
  const long long share = (((long long)vocab + SC_CLUSTER * 4 - 1) / (SC_CLUSTER * 4)) * 4;
  if (share <= 16ll * SC_THREADS) return 16;
  if (share <= 32ll * SC_THREADS) return 32;
  if (share <= 64ll * SC_THREADS) return 64;
  return 0;
}

// How many of a kernel's clusters of SC_CLUSTER blocks the device holds at once (0 if the query fails).
template <typename Kernel>
int sample_clusters_resident(Kernel kernel) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(SC_CLUSTER, 1);
  config.blockDim = dim3(SC_THREADS);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SC_CLUSTER;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

template <int VPT>
void launch_sample_cluster(const float* logits, int n_rows, int vocab, float temperature, int top_k,
                           unsigned long long seed, const int* request, const int* step, int* tokens, int* status,
                           const MllDeviceErrorWords& errors, cudaStream_t stream) {
  if (top_k == 0)
    MLL_LAUNCH((sample_temperature_cluster_kernel<VPT>), dim3(SC_CLUSTER, n_rows), SC_THREADS, 0, stream, logits, vocab,
               temperature, seed, request, step, tokens, status, errors);
  else
    MLL_LAUNCH((sample_top_k_cluster_kernel<VPT>), dim3(SC_CLUSTER, n_rows), SC_THREADS, 0, stream, logits, vocab, top_k,
               temperature, seed, request, step, tokens, status, errors);
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

// Clusters (one per row) of the large-vocabulary sampling kernel for this vocabulary that are resident at once:
// top_k == 0 the temperature kernel, else the top-k kernel; 0 where the one-block kernels run.
MLL_API int mll_sample_resident_rows(int vocab, int top_k) {
  const int run = mll::sample_cluster_run(vocab);
  if (run == 0) return 0;
  if (run == 16)
    return top_k == 0 ? mll::sample_clusters_resident(mll::sample_temperature_cluster_kernel<16>)
                      : mll::sample_clusters_resident(mll::sample_top_k_cluster_kernel<16>);
  if (run == 32)
    return top_k == 0 ? mll::sample_clusters_resident(mll::sample_temperature_cluster_kernel<32>)
                      : mll::sample_clusters_resident(mll::sample_top_k_cluster_kernel<32>);
  return top_k == 0 ? mll::sample_clusters_resident(mll::sample_temperature_cluster_kernel<64>)
                    : mll::sample_clusters_resident(mll::sample_top_k_cluster_kernel<64>);
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
  const int run = n_rows <= 65535 ? mll::sample_cluster_run(vocab) : 0;
  if (run != 0) {
    // a cluster per row, the row in registers
    if (run == 16)
      mll::launch_sample_cluster<16>(logits, n_rows, vocab, temperature, top_k, seed, request, step, tokens, status, errors, stream);
    else if (run == 32)
      mll::launch_sample_cluster<32>(logits, n_rows, vocab, temperature, top_k, seed, request, step, tokens, status, errors, stream);
    else
      mll::launch_sample_cluster<64>(logits, n_rows, vocab, temperature, top_k, seed, request, step, tokens, status, errors, stream);
  } else if (top_k == 0) {
    MLL_LAUNCH((mll::sample_temperature_kernel), n_rows, mll::SAMPLE_THREADS, 0, stream, logits, vocab, temperature, seed, request, step, tokens, status, errors);
  } else {
    MLL_LAUNCH((mll::sample_top_k_kernel), n_rows, mll::SAMPLE_THREADS, 0, stream, logits, vocab, top_k, temperature, seed, request, step, tokens, status, errors);
  }
  MLL_LAUNCH_CHECK();
  return 0;
}
