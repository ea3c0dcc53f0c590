// Next-token selection over float logits [rows, vocab]: argmax, and temperature
// sampling with joint top-k / top-p.
//
// Semantics (reference: src/engine/sampling.rs:241-269, :409-428): temperature
// <= 0 or top_p == 0 is argmax; else probs = softmax(logits / T) in float; both
// cut-offs are taken on that one distribution and ties at a cut-off are kept:
// the k-th largest probability, and the probability at which the descending
// cumulative sum first reaches top_p; what lies below either is dropped, the
// rest is renormalised and one token is drawn.
//
// The reference draws with a library sampler fed from libtorch's global Philox
// state (src/engine/sampling_bridge.cpp:20-28), so a request's tokens depend on
// what else was sampled before.  Here the uniform number is Philox4x32-10 keyed
// by the row's (seed, counter) alone and the draw is an inverse CDF in vocabulary
// order: the same request, seed and output index give the same token in any batch.
//
// The joint cut-off needs no sort: "keep p >= t" with
//   t = max{ t : count(p >= t) >= k  or  mass(p >= t) >= top_p }
// is found by bisection over the bit patterns of positive floats.
#include <cooperative_groups.h>
#include <math.h>

#include "common.cuh"

namespace cg = cooperative_groups;

struct SampleRow {          // 32 bytes, filled by the host
  float temperature;
  int top_k;
  float top_p;
  unsigned seed_lo, seed_hi;
  unsigned counter;
  int pad0, pad1;
};

constexpr int THREADS = 1024;

__device__ __forceinline__ void philox_round(unsigned (&c)[4], unsigned k0, unsigned k1) {
  const unsigned long long p0 = 0xD2511F53ull * c[0], p1 = 0xCD9E8D57ull * c[2];
  const unsigned hi0 = static_cast<unsigned>(p0 >> 32), lo0 = static_cast<unsigned>(p0);
  const unsigned hi1 = static_cast<unsigned>(p1 >> 32), lo1 = static_cast<unsigned>(p1);
  c[0] = hi1 ^ c[1] ^ k0; c[1] = lo1; c[2] = hi0 ^ c[3] ^ k1; c[3] = lo0;
}

__device__ __forceinline__ float philox_uniform(unsigned seed_lo, unsigned seed_hi, unsigned counter) {
  unsigned c[4] = {counter, 0u, 0x1234567u, 0u};
  unsigned k0 = seed_lo, k1 = seed_hi;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);     // [0, 1)
}

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;      // ties: the lowest index
}

__device__ MaxIdx block_argmax(const float* __restrict__ row, int vocab, MaxIdx* sh, int begin = 0) {
  MaxIdx best = {-INFINITY, 0x7fffffff};
  // four logits a load where the row allows it (its start and `begin` on 16-byte steps), the rest one by one
  const bool wide = reinterpret_cast<uintptr_t>(row) % 16 == 0 && begin % 4 == 0;
  const int wide_end = wide ? begin + (vocab - begin) / 4 * 4 : begin;
  for (int i = begin + 4 * threadIdx.x; i < wide_end; i += 4 * blockDim.x) {
    const float4 v4 = *reinterpret_cast<const float4*>(row + i);
    const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (!(v[e] != v[e])) best = better(best, MaxIdx{v[e], i + e});   // NaN never wins
  }
  for (int i = wide_end + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (!(v != v)) best = better(best, MaxIdx{v, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    MaxIdx b = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other = {__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
    if (threadIdx.x == 0) sh[32] = b;
  }
  __syncthreads();
  return sh[32];
}

// A large vocabulary is shared by a cluster of ARGMAX_CLUSTER CTAs per row: every CTA scans one slice, sends
// its best (value, index) to the first CTA of the cluster through distributed shared memory, and that one
// picks the winner (ties: the lowest index, as in the one-CTA kernel).
constexpr int ARGMAX_CLUSTER = 8;

__global__ void __launch_bounds__(THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int* __restrict__ out, int* err) {
  __shared__ MaxIdx sh[33];
  __shared__ MaxIdx partial[ARGMAX_CLUSTER];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int row = blockIdx.x / ARGMAX_CLUSTER;
  const int slice = (vocab + ARGMAX_CLUSTER - 1) / ARGMAX_CLUSTER;
  const int begin = min(vocab, rank * slice), end = min(vocab, begin + slice);
  const MaxIdx b = block_argmax(logits + row * row_stride, end, sh, begin);
  if (threadIdx.x == 0) *cluster.map_shared_rank(&partial[rank], 0) = b;
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    MaxIdx best = partial[0];
    for (int r = 1; r < ARGMAX_CLUSTER; ++r) best = better(best, partial[r]);
    if (best.i >= vocab) { atomicOr(err, B200_ERR_SAMPLING); out[row] = -1; }
    else out[row] = best.i;
  }
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int* __restrict__ out, int* err) {
  __shared__ MaxIdx sh[33];
  const MaxIdx b = block_argmax(logits + blockIdx.x * row_stride, vocab, sh);
  if (threadIdx.x == 0) {
    if (b.i >= vocab) { atomicOr(err, B200_ERR_SAMPLING); out[blockIdx.x] = -1; }
    else out[blockIdx.x] = b.i;
  }
}

__device__ __forceinline__ float2 block_sum2(float2 v, float2* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { v.x += __shfl_xor_sync(0xffffffffu, v.x, o); v.y += __shfl_xor_sync(0xffffffffu, v.y, o); }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float2 t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : make_float2(0.f, 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { t.x += __shfl_xor_sync(0xffffffffu, t.x, o); t.y += __shfl_xor_sync(0xffffffffu, t.y, o); }
    if (threadIdx.x == 0) sh[32] = t;
  }
  __syncthreads();
  return sh[32];
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, const SampleRow* __restrict__ params,
              int* __restrict__ out, float* __restrict__ uniforms, int* err) {
  __shared__ MaxIdx shm[33];
  __shared__ float2 sh2[33];
  __shared__ float scan[THREADS];
  __shared__ int chosen;
  const float* row = logits + blockIdx.x * row_stride;
  const SampleRow p = params[blockIdx.x];
  const MaxIdx top = block_argmax(row, vocab, shm);
  if (top.i >= vocab) {
    if (threadIdx.x == 0) { atomicOr(err, B200_ERR_SAMPLING); out[blockIdx.x] = -1; }
    return;
  }
  if (!(p.temperature > 0.0f) || p.top_p == 0.0f) {
    if (threadIdx.x == 0) out[blockIdx.x] = top.i;
    return;
  }
  const float inv_t = 1.0f / p.temperature;
  // Z = sum exp((l - max) / T)
  float z = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += expf((row[i] - top.v) * inv_t);
  const float zsum = block_sum2(make_float2(z, 0.0f), sh2).x;
  const float inv_z = 1.0f / zsum;
  const int k = (p.top_k > 0 && p.top_k < vocab) ? p.top_k : vocab;
  const bool use_p = p.top_p < 1.0f;
  float cut = 0.0f;
  if (k < vocab || use_p) {
    // Bisection over float bit patterns in (0, 1]: the largest t whose keep-set still
    // has k members or top_p of the mass.
    unsigned lo = 0u, hi = __float_as_uint(1.0f);          // pred(lo) is true, pred(hi + 1) is false
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      const float t = __uint_as_float(mid);
      float cnt = 0.0f, mass = 0.0f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float pr = expf((row[i] - top.v) * inv_t) * inv_z;
        if (pr >= t) { cnt += 1.0f; mass += pr; }
      }
      const float2 tot = block_sum2(make_float2(cnt, mass), sh2);
      const bool pred = (k < vocab && tot.x >= static_cast<float>(k)) || (use_p && tot.y >= p.top_p);
      if (pred) lo = mid; else hi = mid - 1u;
    }
    cut = __uint_as_float(lo);
  }
  // Inverse CDF in vocabulary order over the kept probabilities.
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, static_cast<int>(threadIdx.x) * chunk), end = min(vocab, begin + chunk);
  float local = 0.0f;
  for (int i = begin; i < end; ++i) {
    const float pr = expf((row[i] - top.v) * inv_t) * inv_z;
    if (pr >= cut) local += pr;
  }
  scan[threadIdx.x] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.0f;
    for (int t = 0; t < blockDim.x; ++t) total += scan[t];
    const float u = philox_uniform(p.seed_lo, p.seed_hi, p.counter);
    if (uniforms) uniforms[blockIdx.x] = u;
    const float target = u * total;
    float run = 0.0f;
    int owner = -1;
    for (int t = 0; t < blockDim.x; ++t) {
      if (scan[t] > 0.0f) {
        owner = t;                                  // the last thread with mass takes what rounding leaves over
        if (run + scan[t] > target) break;
        run += scan[t];
      }
    }
    // Walk the owner's chunk.
    int pick = -1;
    if (owner >= 0) {
      const int b = min(vocab, owner * chunk), e = min(vocab, b + chunk);
      for (int i = b; i < e; ++i) {
        const float pr = expf((row[i] - top.v) * inv_t) * inv_z;
        if (pr >= cut) {
          pick = i;
          if (run + pr > target) break;
          run += pr;
        }
      }
    }
    chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (chosen < 0) { atomicOr(err, B200_ERR_SAMPLING); out[blockIdx.x] = -1; }
    else out[blockIdx.x] = chosen;
  }
}

B200_EXPORT int b200_argmax(const float* logits, long long row_stride, int rows, int vocab, int* out, int* err,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return B200_BAD_SIZE;
  if (vocab >= 16384 && rows <= 4096) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(rows * ARGMAX_CLUSTER);
    config.blockDim = dim3(THREADS);
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ARGMAX_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&config, argmax_cluster_kernel, logits, row_stride, vocab, out, err);
    return e == cudaSuccess ? b200_check_launch() : static_cast<int>(e);
  }
  argmax_kernel<<<rows, THREADS, 0, stream>>>(logits, row_stride, vocab, out, err);
  return b200_check_launch();
}

// `params`: one 32-byte SampleRow per row, on the device.  `uniforms` (optional) receives the uniform
// number that each sampling row drew.
B200_EXPORT int b200_sample(const float* logits, long long row_stride, int rows, int vocab, const void* params,
                            int* out, float* uniforms, int* err, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return B200_BAD_SIZE;
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, row_stride, vocab, static_cast<const SampleRow*>(params),
                                              out, uniforms, err);
  return b200_check_launch();
}
