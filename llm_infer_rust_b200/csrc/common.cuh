// Small device utilities shared by the kernels of this package (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes of the C interface
enum : int { B200_F32 = 0, B200_BF16 = 1 };

// error bits that kernels OR into the engine's device error word
enum : int {
  B200_ERR_TOKEN_RANGE = 1,      // token id outside the embedding table
  B200_ERR_SLOT_RANGE = 2,       // cache slot outside the pool
  B200_ERR_POSITION_RANGE = 4,   // position beyond the rotary table
  B200_ERR_SAMPLING = 8,         // no valid token could be drawn
  B200_ERR_WAIT_TIMEOUT = 16,    // a bounded wait inside a kernel ran out
};

// return codes of launchers: 0 ok, > 0 a cudaError_t, < 0 refused arguments
enum : int { B200_BAD_DTYPE = -1, B200_BAD_SIZE = -2, B200_BAD_ALIGN = -3 };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.  The order of the additions is
// fixed by the thread layout, so a row's sum does not depend on other rows.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// 16-byte vector of elements of T, converted to floats on load.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void load(const float* p, float* out) {
    float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void load(const __nv_bfloat16* p, float* out) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// N consecutive elements of T as floats, fetched with 16-byte loads (8-byte for four bfloat16): N * sizeof(T) is 8,
// 16 or 32 bytes and p is aligned to the load's size.
template <typename T, int N>
__device__ __forceinline__ void load_floats(const T* p, float* out) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + i);
      out[i] = v.x; out[i + 1] = v.y; out[i + 2] = v.z; out[i + 3] = v.w;
    }
  } else if constexpr (N == 8) {
    Vec16<T>::load(p, out);
  } else {
    static_assert(N == 4, "four or eight elements");
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
  }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  // Copies 16 bytes, or writes 16 zero bytes when !valid (src-size 0).
  uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// One poll of an mbarrier's phase (the instruction itself may suspend the thread for a short, bounded while).
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Waits for a phase of the barrier, but never for ever: after about a second it gives up, flags the engine's
// error word and returns false (the caller's results are then meaningless, not hung).  Reading the global timer
// costs far more than a poll and would sit between the barrier's completion and the waiter's next instruction,
// so the clock is looked at only on every 64th failed poll.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t start = 0;
  for (uint32_t polls = 1;; ++polls) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((polls & 63u) == 0u) {
      const uint64_t now = global_ns();
      if (start == 0) start = now;
      if (now - start > 1000000000ull) {
        atomicOr(err, B200_ERR_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}

// Programmatic dependent launch.  A kernel launched with b200_launch (below) may be scheduled while the kernel
// before it in the stream is still running: what does not depend on that kernel (barrier set-up, fetching
// weights) then overlaps its tail.  EVERY block of such a kernel calls pdl_wait() before it touches anything
// the earlier kernel may have written, and before it exits: the wait returns when the earlier kernel has
// finished and its writes are visible (at once, when the launch carried no such dependency).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// Lets the kernel after this one be scheduled from now on (it still waits in its own pdl_wait()).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

static inline int b200_check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Launches `kernel` so that it may overlap the tail of the kernel before it (see pdl_wait), optionally as
// clusters of `cluster_x` blocks.
template <typename... KernelArgs, typename... Args>
static inline int b200_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = 1;
  ++n;
  if (cluster_x > 0) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  config.attrs = attr;
  config.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  return e == cudaSuccess ? b200_check_launch() : static_cast<int>(e);
}
