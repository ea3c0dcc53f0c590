// Row-wise and element-wise kernels: embedding gather, RMSNorm, residual
// add + RMSNorm, SiLU(gate) * up, dtype casts.
//
// Numerics (reference: src/layers/fused_ops.cu:49-106, :135-171): sums of
// squares, the mean, rsqrt, the residual sum and the activation are computed
// in float; a value is rounded once, when it is stored.  The residual add
// normalises the UNROUNDED float sum and stores the rounded sum as the new
// residual.  Each row is reduced by one block in an order fixed by the thread
// layout, so a row's result does not depend on which rows run beside it.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
template <typename TA, typename TW>
__global__ void embedding_kernel(TA* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int width, int vocab, int* err) {
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(err, B200_ERR_TOKEN_RANGE);
  const TW* src = table + static_cast<size_t>(ok ? id : 0) * width;
  TA* dst = out + static_cast<size_t>(row) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = ok ? from_f32<TA>(to_f32<TW>(src[i])) : from_f32<TA>(0.0f);
}

// ------------------------------------------------------------------ norms
// out[r] = rms_norm(x[src(r)] (+ residual[src(r)])) * w, src(r) = rows ? rows[r] : r.
// With ADD the rounded sum is written back to residual[src(r)] when write_residual != 0.
// `out` may be `x` itself when rows == nullptr.
template <typename TA, typename TW, bool ADD>
__global__ void rms_norm_kernel(TA* out, const TA* x, TA* residual, const TW* __restrict__ w,
                                const int* __restrict__ rows, int width, float eps, int write_residual) {
  extern __shared__ float row_buf[];          // width floats, then 33 for the reduction
  float* scratch = row_buf + width;
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * width;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_f32<TA>(x[src + i]);
    if (ADD) {
      v += to_f32<TA>(residual[src + i]);
      if (write_residual) residual[src + i] = from_f32<TA>(v);
    }
    row_buf[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float scale = rsqrtf(total / static_cast<float>(width) + eps);
  TA* dst = out + static_cast<size_t>(r) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = from_f32<TA>(row_buf[i] * scale * to_f32<TW>(w[i]));
}

// Rows whose width is a multiple of the 16-byte vector and at most 32 * VPL vectors: one WARP per row, the row's
// values stay in registers between the sum of squares and the scaling, loads and stores are 16 bytes wide.
// The sum runs over the lanes' partial sums in a fixed order, so a row's result does not depend on other rows.
template <typename TA, typename TW, bool ADD, int VPL>
__global__ void __launch_bounds__(256)
rms_norm_warp_kernel(TA* out, const TA* x, TA* residual, const TW* __restrict__ w, const int* __restrict__ rows,
                     int n_rows, int width, float eps, int write_residual) {
  constexpr int N = Vec16<TA>::N;
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * width;
  const int vectors = width / N;
  float v[VPL][N];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * N;
    if (i * 32 + lane < vectors) {
      Vec16<TA>::load(x + src + c, v[i]);
      if (ADD) {
        float b[N];
        Vec16<TA>::load(residual + src + c, b);
        __align__(16) TA rounded[N];
#pragma unroll
        for (int e = 0; e < N; ++e) { v[i][e] += b[e]; rounded[e] = from_f32<TA>(v[i][e]); }
        if (write_residual) *reinterpret_cast<uint4*>(residual + src + c) = *reinterpret_cast<const uint4*>(rounded);
      }
#pragma unroll
      for (int e = 0; e < N; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  const float scale = rsqrtf(ss / static_cast<float>(width) + eps);
  TA* dst = out + static_cast<size_t>(r) * width;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * 32 + lane) * N;
    if (i * 32 + lane < vectors) {
      __align__(16) TA y[N];
      float wv[N];
      load_floats<TW, N>(w + c, wv);
#pragma unroll
      for (int e = 0; e < N; ++e) y[e] = from_f32<TA>(v[i][e] * scale * wv[e]);
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(y);
    }
  }
}

// ------------------------------------------------------------------ SwiGLU activation
template <typename TA>
__global__ void silu_mul_kernel(TA* __restrict__ out, const TA* __restrict__ gate_up, int width,
                                size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / width, col = i - row * width;
    const float g = to_f32<TA>(gate_up[row * 2 * width + col]);
    const float u = to_f32<TA>(gate_up[row * 2 * width + width + col]);
    out[i] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
  }
}

// The same with 16-byte loads and stores: `width` is a multiple of the vector length and the pointers are aligned.
// A thread takes two vectors a turn, with all four loads in flight before the arithmetic.  bfloat16 results take
// the fast exponential and division (their error is far below the rounding to 8 bits); float32 takes the exact ones.
template <typename TA>
__device__ __forceinline__ float silu_times(float g, float u) {
  if constexpr (sizeof(TA) == 2) return __fdividef(g, 1.0f + __expf(-g)) * u;
  else return g / (1.0f + expf(-g)) * u;
}

template <typename TA>
__global__ void __launch_bounds__(256)
silu_mul_vec_kernel(TA* __restrict__ out, const TA* __restrict__ gate_up, int width, size_t vectors) {
  constexpr int N = Vec16<TA>::N;
  const int per_row = width / N;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < vectors; i0 += 2 * stride) {
    float g[2][N], u[2][N];
    size_t dst[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const size_t i = i0 + j * stride;
      if (i < vectors) {
        const size_t row = i / per_row;
        const int col = static_cast<int>(i - row * per_row) * N;
        Vec16<TA>::load(gate_up + row * 2 * width + col, g[j]);
        Vec16<TA>::load(gate_up + row * 2 * width + width + col, u[j]);
        dst[j] = row * width + col;
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      if (i0 + j * stride < vectors) {
        __align__(16) TA r[N];
#pragma unroll
        for (int e = 0; e < N; ++e) r[e] = from_f32<TA>(silu_times<TA>(g[j][e], u[j][e]));
        *reinterpret_cast<uint4*>(out + dst[j]) = *reinterpret_cast<const uint4*>(r);
      }
    }
  }
}

template <typename TO, typename TI>
__global__ void cast_kernel(TO* __restrict__ out, const TI* __restrict__ in, size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}

// ------------------------------------------------------------------ launchers
#define DISPATCH2(act, wt, CALL)                                                        \
  if (act == B200_F32 && wt == B200_F32) { CALL(float, float); }                        \
  else if (act == B200_BF16 && wt == B200_BF16) { CALL(__nv_bfloat16, __nv_bfloat16); } \
  else if (act == B200_BF16 && wt == B200_F32) { CALL(__nv_bfloat16, float); }          \
  else if (act == B200_F32 && wt == B200_BF16) { CALL(float, __nv_bfloat16); }          \
  else return B200_BAD_DTYPE;

B200_EXPORT int b200_embedding(void* out, const void* table, const int* ids, int tokens, int width,
                               int vocab, int act_dtype, int table_dtype, int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0 || vocab <= 0) return B200_BAD_SIZE;
#define CALL(TA, TW) embedding_kernel<TA, TW><<<tokens, 256, 0, stream>>>( \
    static_cast<TA*>(out), static_cast<const TW*>(table), ids, width, vocab, err)
  DISPATCH2(act_dtype, table_dtype, CALL)
#undef CALL
  return b200_check_launch();
}

B200_EXPORT int b200_rms_norm(void* out, const void* x, void* residual, const void* w, const int* rows,
                              int n_rows, int width, float eps, int write_residual, int act_dtype,
                              int w_dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  {
    // The warp-per-row kernel where it applies (16-byte aligned rows of at most 32 * 4 vectors).
    const int vec = act_dtype == B200_F32 ? 4 : 8;
    const bool aligned = reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(residual) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
    if (width % vec == 0 && width / vec <= 32 * 16 && aligned) {
      const int blocks = (n_rows + 7) / 8;
      const bool small = width / vec <= 32 * 4;
#define LAUNCHW(TA, TW, ADD, VPL)                                                                            \
      rms_norm_warp_kernel<TA, TW, ADD, VPL><<<blocks, 256, 0, stream>>>(static_cast<TA*>(out),               \
          static_cast<const TA*>(x), static_cast<TA*>(residual), static_cast<const TW*>(w), rows, n_rows, width, eps, \
          write_residual)
#define CALLW(TA, TW)                                                                                        \
      if (residual) { if (small) LAUNCHW(TA, TW, true, 4); else LAUNCHW(TA, TW, true, 16); }                 \
      else { if (small) LAUNCHW(TA, TW, false, 4); else LAUNCHW(TA, TW, false, 16); }
      DISPATCH2(act_dtype, w_dtype, CALLW)
#undef CALLW
#undef LAUNCHW
      return b200_check_launch();
    }
  }
  const size_t smem = (static_cast<size_t>(width) + 33) * sizeof(float);
  if (smem > 200 * 1024) return B200_BAD_SIZE;
  const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
#define CALL(TA, TW)                                                                                  \
  if (residual) {                                                                                     \
    if (smem > 48 * 1024) cudaFuncSetAttribute(rms_norm_kernel<TA, TW, true>,                         \
        cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                         \
    rms_norm_kernel<TA, TW, true><<<n_rows, threads, smem, stream>>>(static_cast<TA*>(out),           \
        static_cast<const TA*>(x), static_cast<TA*>(residual), static_cast<const TW*>(w), rows, width, \
        eps, write_residual);                                                                         \
  } else {                                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(rms_norm_kernel<TA, TW, false>,                        \
        cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                         \
    rms_norm_kernel<TA, TW, false><<<n_rows, threads, smem, stream>>>(static_cast<TA*>(out),          \
        static_cast<const TA*>(x), nullptr, static_cast<const TW*>(w), rows, width, eps, 0);          \
  }
  DISPATCH2(act_dtype, w_dtype, CALL)
#undef CALL
  return b200_check_launch();
}

B200_EXPORT int b200_silu_mul(void* out, const void* gate_up, int tokens, int width, int act_dtype,
                              cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (width <= 0) return B200_BAD_SIZE;
  const size_t total = static_cast<size_t>(tokens) * width;
  const int vec = act_dtype == B200_F32 ? 4 : 8;
  if (width % vec == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0) {
    const size_t vectors = total / vec;
    const int vblocks = static_cast<int>(min(static_cast<size_t>(148 * 16), (vectors + 511) / 512));
    if (act_dtype == B200_F32)
      silu_mul_vec_kernel<float><<<vblocks, 256, 0, stream>>>(static_cast<float*>(out), static_cast<const float*>(gate_up),
                                                              width, vectors);
    else if (act_dtype == B200_BF16)
      silu_mul_vec_kernel<__nv_bfloat16><<<vblocks, 256, 0, stream>>>(
          static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), width, vectors);
    else return B200_BAD_DTYPE;
    return b200_check_launch();
  }
  const int blocks = static_cast<int>(min(static_cast<size_t>(148 * 16), (total + 255) / 256));
  if (act_dtype == B200_F32)
    silu_mul_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(out),
                                                       static_cast<const float*>(gate_up), width, total);
  else if (act_dtype == B200_BF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), width, total);
  else return B200_BAD_DTYPE;
  return b200_check_launch();
}

B200_EXPORT int b200_cast(void* out, const void* in, long long total, int out_dtype, int in_dtype,
                          cudaStream_t stream) {
  if (total <= 0) return 0;
  const int blocks = static_cast<int>(min(static_cast<long long>(148 * 16), (total + 255) / 256));
#define CALL(TO, TI) cast_kernel<TO, TI><<<blocks, 256, 0, stream>>>( \
    static_cast<TO*>(out), static_cast<const TI*>(in), static_cast<size_t>(total))
  DISPATCH2(out_dtype, in_dtype, CALL)
#undef CALL
  return b200_check_launch();
}
