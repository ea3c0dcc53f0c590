// C[M, N] = A[M, K] . W[N, K]^T in true 32-bit: FFMA on CUDA cores only, no
// tensor cores and no reduced-precision mode.  This is the matrix product of the
// float32 engine (the reference's float path goes through libtorch matmul:
// src/layers/linear.rs:5-7).
//
// Every output element is accumulated over k = 0, 1, ..., K-1 in that order,
// whatever M and N are and wherever the element sits in a tile, so a token's
// result is bit-identical however the batch around it is cut.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

template <bool VEC>
__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;          // this thread loads row lrow, k offsets lk..lk+3
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
    const int am = m0 + lrow, wn = n0 + lrow, kk = k0 + lk;
    if (VEC) {
      if (am < M && kk < K) { const float4 v = *reinterpret_cast<const float4*>(A + static_cast<size_t>(am) * K + kk); a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w; }
      if (wn < N && kk < K) { const float4 v = *reinterpret_cast<const float4*>(W + static_cast<size_t>(wn) * K + kk); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (am < M && kk + i < K) a[i] = A[static_cast<size_t>(am) * K + kk + i];
        if (wn < N && kk + i < K) w[i] = W[static_cast<size_t>(wn) * K + kk + i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) { As[lk + i][lrow] = a[i]; Ws[lk + i][lrow] = w[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[static_cast<size_t>(m) * N + n] = acc[i][j];
    }
  }
}

B200_EXPORT int b200_gemm_f32(const float* a, const float* w, float* c, int m, int n, int k, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0) return B200_BAD_SIZE;
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  const bool vec = (k % 4 == 0) && (reinterpret_cast<uintptr_t>(a) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0);
  if (vec) sgemm_nt_kernel<true><<<grid, 256, 0, stream>>>(a, w, c, m, n, k);
  else sgemm_nt_kernel<false><<<grid, 256, 0, stream>>>(a, w, c, m, n, k);
  return b200_check_launch();
}
