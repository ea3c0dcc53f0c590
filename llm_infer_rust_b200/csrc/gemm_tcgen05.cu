// C = A . W^T on the fifth-generation tensor cores, for many rows (prompt portions):
// A [M, K] and W [N, K] are bfloat16, row-major (K contiguous), the sums are float in tensor memory, C is bfloat16.
// Optionally the SwiGLU activation is the epilogue: W = [gate rows; up rows] ([2 I, K]) and the kernel writes
// silu(gate) * up ([M, I]) without the projection ever going to memory (reference: src/layers/mlp.rs:21-24,
// src/layers/fused_ops.cu:142-144; gate and up are rounded to bfloat16 first, as the unfused path stores them).
//
// The kernel is persistent (one CTA per SM walks over tiles) and tensor memory holds two accumulators, so the
// epilogue of a tile runs under the MMAs of the next.
// A tile is 128 rows x 256 columns (SwiGLU: 128 gate + the same 128 up columns):
//   warp 0      one lane feeds a ring of 4 stages with TMA: a box of A (128 rows x 64 k) and two boxes of W
//               (128 rows x 64 k each), 128-byte swizzle, 48 KB a stage, reported to the stage's `full` barrier;
//   warp 1      allocates 512 columns of tensor memory (two accumulators); one lane issues tcgen05.mma (M 128,
//               N 256, K 16; four per stage) from shared-memory descriptors, commits each stage to its `empty`
//               barrier and a tile's last one to the accumulator's `acc_full` barrier; frees the tensor memory
//               at the end;
//   warps 2-5   wait for `acc_full`, read their 32 lanes of tensor memory (tcgen05.ld, 32 columns at a time),
//               apply the epilogue, store bfloat16 rows and hand the accumulator back (`acc_empty`).
// Rows beyond M, columns beyond N and k beyond K are zero-filled by TMA and masked in the epilogue.
// Every wait is bounded by the clock; a wait that runs out flags the engine's error word, and every path still
// reaches the end of the kernel, where the tensor memory is given back.
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int B_BYTES = BN * BK * 2;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 48 KB
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;

enum : int { GEMM_PLAIN = 0, GEMM_SWIGLU = 1 };

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart (stride byte offset), leading byte offset 1 (not used by swizzled K-major tiles), descriptor
// version 1 (this architecture), layout type 2 (128-byte swizzle).  `addr` is the shared-memory byte address of
// the tile (1024-byte aligned) plus 32 bytes for every 16 k already consumed.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// Instruction descriptor: float accumulator, bfloat16 A and B, both K-major, N = 256, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((BM >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {      // the barrier is arrived on when all earlier MMAs are done
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
               "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent: CTA b works on tiles b, b + gridDim.x, ...  Tensor memory holds two accumulators of 256 columns,
// so the epilogue of one tile runs under the MMAs of the next (acc_full / acc_empty hand them over).
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap wmap,
                    bf16* __restrict__ out, int M, int N, int K, int mode, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;          // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM;
  const int nkb = (K + BK - 1) / BK;
  const int half = mode == GEMM_SWIGLU ? N / 2 : 0;                         // I
  const int cols = mode == GEMM_SWIGLU ? half : N;
  const int n_tiles = mode == GEMM_SWIGLU ? (cols + 127) / 128 : (cols + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {                                                          // the whole warp allocates tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(2 * TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                                                               // A comes from the kernel before this one

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                                           // k-blocks fetched so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int tile_m = tile % m_tiles, tile_n = tile / m_tiles;         // CTAs that run together share a W tile
        const int w_row0 = mode == GEMM_SWIGLU ? tile_n * 128 : tile_n * BN;
        const int w_row1 = mode == GEMM_SWIGLU ? half + tile_n * 128 : tile_n * BN + 128;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES, use = it / STAGES;
          if (use > 0 && !mbar_wait(empty + s, (use - 1) & 1, err)) { ok = false; break; }
          unsigned char* st = ring + s * STAGE_BYTES;
          mbar_expect_tx(full + s, STAGE_BYTES);
          tma_load_2d(st, &amap, kb * BK, tile_m * BM, full + s);
          tma_load_2d(st + A_BYTES, &wmap, kb * BK, w_row0, full + s);
          tma_load_2d(st + A_BYTES + B_BYTES / 2, &wmap, kb * BK, w_row1, full + s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1, use = local >> 1;
        if (use > 0) ok = mbar_wait(acc_empty + acc, (use - 1) & 1, err);     // the epilogue has read this accumulator
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_c = tmem_base + acc * TMEM_COLS;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(full + s, (it / STAGES) & 1, err);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_c, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);                                           // the stage is free when these MMAs have read it
        }
        umma_commit(acc_full + acc);                                        // the tile's sums are complete
      }
    }
  } else {
    // Epilogue: warp w reads lanes 32 (w mod 4) .. + 31 of tensor memory; a lane is one row of the tile.
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int tile_m = tile % m_tiles, tile_n = tile / m_tiles;
      const int acc = local & 1;
      const int row = tile_m * BM + quarter * 32 + lane;
      if (!mbar_wait(acc_full + acc, (local >> 1) & 1, err)) break;
      tc_fence_after();
      const uint32_t lane_base = tmem_base + acc * TMEM_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
      if (mode == GEMM_PLAIN) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld32(lane_base + c * 32, v);
          const int col0 = tile_n * BN + c * 32;
          if (row < M && col0 < N) {
            bf16* dst = out + static_cast<size_t>(row) * N + col0;
            if (col0 + 32 <= N && (N % 8) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __align__(16) bf16 r[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) r[e] = __float2bfloat16_rn(v[q * 8 + e]);
                *reinterpret_cast<uint4*>(dst + q * 8) = *reinterpret_cast<const uint4*>(r);
              }
            } else {
              for (int e = 0; e < 32 && col0 + e < N; ++e) dst[e] = __float2bfloat16_rn(v[e]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {                                       // gate columns c * 32 .., up columns 128 + c * 32 ..
          float g[32], u[32];
          tmem_ld32(lane_base + c * 32, g);
          tmem_ld32(lane_base + 128 + c * 32, u);
          const int col0 = tile_n * 128 + c * 32;
          if (row < M && col0 < half) {
            bf16* dst = out + static_cast<size_t>(row) * half + col0;
            __align__(16) bf16 r[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float gate = __bfloat162float(__float2bfloat16_rn(g[e]));
              const float up = __bfloat162float(__float2bfloat16_rn(u[e]));
              r[e] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
            }
            if (col0 + 32 <= half && (half % 8) == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = *reinterpret_cast<const uint4*>(r + q * 8);
            } else {
              for (int e = 0; e < 32 && col0 + e < half; ++e) dst[e] = r[e];
            }
          }
        }
      }
      tc_fence_before();                                                    // the loads of this accumulator are done
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + acc);
    }
  }
  // Everybody meets here on every path; then the allocating warp gives the tensor memory back.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes into `out_map` (128 bytes) the TMA descriptor of a row-major bfloat16 matrix [rows, cols], fetched in
// boxes of 128 rows x 64 columns with the 128-byte swizzle; what lies outside reads as zeros.
B200_EXPORT int b200_gemm_tensor_map(void* out_map, const void* matrix, long long rows, long long cols) {
  if (rows <= 0 || cols <= 0 || cols % 8 != 0) return B200_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(matrix) % 16 != 0) return B200_BAD_ALIGN;
  static EncodeTiledFn encode = nullptr;
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (fn == nullptr || found != cudaDriverEntryPointSuccess) return static_cast<int>(cudaErrorNotSupported);
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(bf16)};
  const cuuint32_t box[2] = {64u, 128u};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(matrix), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
  memcpy(out_map, &map, sizeof(map));
  return 0;
}

// out = a . w^T (mode 0: [m, n]) or silu(a . gate^T) * (a . up^T) (mode 1: w = [gate; up], out [m, n / 2]).
// `a_map`, `w_map`: descriptors of b200_gemm_tensor_map for a [m, k] and w [n, k].
B200_EXPORT int b200_gemm_tcgen05(const void* a_map, const void* w_map, void* out, int m, int n, int k, int mode, int* err,
                                  cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || k % 8 != 0 || (mode != GEMM_PLAIN && mode != GEMM_SWIGLU)) return B200_BAD_SIZE;
  if (mode == GEMM_SWIGLU && n % 2 != 0) return B200_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(out) % 16 != 0) return B200_BAD_ALIGN;
  const size_t smem = 1024 + static_cast<size_t>(STAGES) * STAGE_BYTES + (2 * STAGES + 4) * sizeof(uint64_t) + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  CUtensorMap amap, wmap;
  memcpy(&amap, a_map, sizeof(amap));
  memcpy(&wmap, w_map, sizeof(wmap));
  const int m_tiles = (m + BM - 1) / BM;
  const int cols = mode == GEMM_SWIGLU ? n / 2 : n;
  const int n_tiles = mode == GEMM_SWIGLU ? (cols + 127) / 128 : (cols + BN - 1) / BN;
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int grid = m_tiles * n_tiles < sms ? m_tiles * n_tiles : sms;       // persistent: at most one CTA per SM
  return b200_launch(gemm_tcgen05_kernel, dim3(grid), dim3(THREADS), smem, stream, 0, amap, wmap,
                     static_cast<bf16*>(out), m, n, k, mode, err);
}
