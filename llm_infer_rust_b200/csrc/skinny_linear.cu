// y = epilogue(prologue(x) . W^T) for a handful of rows (decode steps): the weights are streamed once,
// at the speed of memory, and what stands before and after the product is fused into the same kernel.
//
//   prologue  none, or residual add + RMSNorm: s = x + residual in float, residual_out = round(s),
//             x' = s * rsqrt(mean(s^2) + eps) * w (the unrounded sum is normalised; reference:
//             src/layers/fused_ops.cu:95-105).  Every CTA recomputes the row statistics (the rows are few
//             and sit in L2); the CTA with index 0 writes residual_out.  The row's scale is a scalar, so it is
//             applied to the finished product: the operand in shared memory is round(s * w).
//   product   W is [N, K] bfloat16, row-major.  A CTA owns BN = 64 * MT weight rows and a range of K; TMA
//             brings boxes of BN rows x 64 columns (128-byte swizzle) into a ring of stages, the rows of
//             x' (at most 16) wait in shared memory, and mma.sync m16n8k16 multiplies with the WEIGHT rows
//             on the 16-row side of the instruction, so no tensor work is wasted on padding the rows.
//             A CTA has four groups of four warps (group g multiplies the k-blocks g, g + 4, ...; the groups'
//             sums are added at the end) and one more warp that only feeds the ring.
//             Where N / BN alone would leave SMs idle, a thread-block cluster of up to 8 CTAs splits K; the
//             partial sums meet in the first CTA's shared memory (distributed shared memory), added in
//             rank order, so the result does not depend on timing.
//   epilogue  PLAIN   out[m, n] (bfloat16 or float)
//             SWIGLU  W = [gate rows; up rows] ([2 I, K]); a CTA takes BN/2 gate rows and the same up rows
//                     and writes silu(gate) * up (reference: src/layers/fused_ops.cu:142-144)
//             QKV     BN = head_dim: a CTA owns one head of the packed q, k, v rows; per-head RMSNorm,
//                     half-split rotary encoding, q to q_out, k and v into the paged cache (the work of
//                     qkv_post.cu, with the same error flags).
// Every wait on a barrier is bounded by the clock; a wait that runs out flags the engine's error word.
#include <cooperative_groups.h>
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

namespace cg = cooperative_groups;
typedef __nv_bfloat16 bf16;

constexpr int BK = 64;                 // k per stage: 128 bytes of a weight row
constexpr int MMAX = 16;               // rows of x
constexpr int ROW_WARPS = 4;           // warps that share the weight rows of a tile
constexpr int GROUPS = 4;              // groups of ROW_WARPS warps; group g multiplies the k-blocks g, g + 4, ...
constexpr int WARPS = ROW_WARPS * GROUPS;          // consumer warps; one more warp feeds the ring
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int XS_BYTES = 64 * 1024;    // the rows of x' that a CTA multiplies with
constexpr int W_RING_BYTES = 128 * 1024;

enum : int { EPI_PLAIN_BF16 = 0, EPI_PLAIN_F32 = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };

struct SkinnyParams {
  // prologue
  const bf16* x;            // [rows of x, K]
  const int* x_rows;        // optional gather: row m of the product is x[x_rows[m]]
  const bf16* residual;     // null: no norm prologue
  bf16* residual_out;       // null: the sum is not stored
  const void* norm_w;       // [K] bfloat16 or float
  int norm_w_f32;
  float eps;
  // product
  int M, N, K, ksplit;
  // epilogue
  int mode;
  void* out;                // PLAIN: [M, N]; SWIGLU: [M, N / 2]; QKV: q_out [M, nh * d]
  // QKV
  int nh, nkv, rot_dim, max_pos, page_size;
  long long cache_slots;
  float qk_eps;
  const void* q_w;          // [d] per-head norm weights (null: no norm), bfloat16 or float
  const void* k_w;
  int qk_w_f32;
  const float* cos_table;   // [max_pos, rot_dim / 2] (null: no rotation)
  const float* sin_table;
  const int* positions;     // [M]
  const int* slots;         // [M] (null: nothing is stored)
  bf16* k_cache;            // [pages + 1, nkv, page_size, d]
  bf16* v_cache;
  int* err;
};

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float norm_weight(const void* w, int f32, int i) {
  return f32 ? static_cast<const float*>(w)[i] : __bfloat162float(static_cast<const bf16*>(w)[i]);
}

// MT: 64-row units of the weight tile (BN = 64 MT rows; a warp owns 16 MT of them).  EARLY_W: the norm's weights
// of a warp's first pass over a row are fetched ahead of the dependency wait (see `launch` for when).
template <int MT, bool EARLY_W>
__global__ void __launch_bounds__(THREADS, 1)
skinny_linear_kernel(const __grid_constant__ CUtensorMap wmap, const SkinnyParams p) {
  constexpr int BN = 64 * MT;
  constexpr int STAGE_BYTES = BN * 128;
  constexpr int STAGES = W_RING_BYTES / STAGE_BYTES;
  // A stage's uses all fall to one group (k-block it -> stage it % STAGES, group it % GROUPS), so that group waits
  // for every phase of the stage's barrier in order; a waiter by parity that skipped a phase could pass too early.
  static_assert(STAGES % GROUPS == 0, "every stage of the ring must belong to one group of warps");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  bf16* xs = reinterpret_cast<bf16*>(ring + W_RING_BYTES);                     // [mpad][ldx]
  float* red = reinterpret_cast<float*>(ring + W_RING_BYTES + XS_BYTES);       // [MMAX][BN + 1]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + MMAX * (BN + 1));
  uint64_t* empty = full + STAGES;
  float* row_scale = reinterpret_cast<float*>(empty + STAGES);                 // [MMAX]

  pdl_launch_dependents();         // the kernel after this one may set itself up from now on (it waits before it reads)
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int tile = blockIdx.x / p.ksplit;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int M = p.M, K = p.K;
  const int mpad = M <= 8 ? 8 : 16;
  const int kblocks = (K + BK - 1) / BK;
  const int kb_per = (kblocks + p.ksplit - 1) / p.ksplit;
  const int kb_lo = min(kblocks, rank * kb_per), kb_hi = min(kblocks, kb_lo + kb_per);
  const int nkb = kb_hi - kb_lo;
  const int k_lo = kb_lo * BK, kc = nkb * BK;                                  // this CTA's columns, padded to 64
  const int ldx = kc + 8;                                                      // padded row: conflict-free ldmatrix

  if (threadIdx.x < STAGES) { mbar_init(full + threadIdx.x, 1); mbar_init(empty + threadIdx.x, ROW_WARPS); }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();

  // Weight rows of this tile: PLAIN / QKV: BN consecutive rows; SWIGLU: BN/2 gate rows, then the same up rows.
  const int w_row0 = p.mode == EPI_SWIGLU ? tile * (BN / 2) : tile * BN;
  const int up_row0 = p.N / 2 + tile * (BN / 2);
  auto issue = [&](int j) {      // one thread: fetch k-block j of this CTA into its stage
    const int s = j % STAGES;
    unsigned char* dst = ring + s * STAGE_BYTES;
    mbar_expect_tx(full + s, STAGE_BYTES);
    if (p.mode == EPI_SWIGLU) {
      tma_load_2d(dst, &wmap, (kb_lo + j) * BK, w_row0, full + s);
      tma_load_2d(dst + STAGE_BYTES / 2, &wmap, (kb_lo + j) * BK, up_row0, full + s);
    } else {
      tma_load_2d(dst, &wmap, (kb_lo + j) * BK, w_row0, full + s);
    }
  };
  // The weights do not depend on the prologue: the feeding warp starts streaming them at once.
  const bool feeder = warp == WARPS;
  if (feeder && lane == 0)
    for (int j = 0; j < STAGES && j < nkb; ++j) issue(j);
  // What the QKV epilogue needs of the step's index arrays and of the rotary tables does not depend on the kernels
  // before either: warp m fetches row m's position, cache slot and angles now, not at the end of the kernel, where
  // two dependent loads would stand between the product and the store.
  constexpr int ROT_PER_LANE = BN / 64;              // a head of BN dims rotates at most BN / 2 pairs: 32 lanes x BN / 64
  int epi_pos = 0, epi_slot = 0;
  float epi_cos[ROT_PER_LANE], epi_sin[ROT_PER_LANE];
  bool epi_rotate = false;
  if (p.mode == EPI_QKV && warp < p.M) {
    if (p.slots != nullptr) epi_slot = p.slots[warp];
    const int half = p.rot_dim / 2;
    if (p.cos_table != nullptr && half > 0) {
      epi_pos = p.positions[warp];
      epi_rotate = epi_pos >= 0 && epi_pos < p.max_pos;
      if (epi_rotate) {
#pragma unroll
        for (int j = 0; j < ROT_PER_LANE; ++j) {
          const int i = lane + 32 * j;
          epi_cos[j] = i < half ? p.cos_table[static_cast<size_t>(epi_pos) * half + i] : 1.0f;
          epi_sin[j] = i < half ? p.sin_table[static_cast<size_t>(epi_pos) * half + i] : 0.0f;
        }
      }
    }
  }
  // The norm's weights for the columns that this lane takes in the first pass over a row (the only pass up to 1,024
  // columns): the same for every row and not written by the kernels before, so they are fetched ahead of the wait.
  // Widened to 32-bit here: kept packed, the loads were found to be scheduled after the wait.
  float first_w[EARLY_W ? 4 : 1][8];
  if (EARLY_W && p.residual != nullptr) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = (u * 32 + lane) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) first_w[u][i] = k + i < K ? norm_weight(p.norm_w, p.norm_w_f32, k + i) : 0.0f;
    }
  }
  pdl_wait();                      // x, the residual and the cache belong to the kernels before this one

  // ---- prologue: the rows of x' for columns [k_lo, k_lo + kc) as bfloat16 in shared memory
  constexpr int ALL_WARPS = WARPS + 1;
  if (p.residual != nullptr) {
    // One warp per row, one pass: the sum s = x + residual is stored rounded (by the writer CTA), its squares
    // are summed, and s * w goes to shared memory as bfloat16.  The row's scale rsqrt(mean(s^2) + eps) is a
    // scalar, so it multiplies the finished product instead (in the epilogue): the weights' product need not
    // wait for the statistics.
    const bool writer = blockIdx.x == 0 && p.residual_out != nullptr;
    const int k_pad = (K + 7) / 8 * 8;
    for (int m = warp; m < mpad; m += ALL_WARPS) {
      if (m >= M) {                                                            // padding rows of x' are zeros
        for (int k = lane * 8; k < kc; k += 32 * 8) *reinterpret_cast<uint4*>(xs + m * ldx + k) = make_uint4(0u, 0u, 0u, 0u);
        continue;
      }
      const size_t src = static_cast<size_t>(p.x_rows ? p.x_rows[m] : m) * K;
      float ss = 0.0f;
      for (int k0 = 0; k0 < max(k_pad, k_lo + kc); k0 += 4 * 32 * 8) {           // four 16-byte loads in flight per tensor
        uint4 xa[4], xb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + (u * 32 + lane) * 8;
          xa[u] = xb[u] = make_uint4(0u, 0u, 0u, 0u);
          if (k < K) {
            xa[u] = *reinterpret_cast<const uint4*>(p.x + src + k);
            xb[u] = *reinterpret_cast<const uint4*>(p.residual + src + k);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int k = k0 + (u * 32 + lane) * 8;
          const uint32_t wa[4] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w}, wb[4] = {xb[u].x, xb[u].y, xb[u].z, xb[u].w};
          float sum[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            sum[2 * i] = __uint_as_float(wa[i] << 16) + __uint_as_float(wb[i] << 16);
            sum[2 * i + 1] = __uint_as_float(wa[i] & 0xffff0000u) + __uint_as_float(wb[i] & 0xffff0000u);
            ss += sum[2 * i] * sum[2 * i] + sum[2 * i + 1] * sum[2 * i + 1];
          }
          if (writer && k < K) {
            __align__(16) bf16 rounded[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) rounded[i] = __float2bfloat16_rn(sum[i]);
            *reinterpret_cast<uint4*>(p.residual_out + src + k) = *reinterpret_cast<uint4*>(rounded);
          }
          if (k >= k_lo && k < k_lo + kc) {
            __align__(16) bf16 weighted[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              weighted[i] = __float2bfloat16_rn(k >= K ? 0.0f : sum[i] * (EARLY_W && k0 == 0 ? first_w[EARLY_W ? u : 0][i] : norm_weight(p.norm_w, p.norm_w_f32, k + i)));
            *reinterpret_cast<uint4*>(xs + m * ldx + (k - k_lo)) = *reinterpret_cast<uint4*>(weighted);
          }
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) row_scale[m] = rsqrtf(ss / static_cast<float>(K) + p.eps);
    }
  } else {
    const int chunks = kc / 8;
    for (int c = threadIdx.x; c < mpad * chunks; c += THREADS) {
      const int m = c / chunks, k = k_lo + (c - m * chunks) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (m < M && k < K) v = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(p.x_rows ? p.x_rows[m] : m) * K + k);
      *reinterpret_cast<uint4*>(xs + m * ldx + (k - k_lo)) = v;
    }
  }
  __syncthreads();

  // ---- product: group `grp` takes the k-blocks grp, grp + GROUPS, ...; inside a group warp `rw` owns 16 MT weight rows
  float acc[MT][2][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int n = 0; n < 2; ++n) { acc[i][n][0] = acc[i][n][1] = acc[i][n][2] = acc[i][n][3] = 0.0f; }
  const int mi = lane >> 3, r8 = lane & 7;
  const int grp = warp / ROW_WARPS, rw = warp % ROW_WARPS;
  bool ok = true;
  if (feeder) {
    if (lane == 0) {
      for (int j = STAGES; j < nkb && ok; ++j) {
        ok = mbar_wait(empty + j % STAGES, (j / STAGES - 1) & 1, p.err);      // the group that had this stage has left it
        if (ok) issue(j);
      }
    }
  } else {
    for (int it = grp; it < nkb; it += GROUPS) {
      const int s = it % STAGES;
      if (!mbar_wait(full + s, (it / STAGES) & 1, p.err)) { ok = false; break; }
      const unsigned char* wt = ring + s * STAGE_BYTES;
#pragma unroll
      for (int ks = 0; ks < BK / 16; ++ks) {
        // B operand: x'[m][k], two 8-row groups (m 0..7, 8..15), k and k + 8
        // (with 8 rows of x' only, the lanes of the second group point at the first: its result is not used)
        uint32_t b[4];
        ldmatrix_x4(b, xs + ((mpad > 8 ? (mi >> 1) * 8 : 0) + r8) * ldx + it * BK + ks * 16 + (mi & 1) * 8);
#pragma unroll
        for (int i = 0; i < MT; ++i) {
          const int r = rw * (16 * MT) + i * 16 + (lane & 15);                 // weight row inside the tile
          const int c = ks * 2 + (lane >> 4);                                  // 16-byte chunk of the 128-byte row
          uint32_t a[4];
          ldmatrix_x4(a, wt + r * 128 + ((c ^ (r & 7)) << 4));
          mma_bf16(acc[i][0], a, b[0], b[1]);
          if (mpad > 8) mma_bf16(acc[i][1], a, b[2], b[3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
  }

  // ---- the groups' sums are added in shared memory, group after group
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  for (int turn = 0; turn < GROUPS; ++turn) {
    if (!feeder && grp == turn) {
#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int n = rw * (16 * MT) + i * 16 + g;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int m = nt * 8 + t2;
          if (m < mpad) {
            float* r0 = red + m * (BN + 1) + n;
            float* r1 = red + (m + 1) * (BN + 1) + n;
            if (turn == 0) { r0[0] = acc[i][nt][0]; r1[0] = acc[i][nt][1]; r0[8] = acc[i][nt][2]; r1[8] = acc[i][nt][3]; }
            else { r0[0] += acc[i][nt][0]; r1[0] += acc[i][nt][1]; r0[8] += acc[i][nt][2]; r1[8] += acc[i][nt][3]; }
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- the partial sums of the cluster meet in rank 0, added in rank order
  cluster.sync();
  if (rank == 0 && p.ksplit > 1) {
    for (int i = threadIdx.x; i < mpad * BN; i += blockDim.x) {
      const int m = i / BN, n = i - m * BN;
      float part[8];
#pragma unroll
      for (int r = 1; r < 8; ++r) part[r] = r < p.ksplit ? cluster.map_shared_rank(red, r)[m * (BN + 1) + n] : 0.0f;
      float sum = red[m * (BN + 1) + n];
#pragma unroll
      for (int r = 1; r < 8; ++r) sum += part[r];
      red[m * (BN + 1) + n] = sum;
    }
  }
  cluster.sync();                    // the others' shared memory has been read: they may leave
  if (rank != 0 || !ok) return;
  if (p.residual != nullptr) {       // the norm's row scale, left out of x' by the prologue
    for (int i = threadIdx.x; i < M * BN; i += blockDim.x) {
      const int m = i / BN, n = i - m * BN;
      red[m * (BN + 1) + n] *= row_scale[m];
    }
    __syncthreads();
  }

  // ---- epilogue on red[m][n] (float)
  if (p.mode == EPI_PLAIN_BF16 || p.mode == EPI_PLAIN_F32) {
    for (int i = threadIdx.x; i < M * BN; i += blockDim.x) {
      const int m = i / BN, n = i - m * BN, col = tile * BN + n;
      if (col >= p.N) continue;
      const float v = red[m * (BN + 1) + n];
      if (p.mode == EPI_PLAIN_F32) static_cast<float*>(p.out)[static_cast<size_t>(m) * p.N + col] = v;
      else static_cast<bf16*>(p.out)[static_cast<size_t>(m) * p.N + col] = __float2bfloat16_rn(v);
    }
  } else if (p.mode == EPI_SWIGLU) {
    const int inter = p.N / 2;
    for (int i = threadIdx.x; i < M * (BN / 2); i += blockDim.x) {
      const int m = i / (BN / 2), n = i - m * (BN / 2), col = tile * (BN / 2) + n;
      if (col >= inter) continue;
      // gate and up leave the product as bfloat16 values in the unfused path; the same rounding here
      const float gate = __bfloat162float(__float2bfloat16_rn(red[m * (BN + 1) + n]));
      const float up = __bfloat162float(__float2bfloat16_rn(red[m * (BN + 1) + BN / 2 + n]));
      static_cast<bf16*>(p.out)[static_cast<size_t>(m) * inter + col] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
  } else {                                                                   // EPI_QKV: tile = one head, BN = head_dim
    constexpr int d = BN;
    const int head = tile;
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
    static_assert(MMAX <= WARPS + 1, "one warp per row in the QKV epilogue");
    if (warp < M) {
      const int m = warp;                                                    // (its position, slot and angles were fetched at the start)
      float* row = red + m * (BN + 1);
      // the projection's output is a bfloat16 tensor in the unfused path; the same rounding here
      for (int i = lane; i < d; i += 32) row[i] = __bfloat162float(__float2bfloat16_rn(row[i]));
      __syncwarp();
      bf16* dst = nullptr;
      if (is_q) {
        dst = static_cast<bf16*>(p.out) + (static_cast<size_t>(m) * p.nh + head) * d;
      } else if (p.slots != nullptr && epi_slot != 0) {
        if (epi_slot < 0 || epi_slot >= p.cache_slots) {
          if (lane == 0) atomicOr(p.err, B200_ERR_SLOT_RANGE);
        } else {
          const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
          const int page = epi_slot / p.page_size, offset = epi_slot - page * p.page_size;
          dst = (is_k ? p.k_cache : p.v_cache) + ((static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + offset) * d;
        }
      }
      if (dst != nullptr && !is_q && !is_k) {
        for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
      } else if (dst != nullptr) {
        const void* w = is_q ? p.q_w : p.k_w;
        if (w != nullptr) {
          float ss = 0.0f;
          for (int i = lane; i < d; i += 32) ss += row[i] * row[i];
          ss = warp_sum(ss);
          const float scale = rsqrtf(ss / static_cast<float>(d) + p.qk_eps);
          for (int i = lane; i < d; i += 32) row[i] = row[i] * scale * norm_weight(w, p.qk_w_f32, i);
          __syncwarp();
        }
        const int half = p.rot_dim / 2;
        const bool wanted = p.cos_table != nullptr && half > 0;
        if (wanted && !epi_rotate && lane == 0) atomicOr(p.err, B200_ERR_POSITION_RANGE);
        if (wanted && epi_rotate) {
#pragma unroll
          for (int j = 0; j < ROT_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            if (i < half) {
              const float a = row[i], b = row[i + half];
              dst[i] = __float2bfloat16_rn(a * epi_cos[j] - b * epi_sin[j]);
              dst[i + half] = __float2bfloat16_rn(b * epi_cos[j] + a * epi_sin[j]);
            }
          }
          for (int i = p.rot_dim + lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
        } else {
          for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes into `out_map` (128 bytes) the TMA descriptor of a bfloat16 weight matrix [n, k], fetched in boxes of
// `box_rows` rows x 64 columns with the 128-byte swizzle.  Rows beyond n and columns beyond k read as zeros.
B200_EXPORT int b200_weight_tensor_map(void* out_map, const void* weight, long long n, long long k, int box_rows) {
  if (n <= 0 || k <= 0 || box_rows <= 0 || box_rows > 256 || k % 8 != 0) return B200_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(weight) % 16 != 0) return B200_BAD_ALIGN;
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
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(n)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * sizeof(bf16)};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(weight), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
  memcpy(out_map, &map, sizeof(map));
  return 0;
}

// Rows of the weight tile that a CTA owns: QKV: the head size (64, 128 or 256; 0: refused); else 128, or 256 for
// a matrix of so many rows (a vocabulary) that tiles of 256 still make four waves of CTAs: every CTA normalises
// the rows of x and fills its ring once, whatever its tile's size.
B200_EXPORT int b200_skinny_tile_rows(int mode, int head_dim, int n, int sm_count) {
  if (mode == EPI_QKV) return (head_dim == 64 || head_dim == 128 || head_dim == 256) ? head_dim : 0;
  if (mode != EPI_SWIGLU && n >= 4 * 256 * (sm_count > 0 ? sm_count : 148)) return 256;
  return 128;
}

// Rows of a weight box that b200_weight_tensor_map must be given.
B200_EXPORT int b200_skinny_box_rows(int mode, int head_dim, int n, int sm_count) {
  const int bn = b200_skinny_tile_rows(mode, head_dim, n, sm_count);
  return mode == EPI_SWIGLU ? bn / 2 : bn;
}

// Largest K range of one CTA for `m` rows, and from it the cluster size (CTAs that split K); 0: the product is refused.
static int choose_ksplit(int m, int n_tiles, int k, int sm_count) {
  const int mpad = m <= 8 ? 8 : 16;
  const int kc_max = ((XS_BYTES / (mpad * 2)) - 8) / BK * BK;
  const int kblocks = (k + BK - 1) / BK;
  const int need = (k + kc_max - 1) / kc_max;
  if (need > 8) return 0;
  // Clusters of 3, 5, 6 or 7 are only taken while the grid stays under half the machine: measured at the Qwen3-8B
  // sizes, 192 clusters of 3 ran 20 % longer than 192 clusters of 2 (a cluster is placed on whole pairs of SMs, so an
  // odd one leaves an SM idle), while 8 clusters of 3 beat 8 of 2.
  auto allowed = [&](int split) {
    return split == need || (split & (split - 1)) == 0 || 2ll * n_tiles * split <= sm_count;
  };
  // A grid that fits one wave of the SMs is bound by how fast ONE SM takes its share in, not by memory: as many CTAs
  // as fit the wave, down to eight k-blocks (64 KB of weights at 64 rows) a CTA.  Measured at the Qwen3-0.6B sizes
  // (decode, batch 8 / batch 1): 1.69 -> 1.56 ms and 1.16 -> 1.02 ms a step against a floor of sixteen k-blocks; a
  // floor of four was slower again (1.66 ms): the cluster's hand-over then costs more than the SMs it wins.
  int one_wave = 0;
  for (int split = need; split <= 8; ++split) {
    if (split > need && kblocks / split < 8) break;
    if (static_cast<long long>(n_tiles) * split > sm_count) break;
    if (allowed(split)) one_wave = split;
  }
  if (one_wave > 0) return one_wave;
  // Several waves: every CTA pays its set-up again, so a CTA keeps at least sixteen k-blocks, and among those cluster
  // sizes the one whose CTAs fill whole waves best wins (a larger cluster must win by a margin: its hand-over is
  // longer).  At the Qwen3-8B sizes the floor of eight k-blocks made a step 7.7 ms instead of 5.0.
  int best = need;
  double best_fill = 0.0;
  for (int split = need; split <= 8; ++split) {
    if (split > need && kblocks / split < 16) break;
    if (!allowed(split)) continue;
    const long long ctas = static_cast<long long>(n_tiles) * split;
    const long long waves = (ctas + sm_count - 1) / sm_count;
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * sm_count);
    if (fill > best_fill + 0.04) { best = split; best_fill = fill; }
  }
  return best;
}

template <int MT, bool EARLY_W>
static int launch_as(const CUtensorMap& map, const SkinnyParams& p, int n_tiles, cudaStream_t stream) {
  constexpr int BN = 64 * MT;
  constexpr int STAGES = W_RING_BYTES / (BN * 128);
  const size_t smem = 1024 + W_RING_BYTES + XS_BYTES + MMAX * (BN + 1) * sizeof(float) + 2 * STAGES * sizeof(uint64_t) +
                      MMAX * sizeof(float) + 64;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(skinny_linear_kernel<MT, EARLY_W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return b200_launch(skinny_linear_kernel<MT, EARLY_W>, dim3(n_tiles * p.ksplit), dim3(THREADS), smem, stream, p.ksplit,
                     map, p);
}

// Which of the two compiled variants runs is a matter of measurement (decode steps at batch 8, both variants for
// every product): rows under 4,096 columns are faster with the early fetch compiled in, also the products that have
// no norm and skip it (1.735 against 1.79 ms a step at the 0.6B sizes); from 4,096 columns on the variant without
// it wins (5.01 against 5.17 ms at the 8B sizes), where a warp passes over a row four times or more.
template <int MT>
static int launch(const CUtensorMap& map, const SkinnyParams& p, int n_tiles, cudaStream_t stream) {
  if (p.K < 4096) return launch_as<MT, true>(map, p, n_tiles, stream);
  return launch_as<MT, false>(map, p, n_tiles, stream);
}

// `params`: a SkinnyParams filled by the caller (ksplit is chosen here); `w_map`: the descriptor of the weight.
// Refuses (B200_BAD_SIZE) more than 16 rows, a K that is no multiple of 8 or too long for a cluster of 8, and
// head sizes other than 64 / 128 / 256 in QKV mode.
B200_EXPORT int b200_skinny_linear(const void* w_map, const void* params, int head_dim, int sm_count, cudaStream_t stream) {
  SkinnyParams p;
  memcpy(&p, params, sizeof(p));
  if (p.M <= 0) return 0;
  if (p.M > MMAX || p.N <= 0 || p.K <= 0 || p.K % 8 != 0) return B200_BAD_SIZE;
  if (p.mode < EPI_PLAIN_BF16 || p.mode > EPI_QKV) return B200_BAD_SIZE;
  if (p.mode == EPI_SWIGLU && p.N % 2 != 0) return B200_BAD_SIZE;
  const int bn = b200_skinny_tile_rows(p.mode, head_dim, p.N, sm_count);
  if (bn == 0) return B200_BAD_SIZE;
  if (p.mode == EPI_QKV && (p.N != (p.nh + 2 * p.nkv) * head_dim || p.rot_dim < 0 || p.rot_dim > head_dim || (p.rot_dim & 1)))
    return B200_BAD_SIZE;
  const int cols = p.mode == EPI_SWIGLU ? p.N / 2 : p.N;
  const int tile_cols = p.mode == EPI_SWIGLU ? bn / 2 : bn;
  const int n_tiles = (cols + tile_cols - 1) / tile_cols;
  p.ksplit = choose_ksplit(p.M, n_tiles, p.K, sm_count > 0 ? sm_count : 148);
  if (p.ksplit == 0) return B200_BAD_SIZE;
  CUtensorMap map;
  memcpy(&map, w_map, sizeof(map));
  if (bn == 64) return launch<1>(map, p, n_tiles, stream);
  if (bn == 128) return launch<2>(map, p, n_tiles, stream);
  return launch<4>(map, p, n_tiles, stream);
}

B200_EXPORT int b200_skinny_params_size() { return static_cast<int>(sizeof(SkinnyParams)); }
