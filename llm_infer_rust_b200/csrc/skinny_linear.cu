// y = epilogue(prologue(x) . W^T) for a handful of rows (decode steps): the weights are streamed once,
// at the speed of memory, and what stands before and after the product is fused into the same kernel.
//
//   prologue  none, or residual add + RMSNorm: s = x + residual in float, residual_out = round(s),
//             x' = s * rsqrt(mean(s^2) + eps) * w (the unrounded sum is normalised; reference:
//             src/layers/fused_ops.cu:95-105).  The row's scale is a scalar, so it is applied to the finished
//             product: the operand in shared memory is round(s * w).  Two ways to the rows' statistics:
//             every CTA reads whole rows (they are few and sit in L2; the CTA with index 0 writes residual_out),
//             or, when the product BEFORE this one was a PLAIN product of this kernel, that product's epilogue
//             has stored round(y + residual) and, per tile of its columns, the rows' sums of squares
//             (post_* / stats_in below): then a CTA reads its own columns only.  At 4,096 columns the whole-row
//             read by every CTA took 5 of a product's 20 us.
//   product   W is [N, K] bfloat16, row-major.  A CTA owns BN = 64 * MT weight rows and a range of K; TMA
//             brings boxes of BN rows x 64 columns (128-byte swizzle) into a ring of stages, the rows of
//             x' (at most 16) wait in shared memory, and mma.sync m16n8k16 multiplies with the WEIGHT rows
//             on the 16-row side of the instruction, so no tensor work is wasted on padding the rows.
//             A CTA has groups of four warps (group g multiplies the k-blocks g, g + GROUPS, ...; every warp leaves
//             its sums in the ring stage of its group, they are added in the groups' order) and one more warp that
//             only feeds the ring.  Two shapes: one CTA an SM with four groups, or two CTAs an SM with two (see Shape).
//             Where N / BN alone would leave SMs idle, a thread-block cluster of up to 8 CTAs splits K; the
//             partial sums meet in the first CTA's shared memory: the others store them there (st.async, counted
//             by a barrier of the first CTA), or the first reads them (distributed shared memory) where that space
//             does not reach; added in rank order, so the result does not depend on timing.
//   epilogue  PLAIN   out[m, n] (bfloat16 or float), and optionally the beginning of the norm that follows (above)
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
// Two shapes of a CTA.  OCC = 1: one CTA an SM, four groups of warps, a ring of 128 KB: for grids of one wave, where
// a CTA's share is all that its SM does.  OCC = 2: two CTAs an SM, each with two groups and a ring of 64 KB: for
// grids of several waves, where one CTA streams while its neighbour prepares its rows of x or adds up its tile.
template <int OCC>
struct Shape {
  static constexpr int GROUPS = OCC == 1 ? 4 : 2;        // groups of ROW_WARPS warps; group g multiplies the k-blocks g, g + GROUPS, ...
  static constexpr int WARPS = ROW_WARPS * GROUPS;       // consumer warps; one more warp feeds the ring
  static constexpr int THREADS = (WARPS + 1) * 32;
  static constexpr int XS_BYTES = OCC == 1 ? 64 * 1024 : 36 * 1024;      // the rows of x' that a CTA multiplies with
  static constexpr int W_RING_BYTES = OCC == 1 ? 128 * 1024 : 64 * 1024;
};

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
  // the norm AFTER a PLAIN bfloat16 product, begun in its epilogue: the rounded sum y + post_residual goes to
  // post_sum_out and the sum of its squares over the tile's columns to post_stats[tile][row]; the product that
  // follows takes them as stats_in (with x = y and residual = post_residual) and reads no whole rows
  const bf16* post_residual;
  bf16* post_sum_out;
  float* post_stats;        // [tiles][MMAX]
  const float* stats_in;    // [stats_tiles][MMAX]; null: this product's prologue reads the rows itself
  int stats_tiles;
  long long* trace;         // for tuning (null in service): [4096 CTAs][32]: nanosecond clocks at the kernel's phases, then the SM's cycle counter at the same places
};

// Compiled with -DSKINNY_TRACE (a tuning aid), the first thread of every CTA leaves both clocks at the kernel's phases.
#ifdef SKINNY_TRACE
__device__ __forceinline__ void stamp(const SkinnyParams& p, int slot) {
  if (threadIdx.x == 0 && p.trace != nullptr && blockIdx.x < 4096) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[blockIdx.x * 32 + slot] = static_cast<long long>(t);
    p.trace[blockIdx.x * 32 + 16 + slot] = clock64();
  }
}
#define STAMP(slot) stamp(p, slot)
#else
#define STAMP(slot)
#endif

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

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

// The address, in the cluster's shared window, of this CTA's shared-memory address `addr` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, int rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
// Stores 16 bytes into another CTA's shared memory; when they have landed, the barrier there (`bar`) counts them.
__device__ __forceinline__ void store_remote_counted(uint32_t addr, const float4& v, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];\n"
               ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(bar) : "memory");
}

// Eight bfloat16 values of a 16-byte vector as floats, in memory order.
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&out)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int N> struct Count { static constexpr int value = N; };

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  __align__(16) bf16 h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = __float2bfloat16_rn(v[i]);
  return *reinterpret_cast<uint4*>(h);
}

// Four neighbouring sums of a CTA, row m from column n (a multiple of 4) on, out of the parts that its groups of warps
// left in their ring stages (see the kernel): added in the order of the groups.
template <int MT, int GROUPS>
__device__ __forceinline__ float4 own_sums(const unsigned char* ring, int m, int n) {
  constexpr int WN = 16 * MT, STAGE_FLOATS = 64 * MT * 128 / 4;
  const float* part = reinterpret_cast<const float*>(ring + (n / WN) * (WN * 128)) + m * (WN + 4) + n % WN;
  float4 more[GROUPS];
#pragma unroll
  for (int gg = 0; gg < GROUPS; ++gg) more[gg] = *reinterpret_cast<const float4*>(part + gg * STAGE_FLOATS);
  float4 sum = more[0];
#pragma unroll
  for (int gg = 1; gg < GROUPS; ++gg) { sum.x += more[gg].x; sum.y += more[gg].y; sum.z += more[gg].z; sum.w += more[gg].w; }
  return sum;
}

__device__ __forceinline__ float norm_weight(const void* w, int f32, int i) {
  return f32 ? static_cast<const float*>(w)[i] : __bfloat162float(static_cast<const bf16*>(w)[i]);
}

// MT: 64-row units of the weight tile (BN = 64 MT rows; a warp owns 16 MT of them).  OCC: the CTA's shape (above).
// Prologues and epilogues are chosen at run time inside ONE kernel per (MT, OCC): a decode step runs the products of a
// layer one after the other for a few microseconds each, and what they share of their code stays in the instruction
// caches from one launch to the next.  (A kernel of its own per epilogue and prologue was measured: every launch
// then began on cold instruction caches and the step took 8 % longer.)
template <int MT, int OCC>
__global__ void __launch_bounds__(Shape<OCC>::THREADS, OCC)
skinny_linear_kernel(const __grid_constant__ CUtensorMap wmap, const SkinnyParams p) {
  constexpr int GROUPS = Shape<OCC>::GROUPS, WARPS = Shape<OCC>::WARPS, THREADS = Shape<OCC>::THREADS;
  constexpr int XS_BYTES = Shape<OCC>::XS_BYTES, W_RING_BYTES = Shape<OCC>::W_RING_BYTES;
  constexpr int ALL_WARPS = WARPS + 1;
  constexpr int ROWS_PER_WARP = (MMAX + ALL_WARPS - 1) / ALL_WARPS;          // rows that a warp takes where a row is a warp's work
  constexpr int BN = 64 * MT;
  constexpr int QUADS = BN / 4;
  constexpr int STAGE_BYTES = BN * 128;
  constexpr int STAGES = W_RING_BYTES / STAGE_BYTES;
  // A stage's uses all fall to one group (k-block it -> stage it % STAGES, group it % GROUPS), so that group waits
  // for every phase of the stage's barrier in order; a waiter by parity that skipped a phase could pass too early.
  static_assert(STAGES % GROUPS == 0, "every stage of the ring must belong to one group of warps");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* xregion = ring + W_RING_BYTES;    // rows of x' [mpad][ldx], then the norm's weights, then the other ranks' sums
  bf16* xs = reinterpret_cast<bf16*>(xregion);
  constexpr int RS = BN + 4;                                                   // a row of sums: 16-byte steps, no bank conflicts
  float* red = reinterpret_cast<float*>(ring + W_RING_BYTES + XS_BYTES);       // [MMAX][RS]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + MMAX * RS);
  uint64_t* empty = full + STAGES;
  uint64_t* gather = empty + STAGES;                                           // rank 0: the other ranks' sums have landed
  float* row_scale = reinterpret_cast<float*>(gather + 2);                     // [MMAX]
  float* row_ss = row_scale + MMAX;                                            // [32]: sums of squares of parts of rows

  pdl_launch_dependents();         // the kernel after this one may set itself up from now on (it waits before it reads)
  STAMP(0);
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
  const bool has_norm = p.residual != nullptr, has_stats = has_norm && p.stats_in != nullptr;

  // The x region of every rank is laid out for the rank with the most columns, so all CTAs of a cluster decide alike.
  const int xs_bytes = mpad * (kb_per * BK + 8) * 2;
  const int ws_bytes = has_norm ? kb_per * BK * 4 : 0;
  float* ws = reinterpret_cast<float*>(xregion + xs_bytes);                    // [kc] the norm's weights of this CTA's columns
  float* slots = reinterpret_cast<float*>(xregion + xs_bytes + ws_bytes);      // [ksplit - 1][M][BN]
  // How the cluster's partial sums meet in rank 0.  push: the other ranks store theirs into rank 0's shared memory
  // and a barrier there counts the bytes (one trip across the cluster).  pull, when that space does not reach:
  // rank 0 reads them from the others' shared memory after a cluster barrier (three trips).
  const int slot_bytes = (p.ksplit - 1) * M * BN * 4;
  const bool push = p.ksplit > 1 && xs_bytes + ws_bytes + slot_bytes <= XS_BYTES;
  const bool pull = p.ksplit > 1 && !push;
  if (threadIdx.x < STAGES) { mbar_init(full + threadIdx.x, 1); mbar_init(empty + threadIdx.x, ROW_WARPS); }
  if (threadIdx.x == 0) {
    mbar_init(gather, 1);
    if (push && rank == 0) mbar_expect_tx(gather, static_cast<uint32_t>(slot_bytes));
  }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();
  if (push) cluster_arrive();      // (waited for before the first store into rank 0: its barrier is set up by then)

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

  // What does not depend on the kernels before is fetched ahead of the dependency wait.
  // QKV: warp m fetches row m's cache slot and rotary angles, and every warp the per-head norm's weights of this head.
  constexpr int ROT_PER_LANE = BN / 64;              // a head of BN dims rotates at most BN / 2 pairs: 32 lanes x BN / 64
  int epi_slot[ROWS_PER_WARP];
  float epi_cos[ROWS_PER_WARP][ROT_PER_LANE], epi_sin[ROWS_PER_WARP][ROT_PER_LANE];
  bool epi_rotate[ROWS_PER_WARP];
  float epi_w[2 * MT];
  bool epi_norm = false;
  if (p.mode == EPI_QKV) {
#pragma unroll
    for (int rr = 0; rr < ROWS_PER_WARP; ++rr) {
      const int m = warp + rr * ALL_WARPS;
      epi_slot[rr] = 0;
      epi_rotate[rr] = false;
      if (m < M) {
        if (p.slots != nullptr) epi_slot[rr] = p.slots[m];
        const int half = p.rot_dim / 2;
        if (p.cos_table != nullptr && half > 0) {
          const int pos = p.positions[m];
          epi_rotate[rr] = pos >= 0 && pos < p.max_pos;
          if (epi_rotate[rr]) {
#pragma unroll
            for (int j = 0; j < ROT_PER_LANE; ++j) {
              const int i = lane + 32 * j;
              epi_cos[rr][j] = i < half ? p.cos_table[static_cast<size_t>(pos) * half + i] : 1.0f;
              epi_sin[rr][j] = i < half ? p.sin_table[static_cast<size_t>(pos) * half + i] : 0.0f;
            }
          }
        }
      }
    }
    const void* w = tile < p.nh ? p.q_w : tile < p.nh + p.nkv ? p.k_w : nullptr;
    if (w != nullptr) {
      epi_norm = true;
#pragma unroll
      for (int j = 0; j < 2 * MT; ++j) epi_w[j] = norm_weight(w, p.qk_w_f32, lane + 32 * j);
    }
  }
  // The norm's weights of this CTA's columns go to shared memory as floats (columns beyond K: zeros): they are the
  // same for every row and for every way of staging the rows below.
  if (has_norm) {
    const int per = p.norm_w_f32 ? 4 : 8;            // weights in a 16-byte load
#pragma unroll 1
    for (int e = threadIdx.x * per; e < kc; e += THREADS * per) {
      float w[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      if (k_lo + e < K) {
        if (reinterpret_cast<uintptr_t>(p.norm_w) % 16 != 0) {          // (a view into a larger tensor: one by one)
          for (int i = 0; i < per; ++i) w[i] = norm_weight(p.norm_w, p.norm_w_f32, k_lo + e + i);
        } else if (p.norm_w_f32) {
          const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(p.norm_w) + k_lo + e);
          w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
          unpack_bf16x8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.norm_w) + k_lo + e), w);
        }
      }
      *reinterpret_cast<float4*>(ws + e) = make_float4(w[0], w[1], w[2], w[3]);
      if (!p.norm_w_f32) *reinterpret_cast<float4*>(ws + e + 4) = make_float4(w[4], w[5], w[6], w[7]);
    }
  }
  pdl_wait();                      // x, the residual and the cache belong to the kernels before this one
  STAMP(1);
  if (has_norm) __syncthreads();   // the weights above are read by other threads than wrote them

  // ---- prologue: the rows of x' for columns [k_lo, k_lo + kc) as bfloat16 in shared memory
  if (has_norm && !has_stats) {
    // The residual add and the norm over whole rows.  One pass: the sum s = x + residual is stored rounded (by the
    // writer CTA), its squares are summed, and s * w goes to shared memory as bfloat16.  The row's scale
    // rsqrt(mean(s^2) + eps) is a scalar, so it multiplies the finished product instead (in the epilogue): the
    // weights' product need not wait for the statistics.  Warps that share a row (as many as the CTA has warps
    // for its rows) take its columns in turns of 1,024, four 16-byte loads in flight per tensor.
    const int warps_per_row = max(1, min(ALL_WARPS / M, (K + 1023) / 1024));
    const bool writer = blockIdx.x == 0 && p.residual_out != nullptr;
    const int k_end = max((K + 7) / 8 * 8, k_lo + kc);
#pragma unroll 1
    for (int unit = warp; unit < M * warps_per_row; unit += ALL_WARPS) {
      const int m = unit % M, turn = unit / M;
      float ss = 0.0f;
      const size_t src = static_cast<size_t>(p.x_rows ? p.x_rows[m] : m) * K;
#pragma unroll 1
      for (int k0 = turn * 1024; k0 < k_end; k0 += warps_per_row * 1024) {
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
          float sum[8], other[8];
          unpack_bf16x8(xa[u], sum);
          unpack_bf16x8(xb[u], other);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            sum[i] += other[i];
            ss += sum[i] * sum[i];
          }
          if (writer && k < K) *reinterpret_cast<uint4*>(p.residual_out + src + k) = pack_bf16x8(sum);
          if (k >= k_lo && k < k_lo + kc) {
            const float4 w0 = *reinterpret_cast<const float4*>(ws + (k - k_lo)), w1 = *reinterpret_cast<const float4*>(ws + (k - k_lo) + 4);
            sum[0] *= w0.x; sum[1] *= w0.y; sum[2] *= w0.z; sum[3] *= w0.w;
            sum[4] *= w1.x; sum[5] *= w1.y; sum[6] *= w1.z; sum[7] *= w1.w;
            *reinterpret_cast<uint4*>(xs + m * ldx + (k - k_lo)) = pack_bf16x8(sum);
          }
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) row_ss[unit] = ss;
    }
    __syncthreads();
    if (threadIdx.x < M) {           // (read after later barriers only)
      float ss = 0.0f;
      for (int turn = 0; turn < warps_per_row; ++turn) ss += row_ss[turn * M + threadIdx.x];
      row_scale[threadIdx.x] = rsqrtf(ss / static_cast<float>(K) + p.eps);
    }
  } else {
    // This CTA's columns only, by all threads, four 16-byte loads in flight per tensor: the rows as they are, or
    // (the product before this one left the rounded sums and, per tile of its columns, the rows' sums of squares)
    // x + residual times the norm's weights, with the statistics fetched first and added up last.
    float stat[ROWS_PER_WARP][2];
    if (has_stats) {
#pragma unroll
      for (int rr = 0; rr < ROWS_PER_WARP; ++rr) {
        const int m = warp + rr * ALL_WARPS;
        stat[rr][0] = stat[rr][1] = 0.0f;
        if (m < M) {
          const int row = p.x_rows ? p.x_rows[m] : m;
          if (lane < p.stats_tiles) stat[rr][0] = p.stats_in[lane * MMAX + row];
          if (lane + 32 < p.stats_tiles) stat[rr][1] = p.stats_in[(lane + 32) * MMAX + row];
        }
      }
    }
    const int chunks = kc / 8, total = M * chunks;
    const unsigned inverse = 0xffffffffu / static_cast<unsigned>(chunks) + 1u;   // c / chunks = umulhi(c, inverse) for these small c
    // U chunks of 16 bytes a thread at a time: one where that covers everything (the usual case in a decode step:
    // less code to run through), else four.
    auto stage = [&](auto batch) {
      constexpr int U = decltype(batch)::value;
#pragma unroll 1
      for (int base = 0; base < total; base += U * THREADS) {
        uint4 xa[U], xb[U];
        int at[U], kk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c = base + u * THREADS + threadIdx.x;
          const int m = static_cast<int>(__umulhi(static_cast<unsigned>(c), inverse)), j = (c - m * chunks) * 8;
          at[u] = c < total ? m * ldx + j : -1;
          kk[u] = c < total && k_lo + j < K ? j : -1;
          xa[u] = xb[u] = make_uint4(0u, 0u, 0u, 0u);
          if (kk[u] >= 0) {
            const size_t src = static_cast<size_t>(p.x_rows ? p.x_rows[m] : m) * K + k_lo + j;
            xa[u] = *reinterpret_cast<const uint4*>(p.x + src);
            if (has_stats) xb[u] = *reinterpret_cast<const uint4*>(p.residual + src);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (at[u] < 0) continue;
          if (has_stats && kk[u] >= 0) {
            float sum[8], other[8];
            unpack_bf16x8(xa[u], sum);
            unpack_bf16x8(xb[u], other);
            const float4 w0 = *reinterpret_cast<const float4*>(ws + kk[u]), w1 = *reinterpret_cast<const float4*>(ws + kk[u] + 4);
            sum[0] = (sum[0] + other[0]) * w0.x; sum[1] = (sum[1] + other[1]) * w0.y;
            sum[2] = (sum[2] + other[2]) * w0.z; sum[3] = (sum[3] + other[3]) * w0.w;
            sum[4] = (sum[4] + other[4]) * w1.x; sum[5] = (sum[5] + other[5]) * w1.y;
            sum[6] = (sum[6] + other[6]) * w1.z; sum[7] = (sum[7] + other[7]) * w1.w;
            xa[u] = pack_bf16x8(sum);
          }
          *reinterpret_cast<uint4*>(xs + at[u]) = xa[u];
        }
      }
    };
    if (total <= THREADS) stage(Count<1>());
    else stage(Count<4>());
    if (has_stats) {
#pragma unroll
      for (int rr = 0; rr < ROWS_PER_WARP; ++rr) {
        const int m = warp + rr * ALL_WARPS;
        float ss = stat[rr][0] + stat[rr][1];
        if (m < M) {                                 // (more than 64 tiles: the rest)
          const int row = p.x_rows ? p.x_rows[m] : m;
          for (int t = lane + 64; t < p.stats_tiles; t += 32) ss += p.stats_in[t * MMAX + row];
        }
        ss = warp_sum(ss);
        if (m < M && lane == 0) row_scale[m] = rsqrtf(ss / static_cast<float>(K) + p.eps);
      }
    }
  }
  for (int m = M; m < mpad; ++m)                     // padding rows are zeros
    for (int k = threadIdx.x * 8; k < kc; k += THREADS * 8) *reinterpret_cast<uint4*>(xs + m * ldx + k) = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  STAMP(2);

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
#pragma unroll 1
      for (int j = STAGES; j < nkb && ok; ++j) {
        ok = mbar_wait(empty + j % STAGES, (j / STAGES - 1) & 1, p.err);      // the group that had this stage has left it
        if (ok) issue(j);
      }
    }
  } else {
#pragma unroll 1
    for (int it = grp; it < nkb; it += GROUPS) {
      const int s = it % STAGES;
      if (!mbar_wait(full + s, (it / STAGES) & 1, p.err)) { ok = false; break; }
      const unsigned char* wt = ring + s * STAGE_BYTES;
      // All fragments of (half) a k-block are fetched before the first multiply, so that the fetches' latencies overlap.
      // (Measured: one k-step at a time, rolled or unrolled, makes no difference to a decode step.)
      constexpr int KS = MT == 4 ? 2 : 4;
#pragma unroll
      for (int ks0 = 0; ks0 < BK / 16; ks0 += KS) {
        uint32_t b[KS][4], a[KS][MT][4];
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
          const int ks = ks0 + kk;
          // B operand: x'[m][k], two 8-row groups (m 0..7, 8..15), k and k + 8
          // (with 8 rows of x' only, the lanes of the second group point at the first: its result is not used)
          ldmatrix_x4(b[kk], xs + ((mpad > 8 ? (mi >> 1) * 8 : 0) + r8) * ldx + it * BK + ks * 16 + (mi & 1) * 8);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            const int r = rw * (16 * MT) + i * 16 + (lane & 15);               // weight row inside the tile
            const int c = ks * 2 + (lane >> 4);                                // 16-byte chunk of the 128-byte row
            ldmatrix_x4(a[kk][i], wt + r * 128 + ((c ^ (r & 7)) << 4));
          }
        }
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            mma_bf16(acc[i][0], a[kk][i], b[kk][0], b[kk][1]);
            if (mpad > 8) mma_bf16(acc[i][1], a[kk][i], b[kk][2], b[kk][3]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
  }
  STAMP(3);

  // ---- every warp leaves its sums where its own weight rows lay in a ring stage of its group (stage g is only ever
  // filled for group g, whose copies have all landed, and those rows are read by this warp alone), so no warp waits
  // for another before it stores
  constexpr int WN = 16 * MT;                      // weight rows of a warp
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  if (!feeder) {
    // [mpad][WN + 4]: rows in 16-byte steps, and the four lanes of a quad (rows 2t, 2t + 1) fall on different banks
    float* part = reinterpret_cast<float*>(ring + grp * STAGE_BYTES + rw * (WN * 128));
    static_assert(MMAX * (WN + 4) * 4 <= WN * 128, "a warp's sums fit where its weight rows lay");
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int m = nt * 8 + t2;
        if (m < mpad) {
          float* r0 = part + m * (WN + 4) + i * 16 + g;
          float* r1 = r0 + (WN + 4);
          r0[0] = acc[i][nt][0]; r1[0] = acc[i][nt][1]; r0[8] = acc[i][nt][2]; r1[8] = acc[i][nt][3];
        }
      }
    }
  }
  ok = __syncthreads_and(ok);
  // ---- the cluster's sums meet in rank 0's `red`, scaled by the norm's row scale: this CTA's groups in the groups'
  // order, then the other ranks in rank order, so the result does not depend on timing
  if (p.ksplit > 1 && rank != 0) {
    if (push) cluster_wait();
    const uint32_t slot0 = map_to_rank(smem_u32(slots), 0), bar0 = map_to_rank(smem_u32(gather), 0);
#pragma unroll 1
    for (int i = threadIdx.x; i < (push ? M : mpad) * QUADS; i += THREADS) {
      const int m = i / QUADS, n = (i - m * QUADS) * 4;
      const float4 sum = own_sums<MT, GROUPS>(ring, m, n);
      if (push) store_remote_counted(slot0 + static_cast<uint32_t>((((rank - 1) * M + m) * BN + n) * 4), sum, bar0);
      else *reinterpret_cast<float4*>(red + m * RS + n) = sum;
    }
    if (pull) {
      __syncwarp();
      cluster_arrive(); cluster_wait();              // the sums are written
      cluster_arrive(); cluster_wait();              // rank 0 has read them: this CTA may leave
    }
    STAMP(6);
    return;                        // (after a push, rank 0 stays until the bytes have landed)
  }
  STAMP(4);
  if (push) {
    cluster_wait();
    if (!mbar_wait(gather, 0, p.err)) ok = false;
  }
  if (pull) { cluster_arrive(); cluster_wait(); }
  STAMP(5);
  if (!ok) {                         // a wait ran out (the error word says so): nothing is stored
    if (pull) { cluster_arrive(); cluster_wait(); }
    return;
  }
  {
    const float* theirs[8];
    if (pull) {
#pragma unroll
      for (int r = 1; r < 8; ++r) theirs[r] = r < p.ksplit ? cluster.map_shared_rank(red, r) : red;
    }
#pragma unroll 1
    for (int i = threadIdx.x; i < M * QUADS; i += THREADS) {
      const int m = i / QUADS, n = (i - m * QUADS) * 4;
      float4 sum = own_sums<MT, GROUPS>(ring, m, n);
      if (push) {                                    // (this CTA's own shared memory: a short loop)
        const float* theirs0 = slots + m * BN + n;
#pragma unroll 1
        for (int r = 1; r < p.ksplit; ++r, theirs0 += M * BN) {
          const float4 part = *reinterpret_cast<const float4*>(theirs0);
          sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
        }
      } else if (pull) {
        float4 part[8];                              // every rank's part is fetched before any is used
#pragma unroll
        for (int r = 1; r < 8; ++r)
          part[r] = r < p.ksplit ? *reinterpret_cast<const float4*>(theirs[r] + m * RS + n) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int r = 1; r < 8; ++r) { sum.x += part[r].x; sum.y += part[r].y; sum.z += part[r].z; sum.w += part[r].w; }
      }
      if (has_norm) { const float f = row_scale[m]; sum.x *= f; sum.y *= f; sum.z *= f; sum.w *= f; }
      if (p.mode == EPI_QKV || p.mode == EPI_SWIGLU) {
        // these products' outputs are bfloat16 tensors in the unfused path; the same rounding here
        sum.x = __bfloat162float(__float2bfloat16_rn(sum.x)); sum.y = __bfloat162float(__float2bfloat16_rn(sum.y));
        sum.z = __bfloat162float(__float2bfloat16_rn(sum.z)); sum.w = __bfloat162float(__float2bfloat16_rn(sum.w));
      }
      *reinterpret_cast<float4*>(red + m * RS + n) = sum;
    }
  }
  __syncwarp();
  if (pull) cluster_arrive();        // the others may leave (this CTA looks at the barrier again when it leaves)
  __syncthreads();

  // ---- epilogue on red[m][n] (float)
  if (p.mode == EPI_PLAIN_BF16 || p.mode == EPI_PLAIN_F32) {
    const bool whole = p.N % 4 == 0;               // then four neighbours are stored at once
    const bool post = p.post_stats != nullptr && p.mode == EPI_PLAIN_BF16;
    static_assert(QUADS <= 32 || MT == 4, "a row's quads lie inside one warp");
#pragma unroll 1
    for (int i0 = 0; i0 < M * QUADS; i0 += THREADS) {
      const int i = i0 + threadIdx.x;
      const int m = i / QUADS, q = i - m * QUADS, n = q * 4, col = tile * BN + n;
      const bool valid = i < M * QUADS && col < p.N;
      const size_t at = static_cast<size_t>(m) * p.N + col;
      float ss = 0.0f;
      if (valid) {
        const float4 v = *reinterpret_cast<const float4*>(red + m * RS + n);
        const float f[4] = {v.x, v.y, v.z, v.w};
        if (p.mode == EPI_PLAIN_F32) {
          if (whole) *reinterpret_cast<float4*>(static_cast<float*>(p.out) + at) = v;
          else
            for (int e = 0; e < 4 && col + e < p.N; ++e) static_cast<float*>(p.out)[at + e] = f[e];
        } else {
          __align__(8) bf16 h[4], sums[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = __float2bfloat16_rn(f[e]);
          if (post) {
            // The norm that follows: s = round(y) + residual in float (what its prologue would add up), stored
            // rounded, and the squares of s over this tile's columns.
            __align__(8) bf16 res[4];
            if (whole) *reinterpret_cast<uint2*>(res) = *reinterpret_cast<const uint2*>(p.post_residual + at);
            else
              for (int e = 0; e < 4; ++e) res[e] = col + e < p.N ? p.post_residual[at + e] : __float2bfloat16_rn(0.0f);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float sum = col + e < p.N ? __bfloat162float(h[e]) + __bfloat162float(res[e]) : 0.0f;
              sums[e] = __float2bfloat16_rn(sum);
              ss += sum * sum;
            }
          }
          if (whole) {
            *reinterpret_cast<uint2*>(static_cast<bf16*>(p.out) + at) = *reinterpret_cast<uint2*>(h);
            if (post) *reinterpret_cast<uint2*>(p.post_sum_out + at) = *reinterpret_cast<uint2*>(sums);
          } else {
            for (int e = 0; e < 4 && col + e < p.N; ++e) {
              static_cast<bf16*>(p.out)[at + e] = h[e];
              if (post) p.post_sum_out[at + e] = sums[e];
            }
          }
        }
      }
      if (post) {                                    // a row's quads are neighbouring lanes: their squares meet in the first
        __syncwarp();
#pragma unroll
        for (int off = (QUADS < 32 ? QUADS : 32) / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (i < M * QUADS && q == 0) p.post_stats[tile * MMAX + m] = ss;
      }
    }
  } else if (p.mode == EPI_SWIGLU) {
    const int inter = p.N / 2;
    const bool whole = inter % 4 == 0;
#pragma unroll 1
    for (int i = threadIdx.x; i < M * (QUADS / 2); i += THREADS) {
      const int m = i / (QUADS / 2), n = (i - m * (QUADS / 2)) * 4, col = tile * (BN / 2) + n;
      if (col >= inter) continue;
      const float4 gate4 = *reinterpret_cast<const float4*>(red + m * RS + n), up4 = *reinterpret_cast<const float4*>(red + m * RS + BN / 2 + n);
      const float gf[4] = {gate4.x, gate4.y, gate4.z, gate4.w}, uf[4] = {up4.x, up4.y, up4.z, up4.w};
      __align__(8) bf16 h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __float2bfloat16_rn(gf[e] / (1.0f + expf(-gf[e])) * uf[e]);
      const size_t at = static_cast<size_t>(m) * inter + col;
      if (whole) *reinterpret_cast<uint2*>(static_cast<bf16*>(p.out) + at) = *reinterpret_cast<uint2*>(h);
      else
        for (int e = 0; e < 4 && col + e < inter; ++e) static_cast<bf16*>(p.out)[at + e] = h[e];
    }
  } else {                                                                   // EPI_QKV: tile = one head, BN = head_dim
    constexpr int d = BN;
    const int head = tile;
    const bool is_q = head < p.nh, is_k = !is_q && head < p.nh + p.nkv;
#pragma unroll
    for (int rr = 0; rr < ROWS_PER_WARP; ++rr) {
      const int m = warp + rr * ALL_WARPS;                                   // (its slot and angles were fetched at the start)
      if (m >= M) continue;
      float* row = red + m * RS;
      bf16* dst = nullptr;
      if (is_q) {
        dst = static_cast<bf16*>(p.out) + (static_cast<size_t>(m) * p.nh + head) * d;
      } else if (p.slots != nullptr && epi_slot[rr] != 0) {
        if (epi_slot[rr] < 0 || epi_slot[rr] >= p.cache_slots) {
          if (lane == 0) atomicOr(p.err, B200_ERR_SLOT_RANGE);
        } else {
          const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
          const int page = epi_slot[rr] / p.page_size, offset = epi_slot[rr] - page * p.page_size;
          dst = (is_k ? p.k_cache : p.v_cache) + ((static_cast<size_t>(page) * p.nkv + kvh) * p.page_size + offset) * d;
        }
      }
      if (dst != nullptr && !is_q && !is_k) {
        for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
      } else if (dst != nullptr) {
        if (epi_norm) {
          float ss = 0.0f;
#pragma unroll
          for (int j = 0; j < 2 * MT; ++j) ss += row[lane + 32 * j] * row[lane + 32 * j];
          ss = warp_sum(ss);
          const float scale = rsqrtf(ss / static_cast<float>(d) + p.qk_eps);
#pragma unroll
          for (int j = 0; j < 2 * MT; ++j) row[lane + 32 * j] = row[lane + 32 * j] * scale * epi_w[j];
          __syncwarp();
        }
        const int half = p.rot_dim / 2;
        const bool wanted = p.cos_table != nullptr && half > 0;
        if (wanted && !epi_rotate[rr] && lane == 0) atomicOr(p.err, B200_ERR_POSITION_RANGE);
        if (wanted && epi_rotate[rr]) {
#pragma unroll
          for (int j = 0; j < ROT_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            if (i < half) {
              const float a = row[i], b = row[i + half];
              dst[i] = __float2bfloat16_rn(a * epi_cos[rr][j] - b * epi_sin[rr][j]);
              dst[i + half] = __float2bfloat16_rn(b * epi_cos[rr][j] + a * epi_sin[rr][j]);
            }
          }
          for (int i = p.rot_dim + lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
        } else {
          for (int i = lane; i < d; i += 32) dst[i] = __float2bfloat16_rn(row[i]);
        }
      }
    }
  }
  __syncwarp();
  if (pull) cluster_wait();              // (every arrival is answered by a wait; the others have long arrived)
#ifdef SKINNY_TRACE
  __syncthreads();
  STAMP(7);
#endif
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

// Largest K range of one CTA of shape `occ` for `m` rows, in columns: the rows of x' (with 8 columns of padding) and,
// with a norm, its weights as floats share the CTA's x region.
static int kc_max_of(int m, int occ, bool has_norm) {
  const int mpad = m <= 8 ? 8 : 16;
  const int xs_bytes = occ == 1 ? Shape<1>::XS_BYTES : Shape<2>::XS_BYTES;
  return (xs_bytes - 16 * mpad) / (2 * mpad + (has_norm ? 4 : 0)) / BK * BK;
}

// The CTA's shape (`occ_out`: CTAs an SM) and the cluster size (CTAs that split K); 0: the product is refused.
static int choose_ksplit(int m, int n_tiles, int k, int sm_count, bool has_norm, bool occ2_possible, int* occ_out) {
  const int kblocks = (k + BK - 1) / BK;
  *occ_out = 1;
  const int need = (k + kc_max_of(m, 1, has_norm) - 1) / kc_max_of(m, 1, has_norm);
  const int need2 = (k + kc_max_of(m, 2, has_norm) - 1) / kc_max_of(m, 2, has_norm);
  if (need > 8) return 0;
  // Clusters of 3, 5, 6 or 7 are only taken while the grid stays under half the machine: measured at the Qwen3-8B
  // sizes, 192 clusters of 3 ran 20 % longer than 192 clusters of 2 (a cluster is placed on whole pairs of SMs, so an
  // odd one leaves an SM idle), while 8 clusters of 3 beat 8 of 2.
  auto allowed = [&](int split, int least) {
    return split == least || (split & (split - 1)) == 0 || 2ll * n_tiles * split <= sm_count;
  };
  // A grid that fits one wave of the SMs is bound by how fast ONE SM takes its share in, not by memory: as many CTAs
  // as fit the wave, down to eight k-blocks (64 KB of weights at 64 rows) a CTA.  Measured at the Qwen3-0.6B sizes
  // (decode, batch 8 / batch 1): 1.69 -> 1.56 ms and 1.16 -> 1.02 ms a step against a floor of sixteen k-blocks; a
  // floor of four was slower again (1.66 ms): the cluster's hand-over then costs more than the SMs it wins.
  int one_wave = 0;
  for (int split = need; split <= 8; ++split) {
    if (split > need && kblocks / split < 8) break;
    if (static_cast<long long>(n_tiles) * split > sm_count) break;
    if (allowed(split, need)) one_wave = split;
  }
  if (one_wave > 0) return one_wave;
  // Several waves: every CTA pays its set-up again, so a CTA keeps at least sixteen k-blocks, and among those cluster
  // sizes the one whose CTAs fill whole waves best wins (a larger cluster must win by a margin: its hand-over is
  // longer).  At the Qwen3-8B sizes the floor of eight k-blocks made a step 7.7 ms instead of 5.0.  Two CTAs share an
  // SM where the tile allows it: one streams while the other stages its rows or adds up its tile (5.09 -> 4.89 ms).
  const int occ = occ2_possible && need2 <= 8 ? 2 : 1;
  const int least = occ == 2 ? need2 : need;
  const long long slots = static_cast<long long>(sm_count) * occ;
  int best = least;
  double best_fill = 0.0;
  for (int split = least; split <= 8; ++split) {
    if (split > least && kblocks / split < 16) break;
    if (!allowed(split, least)) continue;
    const long long ctas = static_cast<long long>(n_tiles) * split;
    const long long waves = (ctas + slots - 1) / slots;
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    if (fill > best_fill + 0.04) { best = split; best_fill = fill; }
  }
  *occ_out = occ;
  return best;
}

template <int MT, int OCC>
static int launch_as(const CUtensorMap& map, const SkinnyParams& p, int n_tiles, cudaStream_t stream) {
  constexpr int BN = 64 * MT;
  constexpr int STAGES = Shape<OCC>::W_RING_BYTES / (BN * 128);
  const size_t smem = 1024 + Shape<OCC>::W_RING_BYTES + Shape<OCC>::XS_BYTES + MMAX * (BN + 4) * sizeof(float) +
                      (2 * STAGES + 2) * sizeof(uint64_t) + (MMAX + 32) * sizeof(float) + 64;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(skinny_linear_kernel<MT, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return b200_launch(skinny_linear_kernel<MT, OCC>, dim3(n_tiles * p.ksplit), dim3(Shape<OCC>::THREADS), smem, stream,
                     p.ksplit, map, p);
}

template <int MT>
static int launch(const CUtensorMap& map, const SkinnyParams& p, int n_tiles, int occ, cudaStream_t stream) {
  if constexpr (MT == 2) {
    if (occ == 2) return launch_as<MT, 2>(map, p, n_tiles, stream);
  }
  return launch_as<MT, 1>(map, p, n_tiles, stream);
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
  if (p.post_stats != nullptr && (p.mode != EPI_PLAIN_BF16 || bn > 128 || p.post_residual == nullptr || p.post_sum_out == nullptr))
    return B200_BAD_SIZE;
  if (p.stats_in != nullptr && (p.residual == nullptr || p.stats_tiles <= 0)) return B200_BAD_SIZE;
  if (p.mode == EPI_QKV && (p.N != (p.nh + 2 * p.nkv) * head_dim || p.rot_dim < 0 || p.rot_dim > head_dim || (p.rot_dim & 1)))
    return B200_BAD_SIZE;
  const int cols = p.mode == EPI_SWIGLU ? p.N / 2 : p.N;
  const int tile_cols = p.mode == EPI_SWIGLU ? bn / 2 : bn;
  const int n_tiles = (cols + tile_cols - 1) / tile_cols;
  int occ = 1;
  p.ksplit = choose_ksplit(p.M, n_tiles, p.K, sm_count > 0 ? sm_count : 148, p.residual != nullptr, bn == 128, &occ);
  if (p.ksplit == 0) return B200_BAD_SIZE;
  CUtensorMap map;
  memcpy(&map, w_map, sizeof(map));
  if (bn == 64) return launch<1>(map, p, n_tiles, occ, stream);
  if (bn == 128) return launch<2>(map, p, n_tiles, occ, stream);
  return launch<4>(map, p, n_tiles, occ, stream);
}

B200_EXPORT int b200_skinny_params_size() { return static_cast<int>(sizeof(SkinnyParams)); }
