// Tensor-core attention over the paged bfloat16 cache, for one head size
// (compile with -DHEAD_DIM=<multiple of 16, at most 256>).
//
// Decode (one query position per row) is bound by the bytes of keys and values
// that a step has to read, so this kernel is built around the copy engine.  The
// cache is laid out [page][KV head][offset in page][head_dim]: the rows of one
// page and KV head are one contiguous block, which TMA fetches as boxes of
// (up to 32 rows) x (64 dims = 128 bytes) straight into shared memory in the
// 128-byte swizzle, reporting to an mbarrier.  A CTA owns one (row, KV head,
// split of the keys); each of its warps walks its own blocks of 32 keys through a
// private ring of stages (16 KB per block at head size 128), so that tens of KB
// per SM are in flight and the loop has no block-wide barrier.  Every wait on a
// barrier is bounded by the clock: when it runs out the kernel flags the engine's
// error word, gives the outstanding copies a bounded time to land and returns.
// The arithmetic rides on mma.sync m16n8k16 (bfloat16 in, float accumulate): the
// query heads that share the KV head are the 16 rows of the A operand (at most 16
// heads per KV head; larger groups, page sizes that are no power of two and float
// caches take the CUDA-core kernel of attention.cu), keys and values are read
// from the swizzled tiles with ldmatrix (values transposed).  Scores, the running
// maximum, the running sum and the output are float; probabilities are rounded to
// bfloat16 only as the A operand of P.V, as the values themselves are bfloat16.
//
// Semantics are those of attention.cu (reference: src/models/attention/backend.rs:1455-1498):
// KV head = head / group, score = q.k * scale, keys j <= p (and j > p - W with a
// window), softmax in float, output = P.V.  Value rows at or beyond the sequence
// end are zeroed in shared memory before they are used, key rows there are masked:
// a page that is used again may hold anything.
#include <cuda.h>
#include <math.h>
#include <string.h>

#include <cooperative_groups.h>

#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size, a multiple of 16>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "the tensor-core kernels take head sizes 16..256 in steps of 16");

typedef __nv_bfloat16 bf16;
namespace cg = cooperative_groups;
constexpr int D = HEAD_DIM;
constexpr int LD = D + 8;          // padded row of the query tile (16 bytes of padding): conflict-free ldmatrix
constexpr int KB = 32;             // keys per block
constexpr int NB = (D + 63) / 64;  // 64-dim (128-byte) column boxes per row
constexpr int HALF_BYTES = KB * 128;              // one column box of a block: 32 rows x 128 bytes
constexpr int TILE_BYTES = 2 * NB * HALF_BYTES;   // keys then values of one block
constexpr int QROWS = 16;          // rows of the A operand: query heads of one KV head

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {      // 2^x in one special-function instruction (-inf gives 0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- mbarrier and bulk-copy primitives (the copy engine writes shared memory and signals the barrier)
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

// Byte offset of (row r, 16-byte chunk c of the row's D dims) inside a tile of NB column boxes, each
// [32 rows][128 bytes] in the 128-byte swizzle (chunk index XOR row mod 8; tiles are 1024-byte aligned).
__device__ __forceinline__ int swz(int r, int c) {
  return (c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// One warp fetches keys [first_key, first_key + 32) of one KV head into `tile` (keys, then values).
// The block is cut into sub-blocks of `box_rows` rows (a power of two that divides 32 and the page
// size, so a sub-block never leaves its page); lane j issues the boxes of sub-block j with the page
// id `page` that it looked up one block earlier.  Sub-blocks that start at or beyond kv_end are skipped.
__device__ __forceinline__ void fetch_block(unsigned char* tile, const CUtensorMap* kmap, const CUtensorMap* vmap,
                                            int page, int page_size, int nkv, int kvh, int box_rows, int first_key,
                                            int kv_end, uint64_t* bar, int lane) {
  const int n_sub = (min(KB, kv_end - first_key) + box_rows - 1) / box_rows;
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // earlier reads and writes of the tile come first
  if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_sub) * 2u * NB * box_rows * 128u);
  __syncwarp();
  if (lane < n_sub) {
    const int key0 = first_key + lane * box_rows;
    const int y = (page * nkv + kvh) * page_size + key0 % page_size;
#pragma unroll
    for (int h = 0; h < NB; ++h) {
      tma_load_2d(tile + h * HALF_BYTES + lane * box_rows * 128, kmap, h * 64, y, bar);
      tma_load_2d(tile + (NB + h) * HALF_BYTES + lane * box_rows * 128, vmap, h * 64, y, bar);
    }
  }
}

// Page id of the sub-block that this lane fetches in the block that starts at first_key.  It is loaded one
// block ahead of its use, so that the table's latency is off the copies' critical path.
__device__ __forceinline__ int lane_page(const int* __restrict__ table, int page_size, int box_rows, int first_key,
                                         int kv_end, int lane) {
  const int key0 = first_key + lane * box_rows;
  return (lane * box_rows < KB && key0 < kv_end) ? table[key0 / page_size] : 0;
}

// State of one warp: 16 query rows x D outputs in mma accumulator layout.
struct WarpAcc {
  float o[D / 8][4];
  float m[2], l[2];          // rows lane/4 and lane/4 + 8; l is this thread's part of the row sum
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    m[0] = m[1] = -INFINITY; l[0] = l[1] = 0.0f;
  }
};

// One block of 32 keys against the 16 query rows in `qs`.  `qpos0/1`: position of the query in rows
// lane/4 and lane/4 + 8 (-1: the row is unused).  `scale_log2` = softmax scale * log2(e).
// MASKED = false: the caller knows that every key of the block is visible to every used row of the warp.
template <bool MASKED>
__device__ __forceinline__ void block_mma(const bf16* qs, const unsigned char* ks, const unsigned char* vs, int first_key, int kv_end,
                                          int window, int qpos0, int qpos1, float scale_log2, WarpAcc& st) {
  const int lane = threadIdx.x & 31;
  const int mi = lane >> 3, r8 = lane & 7;
  float s[4][4];
#pragma unroll
  for (int n = 0; n < 4; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f; }
#pragma unroll
  for (int ks16 = 0; ks16 < D / 16; ++ks16) {
    uint32_t a[4];
    ldmatrix_x4(a, qs + (lane & 15) * LD + ks16 * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int n = 0; n < 4; n += 2) {
      uint32_t b[4];
      ldmatrix_x4(b, ks + swz(n * 8 + (mi >> 1) * 8 + r8, ks16 * 2 + (mi & 1)));
      mma_bf16(s[n], a, b[0], b[1]);
      mma_bf16(s[n + 1], a, b[2], b[3]);
    }
  }
  const int t2 = (lane & 3) * 2;
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      bool v0 = qpos0 >= 0, v1 = qpos1 >= 0;
      if (MASKED) {
        const int key = first_key + n * 8 + t2 + e;
        const bool in_seq = key < kv_end;
        v0 = in_seq && v0 && key <= qpos0 && (window <= 0 || key > qpos0 - window);
        v1 = in_seq && v1 && key <= qpos1 && (window <= 0 || key > qpos1 - window);
      }
      s[n][e] = v0 ? s[n][e] * scale_log2 : -INFINITY;
      s[n][2 + e] = v1 ? s[n][2 + e] * scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, s[n][e]);
      mx1 = fmaxf(mx1, s[n][2 + e]);
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float m0 = fmaxf(st.m[0], mx0), m1 = fmaxf(st.m[1], mx1);
  const float c0 = m0 == -INFINITY ? 1.0f : exp2f(st.m[0] - m0);      // exp2(-inf) = 0 on the first visible block
  const float c1 = m1 == -INFINITY ? 1.0f : exp2f(st.m[1] - m1);
  const float base0 = m0 == -INFINITY ? 0.0f : m0, base1 = m1 == -INFINITY ? 0.0f : m1;
  float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      s[n][e] = fast_exp2(s[n][e] - base0);          // a masked score is -inf: exp2 gives 0
      s[n][2 + e] = fast_exp2(s[n][2 + e] - base1);
      sum0 += s[n][e];
      sum1 += s[n][2 + e];
    }
  }
  st.m[0] = m0; st.m[1] = m1;
  st.l[0] = st.l[0] * c0 + sum0;
  st.l[1] = st.l[1] * c1 + sum1;
  if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {       // no row's maximum moved: nothing to rescale
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { st.o[i][0] *= c0; st.o[i][1] *= c0; st.o[i][2] *= c1; st.o[i][3] *= c1; }
  }
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dn = 0; dn < D / 8; dn += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs + swz(kk * 16 + (mi & 1) * 8 + r8, dn + (mi >> 1)));
      mma_bf16(st.o[dn], a, b[0], b[1]);
      mma_bf16(st.o[dn + 1], a, b[2], b[3]);
    }
  }
}

// ------------------------------------------------------------------ decoded tokens
// grid (splits, nkv, decode rows).  Partials: part_acc[((row * nh + head) * splits + split) * D + dim]
// (unnormalised), part_ml[...][2] = (maximum in log2 units, sum).
// Shared memory: [WARPS][STAGES] tiles (1024-byte aligned), the query tile [16][LD], the barriers.
template <int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32, 1)
decode_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part_acc,
                  float* __restrict__ part_ml, const int* __restrict__ block_table, int table_stride,
                  const int* __restrict__ cu_q, const int* __restrict__ kv_len, const int* __restrict__ rows, int nh,
                  int nkv, int page_size, int box_rows, int window, float scale_log2, int cluster_merge, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  bf16* qs = reinterpret_cast<bf16*>(tiles + static_cast<size_t>(WARPS) * STAGES * TILE_BYTES);   // [16][LD]
  uint64_t* bars = reinterpret_cast<uint64_t*>(qs + QROWS * LD);                                   // [WARPS][STAGES]

  pdl_launch_dependents();
  if (threadIdx.x < WARPS * STAGES) mbar_init(bars + threadIdx.x, 1);
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();
  // The kernel before this one in the stream wrote q and the step's newest key and value of every row.  The
  // step's index arrays were uploaded before the step's first kernel, and all other keys and values are older:
  // both may be read while that kernel still runs.
  const int splits = gridDim.x, split = blockIdx.x, kvh = blockIdx.y;
  const int row = rows[blockIdx.z];
  const int group = nh / nkv, head0 = kvh * group;
  const int tok = cu_q[row];
  const int kv_end = kv_len[row];
  const int qp = kv_end - 1;
  int k_begin = window > 0 ? max(0, qp - window + 1) : 0;
  k_begin -= k_begin % KB;
  const int blocks_total = (kv_end - k_begin + KB - 1) / KB;
  const int per_split = (blocks_total + splits - 1) / splits;
  const int blk_lo = split * per_split, blk_hi = min(blocks_total, blk_lo + per_split);
  const int* table = block_table + static_cast<size_t>(row) * table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  unsigned char* my = tiles + static_cast<size_t>(warp) * STAGES * TILE_BYTES;
  uint64_t* my_bars = bars + warp * STAGES;
  int issue = blk_lo + warp;
  int page = 0;
  auto first_fill = [&]() {                            // the ring's first STAGES - 1 blocks of this warp
    page = issue < blk_hi ? lane_page(table, page_size, box_rows, k_begin + issue * KB, kv_end, lane) : 0;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      const int next = issue + WARPS;
      const int next_page = next < blk_hi ? lane_page(table, page_size, box_rows, k_begin + next * KB, kv_end, lane) : 0;
      if (issue < blk_hi)
        fetch_block(my + s * TILE_BYTES, &kmap, &vmap, page, page_size, nkv, kvh, box_rows, k_begin + issue * KB, kv_end,
                    my_bars + s, lane);
      issue = next;
      page = next_page;
    }
  };
  // They are fetched under the tail of the kernel before, unless the newest key (position kv_end - 1) is in them.
  const int last_of_fill = blk_lo + warp + (STAGES - 2) * WARPS;
  const bool early = k_begin + (last_of_fill + 1) * KB <= qp;
  if (early) first_fill();
  pdl_wait();
  if (!early) first_fill();

  for (int c = threadIdx.x; c < QROWS * (D / 8); c += blockDim.x) {
    const int r = c / (D / 8), part = c - r * (D / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < group) v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(tok) * nh + head0 + r) * D + part * 8);
    *reinterpret_cast<uint4*>(qs + r * LD + part * 8) = v;
  }
  __syncthreads();
  const int g = lane >> 2;
  const int qpos0 = g < group ? qp : -1, qpos1 = g + 8 < group ? qp : -1;
  WarpAcc st;
  st.init();
  int stage = 0;
  uint32_t parity = 0;
  for (int blk = blk_lo + warp; blk < blk_hi; blk += WARPS) {
    const int s_issue = stage == 0 ? STAGES - 1 : stage - 1;      // the stage that the previous block left
    const int next = issue + WARPS;
    const int next_page = next < blk_hi ? lane_page(table, page_size, box_rows, k_begin + next * KB, kv_end, lane) : 0;
    if (issue < blk_hi)
      fetch_block(my + s_issue * TILE_BYTES, &kmap, &vmap, page, page_size, nkv, kvh, box_rows, k_begin + issue * KB,
                  kv_end, my_bars + s_issue, lane);
    issue = next;
    page = next_page;
    if (!mbar_wait(my_bars + stage, parity, err)) {
      // Give the copies that are still in flight a bounded time to land before the tiles are reused.
      for (int s = 0; s < STAGES; ++s) mbar_wait(my_bars + s, s < stage ? parity ^ 1u : parity, err);
      break;
    }
    unsigned char* t = my + stage * TILE_BYTES;
    const int first_key = k_begin + blk * KB;
    if (first_key + KB > kv_end && first_key + lane >= kv_end) {
      // Value rows beyond the sequence: whatever the page holds there must not reach P.V.
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int c = 0; c < NB * 8; ++c) *reinterpret_cast<uint4*>(t + NB * HALF_BYTES + (c >> 3) * HALF_BYTES + lane * 128 + (c & 7) * 16) = zero;
    }
    __syncwarp();
    if (first_key + KB <= kv_end && (window <= 0 || first_key > qp - window))
      block_mma<false>(qs, t, t + NB * HALF_BYTES, first_key, kv_end, window, qpos0, qpos1, scale_log2, st);
    else
      block_mma<true>(qs, t, t + NB * HALF_BYTES, first_key, kv_end, window, qpos0, qpos1, scale_log2, st);
    __syncwarp();                                      // every lane is done reading before the stage is refilled
    if (++stage == STAGES) { stage = 0; parity ^= 1u; }
  }
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1); st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1); st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);
  __syncthreads();
  // Merge the warps through shared memory: [WARPS][group][D + 2] floats over the tile area.
  float* merge = reinterpret_cast<float*>(tiles);     // all copies have landed and been used
  constexpr int MS = D + 2;
  float* mine = merge + WARPS * QROWS * MS;           // [group][MS]: the CTA's own combined part
  const int t2 = (lane & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    if (r < group) {
      float* dst = merge + (warp * group + r) * MS;
#pragma unroll
      for (int dn = 0; dn < D / 8; ++dn) {
        dst[dn * 8 + t2] = st.o[dn][2 * half];
        dst[dn * 8 + t2 + 1] = st.o[dn][2 * half + 1];
      }
      if ((lane & 3) == 0) { dst[D] = st.m[half]; dst[D + 1] = st.l[half]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < group * D; i += blockDim.x) {
    const int r = i / D, dim = i - r * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge[(w * group + r) * MS + D]);
    float l = 0.0f, o = 0.0f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = merge + (w * group + r) * MS;
        const float f = exp2f(src[D] - m);
        l += src[D + 1] * f;
        o += src[dim] * f;
      }
    }
    const int head = head0 + r;
    if (splits == 1) {
      out[(static_cast<size_t>(tok) * nh + head) * D + dim] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
    } else if (cluster_merge) {
      mine[r * MS + dim] = o;                          // this CTA's part, for the cluster's first CTA to read
      if (dim == 0) { mine[r * MS + D] = m; mine[r * MS + D + 1] = l; }
    } else {
      const size_t slot = (static_cast<size_t>(blockIdx.z) * nh + head) * splits + split;
      part_acc[slot * D + dim] = o;
      if (dim == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
    }
  }
  if (!cluster_merge) return;
  // The splits of a (row, KV head) pair are the CTAs of one cluster: the first combines all parts out of the others'
  // shared memory (every CTA reaches both barriers, also one whose waits ran out).
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  if (split == 0) {
    for (int i = threadIdx.x; i < group * D; i += blockDim.x) {
      const int r = i / D, dim = i - r * D;
      float m = -INFINITY;
      for (int s = 0; s < splits; ++s) m = fmaxf(m, cluster.map_shared_rank(mine, s)[r * MS + D]);
      float l = 0.0f, o = 0.0f;
      if (m != -INFINITY) {
        for (int s = 0; s < splits; ++s) {
          const float* src = cluster.map_shared_rank(mine, s) + r * MS;
          const float f = exp2f(src[D] - m);
          l += src[D + 1] * f;
          o += src[dim] * f;
        }
      }
      out[(static_cast<size_t>(tok) * nh + head0 + r) * D + dim] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
    }
  }
  cluster.sync();                                      // nobody leaves while its shared memory may still be read
}

// grid (decode rows, nh): combines the splits of one head (maxima are in log2 units).
__global__ void decode_mma_merge_kernel(bf16* __restrict__ out, const float* __restrict__ part_acc,
                                        const float* __restrict__ part_ml, const int* __restrict__ cu_q,
                                        const int* __restrict__ rows, int nh, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.y;
  const int tok = cu_q[rows[blockIdx.x]];
  const size_t base = (static_cast<size_t>(blockIdx.x) * nh + head) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
    float l = 0.0f, o = 0.0f;
    if (m != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float f = exp2f(part_ml[(base + s) * 2] - m);
        l += part_ml[(base + s) * 2 + 1] * f;
        o += part_acc[(base + s) * D + dim] * f;
      }
    }
    out[(static_cast<size_t>(tok) * nh + head) * D + dim] = __float2bfloat16_rn(l > 0.0f ? o / l : 0.0f);
  }
}

// ------------------------------------------------------------------ prompt portions
// grid (query tiles, nkv, prefill rows).  A CTA serves PF_WARPS * 16 query vectors: consecutive
// tokens of one row x the `group` query heads of one KV head; warp w owns vectors 16 w .. 16 w + 15
// (a warp holds 16 / group whole tokens).  All warps read the same key blocks, which one warp fetches
// into a ring of stages: full[s] flips when the boxes of a block have landed, empty[s] when every
// warp has finished with it.  Each query vector has its own position, so the causal mask (and the
// window) is applied per row of the score tile.
constexpr int PF_WARPS = 4;
// Three CTAs share an SM for heads up to 128 wide (the register budget that this leaves is 170 a thread).
constexpr int PF_MIN_CTAS = D <= 128 ? 3 : 1;
constexpr int PF_ROWS = PF_WARPS * 16;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(PF_WARPS * 32, PF_MIN_CTAS)
prefill_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ block_table,
                   int table_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                   const int* __restrict__ prefix_len, const int* __restrict__ rows, int nh, int nkv, int page_size,
                   int box_rows, int window, float scale_log2, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  bf16* qs = reinterpret_cast<bf16*>(tiles + static_cast<size_t>(STAGES) * TILE_BYTES);     // [PF_ROWS][LD]
  uint64_t* full = reinterpret_cast<uint64_t*>(qs + PF_ROWS * LD);
  uint64_t* empty = full + STAGES;

  // Grid: x = KV head, y = row, z = tile order.  CTAs start in the order x, y, z, and a row's last tiles see the
  // most keys: every row's heaviest tiles start first, over all heads, so that the short ones fill the tail.
  const int row = rows[blockIdx.y];
  const int kvh = blockIdx.x;
  const int group = nh / nkv, head0 = kvh * group;
  const int tokens_per_warp = 16 / group;                       // whole tokens per warp
  const int tile_tokens = tokens_per_warp * PF_WARPS;
  const int q_begin = cu_q[row], q_len = cu_q[row + 1] - q_begin;
  const int tile = (q_len + tile_tokens - 1) / tile_tokens - 1 - static_cast<int>(blockIdx.z);
  if (tile < 0) return;
  const int tok0 = tile * tile_tokens;
  const int ntok = min(tile_tokens, q_len - tok0);
  const int prefix = prefix_len[row];
  const int kv_end = min(kv_len[row], prefix + tok0 + ntok);     // causal: nothing later is visible to this tile
  const int p_lo = prefix + tok0;
  int k_begin = window > 0 ? max(0, p_lo - window + 1) : 0;
  k_begin -= k_begin % KB;
  const int nblk = (kv_end - k_begin + KB - 1) / KB;
  const int* table = block_table + static_cast<size_t>(row) * table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int c = threadIdx.x; c < PF_ROWS * (D / 8); c += blockDim.x) {
    const int r = c / (D / 8), part = c - r * (D / 8);
    const int w = r >> 4, i = r & 15;
    const int tok = w * tokens_per_warp + i / group, head = head0 + i % group;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (i < tokens_per_warp * group && tok < ntok)
      v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(q_begin + tok0 + tok) * nh + head) * D + part * 8);
    *reinterpret_cast<uint4*>(qs + r * LD + part * 8) = v;
  }
  if (threadIdx.x < STAGES) { mbar_init(full + threadIdx.x, 1); mbar_init(empty + threadIdx.x, PF_WARPS); }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();

  // Positions of this thread's two score rows (lane / 4 and lane / 4 + 8 of the warp's 16 vectors).
  const int g = lane >> 2;
  int qpos[2], tok_of[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i = g + 8 * h;
    const int tok = warp * tokens_per_warp + i / group;
    const bool used = i < tokens_per_warp * group && tok < ntok;
    tok_of[h] = used ? tok : -1;
    qpos[h] = used ? p_lo + tok : -1;
  }
  // The warp's own range of key blocks: from its first visible key to its last query's position.
  const int w_tok_lo = warp * tokens_per_warp;
  const int w_tok_hi = min(ntok, w_tok_lo + tokens_per_warp) - 1;           // < w_tok_lo: the warp holds no token
  const int w_p_hi = p_lo + w_tok_hi;
  const int w_first_key = window > 0 ? max(0, p_lo + w_tok_lo - window + 1) : 0;

  WarpAcc st;
  st.init();
  const bf16* my_q = qs + warp * 16 * LD;
  bool ok = true;
  int page = 0;
  if (warp == 0) {                                                          // prologue of the producer
    page = nblk > 0 ? lane_page(table, page_size, box_rows, k_begin, kv_end, lane) : 0;
    for (int j = 0; j < STAGES - 1 && j < nblk; ++j) {
      const int next_page = j + 1 < nblk ? lane_page(table, page_size, box_rows, k_begin + (j + 1) * KB, kv_end, lane) : 0;
      fetch_block(tiles + j * TILE_BYTES, &kmap, &vmap, page, page_size, nkv, kvh, box_rows, k_begin + j * KB, kv_end,
                  full + j, lane);
      page = next_page;
    }
  }
  for (int it = 0; it < nblk && ok; ++it) {
    const int s = it % STAGES;
    if (warp == 0) {
      const int j = it + STAGES - 1;
      if (j < nblk) {
        const int sj = j % STAGES, use = j / STAGES;
        const int next_page = j + 1 < nblk ? lane_page(table, page_size, box_rows, k_begin + (j + 1) * KB, kv_end, lane) : 0;
        if (use > 0) ok = mbar_wait(empty + sj, (use - 1) & 1, err);          // every warp has left block j - STAGES
        if (ok)
          fetch_block(tiles + sj * TILE_BYTES, &kmap, &vmap, page, page_size, nkv, kvh, box_rows, k_begin + j * KB,
                      kv_end, full + sj, lane);
        page = next_page;
      }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) break;
    if (!mbar_wait(full + s, (it / STAGES) & 1, err)) { ok = false; break; }
    unsigned char* t = tiles + s * TILE_BYTES;
    const int first_key = k_begin + it * KB;
    if (first_key + KB > kv_end && first_key + lane >= kv_end) {
      // Value rows beyond what this tile may see hold whatever the page or the stage held before (they are
      // masked for every query of the tile): keep them out of P.V.
      const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int c = 0; c < NB * 8; ++c) *reinterpret_cast<uint4*>(t + NB * HALF_BYTES + (c >> 3) * HALF_BYTES + lane * 128 + (c & 7) * 16) = zero;
    }
    __syncwarp();
    if (w_tok_hi >= w_tok_lo && first_key <= w_p_hi && first_key + KB > w_first_key) {
      // All keys of the block lie at or before the warp's first query (and inside its last query's window)?
      const bool all_visible = first_key + KB - 1 <= p_lo + w_tok_lo && first_key + KB <= kv_end &&
                               (window <= 0 || first_key > w_p_hi - window);
      if (all_visible)
        block_mma<false>(my_q, t, t + NB * HALF_BYTES, first_key, kv_end, window, qpos[0], qpos[1], scale_log2, st);
      else
        block_mma<true>(my_q, t, t + NB * HALF_BYTES, first_key, kv_end, window, qpos[0], qpos[1], scale_log2, st);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);
  }
  if (!ok) {
    // A wait ran out: let the copies in flight land (bounded) before the CTA gives up its shared memory.
    for (int s = 0; s < STAGES; ++s) { mbar_wait(full + s, 0, err); }
    return;
  }
  st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 1); st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], 2);
  st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 1); st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], 2);
  const int t2 = (lane & 3) * 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (tok_of[h] < 0) continue;
    const int head = head0 + (g + 8 * h) % group;
    bf16* dst = out + (static_cast<size_t>(q_begin + tok0 + tok_of[h]) * nh + head) * D;
    const float inv = st.l[h] > 0.0f ? 1.0f / st.l[h] : 0.0f;
#pragma unroll
    for (int dn = 0; dn < D / 8; ++dn)
      *reinterpret_cast<uint32_t*>(dst + dn * 8 + t2) = pack_bf16(st.o[dn][2 * h] * inv, st.o[dn][2 * h + 1] * inv);
  }
}

// ------------------------------------------------------------------ launchers
constexpr size_t kSmemLimit = 226 * 1024;
constexpr size_t kQBytes = QROWS * LD * sizeof(bf16);
constexpr size_t kBarBytes = 256;
constexpr size_t kFixedBytes = 1024 + kQBytes + kBarBytes;            // alignment slack, query tile, barriers
// Six warps with two stages where that fits shared memory (head sizes up to 128), else four, else two.
constexpr int kWarps = kFixedBytes + 6 * 2 * TILE_BYTES <= kSmemLimit ? 6 : (kFixedBytes + 4 * 2 * TILE_BYTES <= kSmemLimit ? 4 : 2);
constexpr int kStages = kFixedBytes + kWarps * 3 * TILE_BYTES <= kSmemLimit ? 3 : 2;
static_assert(kFixedBytes + kWarps * kStages * TILE_BYTES <= kSmemLimit, "the key blocks must fit shared memory");
static_assert(kWarps * kStages * sizeof(uint64_t) <= kBarBytes, "barriers");
static_assert(static_cast<size_t>(kWarps + 1) * QROWS * (D + 2) * sizeof(float) <= static_cast<size_t>(kWarps) * kStages * TILE_BYTES,
              "the merge area lies over the tiles");

B200_EXPORT int b200_attention_mma_head_dim() { return D; }
B200_EXPORT int b200_attention_mma_max_group() { return QROWS; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes into `out_map` (128 bytes) the TMA descriptor of one cache tensor [pages + 1, kv_heads, page_size, D]
// seen as a matrix of `rows` = (pages + 1) * kv_heads * page_size rows of D bfloat16, fetched in boxes of
// `box_rows` rows x 64 columns with the 128-byte swizzle.  Columns beyond D read as zeros.
B200_EXPORT int b200_kv_tensor_map(void* out_map, const void* cache, long long rows, int box_rows) {
  if (rows <= 0 || box_rows <= 0 || box_rows > 256) return B200_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(cache) % 16 != 0) return B200_BAD_ALIGN;
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
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(D) * sizeof(bf16)};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
  memcpy(out_map, &map, sizeof(map));
  return 0;
}

// Decoded tokens over a bfloat16 cache.  `k_map`, `v_map`: descriptors from b200_kv_tensor_map with
// box_rows = min(page_size, 32); page_size must be a power of two; at most 16 query heads per KV head.
// `scratch` as for b200_decode_attention of attention.cu.
B200_EXPORT int b200_decode_attention_mma(const void* q, const void* k_map, const void* v_map, void* out,
                                          float* scratch, const int* block_table, int table_stride,
                                          const int* cu_q, const int* kv_len, const int* rows, int n_rows, int nh,
                                          int nkv, int page_size, int window, float scale, int splits,
                                          int* err, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > QROWS || page_size <= 0 || splits <= 0) return B200_BAD_SIZE;
  if ((page_size & (page_size - 1)) != 0) return B200_BAD_SIZE;
  const int box_rows = page_size < KB ? page_size : KB;
  constexpr size_t smem = kFixedBytes + static_cast<size_t>(kWarps) * kStages * TILE_BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<kWarps, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  CUtensorMap kmap, vmap;
  memcpy(&kmap, k_map, sizeof(kmap));
  memcpy(&vmap, v_map, sizeof(vmap));
  float* part_acc = scratch;
  float* part_ml = scratch + static_cast<size_t>(n_rows) * nh * splits * D;
  dim3 grid(splits, nkv, n_rows);
  // Two, four or eight splits are the CTAs of one cluster and combine their parts through distributed shared memory;
  // other counts leave them in `scratch` for a kernel of its own.
  // (Only while the grid is one wave: clusters must be placed whole, and with several waves of one CTA per SM that
  // costs more than the second kernel, 10.1 k against 10.7 k tokens a second at batch 64.)
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0, n = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    sm_count = n;
  }
  const bool cluster_merge = (splits == 2 || splits == 4 || splits == 8) &&
                             static_cast<long long>(splits) * nkv * n_rows <= sm_count;
  int rc = b200_launch(decode_mma_kernel<kWarps, kStages>, grid, dim3(kWarps * 32), smem, stream, cluster_merge ? splits : 0,
                       kmap, vmap, static_cast<const bf16*>(q), static_cast<bf16*>(out), part_acc, part_ml, block_table,
                       table_stride, cu_q, kv_len, rows, nh, nkv, page_size, box_rows, window, scale * 1.4426950408889634f,
                       cluster_merge ? 1 : 0, err);
  if (rc != 0 || splits == 1 || cluster_merge) return rc;
  dim3 mgrid(n_rows, nh);
  return b200_launch(decode_mma_merge_kernel, mgrid, dim3(D >= 128 ? 128 : 64), 0, stream, 0, static_cast<bf16*>(out),
                     static_cast<const float*>(part_acc), static_cast<const float*>(part_ml), cu_q, rows, nh, splits);
}

constexpr size_t kPfQBytes = PF_ROWS * LD * sizeof(bf16);
constexpr size_t kPfFixed = 1024 + kPfQBytes + kBarBytes;
constexpr int kPfStages = D <= 128 ? 3 : kPfFixed + 4 * TILE_BYTES <= kSmemLimit ? 4 : (kPfFixed + 3 * TILE_BYTES <= kSmemLimit ? 3 : 2);
static_assert(kPfFixed + kPfStages * TILE_BYTES <= kSmemLimit, "the key blocks must fit shared memory");

// Portions of prompts over a bfloat16 cache; arguments as b200_prefill_attention of attention.cu, with the
// descriptors of b200_kv_tensor_map in place of the cache pointers.
B200_EXPORT int b200_prefill_attention_mma(const void* q, const void* k_map, const void* v_map, void* out,
                                           const int* block_table, int table_stride, const int* cu_q,
                                           const int* kv_len, const int* prefix_len, const int* rows, int n_rows,
                                           int max_q_len, int nh, int nkv, int page_size, int window, float scale,
                                           int* err, cudaStream_t stream) {
  if (n_rows <= 0 || max_q_len <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > QROWS || page_size <= 0) return B200_BAD_SIZE;
  if ((page_size & (page_size - 1)) != 0) return B200_BAD_SIZE;
  const int box_rows = page_size < KB ? page_size : KB;
  const int tile_tokens = (16 / (nh / nkv)) * PF_WARPS;
  constexpr size_t smem = kPfFixed + static_cast<size_t>(kPfStages) * TILE_BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<kPfStages>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  CUtensorMap kmap, vmap;
  memcpy(&kmap, k_map, sizeof(kmap));
  memcpy(&vmap, v_map, sizeof(vmap));
  const int n_tiles = (max_q_len + tile_tokens - 1) / tile_tokens;
  if (n_rows > 65535 || n_tiles > 65535) return B200_BAD_SIZE;      // the grid's y and z extents
  dim3 grid(nkv, n_rows, n_tiles);
  prefill_mma_kernel<kPfStages><<<grid, PF_WARPS * 32, smem, stream>>>(
      kmap, vmap, static_cast<const bf16*>(q), static_cast<bf16*>(out), block_table, table_stride, cu_q, kv_len,
      prefix_len, rows, nh, nkv, page_size, box_rows, window, scale * 1.4426950408889634f, err);
  return b200_check_launch();
}
