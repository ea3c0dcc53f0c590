// Causal prefill attention over the paged bfloat16 cache on the fifth-generation tensor cores, head size 128.
//
// A CTA serves 128 query vectors: 128 / group consecutive tokens of one row x the `group` query heads of one KV
// head (row r of the tile = token r / group, head r mod group).  It walks the visible keys in blocks of 128:
//   S = Q K^T      tcgen05.mma, M 128, N 128 (keys), K 16 x 8; Q and K are K-major tiles in the 128-byte swizzle
//                  (Q is written there by the softmax warps, K arrives by TMA); S lands in one of TWO score
//                  buffers in tensor memory, so the scores of block i + 1 are computed under the softmax of block i;
//   softmax        four warps, one thread per query row: two passes over the row of S in tensor memory
//                  (tcgen05.ld): the row maximum, then exp2 and the row sum; the bfloat16 probabilities go back
//                  into tensor memory (tcgen05.st), two to a column, over the first half of the scores they
//                  came from;
//   O += P V       tcgen05.mma with the A operand in tensor memory, M 128, N 128 (head dims), K 16 x 8,
//                  accumulating in tensor memory over all blocks; V is used as it lies in the cache (keys x dims,
//                  the dims contiguous: an MN-major B operand).  The tensor pipe runs the MMAs of one thread in
//                  the order of issue, so the scores of block i + 2 overwrite the buffer only behind P V of block i.
//                  The probabilities are taken relative to a reference maximum that is raised only when a row's
//                  maximum has grown by more than 2^8 (then the row's thread rescales its O in tensor memory,
//                  tcgen05.ld / st, once P V of the block before is finished); a stale reference is exact, since
//                  the row sum uses the same one.
// Two warps (one in the two-tile kernel) fetch K blocks (ring of three) and V blocks (ring of two) by TMA, a page's
// box each in turn; one warp owns tensor memory and issues the MMAs.  Semantics as attention.cu (reference: src/models/attention/backend.rs:1455-1498): causal
// mask, optional window, scale as a parameter, softmax in float.  Value rows at or beyond what the tile may see are
// zeroed in shared memory before they are used.  Every wait is bounded by the clock; on a time-out the error word
// is flagged and every path still reaches the end, where tensor memory is given back.
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
static_assert(HEAD_DIM == 128, "the tcgen05 attention kernel is written for head size 128");

typedef __nv_bfloat16 bf16;
constexpr int D = 128;
constexpr int BQ = 128;                  // query vectors per CTA
constexpr int BKV = 128;                 // keys per block
constexpr int HALF = BKV * 128;          // bytes of a [128 rows x 64 columns] half tile
constexpr int TILE = 2 * HALF;           // bytes of a [128 x 128] bfloat16 tile
constexpr int K_STAGES = 3, V_STAGES = 2;
// Warps that issue the copies: warp 0 and the warps behind the softmax warps.  Measured (kernel alone, pages of 16 keys):
// the one-tile kernel with 1 / 2 / 4 / 8 copy warps: 48.1 / 43.3 / 43.7 / 45.3 us at 2,048 tokens x 16 heads and 594 /
// 740 / 709 / 673 TFLOP/s at 16,384 x 32; the two-tile kernel, which fetches half as much a query: 892 / 886 / 869 / 801.
constexpr int COPY_WARPS = 2;
constexpr int PAIR_COPY_WARPS = 1;
constexpr int THREADS = 192 + 32 * (COPY_WARPS - 1);   // one tile per CTA: warp 0 copies, warp 1 MMA, warps 2-5 softmax, warps 6.. copy
constexpr int PAIR_THREADS = 320 + 32 * (PAIR_COPY_WARPS - 1);   // two tiles per CTA: four more softmax warps (2-9), warps 10.. copy
constexpr int TMEM_COLS = 512;           // S buffers (and P in their first 64 columns): columns 0..127 and 128..255; O: 256..383
constexpr float RESCALE_STEP = 8.0f;     // the reference maximum follows only growth beyond 2^8

// Shared memory: V stages, K stages, Q (each tile 32 KB), then the barriers.
constexpr int V_OFF = 0, K_OFF = V_STAGES * TILE, Q_OFF = K_OFF + K_STAGES * TILE, BAR_OFF = Q_OFF + TILE;
constexpr int N_BARS = 2 * K_STAGES + 2 * V_STAGES + 2 + 4;
constexpr int TBL_ENTRIES = 2048;         // page numbers of a row that the copy warp keeps in shared memory (the rest it reads as before)
constexpr int TBL_OFF = BAR_OFF + (N_BARS + 1) * 8;      // (one more slot holds the tensor-memory address)
constexpr int SMEM_BYTES = TBL_OFF + TBL_ENTRIES * 4;

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// All lanes of a warp wait and agree on the outcome: the collective tensor-memory loads that follow need the
// warp whole, also when a wait has run out.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* err) {
  const bool mine = mbar_wait(bar, parity, err);
  return __all_sync(0xffffffffu, mine ? 1 : 0) != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major tile in the 128-byte swizzle: 8-row groups 1024 bytes apart, leading byte offset unused (1).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// MN-major tile in the 128-byte swizzle (rows = k, 64 MN elements = 128 bytes contiguous): 8-row groups 1024 bytes
// apart (stride byte offset), the next 64 MN elements HALF bytes further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (static_cast<uint32_t>(HALF >> 4) << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// float accumulator, bfloat16 operands, M 128, N 128; B is K-major for S = Q K^T and MN-major for P V.
constexpr uint32_t kDescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kDescPV = kDescQK | (1u << 16);

__device__ __forceinline__ void umma(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The A operand from tensor memory: 16-bit elements packed two to a column (k = 2c, 2c + 1 in column c of lane m).
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_c, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_c), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
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
// 64 consecutive columns of this thread's lane, in one load and one wait.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n"
               "tcgen05.wait::ld.sync.aligned;\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
               : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
               "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
               ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                 "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                 "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                 "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                 "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                 "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                 "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                 "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
// 32 columns of this thread's lane from 32 registers; the caller waits (tcgen05.wait::st) before it tells anyone.
__device__ __forceinline__ void tmem_st32_raw(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
               "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                 "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                 "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                 "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {      // 2^x, one special-function instruction (-inf gives 0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Byte offset of (row r, 16-byte chunk c of 16) inside a [128 x 128] bfloat16 tile of two swizzled halves.
__device__ __forceinline__ int swz(int r, int c) { return (c >> 3) * HALF + r * 128 + (((c & 7) ^ (r & 7)) << 4); }

// ---------------------------------------------------------------------------------------------------------------
// What the softmax threads of both kernels do.  A thread owns one query row: lane r of tensor memory.

// The row's Q vector into its K-major tile in the 128-byte swizzle (zeros for a row that is not used).
__device__ __forceinline__ void write_q_row(unsigned char* q_tile, const bf16* src, int r, bool used) {
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (used) v = *reinterpret_cast<const uint4*>(src + c * 8);
    *reinterpret_cast<uint4*>(q_tile + swz(r, c)) = v;
  }
  proxy_fence();
}

// Row r of an MN-major value tile (128 dims in two halves of 128 bytes), set to zero.
__device__ __forceinline__ void zero_value_row(unsigned char* v_tile, int r) {
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(v_tile + (c >> 3) * HALF + r * 128 + (c & 7) * 16) = zero;
}

struct RowState {
  float m_ref = -INFINITY;     // reference maximum (log2 units): follows the row's maximum in steps of RESCALE_STEP
  float l_run = 0.0f;          // sum of the probabilities relative to it
};

// One block of 128 keys for this thread's row.  The scores lie in the 128 columns from s_base on; the bfloat16
// probabilities go back over the first 64 of them, two to a column (the A operand of P V), and are in tensor memory
// when the function returns.  `block` counts the row's blocks from 0; P V of block - 1 commits to `pv_done`.  Every
// phase of that barrier is waited for here, in order: before the accumulator at o_base is rescaled (the row's
// maximum grew by more than the step), else at the end, when that product has long finished.  A wait by parity
// cannot tell "phase b - 1 is not finished" from "phase b - 2 is not finished": a waiter that skipped a phase
// would pass at once.  Returns false when a wait ran out.
__device__ __forceinline__ bool softmax_block(uint32_t s_base, uint32_t o_base, int first_key, int qpos, int kv_end,
                                              int window, bool masked, float scale_log2, int block, uint64_t* pv_done,
                                              RowState& st, int* err) {
  tc_fence_after();
  // pass 1: the row's maximum over the block's visible keys (of the raw scores; the scale is positive)
  float mx = -INFINITY;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    float v[64];
    tmem_ld64(s_base + c * 64, v);
    if (masked) {
#pragma unroll
      for (int e = 0; e < 64; ++e) {
        const int key = first_key + c * 64 + e;
        const bool vis = key <= qpos && key < kv_end && (window <= 0 || key > qpos - window);
        mx = fmaxf(mx, vis ? v[e] : -INFINITY);
      }
    } else {
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains instead of one
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        m4[0] = fmaxf(m4[0], v[e]); m4[1] = fmaxf(m4[1], v[e + 1]); m4[2] = fmaxf(m4[2], v[e + 2]); m4[3] = fmaxf(m4[3], v[e + 3]);
      }
      mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
    }
  }
  mx = qpos >= 0 ? mx * scale_log2 : -INFINITY;
  // The reference follows the maximum when it grew by more than the step (or there was none yet).
  const bool raise = mx > st.m_ref + RESCALE_STEP || (st.m_ref == -INFINITY && mx > -INFINITY);
  const float m_new = raise ? mx : st.m_ref;
  const float corr = raise ? (st.m_ref == -INFINITY ? 0.0f : exp2f(st.m_ref - m_new)) : 1.0f;
  const float base = m_new == -INFINITY ? 0.0f : m_new;
  bool pv_seen = block == 0;
  // The accumulator may be rescaled only between two products: P V of the block before has to be finished.
  if (block > 0 && __any_sync(0xffffffffu, raise ? 1 : 0)) {
    if (!mbar_wait_warp(pv_done, (block - 1) & 1, err)) return false;
    pv_seen = true;
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      float o[32];
      tmem_ld32(o_base + c * 32, o);
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] *= corr;
      tmem_st32(o_base + c * 32, o);
    }
  }
  st.l_run = st.l_run * corr;
  st.m_ref = m_new;
  // pass 2: probabilities relative to the reference and their sum; those of columns 64c .. 64c + 63 go back into
  // tensor memory over the scores that were just read (columns 32c .. 32c + 31)
  const float neg_base = qpos >= 0 ? -base : -INFINITY;      // a row that is not used gets zeros
  float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    float v[64];
    tmem_ld64(s_base + c * 64, v);
    if (masked) {
#pragma unroll
      for (int e = 0; e < 64; ++e) {
        const int key = first_key + c * 64 + e;
        const bool vis = key <= qpos && key < kv_end && (window <= 0 || key > qpos - window);
        v[e] = vis ? fast_exp2(fmaf(v[e], scale_log2, neg_base)) : 0.0f;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 64; ++e) v[e] = fast_exp2(fmaf(v[e], scale_log2, neg_base));
    }
    uint32_t pr[32];
#pragma unroll
    for (int e = 0; e < 64; e += 2) {
      sum4[(e >> 1) & 3] += v[e] + v[e + 1];
      __nv_bfloat162 two = __floats2bfloat162_rn(v[e], v[e + 1]);
      pr[e >> 1] = *reinterpret_cast<uint32_t*>(&two);
    }
    tmem_st32_raw(s_base + c * 32, pr);
  }
  st.l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
  tmem_wait_st();                                      // P is in tensor memory
  return pv_seen || mbar_wait_warp(pv_done, (block - 1) & 1, err);
}

// The finished row: the accumulator over the row's sum, as bfloat16.  (Every lane of the warp takes part in the
// loads, also those whose row is not used.)
__device__ __forceinline__ void store_output(uint32_t o_base, bf16* dst, float l_run, bool used) {
  tc_fence_after();
  const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float o[32];
    tmem_ld32(o_base + c * 32, o);
    if (used) {
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        __align__(16) bf16 y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = __float2bfloat16_rn(o[q4 * 8 + e] * inv);
        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = *reinterpret_cast<const uint4*>(y);
      }
    }
  }
  tc_fence_before();
}

__global__ void __launch_bounds__(THREADS, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                       const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ block_table,
                       int table_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                       const int* __restrict__ prefix_len, const int* __restrict__ rows, int nh, int nkv, int page_size,
                       int box_rows, int window, float scale_log2, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sm + BAR_OFF);      // [3]
  uint64_t* k_empty = k_full + K_STAGES;                             // [3]
  uint64_t* v_full = k_empty + K_STAGES;                             // [2]
  uint64_t* v_empty = v_full + V_STAGES;                             // [2]
  uint64_t* s_full = v_empty + V_STAGES;                             // [2]
  uint64_t* q_full = s_full + 2;
  uint64_t* p_full = q_full + 1;                                     // [2]: one per score buffer, so that a softmax that runs
  uint64_t* pv_done = p_full + 2;                                    //      a block ahead can never lap the MMA thread's wait
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < K_STAGES; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
    for (int s = 0; s < V_STAGES; ++s) { mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
    mbar_init(s_full, 1);
    mbar_init(s_full + 1, 1);
    mbar_init(q_full, 4);
    mbar_init(p_full, 4);
    mbar_init(p_full + 1, 4);
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();                                  // q, the step's index arrays and the newest keys and values come from earlier kernels

  // Grid: x = KV head, y = row, z = tile order.  CTAs start in the order x, y, z, and a row's last tiles see the
  // most keys: every row's heaviest tiles start first, over all heads, and the light ones fill the gaps behind them.
  const int row = rows[blockIdx.y];
  const int kvh = blockIdx.x;
  const int group = nh / nkv, head0 = kvh * group;
  const int tile_tokens = BQ / group;
  const int q_begin = cu_q[row], q_len = cu_q[row + 1] - q_begin;
  const int tile = (q_len + tile_tokens - 1) / tile_tokens - 1 - static_cast<int>(blockIdx.z);
  const bool active = tile >= 0;               // (an idle CTA still walks to the end, where tensor memory is freed)
  const int tok0 = active ? tile * tile_tokens : 0;
  const int ntok = active ? min(tile_tokens, q_len - tok0) : 0;
  const int prefix = prefix_len[row];
  const int kv_end = active ? min(kv_len[row], prefix + tok0 + ntok) : 0;
  const int p_lo = prefix + tok0;
  int k_begin = window > 0 ? max(0, p_lo - window + 1) : 0;
  k_begin -= k_begin % BKV;
  const int nblk = active ? (kv_end - k_begin + BKV - 1) / BKV : 0;
  const int* table = block_table + static_cast<size_t>(row) * table_stride;

  if (warp == 0 || warp >= 6) {
    // ---- copies: COPY_WARPS warps share a block's sub-blocks (box_rows keys each): warp c's lane l fetches the
    // sub-blocks c + COPY_WARPS l, ...  (One SM takes in more through boxes that several warps issue than through
    // as many from one warp: 34 to 37 against 23 GB/s in a probe that only copies pages of 16 keys; all copy warps
    // walk the same stages and wait for the same barriers, the first announces a stage's bytes.  A box that lands
    // before its stage's bytes are announced is no harm: the phase cannot end before the announcing arrival.)
    // Keys run one block further ahead than values (three stages against two): S of block i + 2 is wanted
    // while block i is still in the softmax.
    // The row's page numbers for this tile's keys come into shared memory first: a copy then does not begin with a
    // load from global memory whose answer it needs for its address.
    const int cw = warp == 0 ? 0 : warp - 5;
    bool ok = true;
    int* tbl = reinterpret_cast<int*>(sm + TBL_OFF);
    const int first_page = k_begin / page_size;
    const int n_pages = min(TBL_ENTRIES, (kv_end + page_size - 1) / page_size - first_page);
    for (int t = cw * 32 + lane; t < n_pages; t += 32 * COPY_WARPS) tbl[t] = table[first_page + t];
    asm volatile("bar.sync 1, %0;\n" ::"n"(32 * COPY_WARPS) : "memory");      // (the copy warps only)
    auto fetch = [&](const CUtensorMap* map, unsigned char* dst, uint64_t* bar, int first_key) {
      const int n_sub = (min(BKV, kv_end - first_key) + box_rows - 1) / box_rows;
      proxy_fence();
      if (cw == 0 && lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_sub) * 2u * box_rows * 128u);
      __syncwarp();
      for (int j = cw + COPY_WARPS * lane; j < n_sub; j += 32 * COPY_WARPS) {
        const int key0 = first_key + j * box_rows;
        const int pi = key0 / page_size - first_page;
        const int page = pi < TBL_ENTRIES ? tbl[pi] : table[first_page + pi];
        const int y = (page * nkv + kvh) * page_size + key0 % page_size;
        tma_load_2d(dst + j * box_rows * 128, map, 0, y, bar);
        tma_load_2d(dst + HALF + j * box_rows * 128, map, 64, y, bar);
      }
    };
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {        // every lane waits, then the warp agrees
      const bool mine = mbar_wait(bar, parity, err);
      return __all_sync(0xffffffffu, mine ? 1 : 0) != 0;
    };
    int ik = 0;                                                  // next key block to fetch
    for (int i = 0; i < nblk && ok; ++i) {
      for (; ik < nblk && ik <= i + K_STAGES - 1 && ok; ++ik) {
        const int s = ik % K_STAGES, use = ik / K_STAGES;
        if (use > 0) ok = wait_all(k_empty + s, (use - 1) & 1);
        if (ok) fetch(&kmap, sm + K_OFF + s * TILE, k_full + s, k_begin + ik * BKV);
      }
      if (!ok) break;
      const int s = i % V_STAGES, use = i / V_STAGES;
      if (use > 0) ok = wait_all(v_empty + s, (use - 1) & 1);
      if (ok) fetch(&vmap, sm + V_OFF + s * TILE, v_full + s, k_begin + i * BKV);
    }
  } else if (warp == 1) {
    // ---- MMA issue (one lane): S_0, S_1; then for every block: O += P V of block i, S of block i + 2
    if (lane == 0 && nblk > 0) {
      bool ok = mbar_wait(q_full, 0, err);
      const uint32_t q_addr = smem_u32(sm + Q_OFF);
      const uint32_t tmem_o = tmem_base + 256;
      auto issue_s = [&](int i) {
        const int s = i % K_STAGES;
        if (!mbar_wait(k_full + s, (i / K_STAGES) & 1, err)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sm + K_OFF + s * TILE);
        const uint32_t tmem_s = tmem_base + (i & 1) * 128;
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          const uint32_t off = (j >> 2) * HALF + (j & 3) * 32;
          umma(tmem_s, desc_k_major(q_addr + off), desc_k_major(k_addr + off), kDescQK, j > 0 ? 1u : 0u);
        }
        umma_commit(s_full + (i & 1));
        umma_commit(k_empty + s);
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok && nblk > 1) ok = issue_s(1);
      for (int i = 0; i < nblk && ok; ++i) {
        const int s = i % V_STAGES;
        ok = mbar_wait(p_full + (i & 1), (i >> 1) & 1, err);      // P of block i lies where S of block i lay
        if (ok) ok = mbar_wait(v_full + s, (i / V_STAGES) & 1, err);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sm + V_OFF + s * TILE);
#pragma unroll
        for (int j = 0; j < BKV / 16; ++j)
          umma_a_tmem(tmem_o, tmem_base + (i & 1) * 128 + j * 8, desc_mn_major(v_addr + j * 16 * 128), kDescPV,
                      (i > 0 || j > 0) ? 1u : 0u);
        umma_commit(pv_done);
        umma_commit(v_empty + s);
        if (i + 2 < nblk) ok = issue_s(i + 2);
      }
    }
  } else {
    // ---- softmax warps: thread r owns query row r of the tile (tensor-memory lane r)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int tok = r / group, head = head0 + r % group;
    const bool used = tok < ntok;
    const int qpos = used ? p_lo + tok : -1;
    if (nblk > 0) {
      write_q_row(sm + Q_OFF, q + (static_cast<size_t>(q_begin + tok0 + tok) * nh + head) * D, r, used);
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    RowState st;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    bool ok = true;
    for (int i = 0; i < nblk && ok; ++i) {
      const int first_key = k_begin + i * BKV;
      if (!mbar_wait_warp(s_full + (i & 1), (i >> 1) & 1, err)) { ok = false; break; }
      const bool masked = first_key + BKV - 1 > p_lo || first_key + BKV > kv_end || (window > 0 && first_key <= p_lo + ntok - 1 - window);
      ok = softmax_block(lane_base + (i & 1) * 128, lane_base + 256, first_key, qpos, kv_end, window, masked, scale_log2, i,
                         pv_done, st, err);
      // value rows beyond what the tile may see must not reach P V, whatever the page or the stage held
      if (ok && first_key + BKV > kv_end) {
        const int s = i % V_STAGES;
        ok = mbar_wait_warp(v_full + s, (i / V_STAGES) & 1, err);      // the copies have landed
        if (ok && first_key + r >= kv_end) zero_value_row(sm + V_OFF + s * TILE, r);
        proxy_fence();                                                 // the zeroed rows are visible to the tensor cores
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + (i & 1));
    }
    if (ok && nblk > 0) ok = mbar_wait_warp(pv_done, (nblk - 1) & 1, err);
    if (ok && nblk > 0)
      store_output(lane_base + 256, out + (static_cast<size_t>(q_begin + tok0 + tok) * nh + head) * D, st.l_run, used);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA.  What the kernel above reads per block of keys (K and V, 64 KB from L2) limits it on long
// prompts: the tensor pipe and the softmax wait for the copies.  Here a CTA serves 256 query vectors, two tiles
// A and B of consecutive tokens, and every K and V block is fetched once for both.  Tensor memory holds one score
// buffer and one output accumulator per tile (4 x 128 columns); the MMA thread alternates between the tiles
// (P V of tile A, the next S of tile A, P V of tile B, the next S of tile B), so one tile's products run under the
// other tile's softmax.  Warps 2-5 are tile A's softmax (one thread per query row), warps 6-9 tile B's.
// (Blocks of 64 keys, which leave room for two score buffers per tile, were tried and were slower: twice the
// hand-overs per key.)  A tile's softmax of block b + 1 needs S of block b + 1, which is issued behind P V of block b:
// no barrier of a tile can complete two phases while someone still waits for the first.
constexpr int PAIR_K_STAGES = 2, PAIR_V_STAGES = 2;      // (deeper rings were slower: more copies in flight, same traffic)
constexpr int PAIR_V_OFF = 0, PAIR_K_OFF = PAIR_V_STAGES * TILE, PAIR_Q_OFF = PAIR_K_OFF + PAIR_K_STAGES * TILE;
constexpr int PAIR_BAR_OFF = PAIR_Q_OFF + 2 * TILE;
constexpr int PAIR_N_BARS = 2 * PAIR_K_STAGES + 2 * PAIR_V_STAGES + 2 + 2 + 2 + 1;
constexpr int PAIR_TBL_OFF = PAIR_BAR_OFF + (PAIR_N_BARS + 1) * 8;
constexpr int PAIR_SMEM_BYTES = PAIR_TBL_OFF + TBL_ENTRIES * 4;

__global__ void __launch_bounds__(PAIR_THREADS, 1)
prefill_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                            const bf16* __restrict__ q, bf16* __restrict__ out, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                            const int* __restrict__ prefix_len, const int* __restrict__ rows, int nh, int nkv,
                            int page_size, int box_rows, int window, float scale_log2, int* err) {
  constexpr int KS = PAIR_K_STAGES, VS = PAIR_V_STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sm + PAIR_BAR_OFF);
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + VS;
  uint64_t* s_full = v_empty + VS;                                   // [2]: one per tile
  uint64_t* p_full = s_full + 2;                                     // [2]
  uint64_t* pv_done = p_full + 2;                                    // [2]
  uint64_t* q_full = pv_done + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < KS; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
    for (int s = 0; s < VS; ++s) { mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(s_full + t, 1); mbar_init(p_full + t, 4); mbar_init(pv_done + t, 1); }
    mbar_init(q_full, 8);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;        // columns: S of tile A 0..127, S of tile B 128..255, O of A 256..383, O of B 384..511
  pdl_launch_dependents();
  pdl_wait();

  // Grid as above, with pairs of tiles in z.
  const int row = rows[blockIdx.y];
  const int kvh = blockIdx.x;
  const int group = nh / nkv, head0 = kvh * group;
  const int tile_tokens = BQ / group, pair_tokens = 2 * tile_tokens;
  const int q_begin = cu_q[row], q_len = cu_q[row + 1] - q_begin;
  const int pair = (q_len + pair_tokens - 1) / pair_tokens - 1 - static_cast<int>(blockIdx.z);
  const bool active = pair >= 0;               // (an idle CTA still walks to the end, where tensor memory is freed)
  const int prefix = prefix_len[row];
  int tok0[2], ntok[2], p_lo[2], kv_end[2], nblk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    tok0[t] = active ? pair * pair_tokens + t * tile_tokens : 0;
    ntok[t] = active ? max(0, min(tile_tokens, q_len - tok0[t])) : 0;
    p_lo[t] = prefix + tok0[t];
    kv_end[t] = ntok[t] > 0 ? min(kv_len[row], p_lo[t] + ntok[t]) : 0;
  }
  // Both tiles walk the same blocks, from where tile A's window begins; tile B ends at or after tile A.
  int k_begin = window > 0 ? max(0, p_lo[0] - window + 1) : 0;
  k_begin -= k_begin % BKV;
#pragma unroll
  for (int t = 0; t < 2; ++t) nblk[t] = ntok[t] > 0 ? (kv_end[t] - k_begin + BKV - 1) / BKV : 0;
  const int nblk_all = max(nblk[0], nblk[1]);
  const int kv_end_all = max(kv_end[0], kv_end[1]);
  const int* table = block_table + static_cast<size_t>(row) * table_stride;

  if (warp == 0 || warp >= 10) {
    // ---- copies, as in the kernel above
    const int cw = warp == 0 ? 0 : warp - 9;
    bool ok = true;
    int* tbl = reinterpret_cast<int*>(sm + PAIR_TBL_OFF);
    const int first_page = k_begin / page_size;
    const int n_pages = min(TBL_ENTRIES, (kv_end_all + page_size - 1) / page_size - first_page);
    for (int t = cw * 32 + lane; t < n_pages; t += 32 * PAIR_COPY_WARPS) tbl[t] = table[first_page + t];
    asm volatile("bar.sync 1, %0;\n" ::"n"(32 * PAIR_COPY_WARPS) : "memory");      // (the copy warps only)
    auto fetch = [&](const CUtensorMap* map, unsigned char* dst, uint64_t* bar, int first_key) {
      const int n_sub = (min(BKV, kv_end_all - first_key) + box_rows - 1) / box_rows;
      proxy_fence();
      if (cw == 0 && lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(n_sub) * 2u * box_rows * 128u);
      __syncwarp();
      for (int j = cw + PAIR_COPY_WARPS * lane; j < n_sub; j += 32 * PAIR_COPY_WARPS) {
        const int key0 = first_key + j * box_rows;
        const int pi = key0 / page_size - first_page;
        const int page = pi < TBL_ENTRIES ? tbl[pi] : table[first_page + pi];
        const int y = (page * nkv + kvh) * page_size + key0 % page_size;
        tma_load_2d(dst + j * box_rows * 128, map, 0, y, bar);
        tma_load_2d(dst + HALF + j * box_rows * 128, map, 64, y, bar);
      }
    };
    int ik = 0;
    for (int i = 0; i < nblk_all && ok; ++i) {
      for (; ik < nblk_all && ik <= i + KS - 1 && ok; ++ik) {
        const int s = ik % KS, use = ik / KS;
        if (use > 0) ok = mbar_wait_warp(k_empty + s, (use - 1) & 1, err);
        if (ok) fetch(&kmap, sm + PAIR_K_OFF + s * TILE, k_full + s, k_begin + ik * BKV);
      }
      if (!ok) break;
      const int s = i % VS, use = i / VS;
      if (use > 0) ok = mbar_wait_warp(v_empty + s, (use - 1) & 1, err);
      if (ok) fetch(&vmap, sm + PAIR_V_OFF + s * TILE, v_full + s, k_begin + i * BKV);
    }
  } else if (warp == 1) {
    // ---- MMA issue (one lane)
    if (lane == 0 && nblk_all > 0) {
      bool ok = mbar_wait(q_full, 0, err);
      // The operand descriptors differ only in their start address (the low 14 bits, in units of 16 bytes, which never
      // carry here): built once, then a stage or a tile is an addition.
      uint64_t dq[D / 16], dk[D / 16], dv[BKV / 16];
#pragma unroll
      for (int j = 0; j < D / 16; ++j) {
        const uint32_t off = (j >> 2) * HALF + (j & 3) * 32;
        dq[j] = desc_k_major(smem_u32(sm + PAIR_Q_OFF) + off);
        dk[j] = desc_k_major(smem_u32(sm + PAIR_K_OFF) + off);
      }
#pragma unroll
      for (int j = 0; j < BKV / 16; ++j) dv[j] = desc_mn_major(smem_u32(sm + PAIR_V_OFF) + j * 16 * 128);
      // S of tile t over key block b; the block's last user gives the stage back
      auto issue_s = [&](int t, int b) {                         // (t is a constant at every call)
        const int s = b % KS;
        if (!mbar_wait(k_full + s, (b / KS) & 1, err)) return false;
        tc_fence_after();
        const uint64_t q_step = static_cast<uint64_t>(t * (TILE >> 4)), k_step = static_cast<uint64_t>(s * (TILE >> 4));
#pragma unroll
        for (int j = 0; j < D / 16; ++j) umma(tmem_base + t * 128, dq[j] + q_step, dk[j] + k_step, kDescQK, j > 0 ? 1u : 0u);
        umma_commit(s_full + t);
        if (t == 1 || b >= nblk[1]) umma_commit(k_empty + s);
        return true;
      };
      if (ok && nblk[0] > 0) ok = issue_s(0, 0);
      if (ok && nblk[1] > 0) ok = issue_s(1, 0);
      for (int b = 0; b < nblk_all && ok; ++b) {
        const int s = b % VS;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || b >= nblk[t]) continue;
          ok = mbar_wait(p_full + t, b & 1, err);            // P of block b lies where S of block b lay
          if (ok) ok = mbar_wait(v_full + s, (b / VS) & 1, err);
          if (!ok) continue;
          tc_fence_after();
          const uint64_t v_step = static_cast<uint64_t>(s * (TILE >> 4));
#pragma unroll
          for (int j = 0; j < BKV / 16; ++j)
            umma_a_tmem(tmem_base + 256 + t * 128, tmem_base + t * 128 + j * 8, dv[j] + v_step, kDescPV, (b > 0 || j > 0) ? 1u : 0u);
          umma_commit(pv_done + t);
          if (t == 1 || b >= nblk[1]) umma_commit(v_empty + s);
          if (b + 1 < nblk[t]) ok = issue_s(t, b + 1);
        }
      }
    }
  } else {
    // ---- softmax warps: thread (tile t, row r) owns one query row (tensor-memory lane r of the tile's columns)
    const int t = (warp - 2) >> 2, quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int tok = r / group, head = head0 + r % group;
    const int my_tok0 = t ? tok0[1] : tok0[0], my_ntok = t ? ntok[1] : ntok[0], my_p_lo = t ? p_lo[1] : p_lo[0];
    const int my_kv_end = t ? kv_end[1] : kv_end[0], my_blocks = t ? nblk[1] : nblk[0];
    const bool used = tok < my_ntok;
    const int qpos = used ? my_p_lo + tok : -1;
    if (nblk_all > 0) {
      // (zeros for an unused row, and for all rows of a tile without tokens)
      write_q_row(sm + PAIR_Q_OFF + t * TILE, q + (static_cast<size_t>(q_begin + my_tok0 + tok) * nh + head) * D, r, used);
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    RowState st;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_base = lane_base + t * 128, o_base = lane_base + 256 + t * 128;
    bool ok = true;
    for (int b = 0; b < my_blocks && ok; ++b) {
      const int first_key = k_begin + b * BKV;
      if (!mbar_wait_warp(s_full + t, b & 1, err)) { ok = false; break; }
      const bool masked = first_key + BKV - 1 > my_p_lo || first_key + BKV > my_kv_end ||
                          (window > 0 && first_key <= my_p_lo + my_ntok - 1 - window);
      ok = softmax_block(s_base, o_base, first_key, qpos, my_kv_end, window, masked, scale_log2, b, pv_done + t, st, err);
      // Value rows beyond what the CTA may see must not reach P V, whatever the page or the stage held.  Both tiles
      // write the same zeros, each before its own product.
      if (ok && first_key + BKV > kv_end_all) {
        const int s = b % VS;
        ok = mbar_wait_warp(v_full + s, (b / VS) & 1, err);
        if (ok && first_key + r >= kv_end_all) zero_value_row(sm + PAIR_V_OFF + s * TILE, r);
        proxy_fence();
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + t);
    }
    if (ok && my_blocks > 0) ok = mbar_wait_warp(pv_done + t, (my_blocks - 1) & 1, err);
    if (ok && my_blocks > 0)
      store_output(o_base, out + (static_cast<size_t>(q_begin + my_tok0 + tok) * nh + head) * D, st.l_run, used);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

B200_EXPORT int b200_attention_tcgen05_head_dim() { return D; }

// How many launches took the one-tile and the two-tile kernel so far (tests ask which path a model reached).
static long long g_launches[2] = {0, 0};
B200_EXPORT long long b200_attention_tcgen05_launches(int two_tiles) { return g_launches[two_tiles ? 1 : 0]; }

// Portions of prompts over a bfloat16 cache, head size 128; the number of query heads per KV head must divide 128
// and the page size must be a power of two.  `k_map`, `v_map`: descriptors of b200_kv_tensor_map (attention_mma.cu)
// with box_rows = min(page_size, 32).  Other arguments as b200_prefill_attention of attention.cu.
// `variant`: 1 = one tile of 128 query vectors per CTA, 2 = two tiles per CTA, 0 = two tiles when the longest
// row then still gives every SM a CTA (pairs halve the traffic per query but also the number of CTAs).
B200_EXPORT int b200_prefill_attention_tcgen05(const void* q, const void* k_map, const void* v_map, void* out,
                                               const int* block_table, int table_stride, const int* cu_q,
                                               const int* kv_len, const int* prefix_len, const int* rows, int n_rows,
                                               int max_q_len, int nh, int nkv, int page_size, int window, float scale,
                                               int variant, int* err, cudaStream_t stream) {
  if (n_rows <= 0 || max_q_len <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || (page_size & (page_size - 1)) != 0) return B200_BAD_SIZE;
  if (variant < 0 || variant > 2) return B200_BAD_SIZE;
  const int group = nh / nkv;
  if (group > BQ || BQ % group != 0) return B200_BAD_SIZE;
  const int box_rows = page_size < 32 ? page_size : 32;
  const int tile_tokens = BQ / group;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0, n = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    sm_count = n;
  }
  const int n_pairs = (max_q_len + 2 * tile_tokens - 1) / (2 * tile_tokens);
  const bool pairs = variant == 2 || (variant == 0 && static_cast<long long>(n_pairs) * nkv * n_rows >= sm_count);
  const size_t smem = 1024 + (pairs ? PAIR_SMEM_BYTES : SMEM_BYTES);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 + SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(prefill_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 1024 + PAIR_SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  CUtensorMap kmap, vmap;
  memcpy(&kmap, k_map, sizeof(kmap));
  memcpy(&vmap, v_map, sizeof(vmap));
  const int n_tiles = pairs ? n_pairs : (max_q_len + tile_tokens - 1) / tile_tokens;
  if (n_rows > 65535 || n_tiles > 65535) return B200_BAD_SIZE;      // the grid's y and z extents
  dim3 grid(nkv, n_rows, n_tiles);
  ++g_launches[pairs ? 1 : 0];
  return b200_launch(pairs ? prefill_tcgen05_pair_kernel : prefill_tcgen05_kernel, grid, dim3(pairs ? PAIR_THREADS : THREADS), smem, stream, 0, kmap,
                     vmap, static_cast<const bf16*>(q), static_cast<bf16*>(out), block_table, table_stride, cu_q, kv_len,
                     prefix_len, rows, nh, nkv, page_size, box_rows, window, scale * 1.4426950408889634f, err);
}
