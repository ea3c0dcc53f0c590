// A chain of few-row products in ONE persistent kernel: y_i = epilogue_i(prologue_i(x_i) . W_i^T), i = 0 .. n - 1,
// where x_{i+1} may be y_i (a decode layer's output projection, gate/up, down and the next layer's QKV, say).
//
// Why one kernel.  With a handful of rows every product is a stream of weights; launched one by one, each starts
// its stream cold and the step becomes a chain of launches.  Here the grid (one CTA per SM) stays resident:
//   * a feeding warp walks the whole chain ahead of the multiplying warps and keeps a ring of eight 16 KB TMA
//     stages full, so the weights of product i + 1 are in shared memory while product i is still being finished;
//   * products are separated by a grid-wide barrier instead of a kernel boundary: one add with release semantics
//     per CTA to a counter that never goes back, and polls of that counter by one thread per CTA;
//   * a product's work is cut so that every SM streams its share of the weights:
//       narrow tiles (small matrices, at most 32 rows of x): a tile is 16 weight rows over ALL of K and belongs
//         to one CTA, so nothing is exchanged between CTAs; a stage holds 16 rows x 512 columns, the warps split
//         the columns and add their sums in shared memory in warp order;
//       wide tiles (large matrices): a tile is 128 weight rows, a stage 128 rows x 64 columns; the stages of all
//         tiles are dealt out in tile-major order, CTA c takes [c per, (c + 1) per).  A tile whose stages fall to
//         several CTAs is finished by the CTA that holds its first stages (for which it is the last tile of its
//         range): the others write their partial sums to scratch memory and count themselves on the tile's ticket
//         without waiting; the finisher adds the parts in CTA order and runs the epilogue.  QKV always has wide
//         tiles (its epilogue needs whole heads).
//
//   prologue  0 none; 1 residual add + RMSNorm; 2 RMSNorm.  The operand in shared memory is round(s * w) with
//             s = x (+ residual) in float; the row's scale rsqrt(mean(s^2) + eps) multiplies the finished
//             product (reference: src/layers/fused_ops.cu:95-105 normalises the unrounded sum).  mean(s^2)
//             comes from `stats_in` when the product before this one left it there (see below), else every
//             CTA reads the rows once; the first CTA of the product then also writes residual_out = round(s).
//   epilogue  PLAIN (bfloat16 or float), SWIGLU (a tile is half gate rows, half the same up rows), QKV (per-head
//             RMSNorm, half-split rotation, q to q_out, k and v into the paged cache; head sizes that divide
//             128), as skinny_linear.cu.  A PLAIN bfloat16 product can also do the add of the norm that
//             FOLLOWS it: with `stats_res_in` it writes stats_res_out = round(y + residual) and the sum of
//             squares of (y + residual) of its tile's columns per row into stats_out[tile][row].
//
// Rows: up to 64 (template NT = row groups of 8: 1, 2, 4, 8).  The weight rows are the 16-row side of
// mma.sync m16n8k16, the rows of x the 8-column side.  x is staged in chunks of columns that fit 34 KB.
//
// Every wait is bounded by the clock (one second): a wait that runs out sets the error word and an abort flag
// that every other wait of the grid polls, so the whole grid leaves.  All CTAs must be resident at once: the
// launcher refuses a grid larger than the number of SMs (one CTA per SM by its shared memory).
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

constexpr int BK = 64;                         // columns per k-block: 128 bytes of a weight row
constexpr int BN = 128;                        // weight rows per tile
constexpr int STAGE_BYTES = BN * 128;          // one k-block of one tile
constexpr int STAGES = 8;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;
constexpr int ROW_WARPS = 4;                   // warps that share the weight rows of a tile (32 rows each)
constexpr int GROUPS = 4;                      // groups of ROW_WARPS warps; a k-block belongs to group (sequence number % 4)
constexpr int WARPS = ROW_WARPS * GROUPS;      // multiplying warps; one more warp feeds the ring
constexpr int CONSUMERS = WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;
constexpr int XS_BYTES = 34 * 1024;            // a chunk of the rows of x'
constexpr int MAX_OPS = 6;
constexpr int MAX_M = 64;
constexpr int MIN_SEGMENT = 4;                 // stages a CTA takes at least (64 KB of weights)
constexpr int NARROW_ROWS = 16;                // weight rows of a narrow tile, which one CTA owns over all of K
constexpr int NARROW_COLS = STAGE_BYTES / (NARROW_ROWS * 2);               // 512 columns per stage of a narrow tile
constexpr int TRACE_WORDS = 64;                // per CTA: eight readings for each product
constexpr int SYNC_WORDS = 8;
static_assert(STAGES % GROUPS == 0, "a stage of the ring always belongs to the same group of warps");

enum : int { EPI_PLAIN_BF16 = 0, EPI_PLAIN_F32 = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };
enum : int { PRO_NONE = 0, PRO_ADD_NORM = 1, PRO_NORM = 2 };

struct ChainOp {
  const bf16* x;            // [rows of x, K]
  const int* x_rows;        // optional gather: row m of the product is x[x_rows[m]]
  const bf16* residual;     // PRO_ADD_NORM
  bf16* residual_out;       // PRO_ADD_NORM without stats_in: round(x + residual), written by the product's first CTA
  const void* norm_w;       // [K] bfloat16 or float
  const float* stats_in;    // [stats_tiles][MAX_M] sums of squares left by the product before (null: rows are read)
  float* stats_out;         // PLAIN bfloat16: [tiles][MAX_M] sums of squares of (y + stats_res_in)
  const bf16* stats_res_in;
  bf16* stats_res_out;      // round(y + stats_res_in)
  void* out;                // PLAIN: [M, N]; SWIGLU: [M, N / 2]; QKV: q_out [M, nh * d]
  const void* q_w;          // QKV: [d] per-head norm weights (null: none)
  const void* k_w;
  const float* cos_table;   // [max_pos, rot_dim / 2] (null: no rotation)
  const float* sin_table;
  const int* positions;     // [M]
  const int* slots;         // [M] (null: nothing is stored)
  bf16* k_cache;            // [pages + 1, nkv, page_size, d]
  bf16* v_cache;
  long long cache_slots;
  int prologue, norm_w_f32;
  float eps;
  int stats_tiles;
  int M, N, K, mode;
  int nh, nkv, head_dim, rot_dim, max_pos, page_size, qk_w_f32;
  float qk_eps;
  int narrow;               // 1: tiles of 16 weight rows, each owned by one CTA (see b200_chain_narrow)
  int box_rows;             // rows of the weight's TMA box (see b200_chain_box_rows)
  // schedule, filled by the launcher
  int tiles, kblocks, per, ctas, first_cta, ticket_off;
};

struct ChainParams {
  ChainOp op[MAX_OPS];
  int n_ops;
  int stages;               // stages of the ring in use: 4 or 8
  float* scratch;           // [grid][mpad][BN] partial sums
  int* tickets;             // one per tile of every product, zero between launches
  unsigned* sync;           // [0] arrivals at barriers, ever; [1] barriers of earlier launches; [2] abort
  int* err;
  unsigned long long* trace;  // null, or [grid][TRACE_WORDS] clock readings of every CTA's first thread (for tuning)
};

struct alignas(64) ChainMaps { CUtensorMap m[MAX_OPS]; };

// ---------------------------------------------------------------- primitives
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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(CONSUMERS) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float norm_weight(const void* w, int f32, int i) {
  return f32 ? static_cast<const float*>(w)[i] : __bfloat162float(static_cast<const bf16*>(w)[i]);
}
__device__ __forceinline__ void unpack8(const uint4& v, float* out) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// ---------------------------------------------------------------- the kernel
template <int NT>
__global__ void __launch_bounds__(THREADS, 1)
linear_chain_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams p) {
  constexpr int MPAD = 8 * NT;
  constexpr int CHUNK_COLS = (XS_BYTES / (MPAD * 2) - 8) / BK * BK;        // columns of x' staged at a time
  constexpr int LDX = CHUNK_COLS + 8;                                      // padded row: conflict-free ldmatrix
  constexpr int LDR = BN + 1;
  constexpr int LD16 = NARROW_ROWS + 1;
  constexpr bool CAN_NARROW = NT <= 4;                                     // (the warps' partial tiles must fit shared memory)
  static_assert(CHUNK_COLS >= 4 * BK, "a chunk of x' holds at least four k-blocks");
  static_assert(!CAN_NARROW || CHUNK_COLS >= NARROW_COLS, "a chunk of x' holds a stage of a narrow tile");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  bf16* xs = reinterpret_cast<bf16*>(ring + RING_BYTES);                    // [MPAD][LDX]
  float* red = reinterpret_cast<float*>(ring + RING_BYTES + XS_BYTES);      // [MPAD][LDR]
  float* red16 = red + MPAD * LDR;                                          // [WARPS][MPAD][LD16] (narrow tiles)
  uint64_t* full = reinterpret_cast<uint64_t*>(red16 + (CAN_NARROW ? WARPS * MPAD * LD16 : 0) + 1);
  full = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(full) + 7) & ~uintptr_t(7));
  uint64_t* empty = full + STAGES;
  float* row_scale = reinterpret_cast<float*>(empty + STAGES);              // [MAX_M]
  int* flags = reinterpret_cast<int*>(row_scale + MAX_M);                   // [0] ticket result, [1] give up

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool feeder = warp == WARPS;
  const int G = static_cast<int>(gridDim.x);
  const uint32_t nst = static_cast<uint32_t>(p.stages);
  if (threadIdx.x < STAGES) { mbar_init(full + threadIdx.x, 1); mbar_init(empty + threadIdx.x, ROW_WARPS); }
  if (threadIdx.x == 0) { flags[0] = 0; flags[1] = 0; }
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  __syncthreads();

  // This CTA's range of stages of product i: [lo, hi) in tile-major order.
  auto my_range = [&](const ChainOp& op, int& lo, int& hi) {
    int c = static_cast<int>(blockIdx.x) - op.first_cta;
    if (c < 0) c += G;
    const int total = op.tiles * op.kblocks;
    lo = c < op.ctas ? min(total, c * op.per) : 0;
    hi = c < op.ctas ? min(total, lo + op.per) : 0;
    return c;
  };

  if (feeder) {
    // ---- the feeding warp: the weights of the whole chain, in order, as fast as the ring takes them
    if (lane == 0) {
      uint32_t j = 0;                                 // sequence number of the stage in this CTA's stream
      bool ok = true;
      for (int i = 0; i < p.n_ops && ok; ++i) {
        const ChainOp& op = p.op[i];
        int lo, hi;
        my_range(op, lo, hi);
        for (int b = lo; b < hi; ++b, ++j) {
          const int s = j % nst;
          if (j >= nst) {
            ok = mbar_wait(empty + s, ((j / nst) - 1) & 1, p.err);        // the warps that had this stage have left it
            if (!ok || ld_acquire(p.sync + 2) != 0u) { ok = false; break; }
          }
          const int tile = b / op.kblocks, kb = b - tile * op.kblocks;
          unsigned char* dst = ring + s * STAGE_BYTES;
          if (op.narrow) {
            // 16 weight rows x 512 columns: eight boxes of 64 columns (SwiGLU: 8 gate rows above 8 up rows)
            const int k0 = kb * NARROW_COLS;
            const int boxes = min(NARROW_COLS / BK, (op.K - k0 + BK - 1) / BK);
            mbar_expect_tx(full + s, static_cast<uint32_t>(boxes) * NARROW_ROWS * 128u);
            for (int sb = 0; sb < boxes; ++sb) {
              if (op.mode == EPI_SWIGLU) {
                tma_load_2d(dst + sb * 2048, &maps.m[i], k0 + sb * BK, tile * (NARROW_ROWS / 2), full + s);
                tma_load_2d(dst + sb * 2048 + 1024, &maps.m[i], k0 + sb * BK, op.N / 2 + tile * (NARROW_ROWS / 2), full + s);
              } else {
                tma_load_2d(dst + sb * 2048, &maps.m[i], k0 + sb * BK, tile * NARROW_ROWS, full + s);
              }
            }
          } else {
            mbar_expect_tx(full + s, STAGE_BYTES);
            if (op.mode == EPI_SWIGLU) {
              tma_load_2d(dst, &maps.m[i], kb * BK, tile * (BN / 2), full + s);
              tma_load_2d(dst + STAGE_BYTES / 2, &maps.m[i], kb * BK, op.N / 2 + tile * (BN / 2), full + s);
            } else {
              tma_load_2d(dst, &maps.m[i], kb * BK, tile * BN, full + s);
            }
          }
        }
      }
      if (!ok) atomicExch(p.sync + 2, 1u);
      // Copies that nobody will read (the grid gave up) must still land before the CTA leaves its shared memory.
      const uint32_t issued = j;
      for (uint32_t back = 0; back < nst && back < issued; ++back) {
        const uint32_t jj = issued - 1 - back;
        mbar_wait(full + jj % nst, (jj / nst) & 1, p.err);
      }
    }
    return;
  }

  // ---- the multiplying warps
  pdl_wait();                       // x, residuals and the cache belong to the kernels before this one
  const int tid = threadIdx.x;      // 0 .. CONSUMERS - 1
  const unsigned epoch0 = ld_acquire(p.sync + 1);    // barriers of earlier launches: sync[0] counts every arrival ever
  const int mi = lane >> 3, r8 = lane & 7;
  const int grp = warp / ROW_WARPS, rw = warp % ROW_WARPS;
  const int g = lane >> 2, t2 = (lane & 3) * 2;
  uint32_t j = 0;
  auto stamp = [&](int i, int what) {
    if (p.trace != nullptr && tid == 0) p.trace[static_cast<size_t>(blockIdx.x) * TRACE_WORDS + i * 8 + what] = global_ns();
  };
  bool alive = true;                // changes only where every multiplying thread sees the same flag
  bool failed = false;              // this warp's own wait ran out (told to the others through flags[1])

  for (int i = 0; i < p.n_ops && alive; ++i) {
    const ChainOp& op = p.op[i];
    int lo, hi;
    const int c = my_range(op, lo, hi);
    const int M = op.M, K = op.K;
    const bool narrow = CAN_NARROW && op.narrow != 0;
    stamp(i, 0);
    if (i > 0) {
      // ---- the grid's barrier.  From here on everything that the products before wrote is visible.
      const unsigned target = (epoch0 + static_cast<unsigned>(i)) * static_cast<unsigned>(G);
      consumer_sync();
      if (tid == 0) {
        // One arrival: an add with release semantics (what this CTA's threads stored before the barrier above is
        // visible to whoever sees the count), then polls of the count with acquire semantics.
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(p.sync) : "memory");
        stamp(i, 7);
        uint64_t start = 0;
        for (uint32_t polls = 1;; ++polls) {
          if (static_cast<int>(ld_acquire(p.sync) - target) >= 0) break;
          if ((polls & 15u) == 0u) {
            bool stop = ld_acquire(p.sync + 2) != 0u;
            const uint64_t now = global_ns();
            if (start == 0) start = now;
            if (now - start > 1000000000ull) {
              atomicOr(p.err, B200_ERR_WAIT_TIMEOUT);
              atomicExch(p.sync + 2, 1u);
              stop = true;
            }
            if (stop) { flags[1] = 1; break; }
          }
        }
      }
      consumer_sync();
      if (flags[1] != 0) { alive = false; break; }
    }
    stamp(i, 1);
    if (lo >= hi) continue;

    // ---- the rows' scales.  Sums of squares that the product before left are only fetched here (up to four values a
    // lane: one row a warp, 128 tiles); they are added up after the first columns of x' have been staged, so that both
    // fetches are on their way at the same time.
    constexpr int STATS_PER_LANE = 4;
    float stats_raw[STATS_PER_LANE] = {0.0f, 0.0f, 0.0f, 0.0f};
    const bool stats_late = op.prologue != PRO_NONE && op.stats_in != nullptr && M <= WARPS && op.stats_tiles <= 32 * STATS_PER_LANE;
    if (op.prologue != PRO_NONE) {
      if (stats_late) {
        if (warp < M) {
          const int src_row = op.x_rows ? op.x_rows[warp] : warp;
#pragma unroll
          for (int u = 0; u < STATS_PER_LANE; ++u)
            if (lane + 32 * u < op.stats_tiles) stats_raw[u] = __ldcg(op.stats_in + (lane + 32 * u) * MAX_M + src_row);
        }
      } else if (op.stats_in != nullptr) {
        for (int m = warp; m < M; m += WARPS) {
          const int src_row = op.x_rows ? op.x_rows[m] : m;
          float ss = 0.0f;
          for (int t = lane; t < op.stats_tiles; t += 32) ss += __ldcg(op.stats_in + t * MAX_M + src_row);
          ss = warp_sum(ss);
          if (lane == 0) row_scale[m] = rsqrtf(ss / static_cast<float>(K) + op.eps);
        }
      } else {
        const bool writer = c == 0 && op.residual_out != nullptr && op.prologue == PRO_ADD_NORM;
        for (int m = warp; m < M; m += WARPS) {
          const size_t src = static_cast<size_t>(op.x_rows ? op.x_rows[m] : m) * K;
          float ss = 0.0f;
          for (int k = lane * 8; k < K; k += 32 * 8) {
            float s[8];
            unpack8(__ldcg(reinterpret_cast<const uint4*>(op.x + src + k)), s);
            if (op.prologue == PRO_ADD_NORM) {
              float r[8];
              unpack8(__ldcg(reinterpret_cast<const uint4*>(op.residual + src + k)), r);
#pragma unroll
              for (int e = 0; e < 8; ++e) s[e] += r[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += s[e] * s[e];
            if (writer) {
              __align__(16) bf16 rounded[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) rounded[e] = __float2bfloat16_rn(s[e]);
              *reinterpret_cast<uint4*>(op.residual_out + src + k) = *reinterpret_cast<uint4*>(rounded);
            }
          }
          ss = warp_sum(ss);
          if (lane == 0) row_scale[m] = rsqrtf(ss / static_cast<float>(K) + op.eps);
        }
      }
    }

    stamp(i, 2);
    const int chunk_cols = narrow ? CHUNK_COLS / NARROW_COLS * NARROW_COLS : CHUNK_COLS;
    const int stage_cols = narrow ? NARROW_COLS : BK;
    int staged_lo = 0, staged_hi = 0;                 // columns of x' that shared memory holds (none yet)
    // The rows of x' for columns [k0, k0 + chunk_cols), as bfloat16 in shared memory: all fetches of four vectors a
    // thread are issued before the first is used.
    auto stage_x = [&](int k0) {
      const int cols = min(chunk_cols, (K - k0 + BK - 1) / BK * BK);
      const int vecs = cols / 8, total = MPAD * vecs;
      consumer_sync();                                      // the columns before have been read by every warp
      for (int base = 0; base < total; base += 4 * CONSUMERS) {
        uint4 xa[4], xb[4];
        int at[4], kk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = base + u * CONSUMERS + tid;
          const int m = v / vecs, k = k0 + (v - m * vecs) * 8;
          at[u] = v < total ? m * LDX + (k - k0) : -1;
          kk[u] = (v < total && m < M && k < K) ? k : -1;
          xa[u] = xb[u] = make_uint4(0u, 0u, 0u, 0u);
          if (kk[u] >= 0) {
            const size_t src = static_cast<size_t>(op.x_rows ? op.x_rows[m] : m) * K + k;
            xa[u] = __ldcg(reinterpret_cast<const uint4*>(op.x + src));
            if (op.prologue == PRO_ADD_NORM) xb[u] = __ldcg(reinterpret_cast<const uint4*>(op.residual + src));
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (at[u] < 0) continue;
          uint4 val = xa[u];
          if (op.prologue != PRO_NONE && kk[u] >= 0) {
            float sv[8], wv[8];
            unpack8(xa[u], sv);
            if (op.prologue == PRO_ADD_NORM) {
              float r[8];
              unpack8(xb[u], r);
#pragma unroll
              for (int e = 0; e < 8; ++e) sv[e] += r[e];
            }
            if (op.norm_w_f32) {
              const float4 w0 = *reinterpret_cast<const float4*>(static_cast<const float*>(op.norm_w) + kk[u]);
              const float4 w1 = *reinterpret_cast<const float4*>(static_cast<const float*>(op.norm_w) + kk[u] + 4);
              wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
            } else {
              unpack8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(op.norm_w) + kk[u]), wv);
            }
            __align__(16) bf16 weighted[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) weighted[e] = __float2bfloat16_rn(sv[e] * wv[e]);
            val = *reinterpret_cast<uint4*>(weighted);
          }
          *reinterpret_cast<uint4*>(xs + at[u]) = val;
        }
      }
      staged_lo = k0;
      staged_hi = k0 + cols;
      consumer_sync();
      stamp(i, 3);
    };
    stage_x((lo % op.kblocks) * stage_cols);
    if (stats_late && warp < M) {
      float ss = stats_raw[0] + stats_raw[1] + stats_raw[2] + stats_raw[3];
      ss = warp_sum(ss);
      if (lane == 0) row_scale[warp] = rsqrtf(ss / static_cast<float>(K) + op.eps);
    }

    // ---- the CTA's segments: one per tile that its range touches
    for (int seg_lo = lo; seg_lo < hi;) {
      const int tile = seg_lo / op.kblocks;
      const int seg_hi = min(hi, (tile + 1) * op.kblocks);
      float acc[2][NT][4];
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int n = 0; n < NT; ++n) { acc[a][n][0] = acc[a][n][1] = acc[a][n][2] = acc[a][n][3] = 0.0f; }

      for (int b = seg_lo; b < seg_hi; ++b, ++j) {
        const int k0 = (b - tile * op.kblocks) * stage_cols;
        if (k0 < staged_lo || min(K, k0 + stage_cols) > staged_hi) stage_x(k0);
        // Stage j % STAGES always belongs to group j % GROUPS, whatever the kind of tile: only that group waits
        // for it (and for every one of its phases, in order), only that group frees it.
        if (static_cast<int>(j % GROUPS) != grp) continue;
        const int s = j % nst;
        if (!failed) failed = !__all_sync(0xffffffffu, mbar_wait(full + s, (j / nst) & 1, p.err));
        if (failed) continue;                               // (no more waits: the grid is about to give up)
        const unsigned char* wt = ring + s * STAGE_BYTES;
        const bf16* xk = xs + (k0 - staged_lo);
        if (narrow) {
          // sixteen weight rows: the stage's eight blocks of 64 columns go to the four warps of the group, two each
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int sb = rw * 2 + half;
            if (k0 + sb * BK >= K) continue;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
              uint32_t a[4];
              const int r = lane & 15, cc = ks * 2 + (lane >> 4);
              ldmatrix_x4(a, wt + sb * 2048 + r * 128 + ((cc ^ (r & 7)) << 4));
              const bf16* xb = xk + sb * BK + ks * 16 + (mi & 1) * 8;
              if (NT == 1) {
                uint32_t bb[4];
                ldmatrix_x4(bb, xb + r8 * LDX);
                mma_bf16(acc[0][0], a, bb[0], bb[1]);
              } else {
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                  uint32_t bb[4];
                  ldmatrix_x4(bb, xb + (np * 16 + (mi >> 1) * 8 + r8) * LDX);
                  mma_bf16(acc[0][np * 2], a, bb[0], bb[1]);
                  mma_bf16(acc[0][np * 2 + 1], a, bb[2], bb[3]);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t a[2][4];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int r = rw * 32 + q * 16 + (lane & 15);                 // weight row inside the tile
              const int cc = ks * 2 + (lane >> 4);                          // 16-byte chunk of the 128-byte row
              ldmatrix_x4(a[q], wt + r * 128 + ((cc ^ (r & 7)) << 4));
            }
            if (NT == 1) {
              uint32_t bb[4];
              ldmatrix_x4(bb, xk + r8 * LDX + ks * 16 + (mi & 1) * 8);      // (both halves point at rows 0..7)
              mma_bf16(acc[0][0], a[0], bb[0], bb[1]);
              mma_bf16(acc[1][0], a[1], bb[0], bb[1]);
            } else {
#pragma unroll
              for (int np = 0; np < NT / 2; ++np) {
                uint32_t bb[4];
                ldmatrix_x4(bb, xk + (np * 16 + (mi >> 1) * 8 + r8) * LDX + ks * 16 + (mi & 1) * 8);
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  mma_bf16(acc[q][np * 2], a[q], bb[0], bb[1]);
                  mma_bf16(acc[q][np * 2 + 1], a[q], bb[2], bb[3]);
                }
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
      }
      if (failed) flags[1] = 1;                             // seen by everybody behind the barriers below
      stamp(i, 4);

      const int tile_rows = narrow ? NARROW_ROWS : BN;      // weight rows (outputs) of this tile
      bool finish = true;
      if (narrow) {
        // ---- every warp's sums for its columns of K meet in shared memory, added in warp order
        if (CAN_NARROW) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            float* r0 = red16 + (warp * MPAD + nt * 8 + t2) * LD16 + g;
            r0[0] = acc[0][nt][0]; r0[LD16] = acc[0][nt][1]; r0[8] = acc[0][nt][2]; r0[LD16 + 8] = acc[0][nt][3];
          }
          consumer_sync();
          for (int e = tid; e < MPAD * NARROW_ROWS; e += CONSUMERS) {
            const int m = e / NARROW_ROWS, n = e - m * NARROW_ROWS;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) sum += red16[(w * MPAD + m) * LD16 + n];
            red[m * LDR + n] = sum;
          }
          consumer_sync();
        }
        if (flags[1] != 0) { alive = false; break; }
      } else {
        // ---- the groups' sums are added in shared memory, group after group
        consumer_sync();                                    // (the epilogue of the tile before has read `red`)
        for (int turn = 0; turn < GROUPS; ++turn) {
          if (grp == turn) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int n = rw * 32 + q * 16 + g;
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const int m = nt * 8 + t2;
                float* r0 = red + m * LDR + n;
                float* r1 = red + (m + 1) * LDR + n;
                if (turn == 0) { r0[0] = acc[q][nt][0]; r1[0] = acc[q][nt][1]; r0[8] = acc[q][nt][2]; r1[8] = acc[q][nt][3]; }
                else { r0[0] += acc[q][nt][0]; r1[0] += acc[q][nt][1]; r0[8] += acc[q][nt][2]; r1[8] += acc[q][nt][3]; }
              }
            }
          }
          consumer_sync();
        }
        if (flags[1] != 0) { alive = false; break; }

        // ---- a tile that several CTAs share.  The CTA that holds the tile's FIRST stages finishes it: for that CTA
        // the tile is the last of its range, so the others (for whom it is the first) have long left their partial
        // sums in scratch memory and counted themselves on the tile's ticket with a release; they never wait.
        const int t_lo = tile * op.kblocks, t_hi = t_lo + op.kblocks;
        const int c_first = t_lo / op.per, c_last = (t_hi - 1) / op.per;
        if (c_last > c_first) {
          unsigned* ticket = reinterpret_cast<unsigned*>(p.tickets) + op.ticket_off + tile;
          if (c != c_first) {
            float* mine = p.scratch + static_cast<size_t>(blockIdx.x) * (MPAD * BN);
            for (int e = tid; e < MPAD * BN; e += CONSUMERS) mine[e] = red[(e / BN) * LDR + (e % BN)];
            consumer_sync();
            if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(ticket) : "memory");
            finish = false;
          } else {
            if (tid == 0) {
              const unsigned others = static_cast<unsigned>(c_last - c_first);
              uint64_t start = 0;
              for (uint32_t polls = 1;; ++polls) {
                if (ld_acquire(ticket) >= others) break;
                if ((polls & 15u) == 0u) {
                  bool stop = ld_acquire(p.sync + 2) != 0u;
                  const uint64_t now = global_ns();
                  if (start == 0) start = now;
                  if (now - start > 1000000000ull) {
                    atomicOr(p.err, B200_ERR_WAIT_TIMEOUT);
                    atomicExch(p.sync + 2, 1u);
                    stop = true;
                  }
                  if (stop) { flags[1] = 1; break; }
                }
              }
              *reinterpret_cast<volatile unsigned*>(ticket) = 0u;           // ready for the next launch
            }
            consumer_sync();
            if (flags[1] != 0) { alive = false; break; }
            for (int e = tid; e < MPAD * BN; e += CONSUMERS) {
              float sum = red[(e / BN) * LDR + (e % BN)];                  // CTA order: this CTA's part first
              for (int cc = c_first + 1; cc <= c_last; ++cc) {
                int phys = cc + op.first_cta;
                if (phys >= G) phys -= G;
                sum += __ldcg(p.scratch + static_cast<size_t>(phys) * (MPAD * BN) + e);
              }
              red[(e / BN) * LDR + (e % BN)] = sum;
            }
            consumer_sync();
          }
        }
      }
      stamp(i, 5);
      if (finish) {
        // ---- epilogue on red[m][n] (float), n < tile_rows
        if (op.prologue != PRO_NONE) {
          for (int e = tid; e < M * tile_rows; e += CONSUMERS) red[(e / tile_rows) * LDR + (e % tile_rows)] *= row_scale[e / tile_rows];
          consumer_sync();
        }
        if (op.mode == EPI_PLAIN_BF16 || op.mode == EPI_PLAIN_F32) {
          const int col0 = tile * tile_rows;
          for (int m = warp; m < M; m += WARPS) {
            float ss = 0.0f;
            for (int n = lane; n < tile_rows; n += 32) {
              const int col = col0 + n;
              if (col >= op.N) continue;
              const float v = red[m * LDR + n];
              const size_t at = static_cast<size_t>(m) * op.N + col;
              if (op.mode == EPI_PLAIN_F32) {
                static_cast<float*>(op.out)[at] = v;
              } else {
                const bf16 y = __float2bfloat16_rn(v);
                static_cast<bf16*>(op.out)[at] = y;
                if (op.stats_out != nullptr) {
                  const float s = __bfloat162float(y) + __uint_as_float(static_cast<uint32_t>(__ldcg(reinterpret_cast<const unsigned short*>(op.stats_res_in) + at)) << 16);
                  op.stats_res_out[at] = __float2bfloat16_rn(s);
                  ss += s * s;
                }
              }
            }
            if (op.stats_out != nullptr) {
              ss = warp_sum(ss);
              if (lane == 0) op.stats_out[tile * MAX_M + m] = ss;
            }
          }
        } else if (op.mode == EPI_SWIGLU) {
          const int inter = op.N / 2, half_rows = tile_rows / 2;
          for (int e = tid; e < M * half_rows; e += CONSUMERS) {
            const int m = e / half_rows, n = e - m * half_rows, col = tile * half_rows + n;
            if (col >= inter) continue;
            // gate and up leave the product as bfloat16 values in the unfused path; the same rounding here
            const float gate = __bfloat162float(__float2bfloat16_rn(red[m * LDR + n]));
            const float up = __bfloat162float(__float2bfloat16_rn(red[m * LDR + half_rows + n]));
            static_cast<bf16*>(op.out)[static_cast<size_t>(m) * inter + col] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
          }
        } else {                                                           // EPI_QKV: BN / d heads per tile
          const int d = op.head_dim, per_tile = BN / d, heads = op.nh + 2 * op.nkv;
          const int half = op.rot_dim / 2;
          for (int item = warp; item < M * per_tile; item += WARPS) {
            const int m = item / per_tile, hh = item - m * per_tile, head = tile * per_tile + hh;
            if (head >= heads) continue;
            const bool is_q = head < op.nh, is_k = !is_q && head < op.nh + op.nkv;
            float* row = red + m * LDR + hh * d;
            // the projection's output is a bfloat16 tensor in the unfused path; the same rounding here
            for (int e = lane; e < d; e += 32) row[e] = __bfloat162float(__float2bfloat16_rn(row[e]));
            __syncwarp();
            bf16* dst = nullptr;
            if (is_q) {
              dst = static_cast<bf16*>(op.out) + (static_cast<size_t>(m) * op.nh + head) * d;
            } else if (op.slots != nullptr) {
              const int slot = op.slots[m];
              if (slot < 0 || slot >= op.cache_slots) {
                if (lane == 0) atomicOr(p.err, B200_ERR_SLOT_RANGE);
              } else if (slot != 0) {                                      // (slot 0 is the sink: padding rows write nothing)
                const int kvh = is_k ? head - op.nh : head - op.nh - op.nkv;
                const int page = slot / op.page_size, offset = slot - page * op.page_size;
                dst = (is_k ? op.k_cache : op.v_cache) + ((static_cast<size_t>(page) * op.nkv + kvh) * op.page_size + offset) * d;
              }
            }
            if (dst == nullptr) continue;
            if (!is_q && !is_k) {
              for (int e = lane; e < d; e += 32) dst[e] = __float2bfloat16_rn(row[e]);
              continue;
            }
            const void* w = is_q ? op.q_w : op.k_w;
            if (w != nullptr) {
              float ss = 0.0f;
              for (int e = lane; e < d; e += 32) ss += row[e] * row[e];
              ss = warp_sum(ss);
              const float scale = rsqrtf(ss / static_cast<float>(d) + op.qk_eps);
              for (int e = lane; e < d; e += 32) row[e] = row[e] * scale * norm_weight(w, op.qk_w_f32, e);
              __syncwarp();
            }
            bool rotate = op.cos_table != nullptr && half > 0;
            int pos = 0;
            if (rotate) {
              pos = op.positions[m];
              if (pos < 0 || pos >= op.max_pos) {
                if (lane == 0) atomicOr(p.err, B200_ERR_POSITION_RANGE);
                rotate = false;
              }
            }
            if (rotate) {
              const float* ct = op.cos_table + static_cast<size_t>(pos) * half;
              const float* st = op.sin_table + static_cast<size_t>(pos) * half;
              for (int e = lane; e < half; e += 32) {
                const float a = row[e], b = row[e + half], cs = ct[e], sn = st[e];
                dst[e] = __float2bfloat16_rn(a * cs - b * sn);
                dst[e + half] = __float2bfloat16_rn(b * cs + a * sn);
              }
              for (int e = op.rot_dim + lane; e < d; e += 32) dst[e] = __float2bfloat16_rn(row[e]);
            } else {
              for (int e = lane; e < d; e += 32) dst[e] = __float2bfloat16_rn(row[e]);
            }
          }
        }
      }
      stamp(i, 6);
      seg_lo = seg_hi;
    }
  }
  if (tid == 0) {
    if (!alive) atomicExch(p.sync + 2, 1u);
    // The barriers of this launch are behind every CTA once CTA 0 has passed the last one: the next launch counts on.
    else if (blockIdx.x == 0 && p.n_ops > 1) *reinterpret_cast<volatile unsigned*>(p.sync + 1) = epoch0 + static_cast<unsigned>(p.n_ops - 1);
  }
  // Stages that the feeding warp filled and nobody took (the grid gave up) are the feeding warp's to wait for.
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Writes into `out_map` (128 bytes) the TMA descriptor of a bfloat16 weight matrix [n, k], fetched in boxes of
// `box_rows` rows (b200_chain_box_rows) x 64 columns with the 128-byte swizzle.  Rows beyond n and columns
// beyond k read as zeros.
B200_EXPORT int b200_chain_weight_map(void* out_map, const void* weight, long long n, long long k, int box_rows) {
  if (n <= 0 || k <= 0 || (box_rows != 8 && box_rows != 16 && box_rows != 64 && box_rows != 128) || k % 8 != 0) return B200_BAD_SIZE;
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

B200_EXPORT int b200_chain_op_size() { return static_cast<int>(sizeof(ChainOp)); }
B200_EXPORT int b200_chain_max_ops() { return MAX_OPS; }
B200_EXPORT int b200_chain_max_rows() { return MAX_M; }

// Whether a product runs on narrow tiles: not QKV, at most 32 rows of x in the launch, a weight of at most
// `max_bytes` (for large weights the wide tiles' even split of the stages counts for more than the exchange it costs).
B200_EXPORT int b200_chain_narrow(int mode, int n, int k, int launch_rows, long long max_bytes) {
  if (mode == EPI_QKV || launch_rows > 32) return 0;
  return 2ll * n * k <= max_bytes ? 1 : 0;
}

// Rows of the weight's TMA box.
B200_EXPORT int b200_chain_box_rows(int mode, int narrow) {
  if (narrow) return mode == EPI_SWIGLU ? NARROW_ROWS / 2 : NARROW_ROWS;
  return mode == EPI_SWIGLU ? BN / 2 : BN;
}

// Tiles of one product (for callers that size the ticket and statistics arrays).
B200_EXPORT int b200_chain_tiles(int mode, int n, int narrow) {
  const int cols = mode == EPI_SWIGLU ? n / 2 : n;
  const int rows = narrow ? NARROW_ROWS : BN;
  const int tile_cols = mode == EPI_SWIGLU ? rows / 2 : rows;
  return (cols + tile_cols - 1) / tile_cols;
}

// Floats of scratch memory that a launch on `grid` CTAs needs for products of up to `rows` rows.
B200_EXPORT long long b200_chain_scratch_floats(int rows, int grid) {
  const int mpad = rows <= 8 ? 8 : rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  return static_cast<long long>(grid) * mpad * BN;
}

// Words of the `sync` array.
B200_EXPORT int b200_chain_sync_words() { return SYNC_WORDS; }

template <int NT>
static int launch_chain(const ChainMaps& maps, const ChainParams& p, int grid, cudaStream_t stream) {
  constexpr int MPAD = 8 * NT;
  constexpr size_t red16 = NT <= 4 ? static_cast<size_t>(WARPS) * MPAD * (NARROW_ROWS + 1) * sizeof(float) : 0;
  const size_t smem = 1024 + RING_BYTES + XS_BYTES + (MPAD * (BN + 1) + 2) * sizeof(float) + red16 + 2 * STAGES * sizeof(uint64_t) +
                      MAX_M * sizeof(float) + 64;
  static_assert(1024 + RING_BYTES + XS_BYTES + (MPAD * (BN + 1) + 2) * sizeof(float) + red16 + 2 * STAGES * sizeof(uint64_t) +
                MAX_M * sizeof(float) + 64 <= 227 * 1024, "shared memory of one CTA");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_chain_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  return b200_launch(linear_chain_kernel<NT>, dim3(grid), dim3(THREADS), smem, stream, 0, maps, p);
}

// `ops`: n_ops ChainOp structs filled by the caller (`narrow` and `box_rows` as b200_chain_narrow and
// b200_chain_box_rows say for the largest row count of the launch; the schedule fields are set here); `w_maps`: n_ops
// descriptors from b200_chain_weight_map (128 bytes each); `scratch`: b200_chain_scratch_floats floats; `tickets`: one
// int per tile of every product, zero (the kernel leaves them zero); `sync`: b200_chain_sync_words zeroed words that
// belong to this device's chain launches for good; `trace`: null, or [sm_count][64] words for clock readings.  Refuses (B200_BAD_SIZE) more than 64 rows, more than MAX_OPS
// products, a K that is no multiple of 8, a head size that does not divide 128 in QKV mode, more CTAs than flags.
B200_EXPORT int b200_linear_chain(const void* ops, const void* w_maps, int n_ops, float* scratch, int* tickets,
                                  unsigned* sync, int* err, unsigned long long* trace, int stages, int sm_count, cudaStream_t stream) {
  if (n_ops <= 0) return 0;
  if (n_ops > MAX_OPS || sm_count <= 0 || (stages != 4 && stages != 8)) return B200_BAD_SIZE;
  ChainParams p;
  memset(&p, 0, sizeof(p));
  ChainMaps maps;
  memcpy(&maps.m[0], w_maps, sizeof(CUtensorMap) * n_ops);
  for (int i = n_ops; i < MAX_OPS; ++i) maps.m[i] = maps.m[0];
  memcpy(&p.op[0], ops, sizeof(ChainOp) * n_ops);
  p.n_ops = n_ops;
  p.scratch = scratch;
  p.tickets = tickets;
  p.sync = sync;
  p.err = err;
  p.trace = trace;
  p.stages = stages;
  const int grid = sm_count;
  int rows = 0, ticket_off = 0, first = 0;
  for (int i = 0; i < n_ops; ++i) rows = p.op[i].M > rows ? p.op[i].M : rows;
  for (int i = 0; i < n_ops; ++i) {
    ChainOp& op = p.op[i];
    if (op.M <= 0 || op.M > MAX_M || op.N <= 0 || op.K <= 0 || op.K % 8 != 0) return B200_BAD_SIZE;
    if (op.mode < EPI_PLAIN_BF16 || op.mode > EPI_QKV || op.prologue < PRO_NONE || op.prologue > PRO_NORM) return B200_BAD_SIZE;
    if (op.mode == EPI_SWIGLU && op.N % 2 != 0) return B200_BAD_SIZE;
    if (op.mode == EPI_QKV) {
      const int d = op.head_dim;
      if (d <= 0 || BN % d != 0 || op.N != (op.nh + 2 * op.nkv) * d || op.rot_dim < 0 || op.rot_dim > d || (op.rot_dim & 1))
        return B200_BAD_SIZE;
    }
    if (op.stats_out != nullptr && (op.mode != EPI_PLAIN_BF16 || op.stats_res_in == nullptr || op.stats_res_out == nullptr))
      return B200_BAD_SIZE;
    if (op.prologue != PRO_NONE && op.norm_w == nullptr) return B200_BAD_SIZE;
    if (op.prologue == PRO_ADD_NORM && op.residual == nullptr) return B200_BAD_SIZE;
    op.narrow = op.narrow != 0 ? 1 : 0;
    if (op.narrow && (op.mode == EPI_QKV || rows > 32)) return B200_BAD_SIZE;
    if (op.box_rows != b200_chain_box_rows(op.mode, op.narrow)) return B200_BAD_SIZE;
    op.tiles = b200_chain_tiles(op.mode, op.N, op.narrow);
    op.kblocks = op.narrow ? (op.K + NARROW_COLS - 1) / NARROW_COLS : (op.K + BK - 1) / BK;
    const long long total = static_cast<long long>(op.tiles) * op.kblocks;
    if (total > (1ll << 30)) return B200_BAD_SIZE;
    if (op.narrow) {
      // whole tiles: nothing is exchanged between CTAs
      const int ctas = op.tiles < grid ? op.tiles : grid;
      const int tiles_per = (op.tiles + ctas - 1) / ctas;
      op.per = tiles_per * op.kblocks;
      op.ctas = (op.tiles + tiles_per - 1) / tiles_per;
    } else {
      long long ctas = total / MIN_SEGMENT;
      ctas = ctas < 1 ? 1 : (ctas > grid ? grid : ctas);
      op.per = static_cast<int>((total + ctas - 1) / ctas);
      op.ctas = static_cast<int>((total + op.per - 1) / op.per);
    }
    // Products that do not fill the grid start where the one before ended: the idle CTAs of a product are the
    // ones that fetch ahead for the next.
    op.first_cta = op.ctas >= grid ? 0 : first % grid;
    first = op.ctas >= grid ? 0 : (op.first_cta + op.ctas) % grid;
    op.ticket_off = ticket_off;
    ticket_off += op.tiles;
  }
  if (rows <= 8) return launch_chain<1>(maps, p, grid, stream);
  if (rows <= 16) return launch_chain<2>(maps, p, grid, stream);
  if (rows <= 32) return launch_chain<4>(maps, p, grid, stream);
  return launch_chain<8>(maps, p, grid, stream);
}
