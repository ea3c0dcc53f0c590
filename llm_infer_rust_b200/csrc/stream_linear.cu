// y = epilogue(prologue(x) . W^T) for a handful of rows (decode steps) and a LARGE weight matrix, streamed by every
// thread for itself: no feeding thread, no barrier between the copy and the multiply, no cluster.
//
//   weights   Every weight is read once and nothing shares it.  A thread of a warp (g = lane / 4, t = lane % 4)
//             fetches 16 bytes = 8 consecutive k of weight row g and of row g + 8 with asynchronous copies
//             (cp.async, past the first-level cache) into pieces of shared memory that are ITS OWN, waits for its own
//             copies only (no barrier, not even within the warp) and reads them back into the registers of the
//             multiply.  Two turns of 64 bytes a thread are on their way while a third is multiplied: 96 KB an SM with
//             768 threads.  The four threads of a row cover a CHUNK of 32 consecutive k.  mma.sync m16n8k16 has the
//             WEIGHT rows on its 16-row side; it wants, for thread t, the k positions 2t, 2t+1, 2t+8, 2t+9 of a 16-k
//             step, and a sum over k does not care about the order of k, so the chunk's k are assigned to the
//             positions as they arrive: thread t's elements 0..3 are the step's positions of thread t in a first
//             instruction, elements 4..7 in a second, and the rows of x are read the same way.
//             (Two earlier versions loaded the weights with plain 16-byte loads straight into registers.  Alone they
//             ran as fast as this one.  Inside a decode step they ran twice as long: bytes that a load has asked for
//             wait for their place in the first-level cache, whatever the load's cache hints; beside kernels that take
//             200 KB of shared memory an SM keeps that carve-out, the cache shrinks to about 28 KB, and so did the
//             bytes on their way.  Asking for a smaller carve-out brought the speed back and cost a reconfiguration of
//             every SM at both ends of the kernel, which ate the gain.  Copies into shared memory need no cache.)
//   x         the rows of x' (at most 16) wait in shared memory, as in skinny_linear.cu: ONE CTA an SM stages them
//             once and then walks over many tiles of weight rows.  Where the grid fills the GPU the CTAs are launched
//             as clusters of two that stage half of the rows each and store them into both CTAs' shared memory:
//             else 148 CTAs read the same rows of x and of the residual out of the second-level cache at the same
//             moment (3.9 us of a 38 us launch at the Qwen3-8B gate/up; a decode step of 36 layers 3.92 -> 3.84 ms).
//   split     the CTA's warps are G groups of KS warps.  A group owns a tile of RW x 16 weight rows at a time
//             (SwiGLU: 8 or 16 gate rows and the same up rows); its KS warps split K (warp s takes the chunks
//             [s C / KS, (s+1) C / KS)), leave their sums in shared memory, and the group's epilogue adds them in
//             warp order, so the result does not depend on timing.  Tiles are dealt out round-robin over all groups
//             of all CTAs; the copies run two turns ahead across tiles, so a tile's epilogue has the next tile's
//             first weights on their way.
//   prologue  none, or (residual add +) RMSNorm as in skinny_linear.cu: s = x + residual in float, the operand is
//             round(s * w), the row's scale rsqrt(mean(s^2) + eps) multiplies the finished product.  Every CTA
//             stages whole rows, so it has the rows' sums of squares itself; the CTA with index 0 stores round(s)
//             as residual_out (reference: src/layers/fused_ops.cu:95-105).
//   epilogue  PLAIN (bfloat16 or float; bfloat16 optionally begins the norm that FOLLOWS: round(y + post_residual)
//             and, per tile, the rows' sums of its squares, which skinny_linear.cu takes as stats_in) or SWIGLU
//             (silu(gate) * up; reference: src/layers/fused_ops.cu:142-144).
// Measured on B200, 8 rows, cold weights, one product after the other in a graph: Qwen3-8B gate/up (201 MB) 38.7 us =
// 5.2 TB/s (the ring kernel of skinny_linear.cu 51.6 us, the library's product alone 37.3 us), the Qwen3-8B head
// (1.24 GB) 198 to 202 us = 6.2 TB/s (ring 262, library 209), Qwen3-32B gate/up (524 MB) 92 to 98 us (ring 130, library
// 95), the Qwen3-0.6B head (311 MB) 57.7 us (ring 67.6, library 59.4).  What does not fit: rows of x beyond what shared
// memory holds beside 96 KB of copies (8 rows of about 6,000 columns), so the down projections of these models stay with
// the ring kernel or the library.
// The first weights are on their way before the dependency wait (they do not depend on the kernel before this one).
#include <cuda.h>
#include <math.h>
#include <string.h>

#include "common.cuh"

typedef __nv_bfloat16 bf16;

enum : int { EPI_PLAIN_BF16 = 0, EPI_PLAIN_F32 = 1, EPI_SWIGLU = 2 };
constexpr int MMAX = 16;               // rows of x
constexpr int CHUNK = 32;              // k per chunk: 64 bytes of a weight row, 16 bytes a thread

struct StreamParams {
  // prologue
  const bf16* x;            // [rows of x, K]
  const int* x_rows;        // optional gather: row m of the product is x[x_rows[m]]
  const bf16* residual;     // null: no add
  bf16* residual_out;       // null: the sum is not stored
  const void* norm_w;       // [K] bfloat16 or float; null: no norm (then no residual either)
  int norm_w_f32;
  float eps;
  // product
  const bf16* w;            // [N, K]
  int M, N, K;
  int mode;
  void* out;                // PLAIN: [M, N]; SWIGLU: [M, N / 2]
  // the norm after a PLAIN bfloat16 product, begun here (see skinny_linear.cu)
  const bf16* post_residual;
  bf16* post_sum_out;
  float* post_stats;        // [tiles][MMAX]
  // shape of the launch, 0: chosen by the launcher: groups of 16 weight rows a tile, warps that split K
  int rw, ks;
  int groups, tiles;        // (filled by the launcher: groups of KS warps a CTA, tiles of the product)
  int xd;                   // the rows of x come with the weights' copies instead of waiting in shared memory: 1 yes, 0 no, -1 where they do not fit
  int pair;                 // CTAs are launched as clusters of two that stage half of the rows of x each (1 yes, 0 no, -1 the launcher's choice)
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 two = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&two);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Shared memory: xs [MP][row_bytes] bfloat16 (the rows of x'; row_bytes = 2 K rounded so that neighbouring rows start
// 64 bytes apart modulo 128: the eight rows that a quarter of a warp reads at once hit different banks), then
// red[G][KS][RW * 16][LDR] floats (a warp's sums: weight row x row of x), part[warps][MMAX] (a warp's share of the rows'
// sums of squares), scale[MMAX].
template <int NB> struct Layout { static constexpr int LDR = NB * 8 + 2; };
__host__ __device__ inline int xs_row_bytes(int k) { return (2 * k) % 128 == 0 ? 2 * k + 64 : 2 * k; }

// Shared memory of the other CTA of a cluster of two.
__device__ __forceinline__ uint32_t peer_address(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void store_peer16(uint32_t addr, const uint4& v) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void store_peer_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void group_barrier(int group, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(group + 1), "r"(threads) : "memory");
}

constexpr int MAX_THREADS = 768;
constexpr int TURN_BYTES = 64;         // weights that a thread fetches a turn: four asynchronous copies of 16 bytes
constexpr int TURNS = 2;               // turns on their way (beside the one in registers): 128 bytes a thread, 96 KB an SM

// XD: the rows of x are too long for shared memory (and have no norm before them): every thread fetches its own
// 16 bytes of them a chunk with the weights' copies, from the second-level cache, where the few rows of x stay.
template <int RW, int NB, bool NORM, bool XD>
__global__ void __launch_bounds__(MAX_THREADS, 1) stream_linear_kernel(const StreamParams p) {
  static_assert(!(NORM && XD), "the norm needs whole rows of x in shared memory");
  constexpr int U = TURN_BYTES / 32 / RW;      // chunks a turn
  constexpr int SLOTS = TURN_BYTES / 16;       // 16-byte pieces of weights that a thread fetches a turn
  constexpr int TSLOTS = SLOTS + (XD ? U * NB : 0);   // ... and of the rows of x
  constexpr int LDR = Layout<NB>::LDR;
  constexpr int MP = NB * 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int KS = p.ks, G = p.groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int grp = warp / KS, slice = warp - grp * KS;
  const int K = p.K, M = p.M;
  const int row_bytes = xs_row_bytes(K);
  unsigned char* xs = smem_raw;
  const int xs_bytes = XD ? 0 : MP * row_bytes;
  float* red = reinterpret_cast<float*>(xs + xs_bytes) + grp * KS * RW * 16 * LDR;
  float* part = reinterpret_cast<float*>(xs + xs_bytes) + G * KS * RW * 16 * LDR;
  float* scale = part + G * KS * MMAX;
  // this thread's pieces: piece s of turn r at ((r * SLOTS + s) * threads + thread) * 16 (a warp's 32 pieces side by side)
  unsigned char* ring = reinterpret_cast<unsigned char*>(scale + MMAX) + threadIdx.x * 16;
  const unsigned piece_stride = blockDim.x * 16;
  pdl_launch_dependents();          // the kernel after this one may set itself up from now on (it waits before it reads)
  // (a pair: both CTAs say that they run; waited for before the first store into the other one's shared memory)
  if (p.pair) asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");

  const int chunks = K / CHUNK;
  const int c_lo = static_cast<int>(static_cast<long long>(slice) * chunks / KS);
  const int c_hi = static_cast<int>(static_cast<long long>(slice + 1) * chunks / KS);
  const bool swiglu = p.mode == EPI_SWIGLU;
  const int inter = p.N / 2;
  const int stride = gridDim.x * G;            // tiles are dealt out over all groups of all CTAs
  int tile = grp * gridDim.x + blockIdx.x;

  // the two weight rows of this thread in every group of rows of a tile (rows beyond the matrix: its last row, never
  // stored), as offsets in elements (the launcher refuses matrices of 2^32 elements and more)
  unsigned wrow[RW][2];
  auto rows_of = [&](int tl) {
#pragma unroll
    for (int j = 0; j < RW; ++j) {
      int r0, limit;
      if (swiglu && RW == 1) {                 // 8 gate rows as the instruction's rows 0..7, the same up rows as its rows 8..15
        wrow[j][0] = static_cast<unsigned>(min(tl * 8 + g, inter - 1)) * static_cast<unsigned>(K) + 8u * t;
        wrow[j][1] = static_cast<unsigned>(min(inter + tl * 8 + g, p.N - 1)) * static_cast<unsigned>(K) + 8u * t;
        continue;
      }
      if (swiglu) {                            // (RW = 2: 16 gate rows, then the same up rows)
        r0 = (j == 0 ? 0 : inter) + tl * 16;
        limit = j == 0 ? inter : p.N;
      } else {
        r0 = (tl * RW + j) * 16;
        limit = p.N;
      }
      wrow[j][0] = static_cast<unsigned>(min(r0 + g, limit - 1)) * static_cast<unsigned>(K) + 8u * t;
      wrow[j][1] = static_cast<unsigned>(min(r0 + g + 8, limit - 1)) * static_cast<unsigned>(K) + 8u * t;
    }
  };
  // The turn that is fetched next: U chunks of tile `itile` from chunk `ic` on, into turn `r` of the ring.  A turn is
  // one group of asynchronous copies whether it has any or not, so that "all but the newest TURNS - 1 groups have
  // landed" always means "the turn to be multiplied now has landed".
  int itile = tile, ic = c_lo;
  if (itile < p.tiles) rows_of(itile);
  auto issue_w = [&](int r) {
    if (itile < p.tiles) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const bool in = ic + u < c_hi;           // (beyond the warp's range: zeros, nothing is read)
#pragma unroll
        for (int j = 0; j < RW; ++j)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            cp_async16(ring + (r * TSLOTS + (u * RW + j) * 2 + h) * piece_stride,
                       in ? p.w + (wrow[j][h] + static_cast<unsigned>(ic + u) * CHUNK) : p.w, in);
      }
      ic += U;
      if (ic >= c_hi) {
        ic = c_lo;
        itile += stride;
        if (itile < p.tiles) rows_of(itile);
      }
    }
  };
  // (XD) the same turn's pieces of the rows of x: row n = nb * 8 + g, the chunk's 16 bytes of thread t
  int xtile = tile, xc = c_lo;
  unsigned xoff[NB];
  bool has[NB];
  auto issue_x = [&](int r) {
    if (XD && xtile < p.tiles) {
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const bool in = xc + u < c_hi && has[nb];
          cp_async16(ring + (r * TSLOTS + SLOTS + u * NB + nb) * piece_stride,
                     in ? p.x + (xoff[nb] + static_cast<unsigned>(xc + u) * CHUNK) : p.x, in);
        }
      xc += U;
      if (xc >= c_hi) {
        xc = c_lo;
        xtile += stride;
      }
    }
  };
#pragma unroll
  for (int r = 0; r < TURNS; ++r) {
    issue_w(r);
    if (!XD) cp_async_commit();
  }
  pdl_wait();                       // x and the residual belong to the kernels before this one
  if (XD) {
    // (the first group then holds the weights of all first turns and the first turn's x: whoever waits for a turn's
    // group has that turn's weights too)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int n = nb * 8 + g;
      has[nb] = n < M;
      xoff[nb] = (has[nb] ? static_cast<unsigned>(p.x_rows ? p.x_rows[n] : n) * static_cast<unsigned>(K) : 0u) + 8u * t;
    }
#pragma unroll
    for (int r = 0; r < TURNS; ++r) {
      issue_x(r);
      cp_async_commit();
    }
  }

  // ---- the rows of x' into shared memory, four rows at a time: a thread takes 16 bytes of each of them (their loads
  // are on their way together), so a row's sum of squares is spread over the threads and meets in `part`
  if (!XD) {
    // A cluster of two CTAs stages half of the rows each and stores them into both CTAs' shared memory: every CTA
    // else reads all rows of x and of the residual, 148 times the same 128 KB out of the second-level cache at once.
    const int csize = p.pair ? 2 : 1;
    uint32_t crank = 0;
    if (p.pair) asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(crank));
    const uint32_t peer_xs = p.pair ? peer_address(xs, crank ^ 1u) : 0u;
    if (p.pair) asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    const bool writer = NORM && static_cast<int>(blockIdx.x) < csize && p.residual_out != nullptr;
#pragma unroll 1
    for (int m0 = 4 * static_cast<int>(crank); m0 < MP; m0 += 4 * csize) {
      float ss[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      unsigned src[4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
        src[r] = m0 + r < M ? static_cast<unsigned>(p.x_rows ? p.x_rows[m0 + r] : m0 + r) * static_cast<unsigned>(K) : 0u;
#pragma unroll 1
      for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        uint4 xa[4], xr[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          xa[r] = xr[r] = make_uint4(0u, 0u, 0u, 0u);
          if (m0 + r < M) {
            xa[r] = *reinterpret_cast<const uint4*>(p.x + src[r] + k);
            if (NORM && p.residual != nullptr) xr[r] = *reinterpret_cast<const uint4*>(p.residual + src[r] + k);
          }
        }
        if (NORM) {
          float w[8];
          if (p.norm_w_f32) {
            const float* nw = static_cast<const float*>(p.norm_w) + k;
            const float4 w0 = *reinterpret_cast<const float4*>(nw), w1 = *reinterpret_cast<const float4*>(nw + 4);
            w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
          } else {
            unpack8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.norm_w) + k), w);
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            if (m0 + r < M) {
              float sum[8], other[8];
              unpack8(xa[r], sum);
              unpack8(xr[r], other);
#pragma unroll
              for (int i = 0; i < 8; ++i) sum[i] += other[i];
              if (writer) *reinterpret_cast<uint4*>(p.residual_out + src[r] + k) = pack8(sum);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                ss[r] = fmaf(sum[i], sum[i], ss[r]);
                sum[i] *= w[i];
              }
              xa[r] = pack8(sum);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          *reinterpret_cast<uint4*>(xs + (m0 + r) * row_bytes + 2 * k) = xa[r];   // (rows beyond M: zeros)
          if (p.pair) store_peer16(peer_xs + (m0 + r) * row_bytes + 2 * k, xa[r]);
        }
      }
      if (NORM) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float v = warp_sum(ss[r]);
          if (lane == 0) part[warp * MMAX + m0 + r] = v;
        }
      }
    }
    __syncthreads();
    if (NORM) {
      // (a CTA of a pair has the sums of its own rows only: it gives their scales to the other one too)
      if (threadIdx.x < MP && (threadIdx.x >> 2) % csize == static_cast<int>(crank)) {
        float v = 0.0f;
        for (int w = 0; w < KS * G; ++w) v += part[w * MMAX + threadIdx.x];
        const float sc = rsqrtf(v / static_cast<float>(K) + p.eps);
        scale[threadIdx.x] = sc;
        if (p.pair) store_peer_f32(peer_address(scale + threadIdx.x, crank ^ 1u), sc);
      }
    }
    if (p.pair) cluster_barrier();    // (every thread of both CTAs: the other CTA's rows and scales have landed)
    else if (NORM) __syncthreads();
  } else if (p.pair) {                // (not reached: pairs are launched with staged rows only)
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  }

  // ---- the tiles of this group
  const int gthreads = KS * 32, gt = threadIdx.x - grp * gthreads;
  const unsigned char* xme[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) xme[nb] = xs + (nb * 8 + g) * row_bytes + 16 * t;
  int turn = 0;
#pragma unroll 1
  while (tile < p.tiles) {
    float acc[RW][NB][4];
#pragma unroll
    for (int j = 0; j < RW; ++j)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) acc[j][nb][0] = acc[j][nb][1] = acc[j][nb][2] = acc[j][nb][3] = 0.0f;
    const int next = tile + stride;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; c += U) {
      cp_async_wait<TURNS - 1>();              // this thread's pieces of the turn have landed (it reads no one else's)
      uint4 wv[U][RW][2];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < RW; ++j)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            wv[u][j][h] = *reinterpret_cast<const uint4*>(ring + (turn * TSLOTS + (u * RW + j) * 2 + h) * piece_stride);
      uint4 xb[U][NB];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
          xb[u][nb] = XD ? *reinterpret_cast<const uint4*>(ring + (turn * TSLOTS + SLOTS + u * NB + nb) * piece_stride)
                         : c + u < c_hi ? *reinterpret_cast<const uint4*>(xme[nb] + (c + u) * (CHUNK * 2)) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < RW; ++j)
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            mma_16816(acc[j][nb], wv[u][j][0].x, wv[u][j][1].x, wv[u][j][0].y, wv[u][j][1].y, xb[u][nb].x, xb[u][nb].y);
            mma_16816(acc[j][nb], wv[u][j][0].z, wv[u][j][1].z, wv[u][j][0].w, wv[u][j][1].w, xb[u][nb].z, xb[u][nb].w);
          }
      issue_w(turn);                           // (behind the multiplies: the pieces are in registers before they are overwritten)
      issue_x(turn);
      cp_async_commit();
      turn = turn + 1 == TURNS ? 0 : turn + 1;
    }
    // ---- the warps' sums meet in shared memory
#pragma unroll
    for (int j = 0; j < RW; ++j)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        float* at = red + ((slice * RW + j) * 16 + g) * LDR + nb * 8 + 2 * t;
        *reinterpret_cast<float2*>(at) = make_float2(acc[j][nb][0], acc[j][nb][1]);
        *reinterpret_cast<float2*>(at + 8 * LDR) = make_float2(acc[j][nb][2], acc[j][nb][3]);
      }
    group_barrier(grp, gthreads);

    // ---- epilogue: element i of the tile's [M][columns] block; a row's columns are neighbouring threads
    auto total_of = [&](int rr, int m) {
      float v = 0.0f;
      for (int s = 0; s < KS; ++s) v += red[(s * RW * 16 + rr) * LDR + m];
      return NORM ? v * scale[m] : v;
    };
    if (!swiglu) {
      constexpr int COLS = RW * 16;
      const bool post = p.post_stats != nullptr && p.mode == EPI_PLAIN_BF16;
#pragma unroll 1
      for (int i0 = 0; i0 < M * COLS; i0 += gthreads) {
        const int i = i0 + gt;
        const int m = i / COLS, rr = i - m * COLS, col = tile * COLS + rr;
        const bool valid = i < M * COLS && col < p.N;
        float sq = 0.0f;
        if (valid) {
          const float v = total_of(rr, m);
          const size_t at = static_cast<size_t>(m) * p.N + col;
          if (p.mode == EPI_PLAIN_F32) {
            static_cast<float*>(p.out)[at] = v;
          } else {
            const bf16 h = __float2bfloat16_rn(v);
            static_cast<bf16*>(p.out)[at] = h;
            if (post) {
              // the norm that follows: s = round(y) + residual in float (what its prologue would add up)
              const float sum = __bfloat162float(h) + __bfloat162float(p.post_residual[at]);
              p.post_sum_out[at] = __float2bfloat16_rn(sum);
              sq = sum * sum;
            }
          }
        }
        if (post) {                     // (a row's 16 or 32 columns are one warp or half of one)
#pragma unroll
          for (int off = COLS / 2; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
          if (i < M * COLS && rr == 0) p.post_stats[tile * MMAX + m] = sq;
        }
      }
    } else {
      constexpr int COLS = RW == 1 ? 8 : 16;   // (the up rows' sums lie COLS rows behind the gate rows')
      for (int i = gt; i < M * COLS; i += gthreads) {
        const int m = i / COLS, rr = i - m * COLS, col = tile * COLS + rr;
        if (col >= inter) continue;
        const float gate = total_of(rr, m), up = total_of(COLS + rr, m);
        static_cast<bf16*>(p.out)[static_cast<size_t>(m) * inter + col] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
      }
    }
    group_barrier(grp, gthreads);       // the sums are read: the next tile may overwrite them
    tile = next;
  }
  cp_async_wait<0>();                   // (only empty groups are left)
}

// ------------------------------------------------------------------ host side
typedef void (*StreamKernel)(const StreamParams);
template <int RW, int NB>
static StreamKernel kernel_of(bool norm, bool xd) {
  if (norm) return stream_linear_kernel<RW, NB, true, false>;
  return xd ? stream_linear_kernel<RW, NB, false, true> : stream_linear_kernel<RW, NB, false, false>;
}
static StreamKernel kernel_of(int rw, int nb, bool norm, bool xd) {
  if (rw == 1 && nb == 1) return kernel_of<1, 1>(norm, xd);
  if (rw == 1 && nb == 2) return kernel_of<1, 2>(norm, xd);
  if (rw == 2 && nb == 1) return kernel_of<2, 1>(norm, xd);
  if (rw == 2 && nb == 2) return kernel_of<2, 2>(norm, xd);
  return nullptr;
}
// Shared memory of a CTA of `warps` warps: the rows of x' (not with xd), the warps' sums, the statistics, the pieces.
static size_t smem_of(int rw, int nb, int k, int warps, bool xd) {
  const int u = TURN_BYTES / 32 / rw;
  return (xd ? 0 : static_cast<size_t>(nb) * 8 * xs_row_bytes(k)) +
         (static_cast<size_t>(warps) * rw * 16 * (nb * 8 + 2) + warps * MMAX + MMAX) * sizeof(float) +
         static_cast<size_t>(warps) * 32 * TURNS * (TURN_BYTES + (xd ? u * nb * 16 : 0));
}
constexpr size_t SMEM_LIMIT = 227 * 1024;

// Warps of a group (they split K): every warp wants at least six chunks a tile (Qwen3-32B gate/up, 160 chunks: 91 us
// with 24 warps a group, 98 with 12; Qwen3-8B gate/up, 128 chunks: 40.4 with 24, 38.9 with 12); twelve groups at most
// (a barrier each).
static int choose_ks(int k) {
  const int chunks = k / CHUNK;
  const int choices[] = {24, 12, 8, 6, 4, 3, 2};
  for (int ks : choices)
    if (chunks / ks >= 6) return ks;
  return 2;
}

// The shape of the launch: groups of 16 weight rows a tile (0: the product is refused), warps that split K, groups of
// them a CTA, and whether the rows of x come with the weights' copies (they do not fit shared memory; p.xd forces it).
static int shape_of(const StreamParams& p, int nb, bool norm, int* ks_out, int* groups_out, bool* xd_out) {
  const int rw = p.rw > 0 ? p.rw : (p.mode == EPI_SWIGLU ? 2 : 1);
  const int ks = p.ks > 0 ? p.ks : choose_ks(p.K);
  if (ks > MAX_THREADS / 32 || rw > 2) return 0;
  int groups = MAX_THREADS / 32 / ks;
  if (groups > 12) groups = 12;
  *ks_out = ks;
  *groups_out = groups;
  const bool staged_fits = smem_of(rw, nb, p.K, ks * groups, false) <= SMEM_LIMIT;
  *xd_out = !norm && (p.xd > 0 || (p.xd < 0 && !staged_fits));
  if (!*xd_out) return staged_fits ? rw : 0;
  return smem_of(rw, nb, p.K, ks * groups, true) <= SMEM_LIMIT ? rw : 0;
}

// Whether the kernel takes a product of m rows with a weight [n, k] (the rows of x must fit shared memory).
B200_EXPORT int b200_stream_fits(int mode, int m, int n, int k, int norm) {
  if (k <= 0 || k % CHUNK != 0 || n <= 0 || m <= 0 || m > MMAX || mode < EPI_PLAIN_BF16 || mode > EPI_SWIGLU) return 0;
  if (static_cast<long long>(n) * k >= (1ll << 32)) return 0;
  StreamParams p = {};
  p.M = m; p.N = n; p.K = k; p.mode = mode; p.xd = -1;
  int ks, groups;
  bool xd;
  return shape_of(p, m <= 8 ? 1 : 2, norm != 0, &ks, &groups, &xd) > 0 ? 1 : 0;
}

// Columns of the output that one tile covers for a product [m, n] x [n, k] (the tiles of post_stats): 0 if refused.
B200_EXPORT int b200_stream_tile_cols(int mode, int m, int n, int k, int norm) {
  if (!b200_stream_fits(mode, m, n, k, norm)) return 0;
  return 16;
}

// `params`: a StreamParams filled by the caller.  Refuses (B200_BAD_SIZE) more than 16 rows, a K that is no multiple
// of 32, rows of x behind a norm that do not fit shared memory, a matrix of 2^32 elements or more, an odd N with SwiGLU, a residual
// without a norm, and shapes of the launch that the kernel does not have (rw 1 or 2; ks up to 24).
B200_EXPORT int b200_stream_linear(const void* params, int sm_count, cudaStream_t stream) {
  StreamParams p;
  memcpy(&p, params, sizeof(p));
  if (p.M <= 0) return 0;
  if (p.M > MMAX || p.N <= 0 || p.K <= 0 || p.K % CHUNK != 0) return B200_BAD_SIZE;
  if (static_cast<long long>(p.N) * p.K >= (1ll << 32)) return B200_BAD_SIZE;
  if (p.mode < EPI_PLAIN_BF16 || p.mode > EPI_SWIGLU) return B200_BAD_SIZE;
  const bool swiglu = p.mode == EPI_SWIGLU;
  if (swiglu && p.N % 2 != 0) return B200_BAD_SIZE;
  if (p.norm_w == nullptr && (p.residual != nullptr || p.residual_out != nullptr)) return B200_BAD_SIZE;
  const bool post = p.post_stats != nullptr;
  if (post && (p.mode != EPI_PLAIN_BF16 || p.post_residual == nullptr || p.post_sum_out == nullptr)) return B200_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(p.w) % 16 != 0 || reinterpret_cast<uintptr_t>(p.x) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(p.residual) % 16 != 0 || reinterpret_cast<uintptr_t>(p.residual_out) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(p.norm_w) % 16 != 0)
    return B200_BAD_ALIGN;
  const int nb = p.M <= 8 ? 1 : 2;
  const bool norm = p.norm_w != nullptr;
  int ks = 0, groups = 0;
  bool xd = false;
  const int rw = shape_of(p, nb, norm, &ks, &groups, &xd);
  StreamKernel kernel = kernel_of(rw, nb, norm, xd);
  if (rw == 0 || kernel == nullptr || ks < 1 || (post && rw != 1)) return B200_BAD_SIZE;
  const int cols = swiglu ? p.N / 2 : p.N;
  const int tile_cols = swiglu ? rw * 8 : rw * 16;
  p.rw = rw; p.ks = ks; p.groups = groups;
  p.tiles = (cols + tile_cols - 1) / tile_cols;
  const size_t smem = smem_of(rw, nb, p.K, ks * groups, xd);
  // (once per kernel and device: the attribute belongs to the device's copy of the kernel)
  static bool configured[8][2][2][3];                  // [device][rw][nb][norm / plain / plain with xd]
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 8) device = 0;
  bool& done = configured[device][rw - 1][nb - 1][norm ? 0 : xd ? 2 : 1];
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SMEM_LIMIT));
    if (e != cudaSuccess) return static_cast<int>(e);
    done = true;
  }
  const int sms = sm_count > 0 ? sm_count : 148;
  int ctas = (p.tiles + groups - 1) / groups < sms ? (p.tiles + groups - 1) / groups : sms;
  // pairs where the grid fills the machine (every CTA then reads all rows of x at the same moment) and has them staged
  const bool pair = !xd && ctas >= 2 && (p.pair > 0 || (p.pair < 0 && ctas >= sms - 1));
  if (pair) ctas &= ~1;
  p.pair = pair ? 1 : 0;
  return b200_launch(kernel, dim3(ctas), dim3(ks * groups * 32), smem, stream, pair ? 2 : 0, p);
}

B200_EXPORT int b200_stream_params_size() { return static_cast<int>(sizeof(StreamParams)); }
