// Causal grouped-query attention over the paged cache, for head sizes up to
// HEAD_DIM (compile with -DHEAD_DIM=<multiple of 16>): a kernel for portions of
// prompts (many query positions per row) and a split-KV kernel for single decoded
// tokens, both for float and bfloat16 caches.  These are the all-sizes CUDA-core
// kernels: they serve the float32 engine and are the reference point of the
// tensor-core kernels.  The real head size `hd` (any even number up to HEAD_DIM; the
// reference's configuration allows every even head size: src/models/qwen3/config.rs:160-162)
// is a run-time argument: rows of q, the cache and the output are `hd` wide, the tiles
// in shared memory HEAD_DIM wide with zeros beyond `hd`.
//
// Semantics (reference: src/models/attention/backend.rs:1455-1498): query head h
// reads KV head h / (nh / nkv); score = q.k / sqrt(d) (the scale is a
// parameter); key j is visible to the query at absolute position p iff j <= p,
// and with a window W iff also p - W < j; softmax over the visible keys in
// float; output = P.V.  Keys and values are always read from the cache: the
// step writes them before it attends (src/models/qwen3/model.rs:495-513), so a
// position's result does not depend on how the tokens were cut into steps.
//
// Work split.  A warp owns up to 4 query vectors (a query vector is one
// (token, query head)); it walks blocks of 32 keys: lane j scores key j for the
// warp's vectors (q in shared memory, K rows padded against bank conflicts),
// an online softmax keeps (max, sum) per vector, then every lane accumulates
// its own output dimensions over the 32 keys.  Rows of a key block that lie
// beyond the sequence are zero-filled, never read: a page that is used again may
// hold anything.
#include <math.h>

#include "common.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size, a multiple of 16>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 512, "head size must be a multiple of 16 in [16, 512]");

constexpr int D = HEAD_DIM;
constexpr int NV = 4;                    // query vectors per warp
constexpr int KB = 32;                   // keys per block (one per lane)
constexpr int PAIRS = (D + 63) / 64;     // output dimension pairs per lane: dims 2*lane + 64*k, +1

template <typename T> struct RowGeom {
  static constexpr int CHUNK = 16 / sizeof(T);     // elements per 16 bytes
  static constexpr int CHUNKS = D / CHUNK;         // 16-byte chunks per row
  static constexpr int STRIDE = D + CHUNK;         // padded row: conflict-free 16-byte reads per lane
};

__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) {
  float2 v = *reinterpret_cast<const float2*>(p); a = v.x; b = v.y;
}
__device__ __forceinline__ void load_pair(const __nv_bfloat16* p, float& a, float& b) {
  uint32_t v = *reinterpret_cast<const uint32_t*>(p);
  a = __uint_as_float(v << 16); b = __uint_as_float(v & 0xffff0000u);
}

struct VecState {
  float m[NV], l[NV], acc[NV][2 * PAIRS];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      m[v] = -INFINITY; l[v] = 0.0f;
#pragma unroll
      for (int i = 0; i < 2 * PAIRS; ++i) acc[v][i] = 0.0f;
    }
  }
};

// One block of 32 keys for the warp's NV query vectors.
//  ks, vs : shared memory, 32 rows of RowGeom<T>::STRIDE elements
//  qs     : shared memory, NV rows of D floats, already multiplied by the softmax scale
//  qpos   : absolute position of each vector's query, -1 for an unused vector
//  ps     : shared memory, 32 * NV floats private to the warp
template <typename T>
__device__ __forceinline__ void warp_key_block(const T* ks, const T* vs, const float* qs, const int* qpos,
                                               int first_key, int kv_end, int window, VecState& st,
                                               float* ps) {
  using G = RowGeom<T>;
  const int lane = threadIdx.x & 31;
  float s[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) s[v] = 0.0f;
  const T* krow = ks + lane * G::STRIDE;
#pragma unroll 4
  for (int c = 0; c < G::CHUNKS; ++c) {
    float kf[G::CHUNK];
    Vec16<T>::load(krow + c * G::CHUNK, kf);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const float* qv = qs + v * D + c * G::CHUNK;
#pragma unroll
      for (int e = 0; e < G::CHUNK; e += 4) {
        const float4 q4 = *reinterpret_cast<const float4*>(qv + e);
        s[v] = fmaf(kf[e], q4.x, s[v]);
        s[v] = fmaf(kf[e + 1], q4.y, s[v]);
        s[v] = fmaf(kf[e + 2], q4.z, s[v]);
        s[v] = fmaf(kf[e + 3], q4.w, s[v]);
      }
    }
  }
  const int key = first_key + lane;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int p = qpos[v];
    const bool visible = p >= 0 && key <= p && key < kv_end && (window <= 0 || key > p - window);
    const float sv = visible ? s[v] : -INFINITY;
    const float m_new = fmaxf(st.m[v], warp_max(sv));
    float prob = 0.0f, corr = 1.0f;
    if (m_new != -INFINITY) {
      prob = visible ? expf(sv - m_new) : 0.0f;
      corr = expf(st.m[v] - m_new);          // exp(-inf) = 0 on the first visible block
    }
    st.l[v] = st.l[v] * corr + warp_sum(prob);
    st.m[v] = m_new;
#pragma unroll
    for (int i = 0; i < 2 * PAIRS; ++i) st.acc[v][i] *= corr;
    ps[lane * NV + v] = prob;
  }
  __syncwarp();
#pragma unroll 4
  for (int j = 0; j < KB; ++j) {
    const float4 pj = *reinterpret_cast<const float4*>(ps + j * NV);
    const T* vrow = vs + j * G::STRIDE;
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
      const int dim = 2 * lane + 64 * k;
      if (dim < D) {
        float a, b;
        load_pair(vrow + dim, a, b);
        st.acc[0][2 * k] = fmaf(pj.x, a, st.acc[0][2 * k]); st.acc[0][2 * k + 1] = fmaf(pj.x, b, st.acc[0][2 * k + 1]);
        st.acc[1][2 * k] = fmaf(pj.y, a, st.acc[1][2 * k]); st.acc[1][2 * k + 1] = fmaf(pj.y, b, st.acc[1][2 * k + 1]);
        st.acc[2][2 * k] = fmaf(pj.z, a, st.acc[2][2 * k]); st.acc[2][2 * k + 1] = fmaf(pj.z, b, st.acc[2][2 * k + 1]);
        st.acc[3][2 * k] = fmaf(pj.w, a, st.acc[3][2 * k]); st.acc[3][2 * k + 1] = fmaf(pj.w, b, st.acc[3][2 * k + 1]);
      }
    }
  }
  __syncwarp();
}

// Copies key rows [first_key, first_key + 32) of one KV head into shared memory
// with `nthreads` threads (thread index `tid`); rows at or beyond kv_end become zeros.
template <typename T>
__device__ __forceinline__ void load_key_block(T* dst, const T* __restrict__ cache, const int* __restrict__ table,
                                               int page_size, int nkv, int kvh, int first_key, int kv_end, int hd,
                                               int tid, int nthreads) {
  using G = RowGeom<T>;
  if (hd % G::CHUNK == 0) {
    // rows start on 16-byte boundaries: asynchronous 16-byte copies, zeros beyond the row and beyond the sequence
    const int row_chunks = hd / G::CHUNK;
    for (int c = tid; c < KB * G::CHUNKS; c += nthreads) {
      const int r = c / G::CHUNKS, part = c - r * G::CHUNKS;
      const int key = first_key + r;
      const bool valid = key < kv_end && part < row_chunks;
      const T* src = cache;
      if (valid) {
        const int page = table[key / page_size];       // cache[page][kv head][offset in page][hd]
        const size_t row = (static_cast<size_t>(page) * nkv + kvh) * page_size + key % page_size;
        src = cache + row * hd + part * G::CHUNK;
      }
      cp_async16(dst + r * G::STRIDE + part * G::CHUNK, src, valid);
    }
  } else {
    // an even head size whose rows are not 16-byte aligned: pairs of elements with plain loads
    for (int c = tid; c < KB * (D / 2); c += nthreads) {
      const int r = c / (D / 2), pair = c - r * (D / 2);
      const int key = first_key + r;
      T a = from_f32<T>(0.0f), b = a;
      if (key < kv_end && 2 * pair < hd) {
        const int page = table[key / page_size];
        const size_t row = (static_cast<size_t>(page) * nkv + kvh) * page_size + key % page_size;
        a = cache[row * hd + 2 * pair];
        b = cache[row * hd + 2 * pair + 1];
      }
      dst[r * G::STRIDE + 2 * pair] = a;
      dst[r * G::STRIDE + 2 * pair + 1] = b;
    }
  }
}

// ------------------------------------------------------------------ prompt portions
// grid (query tiles, nkv * head chunks, prefill rows); 8 warps; a tile holds `tile_tokens` consecutive query
// positions of one row and up to 32 of the `group` query heads of one KV head (head chunk hc holds heads
// 32 hc ..): tile_tokens * heads <= 32 vectors.
constexpr int PF_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(PF_WARPS * 32)
prefill_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         T* __restrict__ out, const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                         const int* __restrict__ prefix_len, const int* __restrict__ rows, int nh, int nkv,
                         int page_size, int window, float scale, int tile_tokens, int head_chunks, int hd) {
  using G = RowGeom<T>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                        // [32][D]
  float* ps = qs + 32 * D;                                               // [PF_WARPS][32 * NV]
  T* ks = reinterpret_cast<T*>(ps + PF_WARPS * KB * NV);                 // [32][STRIDE]
  T* vs = ks + KB * G::STRIDE;

  const int row = rows[blockIdx.z];
  const int kvh = blockIdx.y / head_chunks, hc = blockIdx.y - kvh * head_chunks;
  const int head_base = kvh * (nh / nkv) + hc * 32;                      // first query head of this CTA
  const int group = min(32, nh / nkv - hc * 32);                         // query heads of this CTA
  const int q_begin = cu_q[row], q_len = cu_q[row + 1] - q_begin;
  const int tok0 = blockIdx.x * tile_tokens;
  if (tok0 >= q_len) return;
  const int ntok = min(tile_tokens, q_len - tok0);
  const int nvec = ntok * group;
  const int prefix = prefix_len[row];
  const int kv_end = min(kv_len[row], prefix + tok0 + ntok);            // causal: nothing later is visible
  const int p_lo = prefix + tok0;
  int k_begin = window > 0 ? max(0, p_lo - window + 1) : 0;
  k_begin -= k_begin % KB;
  const int* table = block_table + static_cast<size_t>(row) * table_stride;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * D; i += blockDim.x) {
    const int v = i / D, dim = i - v * D;
    float val = 0.0f;
    if (v < nvec && dim < hd) {
      const int tok = v / group, head = head_base + v % group;
      val = to_f32<T>(q[(static_cast<size_t>(q_begin + tok0 + tok) * nh + head) * hd + dim]) * scale;
    }
    qs[i] = val;
  }
  int qpos[NV];
  int warp_p_max = -1, warp_p_min = 0x7fffffff;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int vec = warp * NV + v;
    qpos[v] = vec < nvec ? p_lo + vec / group : -1;
    if (qpos[v] >= 0) { warp_p_max = max(warp_p_max, qpos[v]); warp_p_min = min(warp_p_min, qpos[v]); }
  }
  VecState st;
  st.init();
  for (int kb = k_begin; kb < kv_end; kb += KB) {
    __syncthreads();                                   // the previous block is no longer read
    load_key_block<T>(ks, k_cache, table, page_size, nkv, kvh, kb, kv_end, hd, threadIdx.x, blockDim.x);
    load_key_block<T>(vs, v_cache, table, page_size, nkv, kvh, kb, kv_end, hd, threadIdx.x, blockDim.x);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    const bool touches = warp_p_max >= kb && (window <= 0 || kb + KB - 1 > warp_p_min - window);
    if (touches)
      warp_key_block<T>(ks, vs, qs + warp * NV * D, qpos, kb, kv_end, window, st, ps + warp * KB * NV);
  }
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int vec = warp * NV + v;
    if (vec >= nvec) continue;
    const int tok = vec / group, head = head_base + vec % group;
    T* dst = out + (static_cast<size_t>(q_begin + tok0 + tok) * nh + head) * hd;
    const float inv = st.l[v] > 0.0f ? 1.0f / st.l[v] : 0.0f;
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
      const int dim = 2 * lane + 64 * k;
      if (dim < hd) {
        dst[dim] = from_f32<T>(st.acc[v][2 * k] * inv);
        dst[dim + 1] = from_f32<T>(st.acc[v][2 * k + 1] * inv);
      }
    }
  }
}

// ------------------------------------------------------------------ decoded tokens, split over the keys
// grid (splits, nkv * vector groups, decode rows); DEC_WARPS warps, each walking its own key blocks
// through a private two-stage cp.async pipeline.  A CTA serves up to 4 query heads of one KV head
// (vector group vg holds heads kvh * group + 4 * vg ..).  Split s of a row covers an equal share of
// the row's key blocks; it writes (max, sum, unnormalised output) per head to scratch, or the
// final output when there is one split.
// DEC_WARPS is 4 where the tiles of four warps fit shared memory, else 2 or 1 (large heads in float).
template <typename T, int DEC_WARPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ kv_len, const int* __restrict__ rows, int nh, int nkv,
                        int page_size, int window, float scale, int vec_groups, int stages, int hd) {
  using G = RowGeom<T>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                        // [NV][D]
  float* ps = qs + NV * D;                                               // [DEC_WARPS][32 * NV]
  T* tiles = reinterpret_cast<T*>(ps + DEC_WARPS * KB * NV);             // [DEC_WARPS][stages][2][32][STRIDE]

  const int splits = gridDim.x, split = blockIdx.x;
  const int kvh = blockIdx.y / vec_groups, vg = blockIdx.y - kvh * vec_groups;
  const int row = rows[blockIdx.z];
  const int group = nh / nkv;
  const int head0 = kvh * group + vg * NV;
  const int nvec = min(NV, group - vg * NV);
  const int tok = cu_q[row];
  const int kv_end = kv_len[row];
  const int qp = kv_end - 1;                                             // the decoded token's position
  int k_begin = window > 0 ? max(0, qp - window + 1) : 0;
  k_begin -= k_begin % KB;
  const int blocks_total = (kv_end - k_begin + KB - 1) / KB;
  const int per_split = (blocks_total + splits - 1) / splits;
  const int blk_lo = split * per_split, blk_hi = min(blocks_total, blk_lo + per_split);
  const int* table = block_table + static_cast<size_t>(row) * table_stride;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < NV * D; i += blockDim.x) {
    const int v = i / D, dim = i - v * D;
    qs[i] = (v < nvec && dim < hd) ? to_f32<T>(q[(static_cast<size_t>(tok) * nh + head0 + v) * hd + dim]) * scale : 0.0f;
  }
  __syncthreads();
  int qpos[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) qpos[v] = v < nvec ? qp : -1;

  const int tile_elems = 2 * KB * G::STRIDE;
  T* my_tiles = tiles + static_cast<size_t>(warp) * stages * tile_elems;
  VecState st;
  st.init();
  // Prologue: issue the first `stages - 1` blocks of this warp.
  int issue = blk_lo + warp;
  for (int s = 0; s < stages - 1; ++s) {
    if (issue < blk_hi) {
      T* t = my_tiles + s * tile_elems;
      load_key_block<T>(t, k_cache, table, page_size, nkv, kvh, k_begin + issue * KB, kv_end, hd, lane, 32);
      load_key_block<T>(t + KB * G::STRIDE, v_cache, table, page_size, nkv, kvh, k_begin + issue * KB, kv_end, hd, lane, 32);
    }
    cp_async_commit();
    issue += DEC_WARPS;
  }
  int stage = 0;
  for (int blk = blk_lo + warp; blk < blk_hi; blk += DEC_WARPS) {
    if (stages > 1) {
      const int s_issue = (stage + stages - 1) % stages;
      if (issue < blk_hi) {
        T* t = my_tiles + s_issue * tile_elems;
        load_key_block<T>(t, k_cache, table, page_size, nkv, kvh, k_begin + issue * KB, kv_end, hd, lane, 32);
        load_key_block<T>(t + KB * G::STRIDE, v_cache, table, page_size, nkv, kvh, k_begin + issue * KB, kv_end, hd, lane, 32);
      }
      cp_async_commit();
      issue += DEC_WARPS;
      cp_async_wait<1>();          // stages is 1 or 2: all but the newest group have landed
    } else {
      T* t = my_tiles;
      load_key_block<T>(t, k_cache, table, page_size, nkv, kvh, k_begin + blk * KB, kv_end, hd, lane, 32);
      load_key_block<T>(t + KB * G::STRIDE, v_cache, table, page_size, nkv, kvh, k_begin + blk * KB, kv_end, hd, lane, 32);
      cp_async_commit();
      cp_async_wait<0>();
    }
    __syncwarp();
    const T* t = my_tiles + stage * tile_elems;
    warp_key_block<T>(t, t + KB * G::STRIDE, qs, qpos, k_begin + blk * KB, kv_end, window, st,
                      ps + warp * KB * NV);
    stage = (stage + 1) % stages;
  }
  cp_async_wait<0>();
  __syncthreads();
  // Merge the warps: shared memory is reused as [DEC_WARPS][NV][D + 2] floats.
  float* merge = reinterpret_cast<float*>(tiles);
  constexpr int MS = D + 2;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    float* dst = merge + (warp * NV + v) * MS;
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
      const int dim = 2 * lane + 64 * k;
      if (dim < D) { dst[dim] = st.acc[v][2 * k]; dst[dim + 1] = st.acc[v][2 * k + 1]; }
    }
    if (lane == 0) { dst[D] = st.m[v]; dst[D + 1] = st.l[v]; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nvec * D; i += blockDim.x) {
    const int v = i / D, dim = i - v * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, merge[(w * NV + v) * MS + D]);
    float l = 0.0f, o = 0.0f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float* src = merge + (w * NV + v) * MS;
        const float f = expf(src[D] - m);
        l += src[D + 1] * f;
        o += src[dim] * f;
      }
    }
    const int head = head0 + v;
    if (splits == 1) {
      if (dim < hd) out[(static_cast<size_t>(tok) * nh + head) * hd + dim] = from_f32<T>(l > 0.0f ? o / l : 0.0f);
    } else {
      const size_t slot = (static_cast<size_t>(blockIdx.z) * nh + head) * splits + split;
      part_acc[slot * D + dim] = o;
      if (dim == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
    }
  }
}

// grid (decode rows, nh): combines the splits of one head.
template <typename T>
__global__ void decode_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc,
                                    const float* __restrict__ part_ml, const int* __restrict__ cu_q,
                                    const int* __restrict__ rows, int nh, int splits, int hd) {
  const int head = blockIdx.y;
  const int tok = cu_q[rows[blockIdx.x]];
  const size_t base = (static_cast<size_t>(blockIdx.x) * nh + head) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(base + s) * 2]);
  for (int dim = threadIdx.x; dim < hd; dim += blockDim.x) {
    float l = 0.0f, o = 0.0f;
    if (m != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float f = expf(part_ml[(base + s) * 2] - m);
        l += part_ml[(base + s) * 2 + 1] * f;
        o += part_acc[(base + s) * D + dim] * f;
      }
    }
    out[(static_cast<size_t>(tok) * nh + head) * hd + dim] = from_f32<T>(l > 0.0f ? o / l : 0.0f);
  }
}

// ------------------------------------------------------------------ launchers
template <typename T>
static int launch_prefill(const void* q, const void* kc, const void* vc, void* out, const int* block_table,
                          int table_stride, const int* cu_q, const int* kv_len, const int* prefix_len,
                          const int* rows, int n_rows, int max_q_len, int nh, int nkv, int page_size, int window,
                          float scale, int hd, cudaStream_t stream) {
  using G = RowGeom<T>;
  const int group = nh / nkv;
  const int head_chunks = (group + 31) / 32;                  // more than 32 query heads per KV head: several CTAs
  const int tile_tokens = group >= 32 ? 1 : 32 / group;
  const size_t smem = (32 * D + PF_WARPS * KB * NV) * sizeof(float) + 2 * KB * G::STRIDE * sizeof(T);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  if (static_cast<long long>(nkv) * head_chunks > 65535 || n_rows > 65535) return B200_BAD_SIZE;
  dim3 grid((max_q_len + tile_tokens - 1) / tile_tokens, nkv * head_chunks, n_rows);
  prefill_attention_kernel<T><<<grid, PF_WARPS * 32, smem, stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc), static_cast<T*>(out),
      block_table, table_stride, cu_q, kv_len, prefix_len, rows, nh, nkv, page_size, window, scale, tile_tokens,
      head_chunks, hd);
  return b200_check_launch();
}

template <typename T>
static int launch_decode(const void* q, const void* kc, const void* vc, void* out, float* part_acc, float* part_ml,
                         const int* block_table, int table_stride, const int* cu_q, const int* kv_len,
                         const int* rows, int n_rows, int nh, int nkv, int page_size, int window, float scale,
                         int splits, int hd, cudaStream_t stream) {
  using G = RowGeom<T>;
  const int group = nh / nkv;
  const int vec_groups = (group + NV - 1) / NV;
  constexpr size_t tile_bytes = 2 * KB * G::STRIDE * sizeof(T);
  constexpr size_t limit = 200 * 1024;
  constexpr size_t fixed4 = (NV * D + 4 * KB * NV) * sizeof(float);
  // Four warps with two stages where that fits, else one stage, else fewer warps.
  constexpr int DEC_WARPS = fixed4 + 4 * tile_bytes <= limit ? 4 : (fixed4 + 2 * tile_bytes <= limit ? 2 : 1);
  constexpr size_t fixed = (NV * D + DEC_WARPS * KB * NV) * sizeof(float);
  static_assert(fixed + DEC_WARPS * tile_bytes <= 220 * 1024, "one key block per warp must fit shared memory");
  const int stages = fixed + DEC_WARPS * 2 * tile_bytes <= limit ? 2 : 1;
  size_t smem = fixed + DEC_WARPS * stages * tile_bytes;
  const size_t merge_bytes = DEC_WARPS * NV * (D + 2) * sizeof(float);
  if (fixed + merge_bytes > smem) smem = fixed + merge_bytes;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<T, DEC_WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = smem;
  }
  dim3 grid(splits, nkv * vec_groups, n_rows);
  decode_attention_kernel<T, DEC_WARPS><<<grid, DEC_WARPS * 32, smem, stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(kc), static_cast<const T*>(vc), static_cast<T*>(out),
      part_acc, part_ml, block_table, table_stride, cu_q, kv_len, rows, nh, nkv, page_size, window, scale,
      vec_groups, stages, hd);
  int rc = b200_check_launch();
  if (rc != 0 || splits == 1) return rc;
  dim3 mgrid(n_rows, nh);
  decode_merge_kernel<T><<<mgrid, D >= 128 ? 128 : 64, 0, stream>>>(static_cast<T*>(out), part_acc, part_ml, cu_q,
                                                                   rows, nh, splits, hd);
  return b200_check_launch();
}

B200_EXPORT int b200_attention_head_dim() { return D; }

// Portions of prompts.  `rows` lists the batch rows to serve (n_rows of them); max_q_len bounds their length.
B200_EXPORT int b200_prefill_attention(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const int* block_table, int table_stride, const int* cu_q,
                                       const int* kv_len, const int* prefix_len, const int* rows, int n_rows,
                                       int max_q_len, int nh, int nkv, int page_size, int window, float scale,
                                       int dtype, int head_dim, cudaStream_t stream) {
  if (n_rows <= 0 || max_q_len <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return B200_BAD_SIZE;
  if (head_dim <= 0 || head_dim > D || (head_dim & 1)) return B200_BAD_SIZE;
  if (dtype == B200_F32)
    return launch_prefill<float>(q, k_cache, v_cache, out, block_table, table_stride, cu_q, kv_len, prefix_len,
                                 rows, n_rows, max_q_len, nh, nkv, page_size, window, scale, head_dim, stream);
  if (dtype == B200_BF16)
    return launch_prefill<__nv_bfloat16>(q, k_cache, v_cache, out, block_table, table_stride, cu_q, kv_len,
                                         prefix_len, rows, n_rows, max_q_len, nh, nkv, page_size, window, scale,
                                         head_dim, stream);
  return B200_BAD_DTYPE;
}

// Scratch floats that b200_decode_attention needs for (n_rows, nh, splits): acc then (max, sum); rows of HEAD_DIM
// floats whatever the real head size.
B200_EXPORT long long b200_decode_scratch_floats(int n_rows, int nh, int splits) {
  return splits <= 1 ? 0 : static_cast<long long>(n_rows) * nh * splits * (D + 2);
}

// Single decoded tokens.  `scratch` holds b200_decode_scratch_floats(...) floats (unused when splits == 1).
B200_EXPORT int b200_decode_attention(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      float* scratch, const int* block_table, int table_stride,
                                      const int* cu_q, const int* kv_len, const int* rows, int n_rows, int nh,
                                      int nkv, int page_size, int window, float scale, int splits, int dtype,
                                      int head_dim, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || splits <= 0) return B200_BAD_SIZE;
  if (head_dim <= 0 || head_dim > D || (head_dim & 1)) return B200_BAD_SIZE;
  float* part_acc = scratch;
  float* part_ml = scratch + static_cast<size_t>(n_rows) * nh * splits * D;
  if (dtype == B200_F32)
    return launch_decode<float>(q, k_cache, v_cache, out, part_acc, part_ml, block_table, table_stride, cu_q,
                                kv_len, rows, n_rows, nh, nkv, page_size, window, scale, splits, head_dim, stream);
  if (dtype == B200_BF16)
    return launch_decode<__nv_bfloat16>(q, k_cache, v_cache, out, part_acc, part_ml, block_table, table_stride,
                                        cu_q, kv_len, rows, n_rows, nh, nkv, page_size, window, scale, splits,
                                        head_dim, stream);
  return B200_BAD_DTYPE;
}
