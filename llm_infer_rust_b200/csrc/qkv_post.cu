// What stands between the QKV projection and attention, in one kernel:
// per-head RMSNorm of q and k, half-split rotary position encoding of q and k,
// and the store of k and v into the paged cache.  One warp owns one
// (token, head); the head's values are read once and written once.
//
// Reference semantics: src/layers/fused_ops.cu:69-87 (per-head norm, float sum
// of squares, rsqrt(mean + eps) * weight), :108-133 (rotation in float from a
// float cos/sin table, pairs (i, i + rot/2)), src/models/attention/kv_store.cu:7-33
// (copy to the row of cache slot = page * page_size + offset; slot 0 is skipped).  The reference runs three kernels
// and rounds after the norm and again after the rotation; here both happen in
// float and the value is rounded once.  A position beyond the table or a slot
// outside the pool sets an error bit and the access is skipped (the reference
// skips the first silently and asserts on the second).
#include "common.cuh"

constexpr int MAX_HEAD_DIM = 512;
constexpr int WARPS = 4;

template <typename TA, typename TW>
__global__ void qkv_post_kernel(const TA* __restrict__ qkv, TA* __restrict__ q_out,
                                TA* __restrict__ k_cache, TA* __restrict__ v_cache,
                                const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                int rot_dim, int max_pos, const int* __restrict__ positions,
                                const int* __restrict__ slots, int tokens, int nh, int nkv, int d,
                                int page_size, long long cache_slots, int* err) {
  __shared__ float buf[WARPS][MAX_HEAD_DIM];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = nh + 2 * nkv;
  const long long work = static_cast<long long>(blockIdx.x) * WARPS + warp;
  if (work >= static_cast<long long>(tokens) * heads) return;
  const int t = static_cast<int>(work / heads);
  const int h = static_cast<int>(work - static_cast<long long>(t) * heads);
  const TA* src = qkv + (static_cast<size_t>(t) * heads + h) * d;
  const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;

  TA* dst;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(t) * nh + h) * d;
  } else {
    if (slots == nullptr) return;                 // this execution reads another entry's cache
    const int slot = slots[t];
    if (slot == 0) return;                        // the sink: padding rows write nothing
    if (slot < 0 || slot >= cache_slots) {
      if (lane == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
      return;
    }
    const int kvh = is_k ? h - nh : h - nh - nkv;
    // cache[page][kv head][offset in page][d]: a page's rows of one KV head are contiguous
    const int page = slot / page_size, offset = slot - page * page_size;
    dst = (is_k ? k_cache : v_cache) + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * d;
  }
  if (!is_q && !is_k) {                           // v: a plain copy
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }

  float* row = buf[warp];
  float ss = 0.0f;
  for (int i = lane; i < d; i += 32) {
    const float v = to_f32<TA>(src[i]);
    row[i] = v;
    ss += v * v;
  }
  const TW* w = is_q ? q_w : k_w;
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / static_cast<float>(d) + eps);
    for (int i = lane; i < d; i += 32) row[i] = row[i] * scale * to_f32<TW>(w[i]);
  }
  __syncwarp();
  const int half = rot_dim / 2;
  bool rotate = cos_table != nullptr && half > 0;
  int pos = 0;
  if (rotate) {
    pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
      if (lane == 0) atomicOr(err, B200_ERR_POSITION_RANGE);
      rotate = false;
    }
  }
  if (rotate) {
    const float* c = cos_table + static_cast<size_t>(pos) * half;
    const float* s = sin_table + static_cast<size_t>(pos) * half;
    for (int i = lane; i < half; i += 32) {
      const float a = row[i], b = row[i + half];
      dst[i] = from_f32<TA>(a * c[i] - b * s[i]);
      dst[i + half] = from_f32<TA>(b * c[i] + a * s[i]);
    }
    for (int i = rot_dim + lane; i < d; i += 32) dst[i] = from_f32<TA>(row[i]);
  } else {
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<TA>(row[i]);
  }
}

// The same work with 16-byte accesses, for heads whose size is 16 bytes times a power of two of at most 32 (64,
// 128 or 256 elements in bfloat16) and a rotation over the whole head: a block takes one token at a time, `lanes` =
// head_dim / vector length lanes of it share HPT consecutive heads.  The token's position, slot, cosines and sines
// are read once per thread and token (the norm weights once per thread), no index needs a division, and a lane
// group's loads are all issued before the first is used.  The sum of squares is reduced and the rotation partner
// (element i <-> i + d/2) is fetched with shuffles; nothing passes through shared memory.
constexpr int HPT = 2;                   // heads per lane group

template <typename TW> struct LoadN;     // N consecutive weights / table entries as floats, by 16-byte loads
template <> struct LoadN<float> {
  template <int N> __device__ __forceinline__ static void load(const float* p, float (&out)[N]) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + i);
      out[i] = v.x; out[i + 1] = v.y; out[i + 2] = v.z; out[i + 3] = v.w;
    }
  }
};
template <> struct LoadN<__nv_bfloat16> {
  template <int N> __device__ __forceinline__ static void load(const __nv_bfloat16* p, float (&out)[N]) {
    static_assert(N == 4 || N == 8, "4 or 8 weights");
    if constexpr (N == 8) {
      Vec16<__nv_bfloat16>::load(p, out);
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(p);
      out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
      out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
    }
  }
};

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
qkv_post_vec_kernel(const TA* __restrict__ qkv, TA* __restrict__ q_out, TA* __restrict__ k_cache,
                    TA* __restrict__ v_cache, const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_pos,
                    const int* __restrict__ positions, const int* __restrict__ slots, int tokens, int nh, int nkv,
                    int d, int page_size, long long cache_slots, int lanes_log2, int* err) {
  constexpr int N = Vec16<TA>::N;
  const int heads = nh + 2 * nkv;
  const int chunks = (heads + HPT - 1) / HPT;                   // lane groups' worth of heads in a token
  const int lanes = 1 << lanes_log2;
  const int sub = threadIdx.x & (lanes - 1);                    // this lane's place inside its head
  const int group = threadIdx.x >> lanes_log2, groups = blockDim.x >> lanes_log2;
  const int half_lanes = lanes >> 1;
  const bool first = sub < half_lanes;
  const unsigned full = 0xffffffffu;
  // norm weights: the same for every token
  float wq[N], wk[N];
  if (q_w != nullptr) LoadN<TW>::template load<N>(q_w + sub * N, wq);
  if (k_w != nullptr) LoadN<TW>::template load<N>(k_w + sub * N, wk);

  // A block takes a token at a time; its lane groups take HPT heads each.  (The loops' trip counts are the same
  // for every lane of a warp: the shuffles below need the warp whole.)
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    int slot = 0;
    bool store_kv = false, rotate = false;
    float c[N], sn[N];
    if (slots != nullptr) {
      slot = slots[t];
      if (slot < 0 || slot >= cache_slots) {
        if (threadIdx.x == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
      } else {
        store_kv = slot != 0;
      }
    }
    if (cos_table != nullptr) {
      const int pos = positions[t];
      if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(err, B200_ERR_POSITION_RANGE);
      } else {
        rotate = true;
        const size_t at = static_cast<size_t>(pos) * (d / 2) + (first ? sub : sub - half_lanes) * N;
        LoadN<float>::load<N>(cos_table + at, c);
        LoadN<float>::load<N>(sin_table + at, sn);
        if (first) {                                            // x[i] cos - x[i + d/2] sin  |  x[i + d/2] cos + x[i] sin
#pragma unroll
          for (int e = 0; e < N; ++e) sn[e] = -sn[e];
        }
      }
    }
    const int page = slot / page_size, offset = slot - page * page_size;
    const TA* src = qkv + static_cast<size_t>(t) * heads * d + sub * N;

    for (int c0 = 0; c0 < chunks; c0 += groups) {
      const int h0 = (c0 + group) * HPT;
      float v[HPT][N];
#pragma unroll
      for (int j = 0; j < HPT; ++j) {                           // the heads' loads are in flight together
#pragma unroll
        for (int e = 0; e < N; ++e) v[j][e] = 0.0f;
        if (h0 + j < heads) Vec16<TA>::load(src + static_cast<size_t>(h0 + j) * d, v[j]);
      }
#pragma unroll
      for (int j = 0; j < HPT; ++j) {
        const int h = h0 + j;
        const bool there = h < heads;
        const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
        // Every lane of the warp executes the shuffles (a warp may hold a key head beside a value head); only the
        // lanes of q and k heads use their results.
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < N; ++e) ss += v[j][e] * v[j][e];
        for (int o = half_lanes; o > 0; o >>= 1) ss += __shfl_xor_sync(full, ss, o, lanes);
        if (there && ((is_q && q_w != nullptr) || (is_k && k_w != nullptr))) {
          const float scale = rsqrtf(ss / static_cast<float>(d) + eps);
#pragma unroll
          for (int e = 0; e < N; ++e) v[j][e] = v[j][e] * scale * (is_q ? wq[e] : wk[e]);
        }
        float partner[N];
#pragma unroll
        for (int e = 0; e < N; ++e) partner[e] = __shfl_xor_sync(full, v[j][e], half_lanes, lanes);
        if (there && rotate && (is_q || is_k)) {
#pragma unroll
          for (int e = 0; e < N; ++e) v[j][e] = fmaf(partner[e], sn[e], v[j][e] * c[e]);
        }
        TA* dst = nullptr;
        if (there && is_q) {
          dst = q_out + (static_cast<size_t>(t) * nh + h) * d;
        } else if (there && store_kv) {
          const int kvh = is_k ? h - nh : h - nh - nkv;
          dst = (is_k ? k_cache : v_cache) + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * d;
        }
        if (dst != nullptr) {
          __align__(16) TA r[N];
#pragma unroll
          for (int e = 0; e < N; ++e) r[e] = from_f32<TA>(v[j][e]);
          *reinterpret_cast<uint4*>(dst + sub * N) = *reinterpret_cast<const uint4*>(r);
        }
      }
    }
  }
}

B200_EXPORT int b200_qkv_post(const void* qkv, void* q_out, void* k_cache, void* v_cache, const void* q_w,
                              const void* k_w, float eps, const float* cos_table, const float* sin_table,
                              int rot_dim, int max_pos, const int* positions, const int* slots, int tokens,
                              int nh, int nkv, int d, int page_size, long long cache_slots, int act_dtype, int w_dtype,
                              int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_HEAD_DIM || nh <= 0 || nkv <= 0 || page_size <= 0) return B200_BAD_SIZE;
  if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return B200_BAD_SIZE;
  const long long work = static_cast<long long>(tokens) * (nh + 2 * nkv);
  {
    const int vec = act_dtype == B200_F32 ? 4 : 8;
    const int lanes = d % vec == 0 ? d / vec : 0;
    auto at16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };      // (a null pointer passes)
    const bool aligned = at16(qkv) && at16(q_out) && at16(k_cache) && at16(v_cache) && at16(q_w) && at16(k_w) &&
                         at16(cos_table) && at16(sin_table);
    const bool whole_rotation = cos_table == nullptr || rot_dim == d;
    if (lanes >= 2 && lanes <= 32 && (lanes & (lanes - 1)) == 0 && aligned && whole_rotation) {
      int lanes_log2 = 0;
      while ((1 << lanes_log2) < lanes) ++lanes_log2;
      const unsigned vblocks = static_cast<unsigned>(tokens < 65536 * 16 ? tokens : 65536 * 16);
#define CALLV(TA, TW)                                                                                          \
      qkv_post_vec_kernel<TA, TW><<<vblocks, 256, 0, stream>>>(                                                 \
          static_cast<const TA*>(qkv), static_cast<TA*>(q_out), static_cast<TA*>(k_cache), static_cast<TA*>(v_cache), \
          static_cast<const TW*>(q_w), static_cast<const TW*>(k_w), eps, cos_table, sin_table, max_pos, positions, \
          slots, tokens, nh, nkv, d, page_size, cache_slots, lanes_log2, err)
      if (act_dtype == B200_F32 && w_dtype == B200_F32) { CALLV(float, float); }
      else if (act_dtype == B200_BF16 && w_dtype == B200_BF16) { CALLV(__nv_bfloat16, __nv_bfloat16); }
      else if (act_dtype == B200_BF16 && w_dtype == B200_F32) { CALLV(__nv_bfloat16, float); }
      else if (act_dtype == B200_F32 && w_dtype == B200_BF16) { CALLV(float, __nv_bfloat16); }
      else return B200_BAD_DTYPE;
#undef CALLV
      return b200_check_launch();
    }
  }
  const unsigned blocks = static_cast<unsigned>((work + WARPS - 1) / WARPS);
#define CALL(TA, TW)                                                                                   \
  qkv_post_kernel<TA, TW><<<blocks, WARPS * 32, 0, stream>>>(                                          \
      static_cast<const TA*>(qkv), static_cast<TA*>(q_out), static_cast<TA*>(k_cache),                 \
      static_cast<TA*>(v_cache), static_cast<const TW*>(q_w), static_cast<const TW*>(k_w), eps,        \
      cos_table, sin_table, rot_dim, max_pos, positions, slots, tokens, nh, nkv, d, page_size, cache_slots, err)
  if (act_dtype == B200_F32 && w_dtype == B200_F32) { CALL(float, float); }
  else if (act_dtype == B200_BF16 && w_dtype == B200_BF16) { CALL(__nv_bfloat16, __nv_bfloat16); }
  else if (act_dtype == B200_BF16 && w_dtype == B200_F32) { CALL(__nv_bfloat16, float); }
  else if (act_dtype == B200_F32 && w_dtype == B200_BF16) { CALL(float, __nv_bfloat16); }
  else return B200_BAD_DTYPE;
#undef CALL
  return b200_check_launch();
}
