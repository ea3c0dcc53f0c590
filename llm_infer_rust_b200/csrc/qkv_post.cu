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
// 128 or 256 elements in bfloat16) and a rotation over the whole head: `lanes` = head_dim / vector length lanes
// share one (token, head); the sum of squares is reduced and the rotation partner (element i <-> i + d/2) is
// fetched with shuffles, nothing passes through shared memory.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
qkv_post_vec_kernel(const TA* __restrict__ qkv, TA* __restrict__ q_out, TA* __restrict__ k_cache,
                    TA* __restrict__ v_cache, const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_pos,
                    const int* __restrict__ positions, const int* __restrict__ slots, int tokens, int nh, int nkv,
                    int d, int page_size, long long cache_slots, int lanes, int* err) {
  constexpr int N = Vec16<TA>::N;
  const int heads = nh + 2 * nkv;
  const int sub = threadIdx.x % lanes;                          // this lane's place inside its (token, head)
  const long long work = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) / lanes;
  const bool live = work < static_cast<long long>(tokens) * heads;
  const int t = live ? static_cast<int>(work / heads) : 0;
  const int h = live ? static_cast<int>(work - static_cast<long long>(t) * heads) : 0;
  const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
  // The token's position is fetched first, and the angles as soon as it is known: they depend on nothing else, and
  // fetched where they are used they stood as two more round trips behind the head's values.
  const bool turns = cos_table != nullptr && (is_q || is_k) && live;
  const int pos = turns ? positions[t] : 0;
  float v[N];
#pragma unroll
  for (int e = 0; e < N; ++e) v[e] = 0.0f;
  if (live) Vec16<TA>::load(qkv + (static_cast<size_t>(t) * heads + h) * d + sub * N, v);
  const bool in_table = turns && pos >= 0 && pos < max_pos;
  const bool first = sub < (lanes >> 1);
  float c[N], sn[N];                                          // (one wide load each: a lane's N angles are contiguous)
  if (in_table) {
    const int ci = (first ? sub : sub - (lanes >> 1)) * N;
    load_floats<float, N>(cos_table + static_cast<size_t>(pos) * (d / 2) + ci, c);
    load_floats<float, N>(sin_table + static_cast<size_t>(pos) * (d / 2) + ci, sn);
  }

  TA* dst = nullptr;
  if (live) {
    if (is_q) {
      dst = q_out + (static_cast<size_t>(t) * nh + h) * d;
    } else if (slots != nullptr) {
      const int slot = slots[t];
      if (slot < 0 || slot >= cache_slots) {
        if (sub == 0) atomicOr(err, B200_ERR_SLOT_RANGE);
      } else if (slot != 0) {
        const int kvh = is_k ? h - nh : h - nh - nkv;
        const int page = slot / page_size, offset = slot - page * page_size;
        dst = (is_k ? k_cache : v_cache) + ((static_cast<size_t>(page) * nkv + kvh) * page_size + offset) * d;
      }
    }
  }
  const unsigned full = 0xffffffffu;
  // Every lane of the warp executes the shuffles (a warp may hold a key head beside a value head); only the
  // lanes of q and k heads use their results.
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < N; ++e) ss += v[e] * v[e];
  for (int o = lanes >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(full, ss, o, lanes);
  const TW* w = is_q ? q_w : k_w;
  if ((is_q || is_k) && w != nullptr) {
    const float scale = rsqrtf(ss / static_cast<float>(d) + eps);
    float wv[N];
    load_floats<TW, N>(w + sub * N, wv);
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] = v[e] * scale * wv[e];
  }
  const int half_lanes = lanes >> 1;
  float partner[N];
#pragma unroll
  for (int e = 0; e < N; ++e) partner[e] = __shfl_xor_sync(full, v[e], half_lanes, lanes);
  if (turns) {
    if (!in_table) {
      if (sub == 0) atomicOr(err, B200_ERR_POSITION_RANGE);
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e) v[e] = first ? v[e] * c[e] - partner[e] * sn[e] : v[e] * c[e] + partner[e] * sn[e];
    }
  }
  if (dst != nullptr) {
    __align__(16) TA r[N];
#pragma unroll
    for (int e = 0; e < N; ++e) r[e] = from_f32<TA>(v[e]);
    *reinterpret_cast<uint4*>(dst + sub * N) = *reinterpret_cast<const uint4*>(r);
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
    const bool aligned = reinterpret_cast<uintptr_t>(qkv) % 16 == 0 && reinterpret_cast<uintptr_t>(q_out) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(k_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(q_w) % 16 == 0 && reinterpret_cast<uintptr_t>(k_w) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(cos_table) % 16 == 0 && reinterpret_cast<uintptr_t>(sin_table) % 16 == 0;
    const bool whole_rotation = cos_table == nullptr || rot_dim == d;
    if (lanes >= 2 && lanes <= 32 && (lanes & (lanes - 1)) == 0 && aligned && whole_rotation) {
      const long long threads = work * lanes;
      const unsigned vblocks = static_cast<unsigned>((threads + 255) / 256);
#define CALLV(TA, TW)                                                                                          \
      qkv_post_vec_kernel<TA, TW><<<vblocks, 256, 0, stream>>>(                                                 \
          static_cast<const TA*>(qkv), static_cast<TA*>(q_out), static_cast<TA*>(k_cache), static_cast<TA*>(v_cache), \
          static_cast<const TW*>(q_w), static_cast<const TW*>(k_w), eps, cos_table, sin_table, max_pos, positions, \
          slots, tokens, nh, nkv, d, page_size, cache_slots, lanes, err)
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
