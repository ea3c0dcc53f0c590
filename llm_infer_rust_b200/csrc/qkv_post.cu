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

B200_EXPORT int b200_qkv_post(const void* qkv, void* q_out, void* k_cache, void* v_cache, const void* q_w,
                              const void* k_w, float eps, const float* cos_table, const float* sin_table,
                              int rot_dim, int max_pos, const int* positions, const int* slots, int tokens,
                              int nh, int nkv, int d, int page_size, long long cache_slots, int act_dtype, int w_dtype,
                              int* err, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_HEAD_DIM || nh <= 0 || nkv <= 0 || page_size <= 0) return B200_BAD_SIZE;
  if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return B200_BAD_SIZE;
  const long long work = static_cast<long long>(tokens) * (nh + 2 * nkv);
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
