// Split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference project: it exists for
// callers of this library that must not, or cannot, allocate device memory at the
// moment they need attention computed.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Floats of split-KV scratch that the library holds (fixed at compile time).
long long b200_decode_attention_static_max_floats(void);

// Same arguments and results as b200_decode_attention, without the scratch pointer.
// Returns 0, a cudaError_t (> 0), or a refusal (< 0); -4 means that
// n_rows * nh * splits * (head_dim + 2) exceeds b200_decode_attention_static_max_floats().
int b200_decode_attention_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                 const int* block_table, int table_stride, const int* cu_q,
                                 const int* kv_len, const int* rows, int n_rows, int nh, int nkv,
                                 int page_size, int window, float scale, int splits, int dtype,
                                 cudaStream_t stream);

#ifdef __cplusplus
}
#endif
