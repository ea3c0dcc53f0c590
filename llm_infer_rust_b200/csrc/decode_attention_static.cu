// Decode attention over the paged cache for callers that cannot allocate.
//
// The split-KV kernel needs a place for every split's partial result (an
// unnormalised output vector, a running maximum and a sum per query head).  The
// ordinary entry point, b200_decode_attention, takes that scratch from its caller.
// Some callers have nowhere to get it from: a plug-in inside a host program that
// owns the whole device heap and forbids cudaMalloc to its guests; a serving loop
// that handed every free byte to its own cache pool at start-up, so that an
// allocation would simply fail; a latency-critical path on which an allocation's
// implicit device synchronisation is not acceptable.  For them this file keeps the
// scratch inside the library itself, in a file-scope __device__ array.  Every GPU
// on which the library is loaded holds that array (B200_STATIC_SCRATCH_FLOATS
// floats, 4 MiB by default) from load until the process exits.  The library is
// compiled once per head size (-DHEAD_DIM): each of those libraries carries an
// array of its own, so a process that loads three head sizes holds three arrays
// per GPU, and "one array that all calls share" below means the calls of one
// head size.
//
// What a caller has to know:
//  * Nothing here calls cudaMalloc, cudaFree or any allocating routine; inputs and
//    the output still come from the caller.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it.  In host
//    code the array's name is only a stand-in for the symbol, never a device
//    pointer, so the kernels are always handed the looked-up address.  Make that
//    first call per device before any stream capture starts.
//  * The array that a call uses is the one of the CURRENT device (cudaGetDevice at
//    the time of the call), not of the stream's or the pointers' device: make the
//    device of `stream`, of the inputs and of the output current before calling.
//    An output pointer that belongs to another device is refused (B200_BAD_SIZE).
//  * A problem whose partials do not fit (n_rows * nh * splits * (head_dim + 2)
//    floats) is refused with B200_STATIC_TOO_LARGE; nothing is launched.
//  * All calls on a device share the one array, and it keeps whatever the last
//    call left there.  Nothing in it has to start at zero: every slot that the
//    merge kernel reads is written by the split kernel of the same call first.  But
//    two calls that overlap on the GPU (different streams) would write over each
//    other's partials: run calls of this entry point one after another.
//
// Compile with -DHEAD_DIM=<head size>, like attention.cu, whose kernels it runs.
#include <mutex>

#include "attention.cu"
#include "decode_attention_static.h"

#ifndef B200_STATIC_SCRATCH_FLOATS
#define B200_STATIC_SCRATCH_FLOATS (1 << 20)
#endif

enum : int { B200_STATIC_TOO_LARGE = -4 };

static __device__ __align__(256) float g_static_scratch[B200_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch(float** out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (device < 0 || device >= kMaxDevices) return B200_BAD_SIZE;
  std::lock_guard<std::mutex> guard(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (address == nullptr) return static_cast<int>(cudaErrorInvalidSymbol);
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return 0;
}
}  // namespace

B200_EXPORT long long b200_decode_attention_static_max_floats(void) { return B200_STATIC_SCRATCH_FLOATS; }

B200_EXPORT int b200_decode_attention_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                             const int* block_table, int table_stride, const int* cu_q,
                                             const int* kv_len, const int* rows, int n_rows, int nh, int nkv,
                                             int page_size, int window, float scale, int splits, int dtype,
                                             cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || splits <= 0) return B200_BAD_SIZE;
  if (dtype != B200_F32 && dtype != B200_BF16) return B200_BAD_DTYPE;
  const long long need = splits <= 1 ? 0 : static_cast<long long>(n_rows) * nh * splits * (D + 2);
  if (need > B200_STATIC_SCRATCH_FLOATS) return B200_STATIC_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != 0) return rc;
  {
    // the array belongs to the current device: an output that lives elsewhere would get the wrong device's array
    int device = -1;
    cudaPointerAttributes attr;
    if (cudaGetDevice(&device) == cudaSuccess && cudaPointerGetAttributes(&attr, out) == cudaSuccess &&
        attr.type == cudaMemoryTypeDevice && attr.device != device)
      return B200_BAD_SIZE;
  }
  float* part_acc = scratch;
  float* part_ml = scratch + static_cast<size_t>(n_rows) * nh * splits * D;
  if (dtype == B200_F32)
    return launch_decode<float>(q, k_cache, v_cache, out, part_acc, part_ml, block_table, table_stride, cu_q,
                                kv_len, rows, n_rows, nh, nkv, page_size, window, scale, splits, D, stream);
  return launch_decode<__nv_bfloat16>(q, k_cache, v_cache, out, part_acc, part_ml, block_table, table_stride, cu_q,
                                      kv_len, rows, n_rows, nh, nkv, page_size, window, scale, splits, D, stream);
}
