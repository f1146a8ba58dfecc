// The allocation-free variant of split-context decode attention: same kernels as
// kvcm_attention_decode_bf16, with the partial results kept in a static device array instead of
// a buffer the caller allocates.  See attention_decode_noalloc.h for who needs this and the rules.
#include <cstdio>

#include "attention_decode_noalloc.h"
#include "common.cuh"

// The ordinary entry point (attention_fast.cu); it takes the scratch pointer from its caller.
extern "C" int kvcm_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride,
                                          const void* k_cache, const void* v_cache,
                                          const int* block_tables, int max_blocks,
                                          const int* seq_ctx_len, int seqs, int nh, int nkv, int hd,
                                          int block_size, float scale, int window, int part_size,
                                          int num_parts, float* scratch, int cluster_merge, void* stream);

namespace {

// Partial (output, max, sum) of every (request, head, partition) of one call.  In host code this
// name is only a handle for the runtime, not an address a kernel could use: handing
// `noalloc_scratch` itself to a launch would fault, or on systems where the GPU can reach host
// memory silently use the wrong bytes.  Host code must ask for the device address.
static __device__ __align__(256) float noalloc_scratch[KVCM_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// Device address of the array, per device.  A plain global written without a lock: two threads that
// make their first call on a device at the same moment both look the address up and both store the
// same value, which is harmless.
float* scratch_address[kMaxDevices] = {};
thread_local char last_error[512] = "";

// Once per device, with that device current: the address kernels can use.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return int(e);
  if (dev < 0 || dev >= kMaxDevices) return KVCM_ERR_UNSUPPORTED;
  if (scratch_address[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), noalloc_scratch);
    if (e != cudaSuccess) {
      std::snprintf(last_error, sizeof last_error,
                    "cudaGetSymbolAddress for the built-in scratch array failed on device %d: %s",
                    dev, cudaGetErrorString(e));
      return int(e);
    }
    scratch_address[dev] = p;
  }
  *out = scratch_address[dev];
  return 0;
}

}  // namespace

KVCM_API int kvcm_attention_decode_bf16_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                                const void* k_cache, const void* v_cache,
                                                const int* block_tables, int max_blocks,
                                                const int* seq_ctx_len, int seqs, int nh, int nkv,
                                                int hd, int block_size, float scale, int window,
                                                int part_size, int num_parts, void* stream) {
  last_error[0] = '\0';
  if (seqs < 0 || nh <= 0 || hd <= 0 || num_parts < 1) {
    std::snprintf(last_error, sizeof last_error, "bad sizes: seqs=%d nh=%d hd=%d num_parts=%d", seqs,
                  nh, hd, num_parts);
    return KVCM_ERR_UNSUPPORTED;
  }
  const long long need = num_parts <= 1 ? 0 : (long long)seqs * nh * num_parts * (hd + 2);
  if (need > (long long)KVCM_NOALLOC_SCRATCH_FLOATS) {
    std::snprintf(last_error, sizeof last_error,
                  "decode attention without allocation: %d requests x %d heads x %d partitions x "
                  "(%d + 2) = %lld floats of partial results exceed the built-in scratch array of "
                  "%d floats; use fewer partitions or the entry point that takes a scratch buffer",
                  seqs, nh, num_parts, hd, need, KVCM_NOALLOC_SCRATCH_FLOATS);
    return KVCM_ERR_SCRATCH_TOO_LARGE;
  }
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  rc = kvcm_attention_decode_bf16(q, q_stride, out, out_stride, k_cache, v_cache, block_tables,
                                  max_blocks, seq_ctx_len, seqs, nh, nkv, hd, block_size, scale, window,
                                  part_size, num_parts, scratch, 0, stream);
  if (rc != 0)
    std::snprintf(last_error, sizeof last_error, "decode attention launch failed with code %d", rc);
  return rc;
}

KVCM_API const char* kvcm_attention_decode_noalloc_error(void) { return last_error; }

KVCM_API long long kvcm_attention_decode_noalloc_capacity(void) { return KVCM_NOALLOC_SCRATCH_FLOATS; }
