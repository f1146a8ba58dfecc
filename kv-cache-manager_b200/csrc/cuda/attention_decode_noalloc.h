// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a step that is
// being recorded into a CUDA graph by someone else's framework, a real-time loop that may not
// take the allocator's lock or trigger an implicit device synchronisation, a plugin loaded into
// a host process whose memory pool this library may not touch, and a process that has already
// handed all free device memory to its own pool.  The ordinary entry point
// (kvcm_attention_decode_bf16) leaves the scratch buffer for the split-context partial results to
// its caller, who normally allocates it; this variant brings its own.
//
// How: the partial results live in one file-scope `static __device__` array of
// KVCM_NOALLOC_SCRATCH_FLOATS floats (8 MiB), aligned to 256 bytes.  Every GPU that loads the
// library holds that array from load until the process exits, whether or not this entry point is
// ever called.  The caller still passes all inputs and the output.
//
// Rules for callers:
//  * The FIRST call on each device looks up the array's device address (cudaGetSymbolAddress,
//    once per device, with that device current).  Make that first call outside any stream
//    capture; later calls only launch kernels.
//  * seqs * nh * num_parts * (hd + 2) must not exceed KVCM_NOALLOC_SCRATCH_FLOATS, otherwise the
//    call returns KVCM_ERR_SCRATCH_TOO_LARGE and launches nothing;
//    kvcm_attention_decode_noalloc_error() then returns a sentence with both numbers.
//  * All calls share the one array and it keeps what the last call wrote.  Nothing in it has to
//    start at zero (each partition slot is written before it is read within a call), so there is
//    nothing to clear; but two calls that overlap on the GPU (different streams, or the same graph
//    launched twice at once) race on it.  Order them on one stream.
//  * No cudaMalloc, cudaFree or allocating library routine is called on any path.
#pragma once

#define KVCM_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define KVCM_ERR_SCRATCH_TOO_LARGE 10002

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as kvcm_attention_decode_bf16 without its `scratch` pointer.
// Returns 0, a cudaError_t, KVCM_ERR_UNSUPPORTED (10001) or KVCM_ERR_SCRATCH_TOO_LARGE (10002).
int kvcm_attention_decode_bf16_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                       const void* k_cache, const void* v_cache,
                                       const int* block_tables, int max_blocks,
                                       const int* seq_ctx_len, int seqs, int nh, int nkv, int hd,
                                       int block_size, float scale, int window, int part_size,
                                       int num_parts, void* stream);

// Text of the last error this entry point returned on the calling thread ("" if none).
const char* kvcm_attention_decode_noalloc_error(void);

// Capacity of the built-in scratch array in floats (KVCM_NOALLOC_SCRATCH_FLOATS).
long long kvcm_attention_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
