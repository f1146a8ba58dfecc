// What the engine loop of the CPU core needs of a device: the step's forward pass, the sampling
// kernels, copies, a stream, events and CUDA graphs -- as C function pointers, so that the core is
// built without CUDA and is handed the kernel library's functions (csrc/cuda/runtime_exports.cu,
// step_forward.cu, sampling.cu) at run time.  A test hands it stand-ins that run on the CPU.
// Every function returns 0 on success.
#pragma once
#include <stddef.h>

struct KvcmForwardArgs;

extern "C" {
struct KvcmDeviceBackend {
  int (*forward)(const KvcmForwardArgs* args, int* launches, void* stream);
  // `mirror` (optional): pinned host memory [2 + rows] that the device also writes [status pair | tokens] into
  int (*argmax)(const float* logits, int* out, int rows, int vocab, int* status, int* mirror, void* stream);
  // the batch's integer arrays fetched from pinned host memory by a kernel (ints a multiple of 4)
  int (*fetch_ints)(const int* pinned_src, int* dst, long long ints, void* stream);
  int (*sample)(const float* logits, const float* temperature, const unsigned long long* seed,
                const long long* request_id, const int* position, int* out, int rows, int vocab, int* status,
                void* stream);
  int (*copy_to_device)(void* dst, const void* src, size_t bytes, void* stream);
  int (*copy_to_host)(void* dst, const void* src, size_t bytes, void* stream);
  int (*stream_create)(void** stream);
  int (*stream_destroy)(void* stream);
  int (*stream_sync)(void* stream);
  int (*device_alloc)(void** p, size_t bytes);          // zero-filled
  int (*device_free)(void* p);
  int (*host_alloc)(void** p, size_t bytes);            // pinned
  int (*host_free)(void* p);
  int (*event_create)(void** event);
  int (*event_destroy)(void* event);
  int (*event_record)(void* event, void* stream);
  int (*event_elapsed_ms)(void* first, void* second, float* ms);
  int (*event_sync)(void* event);                       // waits on the host until the event has happened
  int (*graph_begin)(void* stream);
  int (*graph_end)(void* stream, void** graph_exec);
  int (*graph_launch)(void* graph_exec, void* stream);
  int (*graph_destroy)(void* graph_exec);
  int (*clear_errors)(void);                            // reads and clears the kernels' error words
};
}
