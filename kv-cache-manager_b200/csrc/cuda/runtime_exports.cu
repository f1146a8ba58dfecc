// The device side of the CPU core's engine loop: thin C wrappers of the CUDA runtime calls it needs
// (copies, a stream, pinned and device memory, events, graph capture and launch) and one function
// that fills the core's table of function pointers (csrc/include/device_backend.h) with them and
// with this library's forward pass and sampling kernels.  The core is built without CUDA; it gets
// this table at run time.
#include <cuda_runtime.h>

#include "../include/device_backend.h"
#include "common.cuh"

extern "C" {
int kvcm_forward(const KvcmForwardArgs*, int*, void*);
int kvcm_argmax_mirror_f32(const float*, int*, int, int, int*, int*, void*);
int kvcm_fetch_ints(const int*, int*, long long, void*);
int kvcm_sample_status_f32(const float*, const float*, const unsigned long long*, const long long*, const int*, int*, int,
                           int, int*, void*);
int kvcm_stream_error(void);
int kvcm_tcgen05_error(void);
int kvcm_gemm_tcgen05_pair_error(void);
int kvcm_gemm_tcgen05_splitk_error(void);
int kvcm_attention_tcgen05_error(void);
}

namespace {

int rt_copy_to_device(void* dst, const void* src, size_t bytes, void* stream) {
  return int(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
int rt_copy_to_host(void* dst, const void* src, size_t bytes, void* stream) {
  return int(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}
int rt_stream_create(void** stream) {
  cudaStream_t s = nullptr;
  const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
  *stream = s;
  return int(e);
}
int rt_stream_destroy(void* stream) { return int(cudaStreamDestroy((cudaStream_t)stream)); }
int rt_stream_sync(void* stream) { return int(cudaStreamSynchronize((cudaStream_t)stream)); }
int rt_device_alloc(void** p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes ? bytes : 1);
  if (e == cudaSuccess) e = cudaMemset(*p, 0, bytes ? bytes : 1);
  return int(e);
}
int rt_device_free(void* p) { return int(cudaFree(p)); }
int rt_host_alloc(void** p, size_t bytes) { return int(cudaMallocHost(p, bytes ? bytes : 1)); }
int rt_host_free(void* p) { return int(cudaFreeHost(p)); }
int rt_event_create(void** event) {
  cudaEvent_t e = nullptr;
  const cudaError_t rc = cudaEventCreate(&e);
  *event = e;
  return int(rc);
}
int rt_event_destroy(void* event) { return int(cudaEventDestroy((cudaEvent_t)event)); }
int rt_event_record(void* event, void* stream) { return int(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); }
int rt_event_elapsed_ms(void* first, void* second, float* ms) {
  return int(cudaEventElapsedTime(ms, (cudaEvent_t)first, (cudaEvent_t)second));
}
int rt_event_sync(void* event) { return int(cudaEventSynchronize((cudaEvent_t)event)); }
// Recording: everything launched on the stream between begin and end becomes one graph.  Only this
// thread's launches are affected (thread-local capture mode).
int rt_graph_begin(void* stream) {
  return int(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
}
int rt_graph_end(void* stream, void** graph_exec) {
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &g);
  if (e != cudaSuccess) return int(e);
  cudaGraphExec_t x = nullptr;
  e = cudaGraphInstantiate(&x, g, 0);
  cudaGraphDestroy(g);
  *graph_exec = x;
  return int(e);
}
int rt_graph_launch(void* graph_exec, void* stream) {
  return int(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
}
int rt_graph_destroy(void* graph_exec) { return int(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec)); }
int rt_clear_errors(void) {
  kvcm_stream_error();
  kvcm_tcgen05_error();
  kvcm_gemm_tcgen05_pair_error();
  kvcm_gemm_tcgen05_splitk_error();
  kvcm_attention_tcgen05_error();
  return 0;
}

}  // namespace

// Fills the table; returns its size in bytes so that the caller can check the layout.
KVCM_API int kvcm_device_backend(KvcmDeviceBackend* b) {
  b->forward = kvcm_forward;
  b->argmax = kvcm_argmax_mirror_f32;
  b->fetch_ints = kvcm_fetch_ints;
  b->sample = kvcm_sample_status_f32;
  b->copy_to_device = rt_copy_to_device;
  b->copy_to_host = rt_copy_to_host;
  b->stream_create = rt_stream_create;
  b->stream_destroy = rt_stream_destroy;
  b->stream_sync = rt_stream_sync;
  b->device_alloc = rt_device_alloc;
  b->device_free = rt_device_free;
  b->host_alloc = rt_host_alloc;
  b->host_free = rt_host_free;
  b->event_create = rt_event_create;
  b->event_destroy = rt_event_destroy;
  b->event_record = rt_event_record;
  b->event_elapsed_ms = rt_event_elapsed_ms;
  b->event_sync = rt_event_sync;
  b->graph_begin = rt_graph_begin;
  b->graph_end = rt_graph_end;
  b->graph_launch = rt_graph_launch;
  b->graph_destroy = rt_graph_destroy;
  b->clear_errors = rt_clear_errors;
  return int(sizeof(KvcmDeviceBackend));
}
