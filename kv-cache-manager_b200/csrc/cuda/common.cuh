// Shared device helpers of the kernel library: storage-type traits (float | bfloat16), warp and
// block reductions, the exported-symbol macro and the launch-error convention.
//
// Convention of every exported launcher: C ABI, raw device pointers, the CUDA stream last as a
// void*, return value = cudaError_t of the launch as int (0 = ok).  Launchers never allocate,
// never synchronise and never touch a stream other than the one they are given.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KVCM_API extern "C" __attribute__((visibility("default")))
#define KVCM_LAUNCH_RESULT() static_cast<int>(cudaGetLastError())

// Error codes beyond cudaError_t (which stays below 1000): a launcher refuses a size it cannot
// run instead of producing a wrong result.
#define KVCM_ERR_UNSUPPORTED 10001

namespace kvcm {

typedef __nv_bfloat16 bf16;

template <typename T> struct Store;
template <> struct Store<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct Store<bf16> {
  static __device__ __forceinline__ float load(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return Store<T>::load(p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { Store<T>::store(p, v); }

// Rotation of one rotary pair, written with explicit roundings (no fused multiply-add) so that
// every kernel that rotates gives the same bits.
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& ra, float& rb) {
  ra = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
  rb = __fadd_rn(__fmul_rn(b, cs), __fmul_rn(a, sn));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum / max over blockDim.x threads (blockDim.x a multiple of 32, at most 1024).
// `scratch` holds 33 floats of shared memory.  Every thread receives the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();                      // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace kvcm
