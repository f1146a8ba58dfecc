// Picking the next token from float logits: greedy argmax (lowest index among equal maxima, as
// the reference's kernel, src/cuda/kernels.cu:90-119) and temperature sampling (not in the
// reference, which is greedy only).
//
// Temperature sampling draws from softmax(logits / T) by inverse CDF.  The uniform number is a
// pure function of (seed, request id, position of the drawn token), so a request's tokens do not
// depend on what else is in the batch, on how its prompt was cut, or on preemption:
//     z = seed ^ (id * 0x9E3779B97F4A7C15) ^ (position * 0xBF58476D1CE4E5B9)
//     z = splitmix64 finaliser(z + 0x9E3779B97F4A7C15);   u = (z >> 40) * 2^-24
// The vocabulary is cut into 1024 consecutive segments; segment sums are scanned in order, the
// segment that holds u * total is scanned element by element.  Softmax in float.
#include <algorithm>

#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

constexpr int kSampleThreads = 1024;
constexpr int kStatusWords = 5;

// The error words of the kernel families whose waits are bounded (0 = healthy).  The sampling
// kernels read them at the end of a step and write the first that is set beside the sampled
// tokens, so the host learns of a wait that ran out from the copy it makes anyway.
struct StatusWords {
  const int* word[kStatusWords];
};
// A second copy of [status pair | tokens] in pinned host memory that the device writes directly
// (`mirror`, optional): the host then needs no copy command to learn the step's tokens, it watches
// the words change from the -1 it put there.
// status[0] = 1 + index of the first family whose word is set (0 = none), status[1] = that word.
__device__ __forceinline__ void gather_status(const StatusWords& sw, int* status, int* mirror) {
  int first = 0, value = 0;
#pragma unroll
  for (int i = 0; i < kStatusWords; ++i) {
    const int v = sw.word[i] ? *reinterpret_cast<const volatile int*>(sw.word[i]) : 0;
    if (v != 0 && first == 0) { first = i + 1; value = v; }
  }
  status[0] = first;
  status[1] = value;
  if (mirror != nullptr) {
    *reinterpret_cast<volatile int*>(mirror + 1) = value;
    *reinterpret_cast<volatile int*>(mirror) = first;
  }
}

__device__ __forceinline__ void argmax_merge(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

// Block-wide argmax of a row; every thread returns the same (value, index).
__device__ void block_argmax(const float* __restrict__ row, int vocab, float& best, int& index,
                             float* sv, int* si) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // four consecutive logits per load; within a thread indices still ascend
    for (int i = threadIdx.x * 4; i < vocab; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      if (v.x > bv) { bv = v.x; bi = i; }
      if (v.y > bv) { bv = v.y; bi = i + 1; }
      if (v.z > bv) { bv = v.z; bi = i + 2; }
      if (v.w > bv) { bv = v.w; bi = i + 3; }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (v > bv) { bv = v; bi = i; }          // ascending i: the first maximum is kept
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nwarps ? sv[lane] : -INFINITY;
    bi = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) { sv[0] = bv; si[0] = bi; }
  }
  __syncthreads();
  best = sv[0];
  index = si[0];
  __syncthreads();
}

__global__ void __launch_bounds__(kSampleThreads)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, StatusWords sw, int* status,
              int* mirror) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();
  pdl_wait();
  if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) gather_status(sw, status, mirror);
  float best;
  int index;
  block_argmax(logits + size_t(blockIdx.x) * vocab, vocab, best, index, sv, si);
  if (threadIdx.x == 0) {
    out[blockIdx.x] = index;
    if (mirror != nullptr) *reinterpret_cast<volatile int*>(mirror + 2 + blockIdx.x) = index;
  }
}

__device__ __forceinline__ float sampling_uniform(unsigned long long seed, long long id, int position) {
  unsigned long long z = seed ^ (static_cast<unsigned long long>(id) * 0x9E3779B97F4A7C15ULL) ^
                         (static_cast<unsigned long long>(static_cast<long long>(position)) * 0xBF58476D1CE4E5B9ULL);
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ seed, const long long* __restrict__ request_id,
              const int* __restrict__ position, int* __restrict__ out, int vocab, StatusWords sw, int* status) {
  if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) gather_status(sw, status, nullptr);
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float part[kSampleThreads];
  __shared__ int chosen_segment;
  __shared__ float segment_base, target;
  const int r = blockIdx.x;
  const float* row = logits + size_t(r) * vocab;
  float best;
  int index;
  block_argmax(row, vocab, best, index, sv, si);
  const float temp = temperature[r];
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[r] = index;
    return;
  }
  const float inv_t = 1.f / temp;
  const int seg = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int begin = min(threadIdx.x * seg, vocab), end = min(begin + seg, vocab);
  float s = 0.f;
  for (int i = begin; i < end; ++i) s += expf((row[i] - best) * inv_t);
  part[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < kSampleThreads; ++i) total += part[i];
    const float want = sampling_uniform(seed[r], request_id[r], position[r]) * total;
    float run = 0.f;
    int pick = -1;
    for (int i = 0; i < kSampleThreads; ++i) {
      if (part[i] > 0.f) {
        pick = i;                                   // last non-empty segment so far: the fallback
        if (want < run + part[i]) break;
      }
      run += part[i];
    }
    if (pick >= 0 && !(want < run + part[pick])) {  // rounding pushed `want` past the end
      run = 0.f;
      for (int i = 0; i < pick; ++i) run += part[i];
    }
    chosen_segment = pick;
    segment_base = run;
    target = want;
  }
  __syncthreads();
  if (threadIdx.x == chosen_segment) {
    float run = segment_base;
    int pick = end - 1;
    for (int i = begin; i < end; ++i) {
      run += expf((row[i] - best) * inv_t);
      if (target < run) { pick = i; break; }
    }
    out[r] = pick;
  }
}

}  // namespace kvcm

using namespace kvcm;

extern "C" {
const int* kvcm_stream_error_address(void);
const int* kvcm_tcgen05_error_address(void);
const int* kvcm_gemm_tcgen05_pair_error_address(void);
const int* kvcm_gemm_tcgen05_splitk_error_address(void);
const int* kvcm_attention_tcgen05_error_address(void);
}

// The families in the order of the status index (1-based in status[0]): streaming product,
// tiled tcgen05 product, two-SM product, split-K product, tcgen05 prefill attention.
static StatusWords status_words() {
  StatusWords sw;
  sw.word[0] = kvcm_stream_error_address();
  sw.word[1] = kvcm_tcgen05_error_address();
  sw.word[2] = kvcm_gemm_tcgen05_pair_error_address();
  sw.word[3] = kvcm_gemm_tcgen05_splitk_error_address();
  sw.word[4] = kvcm_attention_tcgen05_error_address();
  return sw;
}

// `status` (optional): two ints that receive the first error word that is set, see gather_status.
// `mirror` (optional, needs `status`): pinned host memory [2 + rows] that receives the same status
// pair and tokens by direct stores of the device.
KVCM_API int kvcm_argmax_mirror_f32(const float* logits, int* out, int rows, int vocab, int* status, int* mirror,
                                    void* stream) {
  if (rows == 0) return 0;
  if (mirror != nullptr && status == nullptr) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(argmax_kernel, dim3(rows), dim3(kSampleThreads), 0, (cudaStream_t)stream, logits, out, vocab,
                    status ? status_words() : StatusWords{}, status, mirror);
}

KVCM_API int kvcm_argmax_status_f32(const float* logits, int* out, int rows, int vocab, int* status, void* stream) {
  return kvcm_argmax_mirror_f32(logits, out, rows, vocab, status, nullptr, stream);
}

namespace kvcm {
// The batch's integer arrays from pinned host memory into the device buffer that the step's kernels
// read: a kernel that fetches them itself, as the first launch of a recorded decode step, instead
// of a copy command in front of it (a copy engine needs several microseconds to start, in which the
// SMs would idle).
__global__ void __launch_bounds__(256) fetch_ints_kernel(const int4* __restrict__ src, int4* __restrict__ dst, int vecs) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += gridDim.x * blockDim.x) dst[i] = src[i];
}
}  // namespace kvcm

// `ints` a multiple of 4 (the batch builder pads every array to 16 bytes); both addresses 16-byte aligned.
KVCM_API int kvcm_fetch_ints(const int* pinned_src, int* dst, long long ints, void* stream) {
  if (ints <= 0) return 0;
  if ((ints & 3) || (reinterpret_cast<uintptr_t>(pinned_src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return KVCM_ERR_UNSUPPORTED;
  const int vecs = int(ints / 4);
  fetch_ints_kernel<<<std::min((vecs + 255) / 256, 8), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const int4*>(pinned_src), reinterpret_cast<int4*>(dst), vecs);
  return KVCM_LAUNCH_RESULT();
}

KVCM_API int kvcm_argmax_f32(const float* logits, int* out, int rows, int vocab, void* stream) {
  return kvcm_argmax_status_f32(logits, out, rows, vocab, nullptr, stream);
}

KVCM_API int kvcm_sample_status_f32(const float* logits, const float* temperature, const unsigned long long* seed,
                                    const long long* request_id, const int* position, int* out, int rows,
                                    int vocab, int* status, void* stream) {
  if (rows == 0) return 0;
  sample_kernel<<<rows, kSampleThreads, 0, (cudaStream_t)stream>>>(logits, temperature, seed, request_id, position,
                                                                   out, vocab, status ? status_words() : StatusWords{},
                                                                   status);
  return KVCM_LAUNCH_RESULT();
}

KVCM_API int kvcm_sample_f32(const float* logits, const float* temperature,
                             const unsigned long long* seed, const long long* request_id,
                             const int* position, int* out, int rows, int vocab, void* stream) {
  return kvcm_sample_status_f32(logits, temperature, seed, request_id, position, out, rows, vocab, nullptr, stream);
}

// How many kernel families report through the status words, for the host's table of names.
KVCM_API int kvcm_status_families(void) { return kStatusWords; }
