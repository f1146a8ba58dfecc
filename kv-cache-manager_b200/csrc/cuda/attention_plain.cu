// Plain paged attention: one block per (row, query head), keys walked through the page table in
// chunks with a running (max, sum, accumulator): softmax and P*V in float whatever the storage
// type.  Any head_dim up to 512, any number of heads and groups, any page size, optional window.
// With float storage this is the attention of the true 32-bit path; with bfloat16 it is the twin
// that the fast kernels are checked against.  A row's result depends only on its own position,
// its keys and the window, never on the batch around it.
//
// Arithmetic as the reference's kernel (src/cuda/paged_attention.cu:80-182): q is scaled first,
// the causal mask is the loop bound ctx = position + 1, o = (sum_t p_t v_t) / sum_t p_t.
#include "common.cuh"

namespace kvcm {

constexpr int kPlainThreads = 128;
constexpr int kPlainChunk = 512;
constexpr int kPlainMaxDimsPerThread = 4;     // head_dim <= 4 * 128

template <typename T>
__global__ void __launch_bounds__(kPlainThreads)
attention_plain_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                       const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ block_tables, int max_blocks,
                       const int* __restrict__ row_seq, const int* __restrict__ positions,
                       int nh, int nkv, int hd, int block_size, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;                     // [hd]
  float* sc = qs + hd;                  // [kPlainChunk]
  float* scratch = sc + kPlainChunk;    // [33]
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = h / (nh / nkv);
  const int ctx = positions[row] + 1;
  const int lo = (window > 0 && ctx > window) ? ctx - window : 0;
  const int* table = block_tables + size_t(row_seq[row]) * max_blocks;
  const size_t head_stride = size_t(block_size) * hd;
  const size_t page_stride = head_stride * nkv;

  for (int d = tid; d < hd; d += kPlainThreads)
    qs[d] = ldf(q + size_t(row) * q_stride + size_t(h) * hd + d) * scale;
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[kPlainMaxDimsPerThread] = {0.f, 0.f, 0.f, 0.f};

  for (int c0 = lo; c0 < ctx; c0 += kPlainChunk) {
    const int n = min(kPlainChunk, ctx - c0);
    float local_max = -INFINITY;
    for (int j = tid; j < n; j += kPlainThreads) {
      const int t = c0 + j;
      const int page = table[t / block_size];
      const T* kp = k_cache + size_t(page) * page_stride + size_t(kvh) * head_stride +
                    size_t(t % block_size) * hd;
      float s = 0.f;
      for (int d = 0; d < hd; ++d) s = fmaf(qs[d], ldf(kp + d), s);
      sc[j] = s;
      local_max = fmaxf(local_max, s);
    }
    const float m_new = fmaxf(m, block_max(local_max, scratch));
    const float factor = (m == -INFINITY) ? 0.f : expf(m - m_new);
    float local_sum = 0.f;
    for (int j = tid; j < n; j += kPlainThreads) {
      const float p = expf(sc[j] - m_new);
      sc[j] = p;
      local_sum += p;
    }
    l = l * factor + block_sum(local_sum, scratch);   // the sums' barriers also publish sc[]
    m = m_new;
#pragma unroll
    for (int i = 0; i < kPlainMaxDimsPerThread; ++i) {
      const int d = tid + i * kPlainThreads;
      if (d >= hd) break;
      float a = acc[i] * factor;
      for (int j = 0; j < n; ++j) {
        const int t = c0 + j;
        const int page = table[t / block_size];
        a = fmaf(sc[j], ldf(v_cache + size_t(page) * page_stride + size_t(kvh) * head_stride +
                            size_t(t % block_size) * hd + d), a);
      }
      acc[i] = a;
    }
    __syncthreads();                    // sc[] is overwritten by the next chunk
  }
#pragma unroll
  for (int i = 0; i < kPlainMaxDimsPerThread; ++i) {
    const int d = tid + i * kPlainThreads;
    if (d < hd) stf(out + size_t(row) * out_stride + size_t(h) * hd + d, l > 0.f ? acc[i] / l : 0.f);
  }
}

template <typename T>
int launch_attention_plain(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                           const void* v_cache, const int* block_tables, int max_blocks,
                           const int* row_seq, const int* positions, int rows, int nh, int nkv, int hd,
                           int block_size, float scale, int window, cudaStream_t s) {
  if (rows == 0) return 0;
  if (hd > kPlainMaxDimsPerThread * kPlainThreads || nkv <= 0 || nh % nkv) return KVCM_ERR_UNSUPPORTED;
  const size_t smem = (size_t(hd) + kPlainChunk + 33) * sizeof(float);
  dim3 grid(rows, nh);
  attention_plain_kernel<T><<<grid, kPlainThreads, smem, s>>>(
      (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, block_tables,
      max_blocks, row_seq, positions, nh, nkv, hd, block_size, scale, window);
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_attention_plain_f32(const void* q, int q_stride, void* out, int out_stride,
                                      const void* k_cache, const void* v_cache, const int* block_tables,
                                      int max_blocks, const int* row_seq, const int* positions, int rows,
                                      int nh, int nkv, int hd, int block_size, float scale, int window,
                                      void* stream) {
  return launch_attention_plain<float>(q, q_stride, out, out_stride, k_cache, v_cache, block_tables,
                                       max_blocks, row_seq, positions, rows, nh, nkv, hd, block_size,
                                       scale, window, (cudaStream_t)stream);
}
KVCM_API int kvcm_attention_plain_bf16(const void* q, int q_stride, void* out, int out_stride,
                                       const void* k_cache, const void* v_cache, const int* block_tables,
                                       int max_blocks, const int* row_seq, const int* positions, int rows,
                                       int nh, int nkv, int hd, int block_size, float scale, int window,
                                       void* stream) {
  return launch_attention_plain<bf16>(q, q_stride, out, out_stride, k_cache, v_cache, block_tables,
                                      max_blocks, row_seq, positions, rows, nh, nkv, hd, block_size,
                                      scale, window, (cudaStream_t)stream);
}
