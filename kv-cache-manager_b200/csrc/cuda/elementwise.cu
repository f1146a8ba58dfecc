// Row-wise kernels of the forward pass: embedding gather, RMSNorm fused with the residual add
// that precedes it, rotary position encoding fused with the write of K and V into cache pages,
// and SiLU(gate)*up.  Each is instantiated for float (the true 32-bit path) and bfloat16.
// Statistics, angles and the residual stream are always float.
//
// Formulas after the reference's kernels (src/cuda/kernels.cu:27-88, src/cuda/kv_cache.cu:19-38);
// the fusions (residual+norm, rotary+cache write) are this engine's own.
#include <algorithm>

#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

// Four neighbouring elements as one access (8 bytes of bfloat16, 16 of float).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ------------------------------------------------------------------------------ embedding
// x[t, :] = float(table[ids[t], :]).  An id outside [0, vocab) yields a row of NaN: loud, not wrong.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ x, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= hidden) return;
  const int id = ids[t];
  float* dst = x + size_t(t) * hidden;
  dst[i] = (id < 0 || id >= vocab) ? __int_as_float(0x7fc00000) : ldf(table + size_t(id) * hidden + i);
}

// The same, four elements a thread (hidden % 4 == 0, aligned rows).
template <typename T>
__global__ void embed_vec_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ x, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (i >= hidden) return;
  const int id = ids[t];
  const float nan = __int_as_float(0x7fc00000);
  const float4 v = (id < 0 || id >= vocab) ? make_float4(nan, nan, nan, nan) : load4(table + size_t(id) * hidden + i);
  *reinterpret_cast<float4*>(x + size_t(t) * hidden + i) = v;
}

// -------------------------------------------------------------------------------- RMSNorm
// Optional residual add first: x[r] += delta[r] (written back when rows are not gathered).
// inv = rsqrt(mean(x^2) + eps); out = round(w * round(x * inv)) in the storage type
// (the reference rounds the normalised value before the weight, src/cuda/kernels.cu:46-48).
// `rows` (optional) gathers: output row r is computed from input row rows[r]; nothing is
// written back to x then.  The weight may be float or T (a tensor stored in 32 bits stays so).
template <typename T, typename W>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const W* __restrict__ weight,
               T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];            // hidden floats: the (updated) row
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + size_t(src) * hidden;
  const T* dr = delta ? delta + size_t(src) * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = xr[i];
    if (dr) {
      v += ldf(dr + i);
      if (!rows) xr[i] = v;
    }
    row_cache[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / float(hidden) + eps);
  T* o = out + size_t(r) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float normed = Store<T>::round(row_cache[i] * inv);
    stf(o + i, ldf(weight + i) * normed);
  }
}

// The same for rows of at most 256 * 4 * VEC elements with hidden % 4 == 0: the row stays in
// registers, one pass over global memory, four elements an access.
template <typename T, typename W, int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta, const W* __restrict__ weight,
                   T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* xr = x + size_t(src) * hidden;
  const T* dr = delta ? delta + size_t(src) * hidden : nullptr;
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    const int i = (k * 256 + threadIdx.x) * 4;
    v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < hidden) {
      v[k] = *reinterpret_cast<const float4*>(xr + i);
      if (dr) {
        const float4 d = load4(dr + i);
        v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
        if (!rows) *reinterpret_cast<float4*>(xr + i) = v[k];
      }
      ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / float(hidden) + eps);
  T* o = out + size_t(r) * hidden;
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    const int i = (k * 256 + threadIdx.x) * 4;
    if (i < hidden) {
      const float4 w = load4(weight + i);
      store4(o + i, make_float4(w.x * Store<T>::round(v[k].x * inv), w.y * Store<T>::round(v[k].y * inv),
                                w.z * Store<T>::round(v[k].z * inv), w.w * Store<T>::round(v[k].w * inv)));
    }
  }
}

// Adds the pending delta into the residual stream without a norm: x += delta.
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    x[i] += ldf(delta + i);
}

// ------------------------------------------------------------- rotary + cache page write
// One block per row.  Rotates the first `rotary_dim` elements of every q head and k head of the
// fused row [q heads | k heads | v heads] in place, then copies the (rotated) k heads and the v
// heads into the page slot of the row.  angle = pos * inv_freq[j] with inv_freq given by the
// caller (float), sin/cos in float.  Pairing: rotate-half (j, j + rotary_dim/2) or interleaved
// (2j, 2j+1).  Cache layout per layer: [page][kv head][slot in page][head_dim].
// slot < 0: the row writes nothing (padding).  write_cache = 0: only the q heads are rotated.
template <typename T>
__global__ void __launch_bounds__(256)
rope_cache_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                  const float* __restrict__ inv_freq, int rotary_dim, int interleaved,
                  const int* __restrict__ slot_mapping, T* __restrict__ k_cache,
                  T* __restrict__ v_cache, int nh, int nkv, int hd, int block_size,
                  int write_cache) {
  extern __shared__ float cs_table[];    // [rotary_dim/2] cos, then [rotary_dim/2] sin: once per row
  pdl_launch_dependents();
  pdl_wait();
  // one block per row; one warp per head at a time: q heads [0, nh), k heads [nh, nh+nkv), v after them
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int heads = write_cache ? nh + 2 * nkv : nh;
  const int half = rotary_dim / 2;
  const bool rotate = inv_freq != nullptr && half > 0;
  if (rotate) {
    const float pos = float(positions[t]);
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &cs_table[half + j], &cs_table[j]);
  }
  __syncthreads();
  const int slot = write_cache ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot - page * block_size : 0;
  for (int head = warp; head < heads; head += nwarps) {
    T* base = qkv + size_t(t) * row_stride + size_t(head) * hd;
    if (head < nh + nkv && rotate) {
      for (int j = lane; j < half; j += 32) {
        const float cs = cs_table[j], sn = cs_table[half + j];
        const int ia = interleaved ? 2 * j : j;
        const int ib = interleaved ? 2 * j + 1 : j + half;
        const float a = ldf(base + ia), b = ldf(base + ib);
        float ra, rb;
        rotate_pair(a, b, cs, sn, ra, rb);
        stf(base + ia, ra);
        stf(base + ib, rb);
      }
    }
    if (head < nh || slot < 0) continue;
    __syncwarp();                        // the rotated values of this head are written by this warp
    const bool is_k = head < nh + nkv;
    const int kvh = is_k ? head - nh : head - nh - nkv;
    T* dst = (is_k ? k_cache : v_cache) + ((size_t(page) * nkv + kvh) * block_size + off) * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = base[d];
  }
}

// The same for bfloat16 rows whose heads are rotated over their whole width in rotate-half pairs
// (rotary_dim == hd, hd a multiple of 16, 16-byte aligned rows): a thread takes 8 neighbouring
// pairs of a head, i.e. one 16-byte piece of each half, so every access to qkv and to the cache
// page is a 16-byte vector.  One block per row; the same values as the kernel above.
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(bf16* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                      const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                      bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int nh, int nkv, int hd,
                      int block_size, int write_cache) {
  extern __shared__ float cs_table[];    // [hd/2] cos, then [hd/2] sin: once per row
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = hd / 2, per_head = half / 8;                // pieces of 8 pairs per head
  const float pos = float(positions[t]);
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &cs_table[half + j], &cs_table[j]);
  __syncthreads();
  const int heads = write_cache ? nh + 2 * nkv : nh;
  const int slot = write_cache ? slot_mapping[t] : -1;
  const int page = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot - page * block_size : 0;
  bf16* row = qkv + size_t(t) * row_stride;
  for (int w = threadIdx.x; w < heads * per_head; w += blockDim.x) {
    const int head = w / per_head, j0 = (w - head * per_head) * 8;
    bf16* base = row + size_t(head) * hd;
    uint4 va = *reinterpret_cast<const uint4*>(base + j0);
    uint4 vb = *reinterpret_cast<const uint4*>(base + half + j0);
    if (head < nh + nkv) {
      __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&va);
      __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&vb);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float r0a, r0b, r1a, r1b;
        rotate_pair(__bfloat162float(a2[i].x), __bfloat162float(b2[i].x), cs_table[j0 + 2 * i], cs_table[half + j0 + 2 * i], r0a, r0b);
        rotate_pair(__bfloat162float(a2[i].y), __bfloat162float(b2[i].y), cs_table[j0 + 2 * i + 1], cs_table[half + j0 + 2 * i + 1], r1a, r1b);
        a2[i] = __floats2bfloat162_rn(r0a, r1a);
        b2[i] = __floats2bfloat162_rn(r0b, r1b);
      }
      *reinterpret_cast<uint4*>(base + j0) = va;
      *reinterpret_cast<uint4*>(base + half + j0) = vb;
    }
    if (head < nh || slot < 0) continue;
    const bool is_k = head < nh + nkv;
    const int kvh = is_k ? head - nh : head - nh - nkv;
    bf16* dst = (is_k ? k_cache : v_cache) + ((size_t(page) * nkv + kvh) * block_size + off) * hd;
    *reinterpret_cast<uint4*>(dst + j0) = va;
    *reinterpret_cast<uint4*>(dst + half + j0) = vb;
  }
}

// The angles of a step depend on the rows' positions only, not on the layer: for a step of many
// rows their cosines and sines are computed once (table [rows][hd]: hd/2 cosines, then hd/2 sines)
// and every layer's rotary kernel reads them.  The same values as the kernels above compute.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int rows,
                                  int half, float* __restrict__ table) {
  pdl_launch_dependents();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * half; i += gridDim.x * blockDim.x) {
    const int t = i / half, j = i - t * half;
    float sn, cs;
    sincosf(float(positions[t]) * inv_freq[j], &sn, &cs);
    table[size_t(t) * 2 * half + j] = cs;
    table[size_t(t) * 2 * half + half + j] = sn;
  }
}

// rope_cache_vec_kernel with the angles from that table: no shared memory, no barrier, one item (8
// neighbouring pairs of a head of a row) a thread.
__global__ void __launch_bounds__(256)
rope_cache_table_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ table,
                        const int* __restrict__ slot_mapping, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                        int rows, int nh, int nkv, int hd, int block_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = hd / 2, per_head = half / 8;
  const int heads = write_cache ? nh + 2 * nkv : nh;
  const int per_row = heads * per_head;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * per_row) return;
  const int t = idx / per_row, w = idx - t * per_row;
  const int head = w / per_head, j0 = (w - head * per_head) * 8;
  bf16* base = qkv + size_t(t) * row_stride + size_t(head) * hd;
  uint4 va = *reinterpret_cast<const uint4*>(base + j0);
  uint4 vb = *reinterpret_cast<const uint4*>(base + half + j0);
  if (head < nh + nkv) {
    const float* cs = table + size_t(t) * hd + j0;
    const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half), s1 = *reinterpret_cast<const float4*>(cs + half + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&va);
    __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&vb);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float r0a, r0b, r1a, r1b;
      rotate_pair(__bfloat162float(a2[i].x), __bfloat162float(b2[i].x), c[2 * i], sn[2 * i], r0a, r0b);
      rotate_pair(__bfloat162float(a2[i].y), __bfloat162float(b2[i].y), c[2 * i + 1], sn[2 * i + 1], r1a, r1b);
      a2[i] = __floats2bfloat162_rn(r0a, r1a);
      b2[i] = __floats2bfloat162_rn(r0b, r1b);
    }
    *reinterpret_cast<uint4*>(base + j0) = va;
    *reinterpret_cast<uint4*>(base + half + j0) = vb;
  }
  if (head < nh) return;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int page = slot / block_size, off = slot - page * block_size;
  const bool is_k = head < nh + nkv;
  const int kvh = is_k ? head - nh : head - nh - nkv;
  bf16* dst = (is_k ? k_cache : v_cache) + ((size_t(page) * nkv + kvh) * block_size + off) * hd;
  *reinterpret_cast<uint4*>(dst + j0) = va;
  *reinterpret_cast<uint4*>(dst + half + j0) = vb;
}

// --------------------------------------------------------------------------- SiLU(g) * u
// gate = columns [0, I) of the fused product, up = columns [I, 2I).  silu is rounded to the
// storage type before the product (src/cuda/kernels.cu:72-82).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const T* g = gate_up + size_t(t) * 2 * inter;
  const float x = ldf(g + i);
  const float s = Store<T>::round(x / (1.f + expf(-x)));
  stf(out + size_t(t) * inter + i, s * ldf(g + inter + i));
}

// bfloat16, width a multiple of 8: eight elements per thread through 16-byte loads and stores.
__global__ void silu_mul_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  const bf16* g = gate_up + size_t(t) * 2 * inter;
  const uint4 gv = *reinterpret_cast<const uint4*>(g + i);
  const uint4 uv = *reinterpret_cast<const uint4*>(g + inter + i);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 x = __bfloat1622float2(gp[k]), u = __bfloat1622float2(up[k]);
    const float s0 = Store<bf16>::round(x.x / (1.f + expf(-x.x)));
    const float s1 = Store<bf16>::round(x.y / (1.f + expf(-x.y)));
    op[k] = __floats2bfloat162_rn(s0 * u.x, s1 * u.y);
  }
  *reinterpret_cast<uint4*>(out + size_t(t) * inter + i) = ov;
}

template <typename T>
int launch_silu_mul(const T* gate_up, T* out, int rows, int inter, cudaStream_t s) {
  return pdl_launch(silu_mul_kernel<T>, dim3(rows, (inter + 255) / 256), dim3(256), 0, s, gate_up, out, inter);
}
template <>
int launch_silu_mul<bf16>(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t s) {
  if ((inter % 8) == 0 && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
    return pdl_launch(silu_mul_vec_kernel, dim3(rows, (inter / 8 + 255) / 256), dim3(256), 0, s, gate_up, out, inter);
  return pdl_launch(silu_mul_kernel<bf16>, dim3(rows, (inter + 255) / 256), dim3(256), 0, s, gate_up, out, inter);
}

// Gathers rows of a [*, width] matrix of T into a dense [n, width] matrix (used for the rows
// whose logits are wanted when a part needs them contiguous).
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int* __restrict__ rows,
                                   T* __restrict__ dst, int width) {
  const T* s = src + size_t(rows[blockIdx.x]) * width;
  T* d = dst + size_t(blockIdx.x) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) d[i] = s[i];
}

template <typename T, typename W>
int launch_rmsnorm_w(float* x, const T* delta, const W* weight, T* out, const int* rows, int n_rows,
                     int hidden, float eps, cudaStream_t s) {
  const uintptr_t others = reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(out);
  if ((hidden % 4) == 0 && hidden <= 256 * 4 * 4 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (others & (4 * sizeof(T) - 1)) == 0 && (reinterpret_cast<uintptr_t>(weight) & (4 * sizeof(W) - 1)) == 0) {
    if (hidden <= 1024) return pdl_launch(rmsnorm_vec_kernel<T, W, 1>, dim3(n_rows), dim3(256), 0, s, x, delta, weight, out, rows, hidden, eps);
    if (hidden <= 2048) return pdl_launch(rmsnorm_vec_kernel<T, W, 2>, dim3(n_rows), dim3(256), 0, s, x, delta, weight, out, rows, hidden, eps);
    return pdl_launch(rmsnorm_vec_kernel<T, W, 4>, dim3(n_rows), dim3(256), 0, s, x, delta, weight, out, rows, hidden, eps);
  }
  const size_t smem = size_t(hidden) * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  auto k = rmsnorm_kernel<T, W>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
  }
  return pdl_launch(k, dim3(n_rows), dim3(256), smem, s, x, delta, weight, out, rows, hidden, eps);
}

template <typename T>
int launch_rmsnorm(float* x, const T* delta, const void* weight, int weight_is_f32, T* out,
                   const int* rows, int n_rows, int hidden, float eps, cudaStream_t s) {
  if (n_rows == 0) return 0;
  if (weight_is_f32)
    return launch_rmsnorm_w<T, float>(x, delta, static_cast<const float*>(weight), out, rows, n_rows, hidden, eps, s);
  return launch_rmsnorm_w<T, T>(x, delta, static_cast<const T*>(weight), out, rows, n_rows, hidden, eps, s);
}

// Whether the vector form of the rotary kernel applies.
template <typename T>
bool rope_cache_vec_ok(const void* qkv, int row_stride, const float* inv_freq, int rotary_dim, int interleaved,
                       const void* k_cache, const void* v_cache, int hd) {
  if (sizeof(T) != 2 || inv_freq == nullptr || interleaved || rotary_dim != hd || (hd % 16) || (row_stride % 8)) return false;
  return ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
}

}  // namespace kvcm

using namespace kvcm;

#define KVCM_INSTANTIATE(SUFFIX, T)                                                                   \
  KVCM_API int kvcm_embed_##SUFFIX(const int* ids, const void* table, float* x, int rows, int hidden, \
                                   int vocab, void* stream) {                                         \
    if (rows == 0) return 0;                                                                          \
    if ((hidden % 4) == 0 && (reinterpret_cast<uintptr_t>(table) & (4 * sizeof(T) - 1)) == 0 &&      \
        (reinterpret_cast<uintptr_t>(x) & 15) == 0)                                                   \
      return pdl_launch(embed_vec_kernel<T>, dim3(rows, (hidden / 4 + 255) / 256), dim3(256), 0,     \
                        (cudaStream_t)stream, ids, (const T*)table, x, hidden, vocab);               \
    return pdl_launch(embed_kernel<T>, dim3(rows, (hidden + 255) / 256), dim3(256), 0,               \
                      (cudaStream_t)stream, ids, (const T*)table, x, hidden, vocab);                 \
  }                                                                                                   \
  KVCM_API int kvcm_rmsnorm_##SUFFIX(float* x, const void* delta, const void* weight,                 \
                                     int weight_is_f32, void* out, const int* rows, int n_rows,       \
                                     int hidden, float eps, void* stream) {                           \
    return launch_rmsnorm<T>(x, (const T*)delta, weight, weight_is_f32, (T*)out, rows, n_rows,        \
                             hidden, eps, (cudaStream_t)stream);                                      \
  }                                                                                                   \
  KVCM_API int kvcm_add_residual_##SUFFIX(float* x, const void* delta, long long n, void* stream) {   \
    if (n == 0) return 0;                                                                             \
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);                        \
    add_residual_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(x, (const T*)delta, (size_t)n);  \
    return KVCM_LAUNCH_RESULT();                                                                      \
  }                                                                                                   \
  KVCM_API int kvcm_rope_cache_##SUFFIX(void* qkv, int row_stride, const int* positions,              \
                                        const float* inv_freq, int rotary_dim, int interleaved,       \
                                        const int* slot_mapping, void* k_cache, void* v_cache,        \
                                        int rows, int nh, int nkv, int hd, int block_size,            \
                                        int write_cache, void* stream) {                              \
    if (rows == 0) return 0;                                                                          \
    if (rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return KVCM_ERR_UNSUPPORTED;           \
    if (rope_cache_vec_ok<T>(qkv, row_stride, inv_freq, rotary_dim, interleaved, k_cache, v_cache, hd)) \
      return pdl_launch(rope_cache_vec_kernel, dim3(rows), dim3(256), size_t(hd) * sizeof(float),     \
                        (cudaStream_t)stream, (bf16*)qkv, row_stride, positions, inv_freq,            \
                        slot_mapping, (bf16*)k_cache, (bf16*)v_cache, nh, nkv, hd, block_size,        \
                        write_cache);                                                                 \
    return pdl_launch(rope_cache_kernel<T>, dim3(rows), dim3(256), size_t(rotary_dim) * sizeof(float),\
                      (cudaStream_t)stream, (T*)qkv, row_stride, positions, inv_freq, rotary_dim,     \
                      interleaved, slot_mapping, (T*)k_cache, (T*)v_cache, nh, nkv, hd, block_size,   \
                      write_cache);                                                                   \
  }                                                                                                   \
  KVCM_API int kvcm_silu_mul_##SUFFIX(const void* gate_up, void* out, int rows, int inter,            \
                                      void* stream) {                                                 \
    if (rows == 0) return 0;                                                                          \
    return launch_silu_mul<T>((const T*)gate_up, (T*)out, rows, inter, (cudaStream_t)stream);         \
  }                                                                                                   \
  KVCM_API int kvcm_gather_rows_##SUFFIX(const void* src, const int* rows, void* dst, int n,          \
                                         int width, void* stream) {                                   \
    if (n == 0) return 0;                                                                             \
    gather_rows_kernel<T><<<n, 256, 0, (cudaStream_t)stream>>>((const T*)src, rows, (T*)dst, width);  \
    return KVCM_LAUNCH_RESULT();                                                                      \
  }

KVCM_INSTANTIATE(f32, float)
KVCM_INSTANTIATE(bf16, bf16)

// cos/sin of position * inv_freq for `rows` rows: table[t][0 .. half) cosines, [half .. 2 half) sines.
KVCM_API int kvcm_rope_table_f32(const int* positions, const float* inv_freq, int rows, int half, float* table,
                                 void* stream) {
  if (rows == 0 || half == 0) return 0;
  const int blocks = std::min((rows * half + 255) / 256, 1184);
  return pdl_launch(rope_table_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, positions, inv_freq, rows, half,
                    table);
}

// Whether kvcm_rope_cache_table_bf16 takes these rows (whole-head rotate-half pairing, 16-byte pieces).
KVCM_API int kvcm_rope_cache_table_supports(const void* qkv, int row_stride, const void* k_cache, const void* v_cache,
                                            const void* table, int hd) {
  return (hd % 16) == 0 && (row_stride % 8) == 0 &&
         ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
           reinterpret_cast<uintptr_t>(table)) & 15) == 0;
}

// kvcm_rope_cache_bf16 (rotate-half over the whole head) with the angles' cosines and sines read
// from a table that kvcm_rope_table_f32 filled for the same rows.
KVCM_API int kvcm_rope_cache_table_bf16(void* qkv, int row_stride, const float* table, const int* slot_mapping,
                                        void* k_cache, void* v_cache, int rows, int nh, int nkv, int hd, int block_size,
                                        int write_cache, void* stream) {
  if (rows == 0) return 0;
  if (!kvcm_rope_cache_table_supports(qkv, row_stride, k_cache, v_cache, table, hd)) return KVCM_ERR_UNSUPPORTED;
  const long long items = (long long)rows * (write_cache ? nh + 2 * nkv : nh) * (hd / 16);
  if (items > (1ll << 30)) return KVCM_ERR_UNSUPPORTED;
  return pdl_launch(rope_cache_table_kernel, dim3(unsigned((items + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                    (bf16*)qkv, row_stride, table, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, rows, nh, nkv, hd,
                    block_size, write_cache);
}
