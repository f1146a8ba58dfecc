// Building blocks of the bfloat16 attention kernels: asynchronous copies of cache pages into
// shared memory, ldmatrix fragment loads and the m16n8k16 bfloat16 tensor-core product with
// float accumulators.  Softmax statistics and the output accumulator are float throughout.
//
// Shared-memory tiles are [rows][HD + 8] bfloat16: the 16-byte pad makes the row stride an odd
// multiple of 16 bytes, so the eight rows an ldmatrix reads fall into distinct bank groups.
#pragma once
#include "common.cuh"

namespace kvcm {

constexpr int kKeyTile = 64;          // keys staged per shared-memory tile

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_row)));
}

// D(16x8, float) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copies keys [t0, t0 + kKeyTile) of one KV head from the paged cache into a shared tile
// [kKeyTile][HD + 8].  Keys outside [lo, hi) are zero-filled (their scores are masked by the
// caller; zero keeps 0 * value finite).  All `nthreads` threads of the block take part.
// When the 16-byte chunks of a row divide the block evenly, a thread keeps one chunk column and
// walks the rows, so the page lookup and the address arithmetic happen once per row, not per
// chunk; `log2_block` >= 0 (a power-of-two page size) turns the division into a shift.
template <int HD>
__device__ __forceinline__ void load_kv_tile(bf16* __restrict__ tile, const bf16* __restrict__ cache,
                                             const int* __restrict__ table, int t0, int lo, int hi,
                                             int kvh, int nkv, int block_size, int tid, int nthreads,
                                             int log2_block = -1) {
  constexpr int CH = HD / 8;                      // 16-byte chunks per row
  constexpr int LD = HD + 8;
  if ((128 % CH) == 0 && nthreads == 128) {
    constexpr int RPP = (128 % CH) == 0 ? 128 / CH : 1;      // rows per pass
    const int ch = tid % CH, r0 = tid / CH;
    const size_t head_off = size_t(kvh) * block_size * HD + ch * 8;
    const size_t page_stride = size_t(nkv) * block_size * HD;
#pragma unroll
    for (int key = r0; key < kKeyTile; key += RPP) {
      const int t = t0 + key;
      bf16* dst = tile + key * LD + ch * 8;
      if (t >= lo && t < hi) {
        const int pi = log2_block >= 0 ? (t >> log2_block) : t / block_size;
        const int off = log2_block >= 0 ? (t & (block_size - 1)) : t - pi * block_size;
        cp_async16(dst, cache + size_t(table[pi]) * page_stride + head_off + size_t(off) * HD);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }
  for (int c = tid; c < kKeyTile * CH; c += nthreads) {
    const int key = c / CH, ch = c - key * CH;
    const int t = t0 + key;
    bf16* dst = tile + key * LD + ch * 8;
    if (t >= lo && t < hi) {
      const int page = table[t / block_size];
      const bf16* src = cache + ((size_t(page) * nkv + kvh) * block_size + (t % block_size)) * HD + ch * 8;
      cp_async16(dst, src);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// Loads the K tile and the V tile of keys [t0, t0 + kKeyTile) together (they share the page table
// and every offset).  With 128 threads and a chunk count that divides them, a thread owns one
// 16-byte column and a run of consecutive keys, so it looks a page up only when its run crosses
// into the next page; everything else is one add per key.  Other shapes take load_kv_tile twice.
template <int HD>
__device__ __forceinline__ void load_kv_tiles(bf16* __restrict__ ktile, bf16* __restrict__ vtile,
                                              const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                                              const int* __restrict__ table, int t0, int lo, int hi, int kvh,
                                              int nkv, int block_size, int tid, int nthreads, int log2_block) {
  constexpr int CH = HD / 8;
  constexpr int LD = HD + 8;
  if constexpr ((128 % CH) == 0 && (kKeyTile % (128 / CH)) == 0) {
    if (nthreads == 128) {
      constexpr int RUN = kKeyTile / (128 / CH);            // consecutive keys per thread
      const int ch = tid % CH, first = (tid / CH) * RUN;
      const size_t page_stride = size_t(nkv) * block_size * HD;
      const size_t head_off = size_t(kvh) * block_size * HD + ch * 8;
      int t = t0 + first;
      int pi = log2_block >= 0 ? (t >> log2_block) : t / block_size;
      int off = t - pi * block_size;
      size_t src = 0;
      bool have_page = false;
      bf16* kd = ktile + first * LD + ch * 8;
      bf16* vd = vtile + first * LD + ch * 8;
      if ((block_size % RUN) == 0 && t >= lo && t + RUN <= hi) {
        // the common case: the thread's run lies inside one page and inside the context: one
        // page lookup, copies at constant offsets (little code: a lone warp runs it cold)
        const size_t at = size_t(table[pi]) * page_stride + head_off + size_t(off) * HD;
#pragma unroll
        for (int k = 0; k < RUN; ++k) {
          cp_async16(kd + k * LD, kcache + at + k * HD);
          cp_async16(vd + k * LD, vcache + at + k * HD);
        }
        return;
      }
#pragma unroll
      for (int k = 0; k < RUN; ++k) {
        if (t >= lo && t < hi) {
          if (!have_page) {
            src = size_t(table[pi]) * page_stride + head_off + size_t(off) * HD;
            have_page = true;
          }
          cp_async16(kd, kcache + src);
          cp_async16(vd, vcache + src);
        } else {
          *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
        }
        ++t; ++off; src += HD; kd += LD; vd += LD;
        if (off == block_size) { off = 0; ++pi; have_page = false; }
      }
      return;
    }
  }
  load_kv_tile<HD>(ktile, kcache, table, t0, lo, hi, kvh, nkv, block_size, tid, nthreads, log2_block);
  load_kv_tile<HD>(vtile, vcache, table, t0, lo, hi, kvh, nkv, block_size, tid, nthreads, log2_block);
}

// 2^x by the hardware approximation (one instruction; softmax weights need no more).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// One warp: S(16 x 16 keys) = Q(16 x HD) * K(16 keys x HD)^T.  `qa` holds the A fragments of Q
// for every 16-wide slice of HD; `ktile` points at the first of the 16 keys in the shared tile.
// s[0] = keys 0..7, s[1] = keys 8..15 (accumulator layout).
template <int HD>
__device__ __forceinline__ void qk_16x16(float (&s)[2][4], const uint32_t (&qa)[HD / 16][4],
                                         const bf16* __restrict__ ktile, int lane) {
  constexpr int LD = HD + 8;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
  const int krow = (lane & 7) + ((lane >> 4) << 3);
  const int kcol = ((lane >> 3) & 1) << 3;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    uint32_t b[4];
    ldmatrix_x4(b, ktile + krow * LD + kk * 16 + kcol);
    mma_bf16(s[0], qa[kk], b[0], b[1]);
    mma_bf16(s[1], qa[kk], b[2], b[3]);
  }
}

// One warp: O(16 x HD) += P(16 x 16 keys) * V(16 keys x HD); `pa` = P as an A fragment.
template <int HD>
__device__ __forceinline__ void pv_16x16(float (&o)[HD / 8][4], const uint32_t (&pa)[4],
                                         const bf16* __restrict__ vtile, int lane) {
  constexpr int LD = HD + 8;
  const int vrow = (lane & 7) + (((lane >> 3) & 1) << 3);
  const int vcol = (lane >> 4) << 3;
#pragma unroll
  for (int dd = 0; dd < HD / 16; ++dd) {
    uint32_t b[4];
    ldmatrix_x4_trans(b, vtile + vrow * LD + dd * 16 + vcol);
    mma_bf16(o[2 * dd], pa, b[0], b[1]);
    mma_bf16(o[2 * dd + 1], pa, b[2], b[3]);
  }
}

// Loads the A fragments of a 16-row tile of Q held in shared memory [16][HD + 8].
template <int HD>
__device__ __forceinline__ void load_q_frags(uint32_t (&qa)[HD / 16][4], const bf16* __restrict__ qtile, int lane) {
  constexpr int LD = HD + 8;
  const int row = lane & 15, col = (lane >> 4) << 3;
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) ldmatrix_x4(qa[kk], qtile + row * LD + kk * 16 + col);
}

// Online-softmax update of one warp for a 16 x 16 score tile.  Thread (g = lane/4, t = lane%4)
// owns rows g and g+8 and, in each 8-key half, columns 2t and 2t+1.  Scores arrive already
// multiplied by scale*log2(e) and masked with -inf.  m/l are the running max / sum of rows
// (g, g+8).  Returns P packed as an A fragment and rescales the output accumulator.
template <int HD>
__device__ __forceinline__ void softmax_step(float (&s)[2][4], float (&m)[2], float (&l)[2],
                                             float (&o)[HD / 8][4], uint32_t (&pa)[4]) {
  float mx[2] = {fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])),
                 fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]))};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
  }
  float scale_old[2], m_new[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    m_new[r] = fmaxf(m[r], mx[r]);
    // A row that has seen no key yet keeps m = -inf; exp2(-inf - -inf) must not become NaN.
    scale_old[r] = (m_new[r] == -INFINITY) ? 1.f : fast_exp2(m[r] - m_new[r]);
    m[r] = m_new[r];
  }
  float p[2][4];
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = j >> 1;
      const float e = (m_new[r] == -INFINITY) ? 0.f : fast_exp2(s[h][j] - m_new[r]);
      p[h][j] = e;
      sum[r] += e;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) l[r] = l[r] * scale_old[r] + sum[r];     // per-thread partial sums
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    o[d][0] *= scale_old[0]; o[d][1] *= scale_old[0];
    o[d][2] *= scale_old[1]; o[d][3] *= scale_old[1];
  }
  pa[0] = pack_bf16(p[0][0], p[0][1]);
  pa[1] = pack_bf16(p[0][2], p[0][3]);
  pa[2] = pack_bf16(p[1][0], p[1][1]);
  pa[3] = pack_bf16(p[1][2], p[1][3]);
}

// Head sizes the tensor-core kernels are instantiated for.
#define KVCM_FOR_HEAD_DIMS(X) \
  X(16) X(32) X(48) X(64) X(80) X(96) X(112) X(128) X(160) X(192) X(224) X(256)

constexpr int kAttnThreads = 128;     // 4 warps

}  // namespace kvcm
