// bfloat16 prefill attention over the paged cache with mma.sync (m16n8k16, float accumulate): the
// kernel for head sizes and page sizes the tcgen05 kernel does not take.
// One block per (64 query rows of a request, query head); keys up to each row's own position come
// from the pages, K and V of the portion included (they were written before), so a portion may
// start anywhere in a request.  The reference has no such kernel (it runs prefill rows through the
// decode kernel, docs/design.md:113-114).  Any head_dim that is a multiple of 16 up to 256, any
// page size, any number of heads and groups, optional window (keys t > position - window).
// Scores are scaled in float after the product; softmax by exp2 with log2(e) folded into the
// scale; probabilities are rounded to bfloat16 for the P*V product, sums stay float.
#include "attention_mma.cuh"
#include "pdl.cuh"

namespace kvcm {

struct PrefillParams {
  const bf16* q; int q_stride;
  bf16* out; int out_stride;
  const bf16* k_cache; const bf16* v_cache;
  const int* block_tables; int max_blocks;
  const int* tile_seq; const int* tile_q0;
  const int* seq_q_start; const int* seq_q_len; const int* seq_ctx_len;
  int nh, nkv, block_size, window;
  float scale_log2;
  int log2_block;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads)
attn_prefill_kernel(PrefillParams p) {
  constexpr int LD = HD + 8;
  constexpr bool Q_IN_REGS = HD <= 128;
  constexpr int BM = 64;                                            // query rows per block
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qtile = reinterpret_cast<bf16*>(smem_raw);                  // [64][LD]
  bf16* kbuf = qtile + BM * LD;                                     // [2][64][LD]
  bf16* vbuf = kbuf + 2 * kKeyTile * LD;

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (p.nh / p.nkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int seq = p.tile_seq[tile], q0 = p.tile_q0[tile];
  const int q_start = p.seq_q_start[seq], q_len = p.seq_q_len[seq], ctx = p.seq_ctx_len[seq];
  const int rows_here = min(BM, q_len - q0);
  const int pos0 = ctx - q_len + q0;                                // position of the tile's first row
  const int hi = pos0 + rows_here;                                  // keys [lo, hi) matter to the tile
  const int lo = (p.window > 0) ? max(0, pos0 - p.window + 1) : 0;
  const int* table = p.block_tables + size_t(seq) * p.max_blocks;

  for (int c = tid; c < BM * (HD / 8); c += kAttnThreads) {
    const int r = c / (HD / 8), ch = c - r * (HD / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows_here)
      v = *reinterpret_cast<const uint4*>(p.q + size_t(q_start + q0 + r) * p.q_stride + size_t(head) * HD + ch * 8);
    *reinterpret_cast<uint4*>(qtile + r * LD + ch * 8) = v;
  }
  const int t_first = (lo / kKeyTile) * kKeyTile;
  const int n_tiles = (hi - t_first + kKeyTile - 1) / kKeyTile;
  load_kv_tiles<HD>(kbuf, vbuf, p.k_cache, p.v_cache, table, t_first, lo, hi, kvh, p.nkv, p.block_size, tid,
                    kAttnThreads, p.log2_block);
  cp_async_commit();
  __syncthreads();

  const bf16* qw = qtile + warp * 16 * LD;
  uint32_t qa[Q_IN_REGS ? HD / 16 : 1][4];
  if constexpr (Q_IN_REGS) load_q_frags<HD>(reinterpret_cast<uint32_t(&)[HD / 16][4]>(qa), qw, lane);

  const int row_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};   // positions of this thread's rows
  const bool warp_live = warp * 16 < rows_here;
  const int warp_last_pos = pos0 + min(warp * 16 + 15, rows_here - 1);
  const int warp_first_lo = (p.window > 0) ? pos0 + warp * 16 - p.window + 1 : 0;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  for (int i = 0; i < n_tiles; ++i) {
    const int t0 = t_first + i * kKeyTile;
    if (i + 1 < n_tiles) {
      const int nb = (i + 1) & 1;
      load_kv_tiles<HD>(kbuf + nb * kKeyTile * LD, vbuf + nb * kKeyTile * LD, p.k_cache, p.v_cache, table,
                        t0 + kKeyTile, lo, hi, kvh, p.nkv, p.block_size, tid, kAttnThreads, p.log2_block);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_live && t0 <= warp_last_pos && t0 + kKeyTile > max(lo, warp_first_lo)) {
      const bf16* kt = kbuf + (i & 1) * kKeyTile * LD;
      const bf16* vt = vbuf + (i & 1) * kKeyTile * LD;
      // scores of this warp's 16 rows against the tile's 64 keys: s[2*sub], s[2*sub+1] = keys of sub-block sub
      float s[kKeyTile / 8][4];
#pragma unroll
      for (int n = 0; n < kKeyTile / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
      const int krow = (lane & 7) + ((lane >> 4) << 3), kcol = ((lane >> 3) & 1) << 3;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4];
        if constexpr (Q_IN_REGS) {
          a[0] = qa[kk][0]; a[1] = qa[kk][1]; a[2] = qa[kk][2]; a[3] = qa[kk][3];
        } else {
          ldmatrix_x4(a, qw + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));
        }
#pragma unroll
        for (int sub = 0; sub < kKeyTile / 16; ++sub) {
          if (t0 + sub * 16 > warp_last_pos) continue;               // warp-uniform: beyond every row of the warp
          uint32_t b[4];
          ldmatrix_x4(b, kt + (sub * 16 + krow) * LD + kk * 16 + kcol);
          mma_bf16(s[2 * sub], a, b[0], b[1]);
          mma_bf16(s[2 * sub + 1], a, b[2], b[3]);
        }
      }
      // scale; mask only where the tile touches the diagonal, the window's edge or the key range's edge
      const bool needs_mask = t0 + kKeyTile - 1 > pos0 + warp * 16 || t0 < lo ||
                              (p.window > 0 && t0 <= warp_last_pos - p.window) || t0 + kKeyTile > hi;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < kKeyTile / 8; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float v = s[n][j] * p.scale_log2;
          if (needs_mask) {
            const int key = t0 + 8 * n + 2 * t4 + (j & 1);
            const int rp = row_pos[j >> 1];
            const bool ok = key <= rp && key >= lo && key < hi && (p.window <= 0 || key > rp - p.window);
            v = ok ? v : -INFINITY;
          }
          s[n][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      float scale_old[2], m_new[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        m_new[r] = fmaxf(m[r], mx[r]);
        scale_old[r] = (m_new[r] == -INFINITY) ? 1.f : fast_exp2(m[r] - m_new[r]);
        m[r] = m_new[r];
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < kKeyTile / 8; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = j >> 1;
          const float e = (m_new[r] == -INFINITY) ? 0.f : fast_exp2(s[n][j] - m_new[r]);
          s[n][j] = e;
          sum[r] += e;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) l[r] = l[r] * scale_old[r] + sum[r];
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) {
        o[d][0] *= scale_old[0]; o[d][1] *= scale_old[0];
        o[d][2] *= scale_old[1]; o[d][3] *= scale_old[1];
      }
#pragma unroll
      for (int sub = 0; sub < kKeyTile / 16; ++sub) {
        if (t0 + sub * 16 > warp_last_pos) continue;                 // those probabilities are all zero
        uint32_t pa[4] = {pack_bf16(s[2 * sub][0], s[2 * sub][1]), pack_bf16(s[2 * sub][2], s[2 * sub][3]),
                          pack_bf16(s[2 * sub + 1][0], s[2 * sub + 1][1]), pack_bf16(s[2 * sub + 1][2], s[2 * sub + 1][3])};
        pv_16x16<HD>(o, pa, vt + sub * 16 * LD, lane);
      }
    }
    __syncthreads();
  }
  if (!warp_live) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int local = warp * 16 + g + 8 * r;
    if (local >= rows_here) continue;
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    bf16* dst = p.out + size_t(q_start + q0 + local) * p.out_stride + size_t(head) * HD + 2 * t4;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d)
      *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
  }
}

template <int HD> size_t prefill_smem() { return size_t(64 + 4 * kKeyTile) * (HD + 8) * sizeof(bf16); }

template <int HD>
int launch_prefill(const PrefillParams& p, int tiles, cudaStream_t s) {
  auto kernel = attn_prefill_kernel<HD>;
  const size_t smem = prefill_smem<HD>();
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  dim3 grid(tiles, p.nh);
  return pdl_launch(kernel, grid, dim3(kAttnThreads), smem, s, p);
}


}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_attention_prefill_bf16(const void* q, int q_stride, void* out, int out_stride,
                                         const void* k_cache, const void* v_cache, const int* block_tables,
                                         int max_blocks, const int* tile_seq, const int* tile_q0,
                                         const int* seq_q_start, const int* seq_q_len, const int* seq_ctx_len,
                                         int tiles, int nh, int nkv, int hd, int block_size, float scale,
                                         int window, void* stream) {
  if (tiles == 0) return 0;
  if (nkv <= 0 || nh % nkv) return KVCM_ERR_UNSUPPORTED;
  PrefillParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.seq_q_start = seq_q_start; p.seq_q_len = seq_q_len; p.seq_ctx_len = seq_ctx_len;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.log2_block = -1;
  for (int b = 0; b < 16; ++b) if ((1 << b) == block_size) p.log2_block = b;
  int rc = KVCM_ERR_UNSUPPORTED;
#define X(N) if (hd == N) rc = launch_prefill<N>(p, tiles, (cudaStream_t)stream);
  KVCM_FOR_HEAD_DIMS(X)
#undef X
  return rc;
}
