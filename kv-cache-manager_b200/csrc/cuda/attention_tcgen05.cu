// Causal prefill attention over the paged cache on the fifth-generation tensor cores (head_dim 64
// or 128).
//
// One block per (128 query rows of a request, query head).  Per tile of 64 keys:
//     S = Q K^T  (tcgen05.mma, M 128 x N 64, accumulator in tensor memory, two buffers)
//     softmax    (four warps, one thread per query row: tcgen05.ld of its row of S, running max
//                 and sum, probabilities rounded to bfloat16 into a 128-byte swizzled tile of
//                 shared memory, two buffers)
//     O += P V   (tcgen05.mma with V as the MN-major operand, straight from the page layout; O stays
//                 in tensor memory for the whole block)
// The products run one tile ahead of the softmax (S_(n+1) is computed while the softmax works on
// S_n, O += P_(n-1) V_(n-1) while it writes P_n), so the softmax threads hardly ever wait.
// The running maximum a row scales by is only renewed when the true maximum has grown by more than
// 2^8 since (probabilities then stay below 2^8, harmless in float and bfloat16); only then is the
// row's O in tensor memory rescaled (tcgen05.ld, multiply, tcgen05.st), which after the first
// tiles hardly ever happens.  The same reference maximum enters the row's sum, so the quotient at
// the end is exact softmax.
// Roles: warp 0 brings Q once and K/V pages (cp.async.bulk.tensor, one box per page, 128-byte
// swizzle) into a four-stage ring; one thread of warp 1 issues the products and commits them to
// mbarriers; warps 2-5 do the softmax and the output.  At head_dim 64 two blocks share an SM (112 KB
// of shared memory and 256 columns of tensor memory each); at 128 a block takes 192 KB.  Keys come from the pages, the portion's own
// included (they were written before), so a portion may start anywhere in a request; masks: key <=
// row's position, key > position - window, key < end of the request's computed part.  Scores are
// scaled in float; softmax by exp2 with log2(e) folded into the scale; probabilities are rounded
// to bfloat16 for the product with V, their sums stay float.
// Every wait on an mbarrier is bounded; when one runs out the block records it
// (kvcm_attention_tcgen05_error), stops waiting, frees its tensor memory and leaves.
// The reference has no prefill kernel (it runs prompt rows through its decode kernel,
// docs/design.md:113-114).
#include "pdl.cuh"
#include "tcgen05_common.cuh"

namespace kvcm {

constexpr int kFaThreads = 192;
constexpr int kFaRows = 128;                 // query rows per block
constexpr int kFaKeys = 64;                  // keys per tile
constexpr int kFaStages = 4;                 // K/V tiles in flight
constexpr int kFaTileBytes = 128 * 128;      // [128 rows][64 bf16]: a 64-wide block of Q, a buffer of P
constexpr int kFaKvBlock = kFaKeys * 128;    // [64 keys][64 bf16]: a 64-wide block of a stage of K or of V
constexpr int kFaTmemCols = 256;             // S: two buffers, columns 0..63 and 64..127; O: columns 128..(128 + head_dim)
// head_dim 64 or 128.  Operands wider than 64 elements are kept as blocks of 64 (one 128-byte
// swizzled row each): Q [HD/64][128 rows][64], a stage of K or V [HD/64][64 keys][64]; the
// products step through the blocks (S over head_dim) or write 64 columns of O per block of V.
constexpr float kFaRescaleStep = 8.f;        // in log2 units

__device__ int g_fa_error = 0;

struct PrefillTcParams {
  bf16* out; int out_stride;
  const int* block_tables; int max_blocks;
  const int* tile_seq; const int* tile_q0;                 // tiles of 64 rows; a block takes an even one and its successor
  const int* seq_q_start; const int* seq_q_len; const int* seq_ctx_len;
  int nh, nkv, block_size, window;
  float scale_log2;
};

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Two blocks of six warps share an SM at head_dim 64.  Registers are handed out per scheduler, a
// block's warps in fours, so two blocks of six warps need room for sixteen: at most 128 registers
// a thread, which the bound of 256 threads asks the compiler for (with 132 registers about half of
// the SMs took a single block).
// Blackwell's three-input maximum.
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int HD>
__global__ void __launch_bounds__(HD == 64 ? 256 : kFaThreads, HD == 64 ? 2 : 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, PrefillTcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr int KB = HD / 64;                                  // 64-wide blocks of head_dim
  constexpr int kFaKvBytes = KB * kFaKvBlock;                  // a stage of K or of V
  unsigned char* q_s = smem_raw;                               // [KB][128 rows][64]             16 KB x KB
  unsigned char* k_s = q_s + KB * kFaTileBytes;                // [stages][KB][64 keys][64]      32 KB x KB
  unsigned char* v_s = k_s + kFaStages * kFaKvBytes;           // [stages][KB][64 keys][64]      32 KB x KB
  unsigned char* p_s = v_s + kFaStages * kFaKvBytes;           // [2][128 rows][64 keys]         32 KB
  __shared__ __align__(8) uint64_t q_full, kv_full[kFaStages], kv_empty[kFaStages], s_full[2], s_free[2], p_full[2],
      p_free[2], o_full;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;

  pdl_launch_dependents();
  // Later tiles of a prompt see more keys: the blocks are ordered with the heads fastest and the
  // last tiles first, so all long blocks start at once and the short ones fill the tail.
  const int tile = int(gridDim.y) - 1 - int(blockIdx.y), head = blockIdx.x;
  const int q0 = p.tile_q0[tile];
  if (q0 & (kFaRows - 1)) return;                              // the odd tile of 64 rows belongs to the block before
  if (tc5::s32(smem_raw) & 1023) {                               // the swizzled tiles need this alignment
    if (threadIdx.x == 0) atomicExch(&g_fa_error, (7 << 16) | int(blockIdx.y & 0xffff));
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.tile_seq[tile];
  const int q_start = p.seq_q_start[seq], q_len = p.seq_q_len[seq], ctx = p.seq_ctx_len[seq];
  const int rows_here = min(kFaRows, q_len - q0);
  const int pos0 = ctx - q_len + q0;                           // position of the block's first row
  const int hi = pos0 + rows_here;                             // keys [lo, hi) matter to the block
  const int lo = (p.window > 0 && pos0 + 1 > p.window) ? pos0 + 1 - p.window : 0;
  const int j0 = lo / kFaKeys, n_tiles = (hi - 1) / kFaKeys - j0 + 1;
  const int kvh = head / (p.nh / p.nkv);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    auto init = [](uint64_t* b, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc5::s32(b)), "r"(count)); };
    init(&q_full, 1);
    for (int s = 0; s < kFaStages; ++s) { init(&kv_full[s], 1); init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) {
      init(&s_full[i], 1);
      init(&s_free[i], 4);                                     // the four softmax warps
      init(&p_full[i], 4);
      init(&p_free[i], 1);
    }
    init(&o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // The K/V ring starts as zeros: pages beyond the request's last key are not loaded, and what a
  // slot holds there is multiplied by probability zero, so it must be finite.
  for (int i = threadIdx.x; i < 2 * kFaStages * kFaKvBytes / 16; i += kFaThreads)
    reinterpret_cast<uint4*>(k_s)[i] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5::s32(&tmem_base)), "r"(kFaTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = tmem_base;
  pdl_wait();                                                  // q and this step's keys come from kernels before

  auto fail = [&](int code) {
    atomicExch(&g_fa_error, (code << 16) | int(blockIdx.y & 0xffff));
    abort_flag = 1;
  };

  if (warp == 0) {
    // ---- producer: Q once, then a tile of K and V per round, one box per page (or per half page)
    if (lane == 0) {
      tc5::mbar_expect_tx(&q_full, KB * kFaTileBytes);
      for (int kb = 0; kb < KB; ++kb)
        tc5::tma_load_2d(q_s + kb * kFaTileBytes, &map_q, &q_full, head * HD + kb * 64, q_start + q0);
    }
    const int* table = p.block_tables + size_t(seq) * p.max_blocks;
    const int B = p.block_size;
    const int box = min(B, kFaKeys), per_tile = kFaKeys / box;                 // rows of a box; boxes of a tile
    for (int n = 0; n < n_tiles; ++n) {
      const int s = n % kFaStages;
      int ok = 1;
      if (lane == 0) {
        ok = !abort_flag && tc5::mbar_wait(&kv_empty[s], ((n / kFaStages) & 1) ^ 1);
        if (!ok && !abort_flag) fail(1);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int key0 = (j0 + n) * kFaKeys;
      const int count = min(per_tile, (hi - key0 + box - 1) / box);             // boxes that hold keys below hi
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
                     ::"r"(tc5::s32(&kv_full[s])), "r"(2 * KB * count * box * 128) : "memory");
      __syncwarp();
      for (int i = lane; i < count; i += 32) {
        const int key = key0 + i * box;
        const int page = table[key / B];
        const int row = (page * p.nkv + kvh) * B + key % B;
        for (int kb = 0; kb < KB; ++kb) {
          tc5::tma_load_2d(k_s + s * kFaKvBytes + kb * kFaKvBlock + i * box * 128, &map_k, &kv_full[s], kb * 64, row);
          tc5::tma_load_2d(v_s + s * kFaKvBytes + kb * kFaKvBlock + i * box * 128, &map_v, &kv_full[s], kb * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    // ---- one thread issues the products, S one tile ahead of O:  S_0, S_1, O+=P_0 V_0, S_2, O+=P_1 V_1, ...
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc5::idesc(kFaRows, kFaKeys, false);
      constexpr uint32_t idesc_o = tc5::idesc(kFaRows, 64, true);       // one 64-wide block of V (and of O) per product
      const uint64_t dq = tc5::smem_desc(tc5::s32(q_s));
      bool ok = tc5::mbar_wait(&q_full, 0);
      if (!ok) fail(2);
      for (int n = 0; ok && n <= n_tiles && !abort_flag; ++n) {
        if (n < n_tiles) {                                     // S_n = Q K_n^T into buffer n % 2
          if (!tc5::mbar_wait(&kv_full[n % kFaStages], (n / kFaStages) & 1)) { fail(3); break; }
          if (!tc5::mbar_wait(&s_free[n & 1], ((n >> 1) & 1) ^ 1)) { fail(8); break; }     // the softmax has read S_(n-2)
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint64_t dk = tc5::smem_desc(tc5::s32(k_s + (n % kFaStages) * kFaKvBytes));
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)                      // (descriptor addresses count units of 16 bytes)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc5::mma(tmem + uint32_t((n & 1) * kFaKeys), dq + uint64_t(kb * (kFaTileBytes >> 4) + 2 * j),
                       dk + uint64_t(kb * (kFaKvBlock >> 4) + 2 * j), idesc_s, (kb > 0 || j > 0) ? 1u : 0u);
          tc5::commit(&s_full[n & 1]);
        }
        if (n >= 1) {                                          // O += P_m V_m
          const int m = n - 1;
          if (!tc5::mbar_wait(&p_full[m & 1], (m >> 1) & 1)) { fail(4); break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint64_t dp = tc5::smem_desc(tc5::s32(p_s + (m & 1) * kFaTileBytes));
          const uint32_t v_addr = tc5::s32(v_s + (m % kFaStages) * kFaKvBytes);
#pragma unroll
          for (int j = 0; j < kFaKeys / 16; ++j)               // 16 keys per step: 32 bytes along a row of P,
#pragma unroll
            for (int nb = 0; nb < KB; ++nb)                    // 16 rows down each 64-wide block of V
              tc5::mma(tmem + 128 + nb * 64, dp + uint64_t(2 * j), tc5::smem_desc(v_addr + nb * kFaKvBlock + j * 16 * 128),
                       idesc_o, (m > 0 || j > 0) ? 1u : 0u);
          tc5::commit(&p_free[m & 1]);                           // P_m has been read, O holds tile m
          tc5::commit(&kv_empty[m % kFaStages]);                 // K_m and V_m have been read
        }
      }
      tc5::commit(&o_full);                                      // everything issued is complete: O is final
    }
  } else {
    // ---- softmax and output: this thread owns query row `r` (lane r of tensor memory)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int pos = pos0 + r;                                  // rows beyond rows_here compute and store nothing
    const int first = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;   // first key of the row
    const uint32_t lane_addr = tmem + (uint32_t(quarter * 32) << 16);
    float m = -INFINITY, l = 0.f;                              // m: the maximum the row currently scales by
    for (int n = 0; n < n_tiles; ++n) {
      const bool got_s = !abort_flag && tc5::mbar_wait(&s_full[n & 1], (n >> 1) & 1);
      if (!__all_sync(0xffffffffu, got_s)) {                     // the warp stays together whatever a lane saw
        if (!abort_flag && lane == 0) fail(5);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      uint32_t v[2][32];                                       // the row's 64 scores
#pragma unroll
      for (int c = 0; c < 2; ++c) tc5::ld32(lane_addr + uint32_t((n & 1) * kFaKeys + c * 32), v[c]);
      tc5::ld_wait();
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(&s_free[n & 1]);                // S_(n+2) may be written
      const int key0 = (j0 + n) * kFaKeys;
      // the keys of this tile that the row may see: [a, b) relative to the tile
      const int a = max(first, lo) - key0, b = min(pos + 1, hi) - key0;
      // Masks are needed only where the tile touches the diagonal, the window's edge or the end of
      // the keys; for every other tile (most of a long prompt) there is none.
      const bool full = key0 + kFaKeys - 1 <= pos0 && (p.window <= 0 || key0 >= pos0 + kFaRows - p.window);
      float mx[2] = {-INFINITY, -INFINITY};
      if (full) {
        // eight chains of three-input maxima, four steps deep, instead of two chains of 32
        float part[8];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float t = fa_max3(__uint_as_float(v[c][8 * g]), __uint_as_float(v[c][8 * g + 1]), __uint_as_float(v[c][8 * g + 2]));
            t = fa_max3(t, __uint_as_float(v[c][8 * g + 3]), __uint_as_float(v[c][8 * g + 4]));
            t = fa_max3(t, __uint_as_float(v[c][8 * g + 5]), __uint_as_float(v[c][8 * g + 6]));
            part[c * 4 + g] = fmaxf(t, __uint_as_float(v[c][8 * g + 7]));
          }
        mx[0] = fmaxf(fa_max3(part[0], part[1], part[2]), part[3]);
        mx[1] = fmaxf(fa_max3(part[4], part[5], part[6]), part[7]);
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int t = c * 32 + i;
            mx[c] = (t >= a && t < b) ? fmaxf(mx[c], __uint_as_float(v[c][i])) : mx[c];
          }
      }
      const float m_tile = fmaxf(mx[0], mx[1]) * p.scale_log2;
      // renew the reference maximum only when it is far behind; O and l then move with it
      float alpha = 1.f;
      bool rescale = false;
      if (m == -INFINITY) {
        m = m_tile;                                            // nothing was added yet: no rescaling
      } else if (m_tile > m + kFaRescaleStep) {
        alpha = fa_exp2(m - m_tile);
        m = m_tile;
        rescale = true;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // O must hold tile n - 1 completely and nothing newer: the first is waited for here, the
        // second holds because O += P_n V_n is only issued after this warp has delivered P_n
        const bool got = n == 0 || (!abort_flag && tc5::mbar_wait(&p_free[(n - 1) & 1], ((n - 1) >> 1) & 1));
        if (!__all_sync(0xffffffffu, got)) {
          if (!abort_flag && lane == 0) fail(9);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        uint32_t ov[32];
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          tc5::ld32(lane_addr + uint32_t(128 + c * 32), ov);
          tc5::ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tc5::st32(lane_addr + uint32_t(128 + c * 32), ov);
        }
        tc5::st_wait();
        l *= alpha;
      }
      // The buffer of P_n was last read by O += P_(n-2) V_(n-2).  That product was issued before
      // S_n, and the commit that announced S_n completes only after everything issued before it:
      // having seen S_n, this thread may write P_n without another wait.
      const float m_use = (m == -INFINITY) ? 0.f : m;           // a row that has seen no key yet
      float sum[2] = {0.f, 0.f};
      unsigned char* rowp = p_s + (n & 1) * kFaTileBytes + r * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fa_exp2(__uint_as_float(v[c][i]) * p.scale_log2 - m_use);
            const float p1 = fa_exp2(__uint_as_float(v[c][i + 1]) * p.scale_log2 - m_use);
            sum[c] += p0 + p1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            packed[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int t = c * 32 + i;
            const float p0 = (t >= a && t < b) ? fa_exp2(__uint_as_float(v[c][i]) * p.scale_log2 - m_use) : 0.f;
            const float p1 = (t + 1 >= a && t + 1 < b) ? fa_exp2(__uint_as_float(v[c][i + 1]) * p.scale_log2 - m_use) : 0.f;
            sum[c] += p0 + p1;
            const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            packed[i / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        // 32 keys = four 16-byte chunks of row r; chunk index XOR (r % 8): the 128-byte swizzle
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c * 4 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(rowp + chunk * 16) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l += sum[0] + sum[1];
      // P_n is complete and O is rescaled: O += P_n V_n may go
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(&p_full[n & 1]);
    }
    const bool got_o = !abort_flag && tc5::mbar_wait(&o_full, 0);
    const bool all_o = __all_sync(0xffffffffu, got_o);
    if (!all_o && !abort_flag && lane == 0) fail(6);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (all_o) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + size_t(q_start + q0 + r) * p.out_stride + size_t(head) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ov[32];
        tc5::ld32(lane_addr + uint32_t(128 + c * 32), ov);       // (all lanes of the warp take part in the load)
        tc5::ld_wait();
        if (r < rows_here) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              h[i] = __floats2bfloat162_rn(__uint_as_float(ov[e * 8 + 2 * i]) * inv, __uint_as_float(ov[e * 8 + 2 * i + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + e * 8) = *reinterpret_cast<const uint4*>(h);
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  // every role ends here; after a wait that ran out, copies still in flight get time to land
  // before the shared memory is given up; tensor memory goes back
  if (abort_flag) {
    const unsigned long long t0 = tc5::now_ns();
    while (tc5::now_ns() - t0 < 100000ull) {}
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kFaTmemCols));
  }
}

// ---------------------------------------------------------------------------------- host

}  // namespace kvcm

using namespace kvcm;

// 1 if the tcgen05 prefill kernel takes these sizes: head_dim 64 or 128; pages of 8, 16, 32 or 64 keys, or a
// multiple of 64 (up to 256, the largest box).
KVCM_API int kvcm_attention_tcgen05_supports(int hd, int block_size) {
  if ((hd != 64 && hd != 128) || block_size < 8 || block_size > 256) return 0;
  return block_size <= kFaKeys ? (kFaKeys % block_size) == 0 && (block_size % 8) == 0 : (block_size % kFaKeys) == 0;
}

// q: [total_rows, >= nh*64] rows `q_stride` elements apart (16-byte aligned, q_stride % 8 == 0); the
// tiles are those of 64 query rows that the batch builder makes (tile_seq, tile_q0); the cache is
// [num_pages, nkv, block_size, 64].
KVCM_API int kvcm_attention_prefill_tcgen05_bf16(const void* q, int q_stride, int total_rows, void* out, int out_stride,
                                                 const void* k_cache, const void* v_cache, int num_pages,
                                                 const int* block_tables, int max_blocks, const int* tile_seq,
                                                 const int* tile_q0, const int* seq_q_start, const int* seq_q_len,
                                                 const int* seq_ctx_len, int tiles, int nh, int nkv, int hd,
                                                 int block_size, float scale, int window, void* stream) {
  if (tiles == 0) return 0;
  if (!kvcm_attention_tcgen05_supports(hd, block_size) || nkv <= 0 || nh % nkv) return KVCM_ERR_UNSUPPORTED;
  if ((q_stride % 8) || (out_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return KVCM_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  int rc = tc5::make_map(&mq, q, total_rows, nh * hd, q_stride, kFaRows);
  if (rc) return rc;
  const long long cache_rows = (long long)num_pages * nkv * block_size;
  const int box_rows = block_size < kFaKeys ? block_size : kFaKeys;
  rc = tc5::make_map(&mk, k_cache, cache_rows, hd, hd, box_rows);
  if (rc) return rc;
  rc = tc5::make_map(&mv, v_cache, cache_rows, hd, hd, box_rows);
  if (rc) return rc;
  PrefillTcParams p;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.seq_q_start = seq_q_start; p.seq_q_len = seq_q_len; p.seq_ctx_len = seq_ctx_len;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int KB = hd / 64;
  // 112 KB at head_dim 64 (two blocks fit an SM exactly), 192 KB at 128
  const size_t smem = size_t(KB + 2) * kFaTileBytes + size_t(2) * kFaStages * KB * kFaKvBlock;
  const dim3 grid(nh, tiles), block(kFaThreads);
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 64) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      if (e != cudaSuccess) return int(e);
      configured = true;
    }
    return pdl_launch(attn_prefill_tc_kernel<64>, grid, block, smem, s, mq, mk, mv, p);
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  return pdl_launch(attn_prefill_tc_kernel<128>, grid, block, smem, s, mq, mk, mv, p);
}

// Reads and clears the error word of the kernel (0 = no bounded wait ever ran out); else
// (code << 16) | block: 1 producer waited for a free stage, 2 Q, 3 K/V, 4 P, 5 S, 6 O; 7 shared memory
// Device address of the error word (the sampling kernels copy it out with the step's tokens).
KVCM_API const int* kvcm_attention_tcgen05_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_fa_error) == cudaSuccess ? p : nullptr;
}

// not aligned to 1,024 bytes; 8 a free buffer of S, 9 a free buffer of P.
KVCM_API int kvcm_attention_tcgen05_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fa_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_fa_error, &zero, sizeof zero);
  return v;
}
