// Matrix product for many rows (prefill) on the fifth-generation tensor cores, two SMs to a tile:
//     Y[M, N] = X[M, K] * W[N, K]^T,  bfloat16 operands, float accumulation in tensor memory.
//
// A pair of blocks (a thread-block cluster of two, on the two SMs of one pair) computes a
// 256 x BN tile of Y with tcgen05.mma.cta_group::2: each block brings 128 rows of X and BN / 2 rows
// of W per k-step into its own shared memory and the tensor cores of both SMs read both halves of
// W, so a block fetches 128 + BN / 2 rows from L2 for 128 x BN results, against 128 + BN for the
// one-SM tile (gemm_tcgen05.cu), whose 96 bytes per clock and SM are more than L2 delivers.  Each
// block keeps its 128 rows of the accumulator in its own tensor memory (two accumulators of 256
// columns: the epilogue of one tile runs while the tensor cores work on the next).  Pairs are
// persistent and take tiles pair, pair + pairs, ... of the walk.
//  * warp 0, one thread in each block: TMA of its pieces of X and W into a six-stage ring
//    (cp.async.bulk.tensor.2d.cta_group::2, completion counted on the leading block's barrier).
//  * warp 1, one thread of the leading block: tcgen05.mma (M 256, N = BN, K 16), four per k-step;
//    tcgen05.commit with a multicast arrive hands the ring slot back to both producers and, at the
//    end of a tile, tells both epilogues.
//  * warps 2-5 in each block: epilogue, tcgen05.ld of this block's 128 rows, convert, store; with
//    GATED the tile's columns are BN / 2 gate columns and the BN / 2 up columns of the same outputs
//    and the epilogue stores silu(gate) * up.
// BN is a run-time size (a multiple of 32, of 64 with GATED; up to 256, or up to 512 as two
// products side by side into one accumulator, in a four-stage ring) chosen on the host for
// the least estimated time: wide enough for L2, narrow enough that the last round of pairs is full.
// Tiles are walked row-major, or in bands of eight row tiles when W is too large to stay in L2
// (pair_tile).  When the tiles do not fill the last round of pairs, the pairs instead take equal
// shares of all (tile, k-step) units (PairWalk): a pair that starts in the middle of a tile's k
// range leaves float partial sums in a workspace, the pair that began the tile adds them in a
// fixed order in its epilogue, so the result does not depend on timing.  Rows, columns and k beyond the matrices are
// zero-filled by the TMA unit: any M, N and any K that is a multiple of 8 work.  Every wait on an
// mbarrier is bounded; when one runs out the block records it (kvcm_gemm_tcgen05_pair_error),
// stops waiting, and both blocks meet at the cluster barrier, free their tensor memory and leave.
// The reference calls cuBLAS for these products (src/model/llama.cpp:45-52).
#include "pdl.cuh"
#include "tcgen05_common.cuh"

namespace kvcm {

constexpr int kPairBM = 128;                   // rows of X per block (256 per pair)
constexpr int kPairBK = 64;
constexpr int kPairThreads = 192;
constexpr int kPairABytes = kPairBM * kPairBK * 2;
constexpr int kPairRingBytes = 192 * 1024;     // six stages of 32 KB (BN <= 256) or four of 48 KB (wider tiles)
constexpr int kPairStages = 6;                 // the most
constexpr int kPairAccCols = 256;

__device__ int g_pair_error = 0;

namespace pair {

__device__ __forceinline__ uint32_t cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
// The address of the same shared-memory object in block `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// One box into this block's shared memory; the bytes are counted on a barrier given by its
// cluster address (the leading block's).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(tc5::s32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t instr, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(da), "l"(db), "r"(instr), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both blocks of the pair when every product issued so
// far is complete.
__device__ __forceinline__ void commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(tc5::s32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(bar_cluster_addr) : "memory");
}
// Bounded wait that also acquires what another block of the cluster released.
__device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity) {
  unsigned long long start = 0;
  for (unsigned spin = 0;; ++spin) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(tc5::s32(bar)), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 63) == 63) {
      const unsigned long long now = tc5::now_ns();
      if (start == 0) start = now;
      else if (now - start > tc5::kWaitLimitNs) return false;
    }
  }
}

}  // namespace pair

// Tile t of the walk: bands of `band` row tiles, inside a band the row tiles fastest.  With a band
// of eight the pairs of one round share a few column tiles of W and the band's rows of X, so each
// piece of W comes from memory once per band even when W is larger than L2; a band of one is the
// plain row-major walk.
__device__ __forceinline__ void pair_tile(int t, int m_tiles, int n_tiles, int band_rows, int& mt, int& nt) {
  const int per_band = band_rows * n_tiles;
  const int band = t / per_band, rem = t - band * per_band;
  const int rows = min(band_rows, m_tiles - band * band_rows);
  mt = band * band_rows + rem % rows;
  nt = rem / rows;
}

// The pieces of work of one pair, in order.  Tile by tile (pair, pair + pairs, ... of the walk), or
// with `split` an equal share of all (tile, k-step) units: the pair's first piece may then start in
// the middle of a tile's k range (it leaves partial sums in a workspace) and its last may end in
// the middle of one (it collects the partial sums of the pairs after it, who made them first).
struct PairWalk {
  int nk, tiles, pairs, pair_id, tl;
  bool split;
  long long u, u1;
  __device__ PairWalk(int nk_, int tiles_, int pairs_, int pair_id_, bool split_)
      : nk(nk_), tiles(tiles_), pairs(pairs_), pair_id(pair_id_), tl(0), split(split_) {
    const long long total = (long long)tiles * nk;
    u = total * pair_id / pairs;
    u1 = total * (pair_id + 1) / pairs;
  }
  // First unit of pair q's share.
  __device__ long long first_unit(int q) const { return (long long)tiles * nk * q / pairs; }
  __device__ bool next(int& t, int& kb, int& ke) {
    if (!split) {
      t = pair_id + tl * pairs;
      if (t >= tiles) return false;
      ++tl;
      kb = 0;
      ke = nk;
      return true;
    }
    if (u >= u1) return false;
    t = int(u / nk);
    kb = int(u - (long long)t * nk);
    const long long left = u1 - u;
    ke = (nk - kb) <= left ? nk : kb + int(left);
    u += ke - kb;
    return true;
  }
};

constexpr int kPairPartFloats = 128 * kPairAccCols;      // one block's rows of one accumulator

template <typename OutT, bool GATED, bool WIDE>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         OutT* __restrict__ Y, int M, int N, int K, int ldy, int BN, int band_rows,
                         float* __restrict__ part, int* __restrict__ part_flag) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full[kPairStages], empty[kPairStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair::cta_rank();                      // 0 = the leading block of the pair
  const int pair_id = int(blockIdx.x) >> 1, pairs = int(gridDim.x) >> 1;
  const int bnout = GATED ? BN / 2 : BN;                       // output columns per tile
  constexpr int nmma = WIDE ? 2 : 1;                           // products per 16 k: the instruction takes N <= 256
  const int n_mma = BN / nmma;                                 // N of one product
  const int b_rows = n_mma / 2;                                // rows of W per block, product and k-step
  constexpr int nacc = WIDE ? 1 : 2;                           // accumulators in tensor memory
  constexpr int stage_bytes = kPairABytes + (WIDE ? 2 : 1) * kPairABytes;
  constexpr int stages = kPairRingBytes / stage_bytes;         // 6 or 4
  const int m_tiles = (M + 2 * kPairBM - 1) / (2 * kPairBM), n_tiles = (N + bnout - 1) / bnout;
  const int tiles = m_tiles * n_tiles;
  const int nk = (K + kPairBK - 1) / kPairBK;
  const bool split = part != nullptr;                          // equal shares of (tile, k-step) units

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kPairStages; ++s) {
      tc5::mbar_init(&full[s], 1);                             // the leading producer's expect_tx
      tc5::mbar_init(&empty[s], 1);                            // one commit
    }
    for (int a = 0; a < 2; ++a) {
      tc5::mbar_init(&acc_full[a], 1);
      tc5::mbar_init(&acc_empty[a], 8);                        // four epilogue warps in each block
    }
    tc5::mbar_init_fence();
  }
  if (warp == 1) {                 // the same warp in both blocks: two accumulators of 256 columns in each
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5::s32(&tmem_base)), "r"(2 * kPairAccCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
  }
  tc5::fence_before();
  __syncthreads();
  pair::cluster_sync();            // both blocks' barriers and tensor memory exist before anyone uses them
  tc5::fence_after();
  const uint32_t tmem = tmem_base;

  pdl_launch_dependents();
  pdl_wait();                      // X may come from the kernel before

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t full0 = pair::map_to_rank(tc5::s32(&full[0]), 0);
      const uint32_t stage_tx = 2u * uint32_t(kPairABytes + nmma * b_rows * kPairBK * 2);   // both blocks' bytes
      int s = 0, round = 0;                        // stage, and how often the ring has been walked
      PairWalk walk(nk, tiles, pairs, pair_id, split);
      int t, kb, ke;
      while (!abort_flag && walk.next(t, kb, ke)) {
        int mt, nt;
        pair_tile(t, m_tiles, n_tiles, band_rows, mt, nt);
        const int m0 = mt * 2 * kPairBM + int(rank) * kPairBM;
        const int n0 = nt * bnout;
        // rows of W for product j: with one product the leading block holds the left half of its
        // columns; GATED: the gate rows are the left half of the tile, the up rows the right half
        int w_row[2];
        if constexpr (GATED) {
          w_row[0] = nmma == 2 ? n0 + int(rank) * b_rows : (rank ? N + n0 : n0);
          w_row[1] = N + n0 + int(rank) * b_rows;
        } else {
          w_row[0] = n0 + int(rank) * b_rows;
          w_row[1] = n0 + n_mma + int(rank) * b_rows;
        }
        for (int k = kb; k < ke; ++k) {
          if (!tc5::mbar_wait(&empty[s], (round & 1) ^ 1)) {
            atomicExch(&g_pair_error, (1 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          if (rank == 0) tc5::mbar_expect_tx(&full[s], stage_tx);
          unsigned char* a = ring + s * stage_bytes;
          pair::tma_load_2d(a, &map_x, full0 + uint32_t(s) * 8u, k * kPairBK, m0);
#pragma unroll
          for (int j = 0; j < nmma; ++j)
            pair::tma_load_2d(a + kPairABytes + j * b_rows * kPairBK * 2, &map_w, full0 + uint32_t(s) * 8u,
                              k * kPairBK, w_row[j]);
          if (++s == stages) s = 0, ++round;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = tc5::idesc(2 * kPairBM, n_mma);
      int s = 0, round = 0;
      PairWalk walk(nk, tiles, pairs, pair_id, split);
      int t, kb, ke;
      for (int tl = 0; !abort_flag && walk.next(t, kb, ke); ++tl) {
        const int acc = tl % nacc;
        // both epilogues must have drained this accumulator (the tile that used it before)
        if (!pair::wait_cluster(&acc_empty[acc], ((tl / nacc) & 1) ^ 1)) {
          atomicExch(&g_pair_error, (4 << 16) | int(blockIdx.x & 0xffff));
          abort_flag = 1;
          break;
        }
        tc5::fence_after();
        const uint32_t d_tmem = tmem + uint32_t(acc * kPairAccCols);
        for (int k = kb; k < ke; ++k) {
          if (!tc5::mbar_wait(&full[s], round & 1)) {
            atomicExch(&g_pair_error, (2 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          tc5::fence_after();
          const uint32_t a_addr = tc5::s32(ring + s * stage_bytes);
          const uint64_t da = tc5::smem_desc(a_addr), db = tc5::smem_desc(a_addr + kPairABytes);
#pragma unroll
          for (int h = 0; h < nmma; ++h) {
            const uint64_t dbh = db + uint64_t((h * b_rows * kPairBK * 2) >> 4);
#pragma unroll
            for (int j = 0; j < kPairBK / 16; ++j)
              pair::mma(d_tmem + uint32_t(h * n_mma), da + uint64_t(2 * j), dbh + uint64_t(2 * j), idesc,
                        (k > kb || j > 0) ? 1u : 0u);
          }
          pair::commit_both(&empty[s]);           // the slot is free in both blocks once these have read it
          if (++s == stages) s = 0, ++round;
        }
        if (abort_flag) break;
        pair::commit_both(&acc_full[acc]);
      }
    }
  } else {
    // ---- epilogue: this warp reads lanes 32*(warp % 4) .. +31 of this block's accumulator
    const int quarter = warp & 3;
    const uint32_t acc_empty0 = pair::map_to_rank(tc5::s32(&acc_empty[0]), 0);
    // Partial sums of a piece that does not start its tile's k range: slot (pair, block), laid out
    // [chunk of 32 columns][quarter][column in chunk][lane] so that a warp writes and reads whole
    // lines; one flag per (pair, block, quarter): 1 = written, put back to 0 by the reader.
    const size_t part_slot = (size_t(pair_id) * 2 + rank) * kPairPartFloats;
    PairWalk walk(nk, tiles, pairs, pair_id, split);
    int t, kb, ke;
    for (int tl = 0; walk.next(t, kb, ke); ++tl) {
      const int acc = tl % nacc;
      int mt, nt;
      pair_tile(t, m_tiles, n_tiles, band_rows, mt, nt);
      const int m0 = mt * 2 * kPairBM + int(rank) * kPairBM, n0 = nt * bnout;
      if (abort_flag || !tc5::mbar_wait(&acc_full[acc], (tl / nacc) & 1)) {
        if (!abort_flag && lane == 0) atomicExch(&g_pair_error, (3 << 16) | int(blockIdx.x & 0xffff));
        abort_flag = 1;
        break;
      }
      tc5::fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(acc * kPairAccCols);
      if (kb > 0) {
        // the later part of a tile's k range: leave the sums for the pair that began the tile
        float* dst = part + part_slot + size_t(quarter) * 1024 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tc5::ld32(tbase + uint32_t(c * 32), v);
          tc5::ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[size_t(c) * 4096 + i * 32] = __uint_as_float(v[i]);
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          int* flag = part_flag + (pair_id * 2 + int(rank)) * 4 + quarter;
          asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(flag), "r"(1) : "memory");
        }
      } else {
        // which pairs hold the rest of this tile's k range (none unless this piece ends early)
        int q_end = pair_id + 1;
        if (ke < nk)
          while (q_end < pairs && walk.first_unit(q_end) < (long long)(t + 1) * nk) ++q_end;
        int have_parts = 1;
        if (lane == 0) {
          for (int q = pair_id + 1; q < q_end && have_parts; ++q) {
            const int* flag = part_flag + (q * 2 + int(rank)) * 4 + quarter;
            unsigned long long start = 0;
            for (unsigned spin = 0;; ++spin) {
              int f;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(f) : "l"(flag) : "memory");
              if (f == 1) break;
              if ((spin & 63) == 63) {
                const unsigned long long now = tc5::now_ns();
                if (start == 0) start = now;
                else if (now - start > tc5::kWaitLimitNs) { have_parts = 0; break; }
              }
            }
          }
        }
        have_parts = __shfl_sync(0xffffffffu, have_parts, 0);
        if (!have_parts) {
          if (lane == 0) atomicExch(&g_pair_error, (5 << 16) | int(blockIdx.x & 0xffff));
          abort_flag = 1;
          break;
        }
        // The partial sums of a chunk of 32 columns are fetched one chunk ahead (a round trip to
        // L2 takes about as long as a chunk's other work) and added in the order of the pairs.
        const bool parts = q_end > pair_id + 1;
        constexpr int kFetch = GATED ? 2 : 1;                  // chunks of the accumulator per chunk of output
        float pnext[kFetch][32];
        auto fetch = [&](int c) {
          if (!parts || c >= bnout / 32) return;
#pragma unroll
          for (int h = 0; h < kFetch; ++h) {
            const int chunk = c + h * (bnout >> 5);
            const float* src = part + (size_t(pair_id + 1) * 2 + rank) * kPairPartFloats + size_t(chunk) * 4096 +
                               size_t(quarter) * 1024 + lane;
#pragma unroll
            for (int i = 0; i < 32; ++i) pnext[h][i] = __ldcg(src + i * 32);
            for (int q = pair_id + 2; q < q_end; ++q) {
              src += 2 * kPairPartFloats;
#pragma unroll
              for (int i = 0; i < 32; ++i) pnext[h][i] += __ldcg(src + i * 32);
            }
          }
        };
        fetch(0);
#pragma unroll 1
        for (int c = 0; c < bnout / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;                                  // warp-uniform
          float pcur[kFetch][32];
          if (parts) {
#pragma unroll
            for (int h = 0; h < kFetch; ++h)
#pragma unroll
              for (int i = 0; i < 32; ++i) pcur[h][i] = pnext[h][i];
            fetch(c + 1);
          }
          if constexpr (GATED) {
            uint32_t g[32], u[32];
            tc5::ld32(tbase + uint32_t(c * 32), g);
            tc5::ld32(tbase + uint32_t(bnout + c * 32), u);
            tc5::ld_wait();
            if (parts) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                g[i] = __float_as_uint(__uint_as_float(g[i]) + pcur[0][i]);
                u[i] = __float_as_uint(__uint_as_float(u[i]) + pcur[kFetch - 1][i]);
              }
            }
            if (row < M) {
              bf16* dst = reinterpret_cast<bf16*>(Y) + size_t(row) * ldy + col0;
              __nv_bfloat162 h2[16];
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const float xa = Store<bf16>::round(__uint_as_float(g[i])), xb = Store<bf16>::round(__uint_as_float(u[i]));
                const float sl = Store<bf16>::round(xa / (1.f + expf(-xa)));
                const bf16 y = __float2bfloat16_rn(sl * xb);
                if (i & 1) h2[i / 2].y = y; else h2[i / 2].x = y;
              }
              if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(h2)[i];
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < N) dst[i] = (i & 1) ? h2[i / 2].y : h2[i / 2].x;
              }
            }
          } else {
            uint32_t v[32];
            tc5::ld32(tbase + uint32_t(c * 32), v);
            tc5::ld_wait();
            if (parts) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + pcur[0][i]);
            }
            if (row < M) {
              OutT* dst = Y + size_t(row) * ldy + col0;
              if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                if constexpr (sizeof(OutT) == 2) {
                  uint4 packed[4];
                  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
                  for (int i = 0; i < 16; ++i) h2[i] = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
#pragma unroll
                  for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = packed[i];
                } else {
#pragma unroll
                  for (int i = 0; i < 8; ++i)
                    reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (col0 + i < N) stf(dst + i, __uint_as_float(v[i]));
              }
            }
          }
        }
        // the partial sums have been read: their slots are free for the next launch
        if (parts) {
          __syncwarp();
          if (lane == 0)
            for (int q = pair_id + 1; q < q_end; ++q) part_flag[(q * 2 + int(rank)) * 4 + quarter] = 0;
        }
      }
      // this warp has read its lanes of the accumulator: tell the leading block's tensor-core thread
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) pair::arrive_remote(acc_empty0 + uint32_t(acc) * 8u);
    }
  }
  // every role ends here; neither block leaves (or frees tensor memory) while the other may still
  // reach into it
  tc5::fence_before();
  __syncthreads();
  pair::cluster_sync();
  if (warp == 1) {
    tc5::fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * kPairAccCols));
  }
}

// ---------------------------------------------------------------------------------- host

constexpr size_t kPairSmem = size_t(kPairRingBytes) + 1024;
constexpr long long kPairWInL2 = 64ll << 20;   // a W up to this size stays in L2 between row tiles

// How many pairs of blocks the device runs at a time (74 on a full B200); 0 if it cannot be asked.
template <typename Kernel>
int pair_capacity(Kernel kernel) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// The tile width (accumulator columns) and the kind of walk with the least estimated time, among
// widths whose products are multiples of 64 columns (the tensor cores take a narrower one in the
// same time).  Per k-step a tile costs the larger of the tensor cores' time (2 clocks per column)
// and the time to bring its operands from L2 (measured: about a clock per row and half-column, at
// least 420); tiles wider than 256 columns fill tensor memory, so their epilogue (about 12 clocks
// per column) is not hidden behind the next tile.  Equal shares of (tile, k-step) units of 256-wide
// tiles cost their k-steps, the epilogue, and the partial sums written and read.
struct PairPlan {
  int bn;
  bool split;
};
inline PairPlan pair_plan(int M, int N, int K, int pairs, bool gated, bool may_split) {
  const long long m_tiles = (M + 2 * kPairBM - 1) / (2 * kPairBM);
  const long long nk = (K + kPairBK - 1) / kPairBK;
  const int widths[5] = {256, 512, 384, 192, 128};
  double best_cost = -1;
  PairPlan best = {256, false};
  for (int bn : widths) {
    const int bnout = gated ? bn / 2 : bn;
    const long long tiles = m_tiles * ((N + bnout - 1) / bnout);
    const double rounds = double((tiles + pairs - 1) / pairs);
    double l2 = 256.0 + bn;
    if (l2 < 420.0) l2 = 420.0;
    const double tc = 2.0 * bn;
    const double per_k = bn > 256 ? tc : (tc > l2 ? tc : l2);
    const double epi = 12.0 * bn;
    const double cost = rounds * nk * per_k + (bn > 256 ? rounds * epi : epi);
    if (best_cost < 0 || cost < best_cost * 0.98) best_cost = cost, best = {bn, false};
    if (bn == 256 && may_split && tiles * nk >= pairs) {
      // a pair's share of k-steps, its epilogue, one partial sum written (about 4,000 clocks at an
      // SM's bandwidth to L2) and those of the tile's other pairs read
      const double share = double((tiles * nk + pairs - 1) / pairs);
      const double others = share >= nk ? 1.0 : double(nk) / share;
      const double cost_split = share * per_k + epi + 4000.0 * (1.0 + others);
      if (cost_split < best_cost * 0.95) best_cost = cost_split, best = {bn, true};
    }
  }
  return best;
}

// GATED: N is the number of output columns; W has 2N rows.  bn: 0 = choose.
template <typename OutT, bool GATED, bool WIDE>
int launch_pair_as(const CUtensorMap& mx, const CUtensorMap& mw, void* Y, int M, int N, int K, int ldy, int bn, int band,
                   int grid_pairs, float* part, int* part_flag, cudaStream_t s) {
  auto kernel = gemm_tcgen05_pair_kernel<OutT, GATED, WIDE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  return pdl_launch_cluster(kernel, dim3(2 * grid_pairs), dim3(kPairThreads), kPairSmem, s, 2, mx, mw,
                            reinterpret_cast<OutT*>(Y), M, N, K, ldy, bn, band, part, part_flag);
}

// The workspace of the split walk: partial sums and flags of `slots` pairs (see the kernel).
struct PairWorkspace {
  float* part;
  int* flag;
  int slots;
};

template <typename OutT, bool GATED>
int pair_capacity_of() {
  static int pairs = -1;
  if (pairs < 0) {
    auto kernel = gemm_tcgen05_pair_kernel<OutT, GATED, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmem)) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    pairs = pair_capacity(kernel);
  }
  return pairs;
}

// bn, band: 0 = chosen here.  split: -1 = chosen here, 0 = tile by tile, 1 = equal shares of k-steps.
template <typename OutT, bool GATED>
int launch_pair(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy, int bn,
                int band, int split, PairWorkspace ws, cudaStream_t s) {
  const int pairs = pair_capacity_of<OutT, GATED>();
  if (pairs <= 0) return KVCM_ERR_UNSUPPORTED;
  const bool have_ws = ws.part != nullptr && ws.flag != nullptr && ws.slots >= pairs;
  if (split == 1 && (!have_ws || bn > 256)) return KVCM_ERR_UNSUPPORTED;
  if (bn == 0) {
    const PairPlan plan = pair_plan(M, N, K, pairs, GATED, have_ws && split != 0);
    bn = plan.bn;
    if (split < 0) split = plan.split;
    else if (split == 1) bn = 256;
  }
  if (split < 0) split = 0;
  if (bn < 32 || bn > 512 || bn % (GATED ? 64 : 32) || (split && bn > 256)) return KVCM_ERR_UNSUPPORTED;
  if (band == 0) band = (long long)(GATED ? 2 * N : N) * K * 2 > kPairWInL2 ? 8 : 1;
  if (band < 1) return KVCM_ERR_UNSUPPORTED;
  CUtensorMap mx, mw;
  int rc = tc5::make_map(&mx, X, M, K, ldx, kPairBM);
  if (rc) return rc;
  rc = tc5::make_map(&mw, W, GATED ? 2 * N : N, K, ldw, bn > 256 ? bn / 4 : bn / 2);   // one product's rows per block
  if (rc) return rc;
  const int bnout = GATED ? bn / 2 : bn;
  const long long tiles = (long long)((M + 2 * kPairBM - 1) / (2 * kPairBM)) * ((N + bnout - 1) / bnout);
  const long long units = split ? tiles * ((K + kPairBK - 1) / kPairBK) : tiles;   // every pair gets at least one
  const int grid_pairs = int(units < pairs ? units : pairs);
  float* part = split ? ws.part : nullptr;
  int* flag = split ? ws.flag : nullptr;
  return bn > 256 ? launch_pair_as<OutT, GATED, true>(mx, mw, Y, M, N, K, ldy, bn, band, grid_pairs, part, flag, s)
                  : launch_pair_as<OutT, GATED, false>(mx, mw, Y, M, N, K, ldy, bn, band, grid_pairs, part, flag, s);
}

inline bool pair_operands_ok(const void* X, const void* W, int M, int N, int K, int ldx, int ldw) {
  return M >= 1 && N >= 1 && K >= 8 && (K % 8) == 0 && (ldx % 8) == 0 && (ldw % 8) == 0 &&
         (reinterpret_cast<uintptr_t>(X) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_gemm_tcgen05_pair_supports(int M, int N, int K, int ldx, int ldw) {
  return M >= 1 && N >= 1 && K >= 8 && (K % 8) == 0 && (ldx % 8) == 0 && (ldw % 8) == 0;
}

// How many pairs of blocks run at a time (the workspace of the split walk holds as many slots), and
// the sizes of a slot: floats of partial sums, flags.
KVCM_API int kvcm_gemm_tcgen05_pair_capacity(void) { return pair_capacity_of<bf16, false>(); }
KVCM_API int kvcm_gemm_tcgen05_pair_slot_floats(void) { return 2 * kPairPartFloats; }
KVCM_API int kvcm_gemm_tcgen05_pair_slot_flags(void) { return 8; }

// out_f32: 0 = bfloat16 result, 1 = float result.  bn: tile width (multiple of 32 up to 512),
// band: row tiles walked together (1 = row-major walk); 0 = chosen here.  split: 1 = the pairs take
// equal shares of all (tile, k-step) units and add partial sums through the workspace (`part`:
// slots x slot_floats floats, `part_flag`: slots x slot_flags zeroed ints, both private to the
// stream), 0 = tile by tile, -1 = chosen here.
KVCM_API int kvcm_gemm_tcgen05_pair_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                         int ldy, int out_f32, int bn, int band, int split, void* part,
                                         void* part_flag, int slots, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!pair_operands_ok(X, W, M, N, K, ldx, ldw)) return KVCM_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const PairWorkspace ws = {static_cast<float*>(part), static_cast<int*>(part_flag), slots};
  return out_f32 ? launch_pair<float, false>(X, W, Y, M, N, K, ldx, ldw, ldy, bn, band, split, ws, s)
                 : launch_pair<bf16, false>(X, W, Y, M, N, K, ldx, ldw, ldy, bn, band, split, ws, s);
}

// act[M, I] = silu(X Wg^T) * (X Wu^T) with Wg, Wu the halves of W [2I, K] (gate rows first), the
// roundings of the separate product and activation kernels; bfloat16.  bn: accumulator columns per
// tile (multiple of 64 up to 512: half of them gate, half up); the other arguments as above.
KVCM_API int kvcm_gate_up_silu_tcgen05_pair_bf16(const void* X, const void* W, void* Y, int M, int I, int K, int ldx,
                                                 int ldw, int ldy, int bn, int band, int split, void* part,
                                                 void* part_flag, int slots, void* stream) {
  if (M == 0 || I == 0) return 0;
  if (!pair_operands_ok(X, W, M, I, K, ldx, ldw)) return KVCM_ERR_UNSUPPORTED;
  const PairWorkspace ws = {static_cast<float*>(part), static_cast<int*>(part_flag), slots};
  return launch_pair<bf16, true>(X, W, Y, M, I, K, ldx, ldw, ldy, bn, band, split, ws, (cudaStream_t)stream);
}

// Device address of the error word (the sampling kernels copy it out with the step's tokens).
KVCM_API const int* kvcm_gemm_tcgen05_pair_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_pair_error) == cudaSuccess ? p : nullptr;
}

// Reads and clears the error word (0 = no bounded wait ever ran out).  Synchronises the device.
KVCM_API int kvcm_gemm_tcgen05_pair_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_pair_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_pair_error, &zero, sizeof zero);
  return v;
}
