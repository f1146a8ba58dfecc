// Weight-streaming matrix product for a handful of rows (decode), TMA-pipelined:
//     Y[M, N] = X[M, K] * W[N, K]^T,   M <= 16, bfloat16 operands, float accumulation.
//
// With so few rows the product is bound by reading W once from HBM, and HBM only delivers its
// bandwidth with megabytes in flight.  So W is not loaded by the computing threads at all: one
// producer thread per block issues bulk asynchronous copies (cp.async.bulk, completion on an
// mbarrier) of [16 rows x chunk k] pieces of W into a ring of shared-memory stages ahead of the
// consumers (as many as shared memory holds: 100-190 KB in flight per SM), and keeps issuing across
// tile boundaries.  The chunk is the whole row where K <= 2048: a copy of a whole 4 KB row next to
// its neighbours streams a quarter faster than 2 KB pieces of rows (measured: 46 MB in 10.4 us
// against 14.4 us).  Eight consumer warps take the tensor-
// core product (m16n8k16, "swap AB": 16 rows of W are the 16-row operand, the batch rows are the
// 8 columns) out of the ring, each warp one eighth of a stage along k; their partial sums are
// added in warp order per tile, so results are reproducible bit for bit.
//  * Blocks are persistent: block b takes tiles b, b + grid, ...; the grid is about one block
//    per SM so that the ring of every SM stays full.
//  * Launched as a programmatic dependent: the producer fills the whole ring BEFORE the kernel
//    waits for its predecessor (weights are constants), so HBM streams while the previous kernel
//    still runs; X (which the predecessor wrote) is staged after the wait, by every warp for the
//    columns it multiplies itself, so that no warp waits for another before its first product.
//    What else does not depend on the predecessor is done before the wait too: the padding rows
//    of X, the rotary angles' sines and cosines, the rows' cache slots.
//  * One warp per scheduler running code once gets through an instruction in about ten cycles, so
//    what stands between the wait and the last store is kept short: slots, phases, chunks and tiles
//    are counted along, never derived by division, and loops have forms without bounds checks.
//  * Every wait on an mbarrier is bounded; a wait that runs out sets an error word that the host
//    reads (kvcm_stream_error), lets copies in flight land and leaves.
//  * Where every block has one tile only and K is long (the feed-forward's down projection), X is
//    not staged in shared memory at all: no element of X is used twice by a block then, so the
//    consumers read their pieces of X from L2 straight into registers, one stage ahead, and the
//    ring gets the whole of shared memory (the block's entire tile of W is in flight at once).
//  * The residual stream and its norm can ride along (a decode layer then has no norm launches).
//    A norm is out = w * x * r with r = rsqrt(mean(x^2) + eps) one number per row, so r can be
//    applied after the product that consumes the normed row: (W (w * x)) * r.  The products that
//    end a sublayer (attention output, feed-forward down) add their result into the float residual
//    themselves, write bfloat16(w * x_new) for the product that follows and, per tile of 16 columns
//    and row, the sum of squares of x_new (kResidual); the products that begin the next sublayer
//    add those partial sums up in a fixed order while their weights stream and scale their float
//    sums by r before the epilogue (SCALED).  One rounding of the normed row instead of two.
// The k index inside a 32-wide block is permuted identically for both operands (thread t of a
// quad owns k = 8t..8t+7), which makes every shared-memory read of W and X a 16-byte vector.
// The reference calls cuBLAS here (src/model/llama.cpp:45-52).
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

constexpr int kStreamConsumers = 8;                    // consumer warps
constexpr int kStreamThreads = 32 * (kStreamConsumers + 1);
constexpr int kMaxStages = 12;                         // ring depth is chosen per launch to fill shared memory
constexpr int kChunkUnit = 256;                        // the k elements of a stage are a multiple of this
constexpr int kChunkLong = 2048, kChunkShort = 1024;   // whole rows up to 2048 k; else pieces of 1024 k
// X straight from L2 (XDIRECT): a stage's pieces of X live in registers, so the stage is as long as
// the registers allow (a bulk copy costs its issuer some 60 ns whatever its size: fewer, larger
// copies keep the producer ahead)
__host__ __device__ constexpr int direct_chunk(int MT) { return kChunkShort; }
constexpr int kRowPad = 64;                            // padded stage row: rows g and g+1 sit 64 bytes apart modulo 128,
                                                       // so the eight lanes of a quarter-warp (two rows x four 16-byte
                                                       // columns) read eight distinct bank groups
constexpr int kXPad = 32;                              // the same for the staged X (elements)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // every wait gives up after two seconds

__device__ int g_stream_error = 0;                     // 0 = ok; else (code << 16) | block
// For tests of the failure path only: the wait limit in force, and a stage (index in a block's
// sequence of copies) whose copy is left out, so that its consumers wait for bytes that never come.
__device__ unsigned long long g_stream_wait_limit_ns = kWaitLimitNs;
__device__ int g_stream_skip_stage = -1;

// What happens to a finished tile of 16 output columns x M rows.
//  kStore    : y[m][n] = sum.
//  kRopeCache: the 16 weight rows of a tile are 8 rows j..j+7 of a head and their rotary partners
//              j + hd/2 .. (so one thread owns both halves of each pair): the sums are rounded to
//              bfloat16 as the plain product would store them, q and k heads are rotated by
//              position * inv_freq[j] (float sin/cos), q goes to y, k (rotated) and v go straight
//              into the row's cache page slot.  Bit-for-bit what the separate product + rotary +
//              cache-write kernels produce.
//  kSiluMul  : the 16 weight rows are 8 gate rows i..i+7 and the 8 up rows I+i..: y[m][i] =
//              round(round(silu(round(gate))) * round(up)), as the separate activation kernel.
//  kResidual : resid[m][n] += round(sum) (the float residual stream, in place; the sum rounded to
//              bfloat16 as the plain product would store it), ss_out[tile][m] = the sum over the
//              tile's 16 columns of the new resid[m][n]^2 (what the next norm needs of this tile),
//              and h_out[m][n] = bfloat16(next_w[n] * resid[m][n]): the next norm's row before its
//              scale (left out where next_w is null).
enum StreamEpilogue { kStore = 0, kRopeCache = 1, kSiluMul = 2, kResidual = 3 };
constexpr int kNormRows = 16;                          // row stride of the partial sums of squares

struct StreamParams {
  const bf16* W; int N, K, ldw;
  const bf16* X; int ldx, M;
  void* Y; int ldy;
  int stages;                                          // ring depth (1..kMaxStages)
  int chunk;                                           // k elements per stage (a multiple of kChunkUnit)
  // rows of tile t: first 8 = (t / pair_blocks) * group_stride + 8 * (t % pair_blocks) + r,
  //                 last 8 = those + pair_offset
  int pair_blocks, group_stride, pair_offset;
  // kRopeCache
  const int* positions; const float* inv_freq; const int* slot_mapping;
  bf16* k_cache; bf16* v_cache;
  int nh, nkv, hd, block_size;
  // kResidual
  float* resid; int ldr; float* ss_out; bf16* h_out; int ldh; const bf16* next_w;
  // SCALED: the sums of row m are multiplied by rsqrt(sum over t of ss_in[t][m] / K + eps) before the
  // epilogue (ss_in [ss_tiles][kNormRows] as kResidual leaves it)
  const float* ss_in; int ss_tiles; float eps;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait for the phase with the given parity.  False = gave up after kWaitLimitNs.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  unsigned long long start = 0;
  for (unsigned spin = 0;; ++spin) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(s32(bar)), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 63) == 63) {
      const unsigned long long now = global_ns();
      if (start == 0) start = now;
      else if (now - start > limit_ns) return false;
    }
  }
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(bar)) : "memory");
}

__device__ __forceinline__ void mma_stream(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_wait_dyn(int n) {       // wait until at most n groups are pending
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;\n" ::); break;
    case 1: asm volatile("cp.async.wait_group 1;\n" ::); break;
    case 2: asm volatile("cp.async.wait_group 2;\n" ::); break;
    case 3: asm volatile("cp.async.wait_group 3;\n" ::); break;
    case 4: asm volatile("cp.async.wait_group 4;\n" ::); break;
    case 5: asm volatile("cp.async.wait_group 5;\n" ::); break;
    case 6: asm volatile("cp.async.wait_group 6;\n" ::); break;
    default: asm volatile("cp.async.wait_group 7;\n" ::); break;
  }
}

template <int MT, typename OutT, int EPI, bool XDIRECT, bool SCALED = false>
__global__ void __launch_bounds__(kStreamThreads)
gemm_stream_kernel(StreamParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int kConsumerThreads = 32 * kStreamConsumers;
  constexpr int MB = MT * 8;                                  // batch rows held (padded)
  const int kChunk = p.chunk;
  const int kRowBytes = kChunk * 2 + kRowPad, kStageBytes = 16 * kRowBytes;
  const int Kc = (p.K + kChunk - 1) / kChunk;                 // stages per tile
  const int Kp = XDIRECT ? 0 : Kc * kChunk + kXPad;            // padded row of the staged X
  const int kStages = p.stages;
  unsigned char* ring = smem_raw;                             // [stages][16][kRowBytes]
  bf16* xs = reinterpret_cast<bf16*>(ring + kStages * kStageBytes);          // [MB][Kp]
  float* red = reinterpret_cast<float*>(xs + MB * Kp);                       // [2][warps][16][MB]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * kStreamConsumers * 16 * MB);
  uint64_t* empty = full + kMaxStages;
  __shared__ volatile int abort_flag;
  __shared__ float norm_s[16];                                // SCALED: 1/rms per row

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_tiles = (p.N + 15) / 16;
  const int my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int total = my_tiles * Kc;                            // stages this block consumes

  if (tid == 0) abort_flag = 0;
  if (tid < kStages) {                                        // a barrier pair a thread
    mbar_init(&full[tid], 1);
    mbar_init(&empty[tid], kStreamConsumers);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  // Weight row of local row r (0..15) of a tile whose first row is `base`.  (A lone warp runs cold
  // code at some ten cycles an instruction, so what is on the way of every stage or tile is kept
  // free of divisions: slots, phases, chunks and tiles are counted along, not derived.)
  auto tile_base = [&](int tile) {
    const int q = tile / p.pair_blocks;
    return q * p.group_stride + 8 * (tile - q * p.pair_blocks);
  };
  auto row_in = [&](int base, int r) { return r < 8 ? base + r : base + p.pair_offset + (r - 8); };

  // Producer warp: lane 0 announces the bytes of a stage, lanes 0..15 each copy one row of it
  // (sixteen copies issued side by side).  Stage i holds rows of tile (i / Kc) at k-chunk (i % Kc).
  const unsigned long long wait_limit = g_stream_wait_limit_ns;
  const int skip_stage = g_stream_skip_stage;
  if (warp == kStreamConsumers) {
    int issued = 0, slot = 0, round = 0, kc = 0, tile = blockIdx.x;        // the stage to issue next
    const bf16* row_ptr = nullptr;                                         // this lane's row of W in `tile`
    uint32_t live_rows = 0;
    auto enter_tile = [&]() {
      const int row = lane < 16 ? row_in(tile_base(tile), lane) : p.N;
      row_ptr = row < p.N ? p.W + size_t(row) * p.ldw : nullptr;
      live_rows = uint32_t(__popc(__ballot_sync(0xffffffffu, row_ptr != nullptr)));
    };
    auto issue = [&]() {
      if (issued != skip_stage) {                                          // (tests: the bytes of this stage never arrive)
        const int k0 = kc * kChunk;
        const int kbytes = min(kChunk, p.K - k0) * 2;
        if (lane == 0) mbar_expect_tx(&full[slot], live_rows * kbytes);
        __syncwarp();
        if (row_ptr != nullptr) bulk_copy(ring + slot * kStageBytes + lane * kRowBytes, row_ptr + k0, kbytes, &full[slot]);
      }
      ++issued;
      if (++slot == kStages) { slot = 0; ++round; }
      if (++kc == Kc) {
        kc = 0;
        tile += gridDim.x;
        if (issued < total) enter_tile();
      }
    };
    if (total > 0) enter_tile();
    const int first = min(total, kStages);
    while (issued < first) issue();                                        // fill the ring: weights are constants
    pdl_wait();                                                             // (nothing below reads what the predecessor wrote)
    while (issued < total) {
      int ok = 1;
      if (lane == 0) {
        ok = !abort_flag && mbar_wait(&empty[slot], (round - 1) & 1, wait_limit);   // consumers freed the slot?
        if (!ok && !abort_flag) {
          atomicExch(&g_stream_error, (1 << 16) | int(blockIdx.x));
          abort_flag = 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      issue();
    }
    // Stay until every copy this block issued has landed (shared memory must not be handed to
    // another block with copies still in flight).  Immediate in a healthy run: the consumers
    // have already seen these phases complete.
    if (lane == 0)
      for (int s = 0; s < kStages; ++s) {
        const int fills = issued > s ? (issued - s - 1) / kStages + 1 : 0;
        if (fills > 0) mbar_wait(&full[s], (fills - 1) & 1, wait_limit / 4);
      }
    return;
  }
  // Rotary encoding: the angle's sine and cosine for this thread's element of the block's first
  // tile, before the wait (positions and frequencies are inputs of the step, not of the predecessor).
  float cs0 = 1.f, sn0 = 0.f;
  int slot0 = -1;                                       // ... and the row's slot in the cache pages, for k and v heads
  if constexpr (EPI == kRopeCache) {
    if (my_tiles > 0 && tid < 8 * MB) {
      const int m = tid >> 3, pr = tid & 7;                    // (the epilogue's mapping: a row's 8 pairs side by side)
      const int q = int(blockIdx.x) / p.pair_blocks;
      const int j = 8 * (int(blockIdx.x) - q * p.pair_blocks) + pr;
      if (q < p.nh + p.nkv && m < p.M) sincosf(float(p.positions[m]) * p.inv_freq[j], &sn0, &cs0);
      if (q >= p.nh && m < p.M) slot0 = p.slot_mapping[m];
    }
  }
  // Rows of the staged X beyond M are zero: written here, before the wait, so that the copies after
  // it are those of live rows only.
  if constexpr (!XDIRECT) {
    const int row_vecs = Kp / 8;                                             // (Kp is a multiple of 8)
    for (int c = tid + p.M * row_vecs; c < MB * row_vecs; c += kConsumerThreads)
      *reinterpret_cast<uint4*>(xs + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads));             // (before the wait: it costs nothing there)
  }
  pdl_wait();                                                               // ... the predecessor wrote X

  // ---- consumers.  X is staged k-chunk by k-chunk (one copy group each, zero fill beyond K), so
  // the first tile can start on chunk 0 while the later chunks are still arriving.  Every warp
  // copies the columns of a chunk that it multiplies itself (an eighth): it waits for its own
  // copies and for no other warp.
  const int chunk_vecs = kChunk / 8;                          // (a multiple of 32)
  if constexpr (!XDIRECT) {
    const int warp_vecs = chunk_vecs / kStreamConsumers;
    for (int kc = 0; kc < Kc; ++kc) {
      for (int v = lane; v < warp_vecs; v += 32) {
        const int ch = kc * chunk_vecs + warp * warp_vecs + v;
        const bool kin = ch * 8 < p.K;
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          if (m >= p.M) break;                                 // (zero already)
          const bf16* src = kin ? p.X + size_t(m) * p.ldx + ch * 8 : p.X;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s32(xs + m * Kp + ch * 8)), "l"(src), "r"(kin ? 16 : 0));
        }
      }
      asm volatile("cp.async.commit_group;\n" ::);
    }
  }
  // SCALED: the partial sums of squares of this warp's rows (row warp, and warp + 8 of sixteen) are
  // asked for behind X and added up after the main loop, so that nothing waits for them here.
  constexpr int kPartRegs = 8;                                 // 32 x 8 tiles of 16 columns: hidden sizes to 4,096 without a loop
  float part[SCALED ? MT : 1][SCALED ? kPartRegs : 1];
  if constexpr (SCALED) {
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int m = warp + kStreamConsumers * j;
#pragma unroll
      for (int i = 0; i < kPartRegs; ++i) {
        const int t = lane + 32 * i;
        part[j][i] = (m < p.M && t < p.ss_tiles) ? __ldcg(p.ss_in + t * kNormRows + m) : 0.f;
      }
    }
  }

  const int g = lane >> 2, t4 = lane & 3;
  const int kPerWarp = kChunk / kStreamConsumers;              // k columns of a stage per warp (a multiple of 32)
  // XDIRECT: this thread's pieces of X for one stage (kXBlocks k-blocks of 32), zero beyond M and K.
  constexpr int kXBlocks = direct_chunk(MT) / kStreamConsumers / 32;
  uint4 xcur[XDIRECT ? MT : 1][XDIRECT ? kXBlocks : 1], xnext[XDIRECT ? MT : 1][XDIRECT ? kXBlocks : 1];
  auto fetch_x = [&](uint4 (&dst)[XDIRECT ? MT : 1][XDIRECT ? kXBlocks : 1], int kc) {
#pragma unroll
    for (int j = 0; j < (XDIRECT ? MT : 1); ++j)
#pragma unroll
      for (int kb = 0; kb < (XDIRECT ? kXBlocks : 1); ++kb) {
        const int m = 8 * j + g, k = kc * kChunk + warp * kPerWarp + kb * 32 + 8 * t4;
        dst[j][kb] = (kc < Kc && m < p.M && k < p.K) ? __ldcg(reinterpret_cast<const uint4*>(p.X + size_t(m) * p.ldx + k))
                                                      : make_uint4(0u, 0u, 0u, 0u);
      }
  };
  if constexpr (XDIRECT) fetch_x(xcur, 0);
  int slot = 0;
  uint32_t phase = 0;                                          // of the stage to consume next
  for (int tl = 0; tl < my_tiles; ++tl) {
    const int tile = blockIdx.x + tl * gridDim.x;
    const int base = tile_base(tile);
    float acc[MT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    // kResidual: this thread's element of the residual (it has one: 16 x MB <= the consumer
    // threads), asked for now and used in the epilogue
    float resid_old = 0.f, next_w_mine = 0.f;
    if constexpr (EPI == kResidual) {
      if (tid < 16 * MB) {
        const int m = tid >> 4, r = tid & 15;                  // (the epilogue's mapping: a row's 16 columns side by side)
        const int n = row_in(base, r);
        if (n < p.N && m < p.M) {
          resid_old = __ldcg(p.resid + size_t(m) * p.ldr + n);
          if (p.next_w != nullptr) next_w_mine = ldf(p.next_w + n);
        }
      }
    }
    for (int kc = 0; kc < Kc; ++kc) {
      if constexpr (XDIRECT) {
        fetch_x(xnext, kc + 1);                                // in flight while this stage is worked on
      } else if (tl == 0) {                                    // this warp's columns of the chunk have landed?
        cp_async_wait_dyn(min(Kc - 1 - kc, 7));
        __syncwarp();
      }
      const int s = slot;
      if (!abort_flag && !mbar_wait(&full[s], phase, wait_limit)) {
        if (lane == 0) atomicExch(&g_stream_error, (2 << 16) | int(blockIdx.x));
        abort_flag = 1;                                        // everyone stops waiting, nobody leaves a barrier alone
      }
      if (++slot == kStages) { slot = 0; phase ^= 1u; }
      if (abort_flag) continue;
      const unsigned char* st = ring + s * kStageBytes;
      const int kbase = kc * kChunk + warp * kPerWarp;          // this warp's share of the stage
      // (XDIRECT: the chunk is the short one, so the trip count is a constant and xcur stays in registers)
      const int n_kb = XDIRECT ? kXBlocks : kPerWarp / 32;
      const unsigned char* wa = st + g * kRowBytes + (warp * kPerWarp + 8 * t4) * 2;   // this thread's 16 bytes of rows g, g+8
      const bf16* xa = xs + g * Kp + kbase + 8 * t4;
      auto k_block = [&](int kb, uint4 va, uint4 vb, const uint4 (&xr)[XDIRECT ? MT : 1]) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          uint4 x;
          if constexpr (XDIRECT) x = xr[j];
          else x = *reinterpret_cast<const uint4*>(xa + 8 * j * Kp + kb * 32);
          mma_stream(acc[j], va.x, vb.x, va.y, vb.y, x.x, x.y);
          mma_stream(acc[j], va.z, vb.z, va.w, vb.w, x.z, x.w);
        }
      };
      if constexpr (XDIRECT) {                                 // a constant trip count: xcur stays in registers
#pragma unroll
        for (int kb = 0; kb < kXBlocks; ++kb) {
          if (kbase + kb * 32 >= p.K) break;                   // warp-uniform: the whole k-block lies beyond K
          uint4 va = *reinterpret_cast<const uint4*>(wa + kb * 64);
          uint4 vb = *reinterpret_cast<const uint4*>(wa + 8 * kRowBytes + kb * 64);
          if (kbase + kb * 32 + 8 * t4 >= p.K) {               // this thread's 8 columns lie beyond K: stale bytes
            va = make_uint4(0u, 0u, 0u, 0u);
            vb = make_uint4(0u, 0u, 0u, 0u);
          }
          uint4 xr[MT];
#pragma unroll
          for (int j = 0; j < MT; ++j) xr[j] = xcur[j][kb];
          k_block(kb, va, vb, xr);
        }
      } else if (kbase + kPerWarp <= p.K) {                    // the warp's whole share lies inside K: no checks
        const uint4 none[1] = {};
#pragma unroll 4
        for (int kb = 0; kb < n_kb; ++kb)
          k_block(kb, *reinterpret_cast<const uint4*>(wa + kb * 64),
                  *reinterpret_cast<const uint4*>(wa + 8 * kRowBytes + kb * 64), none);
      } else {
        const uint4 none[1] = {};
#pragma unroll 4
        for (int kb = 0; kb < n_kb; ++kb) {
          if (kbase + kb * 32 >= p.K) break;
          uint4 va = *reinterpret_cast<const uint4*>(wa + kb * 64);
          uint4 vb = *reinterpret_cast<const uint4*>(wa + 8 * kRowBytes + kb * 64);
          if (kbase + kb * 32 + 8 * t4 >= p.K) {
            va = make_uint4(0u, 0u, 0u, 0u);
            vb = make_uint4(0u, 0u, 0u, 0u);
          }
          k_block(kb, va, vb, none);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);                   // this warp is done with the slot
      if constexpr (XDIRECT) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int kb = 0; kb < kXBlocks; ++kb) xcur[j][kb] = xnext[j][kb];
      }
    }
    if constexpr (SCALED) {
      if (tl == 0) {                                           // 1/rms of the rows, in a fixed order of addition
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const int m = warp + kStreamConsumers * j;
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < kPartRegs; ++i) ss += part[j][i];
          if (m < p.M)
            for (int t = lane + 32 * kPartRegs; t < p.ss_tiles; t += 32) ss += __ldcg(p.ss_in + t * kNormRows + m);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0 && m < p.M) norm_s[m] = rsqrtf(ss / float(p.K) + p.eps);
        }
      }
    }
    // acc[j]: c0,c1 = (W row g, batch 8j + 2t, +1); c2,c3 = (W row g+8, same batch rows)
    float* mine = red + ((tl & 1) * kStreamConsumers + warp) * 16 * MB;
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      *reinterpret_cast<float2*>(mine + g * MB + 8 * j + 2 * t4) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * MB + 8 * j + 2 * t4) = make_float2(acc[j][2], acc[j][3]);
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerThreads));
    // The partial sums of the warps are added in warp order: reproducible bit for bit.
    const float* both = red + (tl & 1) * kStreamConsumers * 16 * MB;
    auto total_of = [&](int r, int m) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kStreamConsumers; ++w) sum += both[(w * 16 + r) * MB + m];
      return sum;
    };
    // A thread takes one element of the tile: row m of the batch, column r of the tile's 16, with a
    // row's columns side by side in a half-warp (neighbouring addresses, and the sum of squares
    // over a row's columns is a few shuffles, not a trip through shared memory).
    if constexpr (EPI == kResidual) {
      for (int e = tid; e < 16 * MB; e += kConsumerThreads) {  // (one trip: 16 x MB <= the consumer threads)
        const int m = e >> 4, r = e & 15;
        const int n = row_in(base, r);
        float v = 0.f;
        if (n < p.N && m < p.M) {
          float* x = p.resid + size_t(m) * p.ldr + n;
          v = resid_old + Store<bf16>::round(total_of(r, m));     // (e == tid: the element asked for above)
          *x = v;
          if (p.next_w != nullptr) stf(p.h_out + size_t(m) * p.ldh + n, next_w_mine * v);
        }
        float ss = v * v;                                      // a fixed tree of additions: reproducible
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (r == 0) p.ss_out[tile * kNormRows + m] = ss;
      }
    } else if constexpr (EPI == kStore) {
      OutT* Y = reinterpret_cast<OutT*>(p.Y);
      for (int e = tid; e < 16 * MB; e += kConsumerThreads) {
        const int m = e >> 4, r = e & 15;
        const int n = row_in(base, r);
        if (n < p.N && m < p.M) stf(Y + size_t(m) * p.ldy + n, total_of(r, m));
      }
    } else {
      bf16* Y = reinterpret_cast<bf16*>(p.Y);
      for (int e = tid; e < 8 * MB; e += kConsumerThreads) {
        const int m = e >> 3, pr = e & 7;
        if (m >= p.M) continue;
        const float r = SCALED ? norm_s[m] : 1.f;
        const float xa = Store<bf16>::round(total_of(pr, m) * r);   // what the plain product stores
        const float xb = Store<bf16>::round(total_of(pr + 8, m) * r);
        if constexpr (EPI == kSiluMul) {
          const float sl = Store<bf16>::round(xa / (1.f + expf(-xa)));
          stf(Y + size_t(m) * p.ldy + 8 * tile + pr, sl * xb);
        } else {
          const int head = tile / p.pair_blocks;
          const int j = 8 * (tile - head * p.pair_blocks) + pr;
          const int half = p.hd / 2;
          float ra = xa, rb = xb;
          if (head < p.nh + p.nkv) {
            float sn = sn0, cs = cs0;                               // (e == tid in the first round of the first tile)
            if (tl > 0 || e != tid) sincosf(float(p.positions[m]) * p.inv_freq[j], &sn, &cs);
            rotate_pair(xa, xb, cs, sn, ra, rb);
          }
          if (head < p.nh) {
            stf(Y + size_t(m) * p.ldy + size_t(head) * p.hd + j, ra);
            stf(Y + size_t(m) * p.ldy + size_t(head) * p.hd + j + half, rb);
          } else {
            const int slot = (tl > 0 || e != tid) ? p.slot_mapping[m] : slot0;
            if (slot >= 0) {
              const int page = slot / p.block_size, off = slot - page * p.block_size;
              const bool is_k = head < p.nh + p.nkv;
              const int kvh = is_k ? head - p.nh : head - p.nh - p.nkv;
              bf16* dst = (is_k ? p.k_cache : p.v_cache) + ((size_t(page) * p.nkv + kvh) * p.block_size + off) * p.hd;
              stf(dst + j, ra);
              stf(dst + j + half, rb);
            }
          }
        }
      }
    }
    // the other half of `red` is used by the next tile; this half again two tiles on, after
    // the barrier of the tile in between
  }
}

constexpr size_t kStreamSmemLimit = 224 * 1024;        // of the 227 KB a block may have
constexpr size_t kStreamSmemHalf = 112 * 1024;         // two such blocks share an SM

// Shared memory of a launch with `stages` ring slots of `chunk` k elements.
static size_t stream_smem(int MT, int K, int chunk, int stages) {
  const int Kc = (K + chunk - 1) / chunk;
  return size_t(stages) * 16 * (chunk * 2 + kRowPad) + size_t(MT) * 8 * (Kc * chunk + kXPad) * sizeof(bf16) +
         size_t(2) * kStreamConsumers * 16 * MT * 8 * sizeof(float) + 2 * kMaxStages * sizeof(uint64_t);
}

// The stage length of a launch: whole rows (rounded up to the unit) while at least two such stages
// fit beside X, else the short piece.  0 = not even two short stages fit.
static int stream_chunk(int MT, int K) {
  const int whole = min(kChunkLong, (K + kChunkUnit - 1) / kChunkUnit * kChunkUnit);
  if (stream_smem(MT, K, whole, 2) <= kStreamSmemLimit) return whole;
  const int piece = min(whole, kChunkShort);
  return stream_smem(MT, K, piece, 2) <= kStreamSmemLimit ? piece : 0;
}

// X straight from L2 (no staging): every block has one tile and K is longer than a whole-row stage.
static bool stream_direct(int N, int K, int sm_count) { return (N + 15) / 16 <= sm_count && K > kChunkLong; }

template <int MT, typename OutT, int EPI, bool XDIRECT, bool SCALED = false>
int launch_stream_as(StreamParams p, int sm_count, cudaStream_t s) {
  auto kernel = gemm_stream_kernel<MT, OutT, EPI, XDIRECT, SCALED>;
  const int tiles = (p.N + 15) / 16;
  const int chunk = XDIRECT ? direct_chunk(MT) : stream_chunk(MT, p.K);
  if (chunk == 0) return KVCM_ERR_UNSUPPORTED;
  const int Kc = (p.K + chunk - 1) / chunk;
  // One block per SM; the ring takes what shared memory is left after X, but never more slots than
  // the block has stages to load.
  const int xk = XDIRECT ? 0 : p.K;                               // k extent of the staged X
  int blocks = min(tiles, sm_count);
  // A few tiles more than SMs, and a whole tile of W beside X takes less than half of an SM's
  // shared memory: one block per tile, two to an SM, instead of a second round for a few blocks.
  // (Small blocks also find room while the predecessor kernel is still running.)
  if (tiles > sm_count && tiles <= 2 * sm_count && stream_smem(MT, xk, chunk, Kc) <= kStreamSmemHalf) blocks = tiles;
  const int need = ((tiles + blocks - 1) / blocks) * Kc;
  int stages = kMaxStages;
  while (stages > 1 && (stream_smem(MT, xk, chunk, stages) > kStreamSmemLimit || stages > need)) --stages;
  const size_t smem = stream_smem(MT, xk, chunk, stages);
  if (smem > kStreamSmemLimit) return KVCM_ERR_UNSUPPORTED;
  p.chunk = chunk;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = smem;
  }
  p.stages = stages;
  return pdl_launch(kernel, dim3(blocks), dim3(kStreamThreads), smem, s, p);
}

template <int MT, typename OutT, int EPI>
int launch_stream(StreamParams p, int sm_count, cudaStream_t s) {
  if constexpr (EPI == kStore || EPI == kResidual) {
    if (stream_direct(p.N, p.K, sm_count)) return launch_stream_as<MT, OutT, EPI, true>(p, sm_count, s);
  } else {
    if (p.ss_in != nullptr) return launch_stream_as<MT, OutT, EPI, false, true>(p, sm_count, s);
  }
  return launch_stream_as<MT, OutT, EPI, false>(p, sm_count, s);
}

}  // namespace kvcm

using namespace kvcm;

static int current_sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count <= 0)
      count = 148;
  }
  return count;
}

static bool stream_ok(int M, int N, int K, int sm_count, bool plain_store) {
  if (M < 1 || M > 16 || N < 1 || K < 8 || (K % 8)) return false;
  return stream_chunk(M <= 8 ? 1 : 2, K) != 0 || (plain_store && stream_direct(N, K, sm_count));
}

// The plain product (no fused epilogue) of these sizes on the current device.
KVCM_API int kvcm_gemm_stream_supports(int M, int N, int K) { return stream_ok(M, N, K, current_sm_count(), true); }

// out_f32: 0 = bfloat16 result, 1 = float result.
KVCM_API int kvcm_gemm_stream_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                                   int ldw, int ldy, int out_f32, int sm_count, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!stream_ok(M, N, K, sm_count, true) || (ldw % 8) || (ldx % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return KVCM_ERR_UNSUPPORTED;
  StreamParams p = {};
  p.W = (const bf16*)W; p.N = N; p.K = K; p.ldw = ldw; p.X = (const bf16*)X; p.ldx = ldx; p.M = M;
  p.Y = Y; p.ldy = ldy;
  p.pair_blocks = 1; p.group_stride = 16; p.pair_offset = 8;          // identity: tile t = rows 16t .. 16t+15
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 8) return out_f32 ? launch_stream<1, float, kStore>(p, sm_count, s) : launch_stream<1, bf16, kStore>(p, sm_count, s);
  return out_f32 ? launch_stream<2, float, kStore>(p, sm_count, s) : launch_stream<2, bf16, kStore>(p, sm_count, s);
}

// The product that ends a sublayer: resid[M, N] (float, in place) += round_bf16(X * W^T);
// ss_out[tile][m] (tile = 16 columns, kNormRows floats apart) = the tile's share of the sum of
// squares of the new residual row m (ss_out holds ceil(N / 16) * 16 floats); and, where next_w is
// given, h_out[M, N] = bfloat16(next_w[n] * resid[m][n]): the row the next norm hands on, before
// its scale.
KVCM_API int kvcm_gemm_stream_residual_bf16(const void* X, const void* W, float* resid, float* ss_out, void* h_out,
                                            const void* next_w, int M, int N, int K, int ldx, int ldw, int ldr,
                                            int ldh, int sm_count, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!stream_ok(M, N, K, sm_count, true) || (ldw % 8) || (ldx % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return KVCM_ERR_UNSUPPORTED;
  if (resid == nullptr || ss_out == nullptr || (next_w != nullptr && h_out == nullptr)) return KVCM_ERR_UNSUPPORTED;
  StreamParams p = {};
  p.W = (const bf16*)W; p.N = N; p.K = K; p.ldw = ldw; p.X = (const bf16*)X; p.ldx = ldx; p.M = M;
  p.resid = resid; p.ldr = ldr; p.ss_out = ss_out; p.h_out = (bf16*)h_out; p.ldh = ldh; p.next_w = (const bf16*)next_w;
  p.pair_blocks = 1; p.group_stride = 16; p.pair_offset = 8;
  cudaStream_t s = (cudaStream_t)stream;
  return M <= 8 ? launch_stream<1, bf16, kResidual>(p, sm_count, s) : launch_stream<2, bf16, kResidual>(p, sm_count, s);
}

// Fused decode step of an attention layer's input side: qkv = X * Wqkv^T, rotary encoding of the q
// and k heads (rotate-half pairing over the whole head), q written to Y [M, >= nh*hd], k and v
// written into the rows' cache page slots.  Needs hd a multiple of 16.
// With ss_in (ss_tiles x kNormRows floats as kvcm_gemm_stream_residual_bf16 leaves them): row m of
// the product is scaled by rsqrt(sum of ss_in[.][m] / K + eps) first -- X is then a normed row
// before its scale, and this is the norm in front of the attention layer.
KVCM_API int kvcm_qkv_rope_cache_scaled_bf16(const void* X, const float* ss_in, int ss_tiles, float eps,
                                             const void* Wqkv, void* Yq, int M, int K, int ldx, int ldw, int ldy,
                                             const int* positions, const float* inv_freq, const int* slot_mapping,
                                             void* k_cache, void* v_cache, int nh, int nkv, int hd, int block_size,
                                             int sm_count, void* stream) {
  const int N = (nh + 2 * nkv) * hd;
  if (M == 0) return 0;
  if ((hd % 16) || !stream_ok(M, N, K, sm_count, false) || (ldw % 8) || (ldx % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(Wqkv) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return KVCM_ERR_UNSUPPORTED;
  if (ss_in != nullptr && ss_tiles <= 0) return KVCM_ERR_UNSUPPORTED;
  StreamParams p = {};
  p.W = (const bf16*)Wqkv; p.N = N; p.K = K; p.ldw = ldw; p.X = (const bf16*)X; p.ldx = ldx; p.M = M;
  p.ss_in = ss_in; p.ss_tiles = ss_tiles; p.eps = eps;
  p.Y = Yq; p.ldy = ldy;
  p.pair_blocks = hd / 16; p.group_stride = hd; p.pair_offset = hd / 2;
  p.positions = positions; p.inv_freq = inv_freq; p.slot_mapping = slot_mapping;
  p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache;
  p.nh = nh; p.nkv = nkv; p.hd = hd; p.block_size = block_size;
  cudaStream_t s = (cudaStream_t)stream;
  return M <= 8 ? launch_stream<1, bf16, kRopeCache>(p, sm_count, s) : launch_stream<2, bf16, kRopeCache>(p, sm_count, s);
}

KVCM_API int kvcm_qkv_rope_cache_bf16(const void* X, const void* Wqkv, void* Yq, int M, int K, int ldx, int ldw,
                                      int ldy, const int* positions, const float* inv_freq,
                                      const int* slot_mapping, void* k_cache, void* v_cache, int nh, int nkv,
                                      int hd, int block_size, int sm_count, void* stream) {
  return kvcm_qkv_rope_cache_scaled_bf16(X, nullptr, 0, 0.f, Wqkv, Yq, M, K, ldx, ldw, ldy, positions, inv_freq,
                                         slot_mapping, k_cache, v_cache, nh, nkv, hd, block_size, sm_count, stream);
}

// Fused input side of a gated feed-forward: act[M, I] = silu(X Wg^T) * (X Wu^T) with Wg, Wu the
// two halves of W [2I, K] (gate rows first).  Needs I a multiple of 8.  With ss_in: both products
// scaled per row first (see kvcm_qkv_rope_cache_scaled_bf16): the norm in front of the feed-forward.
KVCM_API int kvcm_gate_up_silu_scaled_bf16(const void* X, const float* ss_in, int ss_tiles, float eps, const void* W,
                                           void* Y, int M, int I, int K, int ldx, int ldw, int ldy, int sm_count,
                                           void* stream) {
  if (M == 0) return 0;
  if ((I % 8) || !stream_ok(M, 2 * I, K, sm_count, false) || (ldw % 8) || (ldx % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return KVCM_ERR_UNSUPPORTED;
  if (ss_in != nullptr && ss_tiles <= 0) return KVCM_ERR_UNSUPPORTED;
  StreamParams p = {};
  p.W = (const bf16*)W; p.N = 2 * I; p.K = K; p.ldw = ldw; p.X = (const bf16*)X; p.ldx = ldx; p.M = M;
  p.ss_in = ss_in; p.ss_tiles = ss_tiles; p.eps = eps;
  p.Y = Y; p.ldy = ldy;
  p.pair_blocks = I / 8; p.group_stride = 0; p.pair_offset = I;
  cudaStream_t s = (cudaStream_t)stream;
  return M <= 8 ? launch_stream<1, bf16, kSiluMul>(p, sm_count, s) : launch_stream<2, bf16, kSiluMul>(p, sm_count, s);
}

KVCM_API int kvcm_gate_up_silu_bf16(const void* X, const void* W, void* Y, int M, int I, int K, int ldx, int ldw,
                                    int ldy, int sm_count, void* stream) {
  return kvcm_gate_up_silu_scaled_bf16(X, nullptr, 0, 0.f, W, Y, M, I, K, ldx, ldw, ldy, sm_count, stream);
}

// The fused products (rotary/cache and gate/up epilogues) of these sizes: X is always staged there.
KVCM_API int kvcm_gemm_stream_fused_supports(int M, int N, int K) { return stream_ok(M, N, K, current_sm_count(), false); }

// Device address of the error word (the sampling kernels copy it out with the step's tokens).
KVCM_API const int* kvcm_stream_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_stream_error) == cudaSuccess ? p : nullptr;
}

// Test hooks of the failure path: the wait limit (0 = the default of two seconds) and the stage
// whose copy is left out (-1 = none).  Not for production use.
KVCM_API int kvcm_stream_test_hooks(unsigned long long wait_limit_ns, int skip_stage) {
  const unsigned long long limit = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  if (cudaMemcpyToSymbol(g_stream_wait_limit_ns, &limit, sizeof limit) != cudaSuccess) return -1;
  if (cudaMemcpyToSymbol(g_stream_skip_stage, &skip_stage, sizeof skip_stage) != cudaSuccess) return -1;
  return 0;
}

// Reads and clears the error word of the streaming kernels (0 = no bounded wait ever ran out).
KVCM_API int kvcm_stream_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_stream_error, &zero, sizeof zero);
  return v;
}
