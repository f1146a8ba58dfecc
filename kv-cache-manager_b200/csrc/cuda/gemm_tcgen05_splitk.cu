// Matrix product for a few dozen to a few hundred rows (decode at larger batches, short prompt
// portions) on the fifth-generation tensor cores:
//     Y[M, N] = X[M, K] * W[N, K]^T,  16 < M <= 256, bfloat16 operands, float accumulation.
//
// With so few rows the product is bound by reading W once, so the roles of the operands are swapped:
// 128 rows of W are the 128-row operand of tcgen05.mma and the (padded) batch is its N, the
// accumulator [128 weight rows x M] sits in tensor memory.  N / 128 tiles alone would leave most of
// the 148 SMs idle, so K is split over the blocks of a thread-block cluster (1, 2, 4 or 8): every
// block streams its 128 x (K / S) slab of W (and the matching columns of X) through a TMA ring of
// up to ten stages, which keeps 150-200 KB of copies in flight per SM.  At the end every block puts
// its partial sums into its own shared memory, the cluster meets, and each block adds the S
// partial sums (always in block order: reproducible) for 128 / S of the weight rows through
// distributed shared memory and stores that part of Y.
// Roles per block: warp 0 one thread TMA, warp 1 one thread tcgen05.mma, warps 2-5 the epilogue.
// Every wait on an mbarrier is bounded; a block whose wait ran out records it
// (kvcm_gemm_tcgen05_splitk_error), contributes nothing more, still meets its cluster and frees
// its tensor memory.  The reference calls cuBLAS for these products (src/model/llama.cpp:45-52).
#include <cooperative_groups.h>

#include "tcgen05_common.cuh"

namespace kvcm {

namespace cg = cooperative_groups;

constexpr int kSkThreads = 192;
constexpr int kSkRows = 128;                 // weight rows per tile
constexpr int kSkBK = 64;                    // k elements per stage
constexpr int kSkMaxStages = 10;
constexpr int kSkWBytes = kSkRows * kSkBK * 2;
constexpr size_t kSkSmemLimit = 200 * 1024;

__device__ int g_splitk_error = 0;

template <typename OutT>
__global__ void __launch_bounds__(kSkThreads)
gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           OutT* __restrict__ Y, int M, int N, int K, int ldy, int Mp, int stages, int tmem_cols) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int stage_bytes = kSkWBytes + Mp * kSkBK * 2;          // W piece, then X piece (both 1,024-byte multiples)
  __shared__ __align__(8) uint64_t full[kSkMaxStages], empty[kSkMaxStages], acc_full;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;

  cg::cluster_group cluster = cg::this_cluster();
  const int S = int(cluster.num_blocks()), rank = int(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = int(blockIdx.x) / S;
  const int n0 = tile * kSkRows;
  const int nk = (K + kSkBK - 1) / kSkBK;
  const int per = (nk + S - 1) / S;                            // k-steps per block of the cluster
  const int k_begin = min(nk, rank * per), k_end = min(nk, k_begin + per);
  const int steps = k_end - k_begin;
  const bool aligned = (tc5::s32(smem_raw) & 1023) == 0;       // the swizzled tiles need this

  if (threadIdx.x == 0) {
    abort_flag = aligned ? 0 : 1;
    if (!aligned) atomicExch(&g_splitk_error, (7 << 16) | int(blockIdx.x & 0xffff));
    for (int s = 0; s < stages; ++s) { tc5::mbar_init(&full[s], 1); tc5::mbar_init(&empty[s], 1); }
    tc5::mbar_init(&acc_full, 1);
    tc5::mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5::s32(&tmem_base)), "r"(tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc5::fence_before();
  __syncthreads();
  tc5::fence_after();
  const uint32_t tmem = tmem_base;

  auto fail = [&](int code) {
    atomicExch(&g_splitk_error, (code << 16) | int(blockIdx.x & 0xffff));
    abort_flag = 1;
  };

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < steps && !abort_flag; ++i) {
        const int s = i % stages;
        if (!tc5::mbar_wait(&empty[s], ((i / stages) & 1) ^ 1)) { fail(1); break; }
        tc5::mbar_expect_tx(&full[s], uint32_t(stage_bytes));
        unsigned char* w_s = smem_raw + size_t(s) * stage_bytes;
        tc5::tma_load_2d(w_s, &map_w, &full[s], (k_begin + i) * kSkBK, n0);
        tc5::tma_load_2d(w_s + kSkWBytes, &map_x, &full[s], (k_begin + i) * kSkBK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t instr = tc5::idesc(kSkRows, Mp);
      for (int i = 0; i < steps && !abort_flag; ++i) {
        const int s = i % stages;
        if (!tc5::mbar_wait(&full[s], (i / stages) & 1)) { fail(2); break; }
        tc5::fence_after();
        const uint32_t w_addr = tc5::s32(smem_raw + size_t(s) * stage_bytes);
        const uint64_t da = tc5::smem_desc(w_addr), db = tc5::smem_desc(w_addr + kSkWBytes);
#pragma unroll
        for (int j = 0; j < kSkBK / 16; ++j)
          tc5::mma(tmem, da + uint64_t(2 * j), db + uint64_t(2 * j), instr, (i > 0 || j > 0) ? 1u : 0u);
        tc5::commit(&empty[s]);                                // the slot is free once these products have read it
      }
      if (!abort_flag) tc5::commit(&acc_full);
    }
  }

  // ---- the block's partial sums go to its shared memory as [Mp][128] floats (the ring is no longer
  // needed: every copy has landed and every product has read it once acc_full completes)
  float* partial = reinterpret_cast<float*>(smem_raw);
  if (warp >= 2) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                       // weight row of the tile = lane of tensor memory
    bool have = steps > 0 && !abort_flag;
    if (have) have = tc5::mbar_wait(&acc_full, 0);
    if (!__all_sync(0xffffffffu, have)) {
      if (steps > 0 && !abort_flag && lane == 0) fail(3);
      have = false;
    }
    tc5::fence_after();
    for (int c = 0; c < Mp / 32 + (Mp % 32 ? 1 : 0); ++c) {
      uint32_t v[32];
      if (have) {
        // (loads of 32 columns; the allocation is a power of two >= Mp rounded up to 32, so the
        // columns beyond Mp exist and are simply not used)
        tc5::ld32(tmem + (uint32_t(quarter * 32) << 16) + uint32_t(c * 32), v);
        tc5::ld_wait();
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int m = c * 32 + i;
        if (m < Mp) partial[m * kSkRows + row] = have ? __uint_as_float(v[i]) : 0.f;
      }
    }
    tc5::fence_before();
  }
  cluster.sync();                                              // every block's partial sums are in place
  {
    // this block adds and stores weight rows [rank * W, (rank + 1) * W) of the tile, for every batch row
    const int Wd = kSkRows / S;
    const float* parts[8];
    for (int q = 0; q < S; ++q) parts[q] = cluster.map_shared_rank(partial, q);
    if (!abort_flag) {
      // four neighbouring weight rows per step (a 16-byte read from every block), four steps with
      // all their reads in flight before the first store (the compiler cannot move a read of
      // another block's memory across a store to Y by itself)
      const int vec = Wd / 4, items = M * vec;                 // Wd is 16, 32, 64 or 128
      constexpr int kBatch = 4;
      for (int e0 = threadIdx.x; e0 < items; e0 += kBatch * kSkThreads) {
        float4 acc[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int e = e0 + u * kSkThreads;
          acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (e < items) {
            const int m = e / vec, j = (e - m * vec) * 4;
            for (int q = 0; q < S; ++q) {
              const float4 t = *reinterpret_cast<const float4*>(parts[q] + m * kSkRows + rank * Wd + j);
              acc[u].x += t.x; acc[u].y += t.y; acc[u].z += t.z; acc[u].w += t.w;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const int e = e0 + u * kSkThreads;
          if (e >= items) break;
          const int m = e / vec, j = (e - m * vec) * 4;
          const int n = n0 + rank * Wd + j;
          OutT* dst = Y + size_t(m) * ldy + n;
          const float r[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (n + i < N) stf(dst + i, r[i]);
        }
      }
    }
  }
  cluster.sync();                                              // nobody leaves while its memory is read
  tc5::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc5::fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(tmem_cols));
  }
}

// How K is split: as many blocks as run at once (one per SM while the tiles are fewer than the SMs),
// at most 8 per tile, at least four k-steps each.
static int splitk_factor(int N, int K, int sm_count) {
  const int tiles = (N + kSkRows - 1) / kSkRows, nk = (K + kSkBK - 1) / kSkBK;
  int S = 1;
  while (S < 8 && tiles * (2 * S) <= sm_count && nk / (2 * S) >= 4) S *= 2;
  return S;
}

template <typename OutT>
int launch_splitk(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy, cudaStream_t s) {
  static int sm_count = 0;
  if (sm_count == 0) sm_count = tc5::current_sm_count();
  const int Mp = (M + 15) / 16 * 16;
  CUtensorMap mw, mx;
  int rc = tc5::make_map(&mw, W, N, K, ldw, kSkRows);
  if (rc) return rc;
  rc = tc5::make_map(&mx, X, M, K, ldx, Mp);
  if (rc) return rc;
  const int stage_bytes = kSkWBytes + Mp * kSkBK * 2;
  const size_t partial_bytes = size_t(Mp) * kSkRows * sizeof(float);
  const int S = splitk_factor(N, K, sm_count);
  const int nk = (K + kSkBK - 1) / kSkBK, per = (nk + S - 1) / S;
  const int tiles_all = (N + kSkRows - 1) / kSkRows;
  // more tiles than SMs: rings of half the size, so that two blocks share an SM instead of queueing
  const size_t budget = tiles_all * S > sm_count ? kSkSmemLimit / 2 : kSkSmemLimit;
  int stages = int(budget / stage_bytes);
  if (stages < 2) stages = int(kSkSmemLimit / stage_bytes) >= 2 ? 2 : 1;
  if (stages > kSkMaxStages) stages = kSkMaxStages;
  if (stages > per) stages = per < 1 ? 1 : per;
  size_t smem = size_t(stages) * stage_bytes;
  if (smem < partial_bytes) smem = partial_bytes;
  if (stages < 1 || smem > kSkSmemLimit + 24 * 1024) return KVCM_ERR_UNSUPPORTED;
  int tmem_cols = 32;
  while (tmem_cols < Mp) tmem_cols *= 2;
  auto kernel = gemm_tcgen05_splitk_kernel<OutT>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = smem;
  }
  const int tiles = (N + kSkRows - 1) / kSkRows;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * S);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return int(cudaLaunchKernelEx(&cfg, kernel, mw, mx, reinterpret_cast<OutT*>(Y), M, N, K, ldy, Mp, stages, tmem_cols));
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_gemm_tcgen05_splitk_supports(int M, int N, int K, int ldx, int ldw) {
  return M >= 1 && M <= 256 && N >= 1 && K >= 8 && (K % 8) == 0 && (ldx % 8) == 0 && (ldw % 8) == 0;
}

// out_f32: 0 = bfloat16 result, 1 = float result.
KVCM_API int kvcm_gemm_tcgen05_splitk_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                           int ldy, int out_f32, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!kvcm_gemm_tcgen05_splitk_supports(M, N, K, ldx, ldw)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return KVCM_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  return out_f32 ? launch_splitk<float>(X, W, Y, M, N, K, ldx, ldw, ldy, s) : launch_splitk<bf16>(X, W, Y, M, N, K, ldx, ldw, ldy, s);
}

// Reads and clears the error word of the kernel (0 = no bounded wait ever ran out); else
// (code << 16) | block: 1 the producer waited for a free stage, 2 the products for data, 3 the
// Device address of the error word (the sampling kernels copy it out with the step's tokens).
KVCM_API const int* kvcm_gemm_tcgen05_splitk_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_splitk_error) == cudaSuccess ? p : nullptr;
}

// epilogue for the accumulator, 7 shared memory not aligned to 1,024 bytes.
KVCM_API int kvcm_gemm_tcgen05_splitk_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_splitk_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_splitk_error, &zero, sizeof zero);
  return v;
}
