// Matrix product for many rows (prefill) on the fifth-generation tensor cores:
//     Y[M, N] = X[M, K] * W[N, K]^T,  bfloat16 operands, float accumulation in tensor memory.
//
// Blocks are persistent (one per SM) and compute 128 x 256 tiles of Y (128 x 128 when that fills the
// last round of blocks better), with two accumulators in tensor memory so that the epilogue of one
// tile runs while the tensor core works on the next:
//  * warp 0, one thread: TMA.  Tiled tensor maps (cp.async.bulk.tensor.2d) bring a [128 x 64] piece
//    of X and a [256 x 64] piece of W per k-step into a four-stage (six for the narrow tile) ring of shared memory, in the
//    128-byte swizzled layout the tensor core reads; completion is counted on an mbarrier.
//  * warp 1, one thread: tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 256, K = 16), four per
//    k-step, accumulating into one of the two accumulators (256 columns each) of tensor memory; tcgen05.commit hands each ring slot
//    back to the producer when the products that read it are done, and signals the epilogue at
//    the end.
//  * warps 2-5: epilogue.  tcgen05.ld reads the accumulator (each warp its quarter of the 128
//    lanes), converts and stores rows of Y (bfloat16 or float).
// Out-of-range rows, columns and k are zero-filled by the TMA unit, so any M, N and any K that
// is a multiple of 8 work.  Every wait on an mbarrier is bounded; when one runs out the block
// records it (kvcm_tcgen05_error), stops waiting, frees its tensor memory and leaves.
// The reference calls cuBLAS for these products (src/model/llama.cpp:45-52).
#include "tcgen05_common.cuh"

namespace kvcm {

constexpr int kTcBM = 128, kTcBK = 64;
constexpr int kTcThreads = 192;
constexpr int kTcABytes = kTcBM * kTcBK * 2;

__device__ int g_tcgen05_error = 0;

// GATED: W is [2N, K], gate rows first; a tile's 256 accumulator columns are 128 gate columns
// n0..n0+127 and the 128 up columns N+n0.., and the epilogue stores
// y[m][n] = round(round(silu(round(gate))) * round(up)) -- the roundings of the separate product
// and activation kernels -- so the [M, 2N] intermediate never goes to memory.
template <typename OutT, int BN, bool GATED>
__global__ void __launch_bounds__(kTcThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    OutT* __restrict__ Y, int M, int N, int K, int ldy) {
  static_assert(!GATED || BN == 256, "the gated tile is 128 + 128 columns");
  constexpr int BNOUT = GATED ? BN / 2 : BN;                   // output columns per tile
  constexpr int kBBytes = BN * kTcBK * 2;
  constexpr int kStageBytes = kTcABytes + kBBytes;
  constexpr int kStages = BN == 256 ? 4 : 6;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + kTcBM - 1) / kTcBM, n_tiles = (N + BNOUT - 1) / BNOUT;
  const int tiles = m_tiles * n_tiles;
  const int nk = (K + kTcBK - 1) / kTcBK;
  // Persistent block: tiles blockIdx.x, + gridDim.x, ...  Neighbouring blocks take different column
  // tiles of the same row tile: the blocks of a round share a few pieces of X and sweep W, all of
  // which stays in L2 at these sizes.
  const int my_tiles = int(blockIdx.x) < tiles ? (tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5::s32(&full[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5::s32(&empty[s])));
    }
    for (int a = 0; a < 2; ++a) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(tc5::s32(&acc_full[a])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;\n" ::"r"(tc5::s32(&acc_empty[a])));   // four epilogue warps
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {                                // one warp allocates two accumulators of BN columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5::s32(&tmem_base)), "r"(2 * BN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                  // running stage counter across tiles
      for (int tl = 0; tl < my_tiles && !abort_flag; ++tl) {
        const int t = int(blockIdx.x) + tl * int(gridDim.x);
        const int m0 = (t / n_tiles) * kTcBM, n0 = (t % n_tiles) * BNOUT;
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % kStages;
          if (!tc5::mbar_wait(&empty[s], ((it / kStages) & 1) ^ 1)) {
            atomicExch(&g_tcgen05_error, (1 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc5::s32(&full[s])), "r"(kStageBytes) : "memory");
          unsigned char* a = ring + s * kStageBytes;
          unsigned char* b = a + kTcABytes;
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                       ::"r"(tc5::s32(a)), "l"(&map_x), "r"(tc5::s32(&full[s])), "r"(k * kTcBK), "r"(m0) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                       ::"r"(tc5::s32(b)), "l"(&map_w), "r"(tc5::s32(&full[s])), "r"(k * kTcBK), "r"(n0) : "memory");
          if constexpr (GATED)                                   // the map's box is 128 rows: the up rows follow
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                         ::"r"(tc5::s32(b + kBBytes / 2)), "l"(&map_w), "r"(tc5::s32(&full[s])), "r"(k * kTcBK), "r"(N + n0) : "memory");
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::idesc(kTcBM, BN);
      int it = 0;
      for (int tl = 0; tl < my_tiles && !abort_flag; ++tl) {
        const int acc = tl & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (!tc5::mbar_wait(&acc_empty[acc], ((tl >> 1) & 1) ^ 1)) {
          atomicExch(&g_tcgen05_error, (4 << 16) | int(blockIdx.x & 0xffff));
          abort_flag = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t d_tmem = tmem + uint32_t(acc * BN);
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % kStages;
          if (!tc5::mbar_wait(&full[s], (it / kStages) & 1)) {
            atomicExch(&g_tcgen05_error, (2 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = tc5::s32(ring + s * kStageBytes);
          const uint64_t da = tc5::smem_desc(a_addr), db = tc5::smem_desc(a_addr + kTcABytes);
#pragma unroll
          for (int j = 0; j < kTcBK / 16; ++j) {
            const uint32_t accumulate = (k > 0 || j > 0) ? 1u : 0u;
            // +32 bytes along k inside the swizzled row = +2 in the descriptor's address field
            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                         ::"r"(d_tmem), "l"(da + uint64_t(2 * j)), "l"(db + uint64_t(2 * j)), "r"(idesc), "r"(accumulate) : "memory");
          }
          // the ring slot is free once these products have read it
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc5::s32(&empty[s])) : "memory");
        }
        if (abort_flag) break;
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tc5::s32(&acc_full[acc])) : "memory");
      }
    }
  } else {
    // ---- epilogue: this warp reads lanes 32*(warp % 4) .. +31 of the accumulator, while the
    // tensor core already fills the other accumulator with the next tile
    const int quarter = warp & 3;
    for (int tl = 0; tl < my_tiles; ++tl) {
      const int acc = tl & 1;
      const int t = int(blockIdx.x) + tl * int(gridDim.x);
      const int m0 = (t / n_tiles) * kTcBM, n0 = (t % n_tiles) * BNOUT;
      if (abort_flag || !tc5::mbar_wait(&acc_full[acc], (tl >> 1) & 1)) {
        if (!abort_flag && lane == 0) atomicExch(&g_tcgen05_error, (3 << 16) | int(blockIdx.x & 0xffff));
        abort_flag = 1;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + quarter * 32 + lane;
      if constexpr (GATED) {
#pragma unroll 1
        for (int c = 0; c < BNOUT / 32; ++c) {
          uint32_t g[32], u[32];
          const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(acc * BN + c * 32);
          tc5::ld32(taddr, g);
          tc5::ld32(taddr + BNOUT, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row < M) {
            const int col0 = n0 + c * 32;
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
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(acc * BN + c * 32);
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                     "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                     "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                       "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                       "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                       "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                     : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        if (row < M) {
          const int col0 = n0 + c * 32;
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
      // this warp has read its lanes of the accumulator: hand it back to the tensor core
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc5::s32(&acc_empty[acc])) : "memory");
    }
  }
  // every role ends here; tensor memory goes back before the block leaves
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN));
  }
}

// ---------------------------------------------------------------------------------- host

// GATED: N is the number of output columns; W has 2N rows.
template <typename OutT, int BN, bool GATED = false>
int launch_tcgen05_bn(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                      int sm_count, cudaStream_t s) {
  CUtensorMap mx, mw;
  int rc = tc5::make_map(&mx, X, M, K, ldx, kTcBM);
  if (rc) return rc;
  rc = GATED ? tc5::make_map(&mw, W, 2 * N, K, ldw, BN / 2) : tc5::make_map(&mw, W, N, K, ldw, BN);
  if (rc) return rc;
  auto kernel = gemm_tcgen05_kernel<OutT, BN, GATED>;
  const size_t smem = size_t(BN == 256 ? 4 : 6) * (kTcABytes + BN * kTcBK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  constexpr int BNOUT = GATED ? BN / 2 : BN;
  const int tiles = ((N + BNOUT - 1) / BNOUT) * ((M + kTcBM - 1) / kTcBM);
  kernel<<<dim3(tiles < sm_count ? tiles : sm_count), kTcThreads, smem, s>>>(mx, mw, reinterpret_cast<OutT*>(Y), M, N, K, ldy);
  return KVCM_LAUNCH_RESULT();
}

template <typename OutT>
int launch_tcgen05(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                   cudaStream_t s) {
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // 128 x 256 tiles unless the narrower 128 x 128 tile fills the last round of blocks better.
  const long long m_tiles = (M + kTcBM - 1) / kTcBM;
  const long long t256 = m_tiles * ((N + 255) / 256), t128 = m_tiles * ((N + 127) / 128);
  const long long cost256 = ((t256 + sm_count - 1) / sm_count) * 256, cost128 = ((t128 + sm_count - 1) / sm_count) * 128;
  if (cost128 * 3 < cost256 * 2) return launch_tcgen05_bn<OutT, 128>(X, W, Y, M, N, K, ldx, ldw, ldy, sm_count, s);
  return launch_tcgen05_bn<OutT, 256>(X, W, Y, M, N, K, ldx, ldw, ldy, sm_count, s);
}

}  // namespace kvcm

using namespace kvcm;

// act[M, I] = silu(X Wg^T) * (X Wu^T) with Wg, Wu the halves of W [2I, K] (gate rows first), the
// roundings of the separate product and activation kernels; bfloat16.
KVCM_API int kvcm_gate_up_silu_tcgen05_bf16(const void* X, const void* W, void* Y, int M, int I, int K, int ldx,
                                            int ldw, int ldy, void* stream) {
  if (M == 0 || I == 0) return 0;
  if (M < 1 || I < 1 || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return KVCM_ERR_UNSUPPORTED;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  return launch_tcgen05_bn<bf16, 256, true>(X, W, Y, M, I, K, ldx, ldw, ldy, sms, (cudaStream_t)stream);
}

KVCM_API int kvcm_gemm_tcgen05_supports(int M, int N, int K, int ldx, int ldw) {
  return M >= 1 && N >= 1 && K >= 8 && (K % 8) == 0 && (ldx % 8) == 0 && (ldw % 8) == 0;
}

// out_f32: 0 = bfloat16 result, 1 = float result.
KVCM_API int kvcm_gemm_tcgen05_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                    int ldy, int out_f32, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!kvcm_gemm_tcgen05_supports(M, N, K, ldx, ldw)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return KVCM_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  return out_f32 ? launch_tcgen05<float>(X, W, Y, M, N, K, ldx, ldw, ldy, s)
                 : launch_tcgen05<bf16>(X, W, Y, M, N, K, ldx, ldw, ldy, s);
}

// Device address of the error word (the sampling kernels copy it out with the step's tokens).
KVCM_API const int* kvcm_tcgen05_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_tcgen05_error) == cudaSuccess ? p : nullptr;
}

// Reads and clears the error word (0 = no bounded wait ever ran out).  Synchronises the device.
KVCM_API int kvcm_tcgen05_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tcgen05_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_tcgen05_error, &zero, sizeof zero);
  return v;
}
