// Weight-streaming matrix product for a handful of rows (decode):
//     Y[M, N] = X[M, K] * W[N, K]^T,   M <= 16, bfloat16 operands, float accumulation.
//
// With so few rows the product is bound by reading W once from HBM, so the kernel is built
// around that stream:
//  * "swap AB": 16 rows of W are the 16-row operand of the tensor-core product (m16n8k16) and the
//    batch rows are its 8 columns, so no tensor-core work is wasted on padding M up to 64 or 128;
//  * W goes from global memory straight to registers in 16-byte loads, a ring of eight k-blocks
//    ahead of the product; the k index inside a 32-wide block is permuted identically for both operands
//    (thread t of a quad owns k = 8t..8t+7), which makes every load of W and X a 16-byte vector;
//  * X (a few KB) is staged once per block in shared memory;
//  * a block of 8 warps covers (8 / KW) tiles of 16 rows of W, KW warps sharing a tile along K;
//    their partial sums are added in warp order, so the result is bit-for-bit reproducible;
//  * launched as a programmatic dependent: the first loads of W are issued before the kernel
//    waits for its predecessor, so streaming starts while the previous kernel drains.
// Output bfloat16, or float (logits).  K must be a multiple of 8; anything else is refused.
// The reference calls cuBLAS here (src/model/llama.cpp:45-52).
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyWarps = 8;
constexpr int kAhead = 8;                 // k-blocks of 32 loaded ahead per warp (16 x 16 B per thread)

struct SkinnyParams {
  const bf16* W; int N, K, ldw;
  const bf16* X; int ldx, M;
  void* Y; int ldy;
  int kw;                                 // warps that share one 16-row tile along K (1, 2, 4, 8)
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, typename OutT>
__global__ void __launch_bounds__(kSkinnyThreads)
gemm_skinny_kernel(SkinnyParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int Kb = (p.K + 31) / 32;                    // k-blocks
  const int Kp = Kb * 32 + 8;                        // padded row of the staged X (odd multiple of 16 B)
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);      // [MT*8][Kp]
  float* red = reinterpret_cast<float*>(xs + MT * 8 * Kp);   // [8 warps][16][MT*8]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int tiles_per_block = kSkinnyWarps / p.kw;
  const int tile = blockIdx.x * tiles_per_block + warp / p.kw;
  const int kpart = warp % p.kw;
  const int n_tiles = (p.N + 15) / 16;
  const bool tile_live = tile < n_tiles;
  const int row_a = min(tile * 16 + g, p.N - 1), row_b = min(tile * 16 + g + 8, p.N - 1);
  const int per = (Kb + p.kw - 1) / p.kw;
  const int kb_begin = kpart * per, kb_end = min(Kb, kb_begin + per);
  const bf16* wa = p.W + size_t(row_a) * p.ldw + 8 * t4;
  const bf16* wb = p.W + size_t(row_b) * p.ldw + 8 * t4;

  auto load_w = [&](int kb, uint4& va, uint4& vb) {
    const int k = kb * 32 + 8 * t4;
    if (tile_live && kb < kb_end && k < p.K) {
      va = ldg_stream(wa + kb * 32);
      vb = ldg_stream(wb + kb * 32);
    } else {
      va = make_uint4(0u, 0u, 0u, 0u);
      vb = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  pdl_launch_dependents();
  uint4 a_cur[kAhead][2];                                        // a ring of kAhead k-blocks in flight
#pragma unroll
  for (int i = 0; i < kAhead; ++i) load_w(kb_begin + i, a_cur[i][0], a_cur[i][1]);   // weights are constants:
  pdl_wait();                                                                        // safe before the wait

  // stage X with asynchronous copies, all in flight at once: rows beyond M and columns beyond K
  // are zero-filled (a copy with source size 0 writes zeros)
  const int chunks = Kp / 8;
  for (int c = tid; c < MT * 8 * chunks; c += kSkinnyThreads) {
    const int m = c / chunks, ch = c - m * chunks;
    const bool live = m < p.M && ch * 8 < p.K;
    const bf16* src = live ? p.X + size_t(m) * p.ldx + ch * 8 : p.X;
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(xs + m * Kp + ch * 8));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(live ? 16 : 0));
  }
  asm volatile("cp.async.commit_group;\n" ::);
  asm volatile("cp.async.wait_group 0;\n" ::);
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int j = 0; j < MT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  for (int kb = kb_begin; kb < kb_end; kb += kAhead) {
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      const uint4 va = a_cur[i][0], vb = a_cur[i][1];
      load_w(kb + kAhead + i, a_cur[i][0], a_cur[i][1]);           // refill the slot at once
      if (kb + i < kb_end) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          const uint4 x = *reinterpret_cast<const uint4*>(xs + (8 * j + g) * Kp + (kb + i) * 32 + 8 * t4);
          mma_16816(acc[j], va.x, vb.x, va.y, vb.y, x.x, x.y);
          mma_16816(acc[j], va.z, vb.z, va.w, vb.w, x.z, x.w);
        }
      }
    }
  }

  // acc[j]: c0,c1 = (W row g, batch 8j + 2t, +1); c2,c3 = (W row g+8, same batch rows)
  float* mine = red + warp * 16 * (MT * 8);
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    mine[g * (MT * 8) + 8 * j + 2 * t4] = acc[j][0];
    mine[g * (MT * 8) + 8 * j + 2 * t4 + 1] = acc[j][1];
    mine[(g + 8) * (MT * 8) + 8 * j + 2 * t4] = acc[j][2];
    mine[(g + 8) * (MT * 8) + 8 * j + 2 * t4 + 1] = acc[j][3];
  }
  __syncthreads();
  // one thread per (tile in block, W row, batch row): sum the KW partials in warp order
  OutT* Y = reinterpret_cast<OutT*>(p.Y);
  for (int i = tid; i < tiles_per_block * 16 * MT * 8; i += kSkinnyThreads) {
    const int tl = i / (16 * MT * 8), rem = i - tl * (16 * MT * 8);
    const int r = rem / (MT * 8), m = rem - r * (MT * 8);
    const int n = (blockIdx.x * tiles_per_block + tl) * 16 + r;
    if (n >= p.N || m >= p.M) continue;
    float s = 0.f;
    for (int w = 0; w < p.kw; ++w) s += red[(tl * p.kw + w) * 16 * (MT * 8) + r * (MT * 8) + m];
    stf(Y + size_t(m) * p.ldy + n, s);
  }
}

template <int MT, typename OutT>
int launch_skinny(const SkinnyParams& p, cudaStream_t s) {
  auto kernel = gemm_skinny_kernel<MT, OutT>;
  const int Kb = (p.K + 31) / 32;
  const size_t smem = size_t(MT) * 8 * (Kb * 32 + 8) * sizeof(bf16) + size_t(kSkinnyWarps) * 16 * MT * 8 * sizeof(float);
  if (smem > 200 * 1024) return KVCM_ERR_UNSUPPORTED;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = smem;
  }
  const int tiles = (p.N + 15) / 16;
  const int tiles_per_block = kSkinnyWarps / p.kw;
  const int blocks = (tiles + tiles_per_block - 1) / tiles_per_block;
  return pdl_launch(kernel, dim3(blocks), dim3(kSkinnyThreads), smem, s, p);
}

}  // namespace kvcm

using namespace kvcm;

// Largest K the kernel can stage for M rows (shared memory), so that callers can ask first.
KVCM_API int kvcm_gemm_skinny_supports(int M, int N, int K) {
  if (M < 1 || M > 16 || N < 1 || K < 8 || (K % 8)) return 0;
  const int MT = M <= 8 ? 1 : 2;
  const int Kb = (K + 31) / 32;
  const size_t smem = size_t(MT) * 8 * (Kb * 32 + 8) * 2 + size_t(kSkinnyWarps) * 16 * MT * 8 * 4;
  return smem <= 200 * 1024;
}

// out_f32: 0 = bfloat16 result, 1 = float result.  kw: warps along K per tile (0 = choose).
KVCM_API int kvcm_gemm_skinny_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                                   int ldw, int ldy, int out_f32, int kw, int sm_count, void* stream) {
  if (M == 0 || N == 0) return 0;
  if (!kvcm_gemm_skinny_supports(M, N, K) || (ldw % 8) || (ldx % 8)) return KVCM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(X) & 15)) return KVCM_ERR_UNSUPPORTED;
  if (kw == 0) {
    // Fewest warps along K that still give about two blocks per SM; each warp keeps >= 4 k-blocks.
    const int tiles = (N + 15) / 16;
    const int Kb = (K + 31) / 32;
    kw = 1;
    while (kw < 8 && (tiles * kw + kSkinnyWarps - 1) / kSkinnyWarps < 2 * sm_count && Kb / (kw * 2) >= 4) kw *= 2;
  }
  if (kw != 1 && kw != 2 && kw != 4 && kw != 8) return KVCM_ERR_UNSUPPORTED;
  SkinnyParams p{(const bf16*)W, N, K, ldw, (const bf16*)X, ldx, M, Y, ldy, kw};
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 8) return out_f32 ? launch_skinny<1, float>(p, s) : launch_skinny<1, bf16>(p, s);
  return out_f32 ? launch_skinny<2, float>(p, s) : launch_skinny<2, bf16>(p, s);
}
