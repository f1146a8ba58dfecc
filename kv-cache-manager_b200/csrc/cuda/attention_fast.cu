// bfloat16 decode attention over the paged cache on tensor cores (m16n8k16, float accumulate).
//
// decode  : one query token per request.  One block per (context partition, KV head x tile of 16
//           query heads, request): the query heads that share a KV head are the 16 rows of the
//           tile, so every key and value is read once for the whole group (the reference's kernel
//           has the same aim, src/cuda/paged_attention.cu:3-4).  The context is split into
//           partitions so that small batches still fill the GPU; partial (max, sum, output) are
//           merged as in the reference's v2 (:186-203): up to 8 partitions are the blocks of one
//           thread-block cluster, which read one another's partial results from shared memory
//           and each write a share of the outputs; more partitions go through global memory and
//           a second kernel.  With one partition the block writes the result itself (v1).
// (Portions of more than one token: attention_tcgen05.cu and attention_prefill_mma.cu.)
// Any head_dim that is a multiple of 16 up to 256, any page size, any number of heads and groups,
// optional window (keys t > position - window).  Scores are scaled in float after the product;
// softmax by exp2 with log2(e) folded into the scale; probabilities are rounded to bfloat16 for
// the P*V product, sums stay float.
#include <cooperative_groups.h>

#include "attention_mma.cuh"
#include "pdl.cuh"

namespace kvcm {

// Decode keeps STAGES key/value tiles in flight per block: 3 when few blocks must hide the memory
// latency themselves, 2 (less shared memory, more blocks per SM) when the grid is large.

struct DecodeParams {
  const bf16* q; int q_stride;
  bf16* out; int out_stride;
  const bf16* k_cache; const bf16* v_cache;
  const int* block_tables; int max_blocks;
  const int* seq_ctx_len;
  float* part_o; float* part_ml;
  int nh, nkv, block_size, window, part_size, num_parts;
  float scale_log2;
  int log2_block;                      // log2(block_size) when it is a power of two, else -1
  int cluster_merge;                   // the partitions of a (request, head group) are one cluster
};

constexpr int kTabMax = 512;         // page-table entries of a partition kept in shared memory
constexpr int kMaxClusterParts = 8;      // the portable cluster size: any GPC can place it

// Four adjacent outputs: one 8-byte store where the address allows it.
__device__ __forceinline__ void store_out4(bf16* dst, float a, float b, float c, float d) {
  if ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    uint2 packed;
    packed.x = pack_bf16(a, b);
    packed.y = pack_bf16(c, d);
    *reinterpret_cast<uint2*>(dst) = packed;
  } else {
    dst[0] = __float2bfloat16_rn(a); dst[1] = __float2bfloat16_rn(b);
    dst[2] = __float2bfloat16_rn(c); dst[3] = __float2bfloat16_rn(d);
  }
}

// Merge of the partitions inside a cluster.  Every block has put its partial result for the 16
// heads of the tile into its own shared memory (bo [16][HD], bm [16] max, bl [16] sum; an empty
// partition has max = -inf).  The outputs are dealt out over the blocks of the cluster; each
// reads all partitions' values through distributed shared memory and adds them in partition
// order.
template <int HD>
__device__ __forceinline__ void cluster_merge_tail(const DecodeParams& p, int seq, int head0, int heads_here,
                                                   float* bo, float* bm, float* bl) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();                                                  // every block's partial result is in place
  const int P = p.num_parts;
  // An item is four adjacent elements of one head's output; the items are dealt out over the blocks
  // of the cluster.  Every block's (max, sum, values) for the item are asked for at once: one trip
  // through the cluster's shared memory, not one per partition; the weights 2^(m_p - M) are
  // formed once per item.
  constexpr int Q4 = HD / 4;
  for (int it = int(cluster.block_rank()) * kAttnThreads + threadIdx.x; it < heads_here * Q4; it += P * kAttnThreads) {
    const int r = it / Q4, d = (it - r * Q4) * 4;
    float mp[kMaxClusterParts], lp[kMaxClusterParts];
    float4 op[kMaxClusterParts];
#pragma unroll
    for (int i = 0; i < kMaxClusterParts; ++i) {
      mp[i] = -INFINITY; lp[i] = 0.f; op[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < P) {
        mp[i] = *cluster.map_shared_rank(bm + r, i);
        lp[i] = *cluster.map_shared_rank(bl + r, i);
        op[i] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(bo + r * HD + d, i));
      }
    }
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxClusterParts; ++i) M = fmaxf(M, mp[i]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxClusterParts; ++i) {
      if (mp[i] == -INFINITY) continue;                            // an empty partition left no output (its bo is not written)
      const float f = fast_exp2(mp[i] - M);
      acc.x = __fmaf_rn(f, op[i].x, acc.x); acc.y = __fmaf_rn(f, op[i].y, acc.y);
      acc.z = __fmaf_rn(f, op[i].z, acc.z); acc.w = __fmaf_rn(f, op[i].w, acc.w);
      L = __fmaf_rn(f, lp[i], L);
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    store_out4(p.out + size_t(seq) * p.out_stride + size_t(head0 + r) * HD + d, acc.x * inv, acc.y * inv, acc.z * inv,
               acc.w * inv);
  }
  cluster.sync();                                                  // nobody leaves while its memory is read
}

// Shared memory of the decode kernel without the page-table slice: the larger of the tiles of
// the key loop and the buffers of the merge that reuse them.
template <int HD, int kKVStages> constexpr size_t decode_core_smem() {
  const size_t tiles = size_t(16 + 2 * kKVStages * kKeyTile) * (HD + 8) * sizeof(bf16);
  const size_t merge = size_t(16) * (HD + 8) * sizeof(bf16) + (size_t(5) * 16 * HD + 2 * 4 * 16 + 32) * sizeof(float);
  return tiles > merge ? tiles : merge;
}

template <int HD, int kKVStages>
__global__ void __launch_bounds__(kAttnThreads)
attn_decode_kernel(DecodeParams p) {
  constexpr int LD = HD + 8;
  constexpr bool Q_IN_REGS = HD <= 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qtile = reinterpret_cast<bf16*>(smem_raw);                 // [16][LD]
  bf16* kbuf = qtile + 16 * LD;                                    // [stages][64][LD]
  bf16* vbuf = kbuf + kKVStages * kKeyTile * LD;                   // [stages][64][LD]
  int* stab = reinterpret_cast<int*>(smem_raw + decode_core_smem<HD, kKVStages>());   // [kTabMax]

  // Until pdl_wait() only what no kernel of this step writes is read: the batch's integer arrays
  // and the keys and values of earlier tokens.  The query and the newest key and value come from
  // the kernel before this one.
  pdl_launch_dependents();
  const int part = blockIdx.x, seq = blockIdx.z;
  const int G = p.nh / p.nkv;
  const int head_tiles = (G + 15) / 16;
  const int kvh = blockIdx.y / head_tiles, ht = blockIdx.y - kvh * head_tiles;
  const int head0 = kvh * G + ht * 16;
  const int heads_here = min(16, G - ht * 16);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int ctx = p.seq_ctx_len[seq];
  const int lo = (p.window > 0 && ctx > p.window) ? ctx - p.window : 0;
  const int begin = max(lo, part * p.part_size);
  const int end = min(ctx, (part + 1) * p.part_size);
  float* mo = reinterpret_cast<float*>(kbuf);                       // [4][16][HD]   (after the key loop)
  float* mm = mo + 4 * 16 * HD;                                     // [4][16]
  float* mlsum = mm + 4 * 16;                                       // [4][16]
  float* bo = mlsum + 4 * 16;                                       // [16][HD] the block's result (cluster merge)
  float* bm = bo + 16 * HD;                                         // [16]
  float* bl = bm + 16;                                              // [16]
  if (begin >= end) pdl_wait();
  if (begin >= end && p.cluster_merge) {                           // nothing to read here, but the cluster waits
    if (tid < 16) { bm[tid] = -INFINITY; bl[tid] = 0.f; }
    cluster_merge_tail<HD>(p, seq, head0, heads_here, bo, bm, bl);
    return;
  }
  if (begin >= end) {                                              // nothing to read here
    for (int i = tid; i < heads_here * HD; i += kAttnThreads) {
      const int r = i / HD, d = i - r * HD;
      if (p.num_parts == 1) {
        p.out[size_t(seq) * p.out_stride + size_t(head0 + r) * HD + d] = __float2bfloat16_rn(0.f);
      } else if (d == 0) {
        float* ml = p.part_ml + ((size_t(seq) * p.nh + head0 + r) * p.num_parts + part) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }
  // The partition's slice of the page table goes to shared memory first: one memory latency
  // here instead of one inside every round of the key loop.
  const int* table = p.block_tables + size_t(seq) * p.max_blocks;
  {
    const int first_page = begin / p.block_size, n_pages = (end - 1) / p.block_size - first_page + 1;
    if (n_pages <= kTabMax) {
      for (int j = tid; j < n_pages; j += kAttnThreads) stab[j] = table[first_page + j];
      table = stab - first_page;
      __syncthreads();
    }
  }

  const int t_first = (begin / kKeyTile) * kKeyTile;
  const int n_tiles = (end - t_first + kKeyTile - 1) / kKeyTile;
  auto load_stage = [&](int i) {                                   // tile i -> ring slot i % stages
    const int sl = i % kKVStages;
    if (i < n_tiles) {
      load_kv_tiles<HD>(kbuf + sl * kKeyTile * LD, vbuf + sl * kKeyTile * LD, p.k_cache, p.v_cache, table,
                        t_first + i * kKeyTile, begin, end, kvh, p.nkv, p.block_size, tid, kAttnThreads, p.log2_block);
    }
    cp_async_commit();                                             // one group per tile, empty ones too
  };
  // Tiles that lie wholly below the newest key (position ctx - 1, written by the kernel before
  // this one) are requested before the wait; the rest of the first stages after it.
  int ahead = 0;
  for (; ahead < kKVStages - 1; ++ahead) {
    if (t_first + (ahead + 1) * kKeyTile > ctx - 1) break;
    load_stage(ahead);
  }
  pdl_wait();
  for (int c = tid; c < 16 * (HD / 8); c += kAttnThreads) {        // Q tile, zero rows beyond the group
    const int r = c / (HD / 8), ch = c - r * (HD / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < heads_here)
      v = *reinterpret_cast<const uint4*>(p.q + size_t(seq) * p.q_stride + size_t(head0 + r) * HD + ch * 8);
    *reinterpret_cast<uint4*>(qtile + r * LD + ch * 8) = v;
  }
  for (int i = ahead; i < kKVStages - 1; ++i) load_stage(i);
  __syncthreads();                                                 // qtile is written

  uint32_t qa[Q_IN_REGS ? HD / 16 : 1][4];
  if constexpr (Q_IN_REGS) load_q_frags<HD>(reinterpret_cast<uint32_t(&)[HD / 16][4]>(qa), qtile, lane);

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  // Where the 16-byte chunks of a key divide a warp, load_kv_tiles gives warp w exactly the keys
  // it works on (16 w .. 16 w + 15 of every tile): the warps then need no barrier in the key loop
  // and drift apart, each hiding the others' latencies.
  constexpr bool kWarpPrivate = (32 % (HD / 8)) == 0;
  auto round_barrier = [&]() {
    if constexpr (kWarpPrivate) __syncwarp(); else __syncthreads();
  };
  int slot = 0;                                                    // ring slot of tile i (counted along: i % stages)
  for (int i = 0; i < n_tiles; ++i) {
    const int t0 = t_first + i * kKeyTile;
    load_stage(i + kKVStages - 1);                                 // its slot was freed by the barrier that
    cp_async_wait<kKVStages - 1>();                                // ended round i - 1; tile i has landed
    round_barrier();
    const int kb = t0 + warp * 16;                                 // this warp's 16 keys
    if (kb < end && kb + 16 > begin) {
      const bf16* kt = kbuf + slot * kKeyTile * LD + warp * 16 * LD;
      const bf16* vt = vbuf + slot * kKeyTile * LD + warp * 16 * LD;
      float s[2][4];
      if constexpr (Q_IN_REGS) {
        qk_16x16<HD>(s, reinterpret_cast<const uint32_t(&)[HD / 16][4]>(qa), kt, lane);
      } else {
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) s[a][b] = 0.f;
        const int krow = (lane & 7) + ((lane >> 4) << 3), kcol = ((lane >> 3) & 1) << 3;
#pragma unroll 4
        for (int kk = 0; kk < HD / 16; ++kk) {
          uint32_t a[4], b[4];
          ldmatrix_x4(a, qtile + (lane & 15) * LD + kk * 16 + ((lane >> 4) << 3));
          ldmatrix_x4(b, kt + krow * LD + kk * 16 + kcol);
          mma_bf16(s[0], a, b[0], b[1]);
          mma_bf16(s[1], a, b[2], b[3]);
        }
      }
      if (kb >= begin && kb + 16 <= end) {                         // all sixteen keys count: no masks
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) s[h][j] *= p.scale_log2;
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int key = kb + 8 * h + 2 * t4 + (j & 1);
            s[h][j] = (key >= begin && key < end) ? s[h][j] * p.scale_log2 : -INFINITY;
          }
      }
      uint32_t pa[4];
      softmax_step<HD>(s, m, l, o, pa);
      pv_16x16<HD>(o, pa, vt, lane);
    }
    round_barrier();                                               // the buffer is loaded again next round
    if (++slot == kKVStages) slot = 0;
  }

  cp_async_wait<0>();
  __syncthreads();                                                 // the tiles give way to the merge buffers
  // ---- merge the four warps (each saw different keys) through shared memory.  An item is four
  // adjacent elements of one head's output: the weights 2^(m_w - M) are formed once per item, the
  // values move as 16-byte vectors.
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) {
    float* base = mo + (warp * 16) * HD + d * 8 + 2 * t4;
    *reinterpret_cast<float2*>(base + g * HD) = make_float2(o[d][0], o[d][1]);
    *reinterpret_cast<float2*>(base + (g + 8) * HD) = make_float2(o[d][2], o[d][3]);
  }
  if (t4 == 0) {
    mm[warp * 16 + g] = m[0];
    mm[warp * 16 + g + 8] = m[1];
    mlsum[warp * 16 + g] = l[0];
    mlsum[warp * 16 + g + 8] = l[1];
  }
  __syncthreads();
  constexpr int Q4 = HD / 4;
  for (int it = tid; it < heads_here * Q4; it += kAttnThreads) {
    const int r = it / Q4, d = (it - r * Q4) * 4;
    float mw[4], M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mw[w] = mm[w * 16 + r];
      M = fmaxf(M, mw[w]);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = (mw[w] == -INFINITY) ? 0.f : fast_exp2(mw[w] - M);
      const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * HD + d);
      acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
      L += f * mlsum[w * 16 + r];
    }
    const int head = head0 + r;
    if (p.cluster_merge) {
      *reinterpret_cast<float4*>(bo + r * HD + d) = acc;
      if (d == 0) {
        bm[r] = M;
        bl[r] = L;
      }
    } else if (p.num_parts == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      store_out4(p.out + size_t(seq) * p.out_stride + size_t(head) * HD + d, acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    } else {
      const size_t idx = (size_t(seq) * p.nh + head) * p.num_parts + part;
      *reinterpret_cast<float4*>(p.part_o + idx * HD + d) = acc;
      if (d == 0) {
        p.part_ml[idx * 2] = M;
        p.part_ml[idx * 2 + 1] = L;
      }
    }
  }
  if (p.cluster_merge) cluster_merge_tail<HD>(p, seq, head0, heads_here, bo, bm, bl);
}

// Merges the partitions of one (request, head): out = sum_p 2^(m_p - M) o_p / sum_p 2^(m_p - M) l_p.
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, int out_stride, int nh, int hd, int num_parts) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y;
  const size_t base = (size_t(seq) * nh + head) * num_parts;
  float M = -INFINITY;
  for (int i = 0; i < num_parts; ++i) M = fmaxf(M, part_ml[(base + i) * 2]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
    for (int i = 0; i < num_parts; ++i) {
      const float mp = part_ml[(base + i) * 2];
      if (mp == -INFINITY) continue;
      const float f = exp2f(mp - M);
      acc = __fmaf_rn(f, part_o[(base + i) * hd + d], acc);
      L = __fmaf_rn(f, part_ml[(base + i) * 2 + 1], L);
    }
    out[size_t(seq) * out_stride + size_t(head) * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
}

template <int HD, int kKVStages> size_t decode_smem() {
  return decode_core_smem<HD, kKVStages>() + kTabMax * sizeof(int);
}

template <int HD, int STAGES>
int launch_decode_staged(const DecodeParams& p, int seqs, cudaStream_t s) {
  auto kernel = attn_decode_kernel<HD, STAGES>;
  const size_t smem = decode_smem<HD, STAGES>();
  static bool configured = false;                                  // per instantiation, set once
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  const int G = p.nh / p.nkv;
  dim3 grid(p.num_parts, p.nkv * ((G + 15) / 16), seqs);
  if (p.cluster_merge) return pdl_launch_cluster(kernel, grid, dim3(kAttnThreads), smem, s, p.num_parts, p);
  return pdl_launch(kernel, grid, dim3(kAttnThreads), smem, s, p);
}

// Blocks of the decode kernel with STAGES key tiles in flight that the device holds at once (0 if
// it cannot say, or if a block of that many stages does not fit an SM).
template <int HD, int STAGES>
int decode_resident_blocks(int sm_count) {
  static int per_sm = -1;
  if (per_sm < 0) {
    auto kernel = attn_decode_kernel<HD, STAGES>;
    const size_t smem = decode_smem<HD, STAGES>();
    int n = 0;
    if (smem > 227 * 1024) n = 0;
    else if (smem > 48 * 1024 &&
             cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) n = 0;
    else if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kAttnThreads, smem) != cudaSuccess) n = 0;
    per_sm = n;
  }
  return per_sm * sm_count;
}

// Key tiles in flight per block: three while all blocks are resident at once; five where the
// partitions are long (a block then works through its keys at one memory latency per four tiles
// instead of per two) and the fewer, larger blocks still all fit; two for a grid too large for
// three (more blocks fit an SM: a second wave of blocks costs more than the shallower pipeline).
template <int HD>
int launch_decode(const DecodeParams& p, int seqs, int sm_count, cudaStream_t s) {
  const int G = p.nh / p.nkv;
  const long long blocks = (long long)p.num_parts * p.nkv * ((G + 15) / 16) * seqs;
  if constexpr (HD <= 128) {                                       // (five stages of larger heads do not fit an SM)
    if (p.part_size >= 5 * kKeyTile && blocks <= decode_resident_blocks<HD, 5>(sm_count))
      return launch_decode_staged<HD, 5>(p, seqs, s);
  }
  if (blocks > decode_resident_blocks<HD, 3>(sm_count)) return launch_decode_staged<HD, 2>(p, seqs, s);
  return launch_decode_staged<HD, 3>(p, seqs, s);
}

}  // namespace kvcm

using namespace kvcm;

// 1 if the tensor-core kernels take this head_dim (else the caller uses the plain kernel).
KVCM_API int kvcm_attention_fast_supports(int hd) {
#define X(N) if (hd == N) return 1;
  KVCM_FOR_HEAD_DIMS(X)
#undef X
  return 0;
}

// Floats of scratch the decode kernel needs for `seqs` requests split into `num_parts`.
KVCM_API long long kvcm_attention_decode_scratch_floats(int seqs, int nh, int hd, int num_parts) {
  return num_parts <= 1 ? 0 : (long long)seqs * nh * num_parts * (hd + 2);
}

// Blocks of the decode kernel (partitions x KV heads x tiles of 16 query heads x requests) that
// run at once with three stages of keys in flight; the caller sizes the partitions by it.
KVCM_API int kvcm_attention_decode_resident_blocks(int hd) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
#define X(N) if (hd == N) return decode_resident_blocks<N, 3>(sms);
  KVCM_FOR_HEAD_DIMS(X)
#undef X
  return 0;
}

// Most partitions that one cluster merges; with more the caller must give scratch.
KVCM_API int kvcm_attention_decode_cluster_parts(void) { return kMaxClusterParts; }

// `scratch`: kvcm_attention_decode_scratch_floats() floats, needed when num_parts > 1 unless the
// merge runs inside a cluster (cluster_merge != 0 and num_parts <= kvcm_attention_decode_cluster_parts()).
KVCM_API int kvcm_attention_decode_bf16(const void* q, int q_stride, void* out, int out_stride,
                                        const void* k_cache, const void* v_cache, const int* block_tables,
                                        int max_blocks, const int* seq_ctx_len, int seqs, int nh, int nkv,
                                        int hd, int block_size, float scale, int window, int part_size,
                                        int num_parts, float* scratch, int cluster_merge, void* stream) {
  if (seqs == 0) return 0;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  if (nkv <= 0 || nh % nkv || part_size <= 0 || part_size % kKeyTile || num_parts < 1) return KVCM_ERR_UNSUPPORTED;
  if (cluster_merge && (num_parts < 2 || num_parts > kMaxClusterParts)) cluster_merge = 0;
  if (num_parts > 1 && !cluster_merge && scratch == nullptr) return KVCM_ERR_UNSUPPORTED;
  DecodeParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.seq_ctx_len = seq_ctx_len;
  p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)seqs * nh * num_parts * hd : nullptr;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.part_size = part_size; p.num_parts = num_parts; p.cluster_merge = cluster_merge;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.log2_block = -1;
  for (int b = 0; b < 16; ++b) if ((1 << b) == block_size) p.log2_block = b;
  int rc = KVCM_ERR_UNSUPPORTED;
#define X(N) if (hd == N) rc = launch_decode<N>(p, seqs, sm_count, (cudaStream_t)stream);
  KVCM_FOR_HEAD_DIMS(X)
#undef X
  if (rc != 0 || num_parts == 1 || cluster_merge) return rc;
  return pdl_launch(attn_decode_merge_kernel, dim3(seqs, nh), dim3(hd < 64 ? 32 : 64), 0, (cudaStream_t)stream,
                    (const float*)p.part_o, (const float*)p.part_ml, p.out, out_stride, nh, hd, num_parts);
}

