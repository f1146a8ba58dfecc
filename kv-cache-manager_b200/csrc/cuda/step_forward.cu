// The forward pass of one step, launched from C++: embedding, every call site of the run order
// (RMSNorm -> paged attention with rotate-half rotary encoding -> RMSNorm -> SiLU-gated
// feed-forward, pre-norm, float residual stream), final norm on the wanted rows and the output head.
//
// This file holds no kernel.  It is the host-side loop that the step function would otherwise run
// in Python, one ctypes call and a few tensor objects per launch (about 8 us each, 3.7 ms for a
// prefill step of 22 layers): the same launchers, in the same order, chosen by the same rules, called
// directly.  The order and the formulas are the reference's forward (src/model/llama.cpp:84-139);
// which product kernel runs is this engine's own dispatch (parts/linear.py gives the reasons):
//   float32 storage  -> the plain kernels throughout (the true 32-bit path);
//   bfloat16 storage -> the weight-streaming kernel for a handful of rows, with the rotary encoding
//                       and the cache write (qkv) or SiLU*up (gate/up) in its epilogue; the tcgen05
//                       kernel with the gated epilogue for the gate/up product of many rows; the
//                       library product (cuBLAS, where the reference calls it too) for the rest.
// The caller (engine/native_forward.py) checks that the model is made of exactly these parts, owns
// every buffer, and falls back to the part-by-part path for anything else.
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "../include/forward_args.h"
#include "common.cuh"

extern "C" {
// launchers of the other files of this library (C ABI; see each file for the contract)
int kvcm_embed_f32(const int*, const void*, float*, int, int, int, void*);
int kvcm_embed_bf16(const int*, const void*, float*, int, int, int, void*);
int kvcm_rmsnorm_f32(float*, const void*, const void*, int, void*, const int*, int, int, float, void*);
int kvcm_rmsnorm_bf16(float*, const void*, const void*, int, void*, const int*, int, int, float, void*);
int kvcm_rope_cache_f32(void*, int, const int*, const float*, int, int, const int*, void*, void*, int, int, int, int, int, int, void*);
int kvcm_rope_cache_bf16(void*, int, const int*, const float*, int, int, const int*, void*, void*, int, int, int, int, int, int, void*);
int kvcm_silu_mul_f32(const void*, void*, int, int, void*);
int kvcm_silu_mul_bf16(const void*, void*, int, int, void*);
int kvcm_gemm_plain_f32(const void*, const void*, void*, int, int, int, int, int, int, void*);
int kvcm_attention_plain_f32(const void*, int, void*, int, const void*, const void*, const int*, int, const int*, const int*,
                             int, int, int, int, int, float, int, void*);
int kvcm_attention_plain_bf16(const void*, int, void*, int, const void*, const void*, const int*, int, const int*, const int*,
                              int, int, int, int, int, float, int, void*);
int kvcm_attention_fast_supports(int);
int kvcm_attention_decode_resident_blocks(int);
int kvcm_attention_decode_cluster_parts(void);
int kvcm_attention_decode_bf16(const void*, int, void*, int, const void*, const void*, const int*, int, const int*, int, int,
                               int, int, int, float, int, int, int, float*, int, void*);
int kvcm_attention_tcgen05_supports(int, int);
int kvcm_attention_prefill_tcgen05_bf16(const void*, int, int, void*, int, const void*, const void*, int, const int*, int,
                                        const int*, const int*, const int*, const int*, const int*, int, int, int, int, int,
                                        float, int, void*);
int kvcm_attention_prefill_bf16(const void*, int, void*, int, const void*, const void*, const int*, int, const int*,
                                const int*, const int*, const int*, const int*, int, int, int, int, int, float, int, void*);
int kvcm_gemm_stream_supports(int, int, int);
int kvcm_gemm_stream_fused_supports(int, int, int);
int kvcm_gemm_stream_bf16(const void*, const void*, void*, int, int, int, int, int, int, int, int, void*);
int kvcm_qkv_rope_cache_bf16(const void*, const void*, void*, int, int, int, int, int, const int*, const float*, const int*,
                             void*, void*, int, int, int, int, int, void*);
int kvcm_gate_up_silu_bf16(const void*, const void*, void*, int, int, int, int, int, int, int, void*);
int kvcm_gemm_tcgen05_supports(int, int, int, int, int);
int kvcm_rope_table_f32(const int*, const float*, int, int, float*, void*);
int kvcm_rope_cache_table_supports(const void*, int, const void*, const void*, const void*, int);
int kvcm_rope_cache_table_bf16(void*, int, const float*, const int*, void*, void*, int, int, int, int, int, int, void*);
int kvcm_gemm_stream_residual_bf16(const void*, const void*, float*, float*, void*, const void*, int, int, int, int, int, int,
                                   int, int, void*);
int kvcm_qkv_rope_cache_scaled_bf16(const void*, const float*, int, float, const void*, void*, int, int, int, int, int,
                                    const int*, const float*, const int*, void*, void*, int, int, int, int, int, void*);
int kvcm_gate_up_silu_scaled_bf16(const void*, const float*, int, float, const void*, void*, int, int, int, int, int, int, int,
                                  void*);
int kvcm_gate_up_silu_tcgen05_bf16(const void*, const void*, void*, int, int, int, int, int, int, void*);
}

namespace {

constexpr int kMaxGroups = KVCM_FORWARD_MAX_GROUPS;
constexpr long long kStreamMaxBytes = 32ll << 20;       // parts/linear.py: STREAM_MAX_BYTES
constexpr int kTcgen05MinRows = 256;                    // TCGEN05_MIN_ROWS
constexpr int kTcgen05GatedMaxHidden = 3072;            // TCGEN05_GATED_MAX_HIDDEN
constexpr int kKeyTile = 64;
constexpr int kRopeTableMinRows = 64;                   // from here on the angles are computed once a step
// Most rows of a step whose norms ride in its products (a decode step of the 1.1B shape, with and
// without: 1 row 881 -> 809 us, 4 rows 902 -> 837, 8 rows 916 -> 869, 16 rows 1171 -> 1180).
constexpr int kNormRideMaxRows = 8;

}  // namespace

namespace {

struct Library {                                        // one cuBLAS handle per device
  cublasHandle_t handle[64] = {};
  std::mutex lock;
  cublasHandle_t get() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> g(lock);
    if (handle[dev] == nullptr && cublasCreate(&handle[dev]) != CUBLAS_STATUS_SUCCESS) handle[dev] = nullptr;
    return handle[dev];
  }
};
Library g_library;

// y[M,N] = x[M,K] w[N,K]^T with the library: bfloat16 operands, float accumulation.
int library_gemm(const KvcmForwardArgs& a, const void* x, const void* w, void* y, int M, int N, int K, bool out_f32,
                 cudaStream_t s) {
  cublasHandle_t h = g_library.get();
  if (h == nullptr) return KVCM_ERR_UNSUPPORTED;
  if (cublasSetStream(h, s) != CUBLAS_STATUS_SUCCESS) return KVCM_ERR_UNSUPPORTED;
  // a workspace of the caller's: the library must not allocate while a CUDA graph is recorded
  if (a.lib_workspace != nullptr &&
      cublasSetWorkspace(h, a.lib_workspace, size_t(a.lib_workspace_bytes)) != CUBLAS_STATUS_SUCCESS)
    return KVCM_ERR_UNSUPPORTED;
  const float alpha = 1.f, beta = 0.f;
  // row-major y = x w^T  <=>  column-major y^T[N,M] = w[K,N]^T x^T[K,M]
  const cublasStatus_t st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, K, x, CUDA_R_16BF, K,
                                         &beta, y, out_f32 ? CUDA_R_32F : CUDA_R_16BF, N, CUBLAS_COMPUTE_32F,
                                         CUBLAS_GEMM_DEFAULT);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 20000 + int(st);
}

// The product of a part: which kernel, by the rules of parts/linear.py ('auto').
int product(const KvcmForwardArgs& a, const void* x, const void* w, void* y, int M, int N, int K, bool out_f32,
            cudaStream_t s) {
  if (M == 0) return 0;
  if (a.f32) return kvcm_gemm_plain_f32(x, w, y, M, N, K, K, K, N, s);
  if ((M <= 8 || (long long)N * K * 2 <= kStreamMaxBytes) && kvcm_gemm_stream_supports(M, N, K))
    return kvcm_gemm_stream_bf16(x, w, y, M, N, K, K, K, N, out_f32 ? 1 : 0, a.sm_count, s);
  return library_gemm(a, x, w, y, M, N, K, out_f32, s);
}

bool tiles_fill_well(int M, int N, int sms) {
  const long long tiles = (long long)((M + 127) / 128) * ((N + 255) / 256);
  const long long rounds = (tiles + sms - 1) / sms;
  return tiles >= sms && tiles * 10 >= 8 * rounds * sms;
}

// How decode attention splits the context (kernels/library.py: decode_partitions, 'auto').
void decode_partitions(int seqs, int nh, int nkv, int hd, int max_ctx, int* size, int* parts) {
  max_ctx = std::max(max_ctx, 1);
  const int G = nh / nkv;
  const int blocks = std::max(1, seqs * nkv * ((G + 15) / 16));
  static int resident_hd = -1, resident = 0;
  if (resident_hd != hd) {
    resident = kvcm_attention_decode_resident_blocks(hd);
    resident_hd = hd;
  }
  int sms = 0, dev = 0;
  if (resident <= 0 && cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int res = resident > 0 ? resident : 3 * std::max(sms, 1);
  const int cluster = kvcm_attention_decode_cluster_parts();
  int p = std::max(1, std::min(res / blocks, max_ctx / 128));
  if (p > cluster) p = std::max(cluster, std::min(p, (max_ctx + 511) / 512));
  *size = ((max_ctx + p - 1) / p + kKeyTile - 1) / kKeyTile * kKeyTile;
  *parts = (max_ctx + *size - 1) / *size;
}

int attention(const KvcmForwardArgs& a, const KvcmForwardLayer& L, const void* q, int q_stride, int& launches,
              cudaStream_t s) {
  const int* tables = a.group_tables[L.group];
  if (a.f32 || !kvcm_attention_fast_supports(a.hd) || a.nh % a.nkv) {
    ++launches;
    return (a.f32 ? kvcm_attention_plain_f32 : kvcm_attention_plain_bf16)(
        q, q_stride, a.attn, a.nh * a.hd, L.k_cache, L.v_cache, tables, a.max_blocks, a.row_seq, a.positions, a.rows, a.nh,
        a.nkv, a.hd, a.block_size, a.scale, L.window, s);
  }
  int rc = 0;
  const int nd = a.decode_seqs;
  if (nd > 0) {
    int size = 0, parts = 1;
    decode_partitions(nd, a.nh, a.nkv, a.hd, a.max_decode_ctx, &size, &parts);
    const int cluster = kvcm_attention_decode_cluster_parts();
    int in_cluster = parts > 1 && parts <= cluster;
    if (parts > 1 && !in_cluster && (long long)nd * a.nh * parts * (a.hd + 2) > a.attn_scratch_floats)
      return KVCM_ERR_UNSUPPORTED;                                  // the caller sizes the scratch for its limits
    rc = kvcm_attention_decode_bf16(q, q_stride, a.attn, a.nh * a.hd, L.k_cache, L.v_cache, tables, a.max_blocks,
                                    a.seq_ctx_len, nd, a.nh, a.nkv, a.hd, a.block_size, a.scale, L.window, size, parts,
                                    a.attn_scratch, in_cluster, s);
    if (rc) return rc;
    launches += (parts > 1 && !in_cluster) ? 2 : 1;
  }
  if (a.rows > nd) {
    if (a.tile_rows != 64) return KVCM_ERR_UNSUPPORTED;
    ++launches;
    if (kvcm_attention_tcgen05_supports(a.hd, a.block_size) && (q_stride % 8) == 0)
      return kvcm_attention_prefill_tcgen05_bf16(q, q_stride, a.rows, a.attn, a.nh * a.hd, L.k_cache, L.v_cache, L.num_pages,
                                                 tables, a.max_blocks, a.tile_seq, a.tile_q0, a.seq_q_start, a.seq_q_len,
                                                 a.seq_ctx_len, a.prefill_tiles, a.nh, a.nkv, a.hd, a.block_size, a.scale,
                                                 L.window, s);
    return kvcm_attention_prefill_bf16(q, q_stride, a.attn, a.nh * a.hd, L.k_cache, L.v_cache, tables, a.max_blocks,
                                       a.tile_seq, a.tile_q0, a.seq_q_start, a.seq_q_len, a.seq_ctx_len, a.prefill_tiles,
                                       a.nh, a.nkv, a.hd, a.block_size, a.scale, L.window, s);
  }
  return rc;
}

}  // namespace

#define KVCM_TRY(expr)        \
  do {                        \
    const int rc_ = (expr);   \
    if (rc_ != 0) return rc_; \
  } while (0)

// Runs the step.  Only enqueues device work on `stream`; returns the first non-zero launch result.
// `launches` (optional) receives the number of launches made.
KVCM_API int kvcm_forward(const KvcmForwardArgs* ap, int* launches, void* stream) {
  const KvcmForwardArgs& a = *ap;
  cudaStream_t s = (cudaStream_t)stream;
  int n = 0;
  if (launches) *launches = 0;
  if (a.rows == 0) return 0;
  if (a.num_layers < 0 || a.H <= 0 || a.nkv <= 0 || a.nh % a.nkv) return KVCM_ERR_UNSUPPORTED;
  const int T = a.rows, H = a.H, I = a.I, QK = a.nh * a.hd, QKV = (a.nh + 2 * a.nkv) * a.hd;
  const auto embed = a.f32 ? kvcm_embed_f32 : kvcm_embed_bf16;
  const auto rmsnorm = a.f32 ? kvcm_rmsnorm_f32 : kvcm_rmsnorm_bf16;
  const auto rope_cache = a.f32 ? kvcm_rope_cache_f32 : kvcm_rope_cache_bf16;
  const auto silu_mul = a.f32 ? kvcm_silu_mul_f32 : kvcm_silu_mul_bf16;

  // A handful of rows: the products that end a sublayer add into the residual themselves, leave
  // partial sums of squares and the next norm's row before its scale (a.h); the products that
  // begin the next sublayer scale their sums by the norm's 1/rms.  No norm launches between them.
  const int ss_tiles = (H + 15) / 16;
  const auto streams = [&](int N, int K) {
    return (T <= 8 || (long long)N * K * 2 <= kStreamMaxBytes) && kvcm_gemm_stream_supports(T, N, K);
  };
  const bool may_ride = !a.f32 && a.norm_partials != nullptr && a.norm_partials_floats >= (long long)ss_tiles * 16 &&
                        T <= kNormRideMaxRows;
  // (each sublayer by itself: where the down product is too wide for the streaming kernel, as at the
  // Llama-3-8B shape, the attention sublayer still closes this way)
  const bool ride_attn = may_ride && streams(H, QK), ride_ffn = may_ride && streams(H, I);
  const bool gate_fused = !a.f32 && (I % 8) == 0 && kvcm_gemm_stream_fused_supports(T, 2 * I, H);
  const auto qkv_fused = [&](const KvcmForwardLayer& L) {
    return !a.f32 && L.writes && (a.hd % 16) == 0 && kvcm_gemm_stream_fused_supports(T, QKV, H);
  };

  KVCM_TRY(embed(a.tokens, a.embed, a.x, T, H, a.V, s)); ++n;
  bool table_filled = false;                            // the step's cosines and sines are in a.rope_table
  const void* pending = nullptr;                        // a sublayer's result not yet added to the residual
  bool handed = false;                                  // a.h and norm_partials hold the next norm's row before its scale
  // ends a sublayer: x += y w^T, one way or the other (next_norm: the norm weight of the product
  // that follows, where that product takes the scaled form)
  const auto close_sublayer = [&](const void* y, const void* w, int K, const void* next_norm, bool ride) {
    pending = nullptr;
    handed = false;
    if (ride) {
      handed = next_norm != nullptr;
      return kvcm_gemm_stream_residual_bf16(y, w, a.x, a.norm_partials, a.h, next_norm, T, H, K, K, K, H, H, a.sm_count, s);
    }
    pending = a.proj;
    return product(a, y, w, a.proj, T, H, K, false, s);
  };
  for (int l = 0; l < a.num_layers; ++l) {
    const KvcmForwardLayer& L = a.layers[l];
    if (L.group < 0 || L.group >= kMaxGroups) return KVCM_ERR_UNSUPPORTED;
    // attention: qkv product, rotary encoding, cache write -- one kernel for a handful of rows
    const void* q = a.qkv;
    int q_stride = QKV;
    if (!handed) { KVCM_TRY(rmsnorm(a.x, pending, L.norm1, 0, a.h, nullptr, T, H, L.eps1, s)); ++n; }
    if (qkv_fused(L)) {
      KVCM_TRY(kvcm_qkv_rope_cache_scaled_bf16(a.h, handed ? a.norm_partials : nullptr, ss_tiles, L.eps1, L.w_qkv, a.qkv, T, H,
                                               H, H, QK, a.positions, a.inv_freq, a.group_slots[L.group], L.k_cache,
                                               L.v_cache, a.nh, a.nkv, a.hd, a.block_size, a.sm_count, s));
      ++n;
      q_stride = QK;
    } else {
      KVCM_TRY(product(a, a.h, L.w_qkv, a.qkv, T, QKV, H, false, s)); ++n;
      // the angles are the same in every layer: with many rows they are computed once a step
      if (!a.f32 && T >= kRopeTableMinRows && a.rope_table != nullptr && a.rope_table_floats >= (long long)T * a.hd &&
          kvcm_rope_cache_table_supports(a.qkv, QKV, L.k_cache, L.v_cache, a.rope_table, a.hd)) {
        if (!table_filled) {
          KVCM_TRY(kvcm_rope_table_f32(a.positions, a.inv_freq, T, a.hd / 2, a.rope_table, s)); ++n;
          table_filled = true;
        }
        KVCM_TRY(kvcm_rope_cache_table_bf16(a.qkv, QKV, a.rope_table, a.group_slots[L.group], L.k_cache, L.v_cache, T, a.nh,
                                            a.nkv, a.hd, a.block_size, L.writes, s));
      } else {
        KVCM_TRY(rope_cache(a.qkv, QKV, a.positions, a.inv_freq, a.hd, 0, a.group_slots[L.group], L.k_cache, L.v_cache, T,
                            a.nh, a.nkv, a.hd, a.block_size, L.writes, s));
      }
      ++n;
    }
    KVCM_TRY(attention(a, L, q, q_stride, n, s));
    KVCM_TRY(close_sublayer(a.attn, L.w_o, QK, gate_fused ? L.norm2 : nullptr, ride_attn)); ++n;
    // feed-forward: gate/up product and activation -- one kernel where one exists for the shape
    if (!handed) { KVCM_TRY(rmsnorm(a.x, pending, L.norm2, 0, a.h, nullptr, T, H, L.eps2, s)); ++n; }
    if (gate_fused) {
      KVCM_TRY(kvcm_gate_up_silu_scaled_bf16(a.h, handed ? a.norm_partials : nullptr, ss_tiles, L.eps2, L.w_gate_up, a.act, T,
                                             I, H, H, H, I, a.sm_count, s));
      ++n;
    } else if (!a.f32 && T >= kTcgen05MinRows && tiles_fill_well(T, 2 * I, a.sm_count) && H <= kTcgen05GatedMaxHidden &&
               kvcm_gemm_tcgen05_supports(T, 2 * I, H, H, H)) {
      KVCM_TRY(kvcm_gate_up_silu_tcgen05_bf16(a.h, L.w_gate_up, a.act, T, I, H, H, H, I, s)); ++n;
    } else {
      KVCM_TRY(product(a, a.h, L.w_gate_up, a.gate_up, T, 2 * I, H, false, s)); ++n;
      KVCM_TRY(silu_mul(a.gate_up, a.act, T, I, s)); ++n;
    }
    const bool next_takes = l + 1 < a.num_layers && qkv_fused(a.layers[l + 1]);
    KVCM_TRY(close_sublayer(a.act, L.w_down, I, next_takes ? a.layers[l + 1].norm1 : nullptr, ride_ffn)); ++n;
  }
  if (a.num_logits > 0) {
    KVCM_TRY(rmsnorm(a.x, pending, a.final_norm, 0, a.h_last, a.logit_rows, a.num_logits, H, a.final_eps, s)); ++n;
    if (a.f32) {
      KVCM_TRY(kvcm_gemm_plain_f32(a.h_last, a.lm_head, a.logits, a.num_logits, a.V, H, H, H, a.V, s));
    } else {
      KVCM_TRY(product(a, a.h_last, a.lm_head, a.logits, a.num_logits, a.V, H, true, s));
    }
    ++n;
  }
  if (launches) *launches = n;
  return 0;
}

KVCM_API int kvcm_forward_args_bytes(void) { return int(sizeof(KvcmForwardArgs)); }
KVCM_API int kvcm_forward_layer_bytes(void) { return int(sizeof(KvcmForwardLayer)); }
