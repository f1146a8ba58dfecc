// The argument blocks of the step's forward pass (csrc/cuda/step_forward.cu: kvcm_forward), shared by
// the kernel library, which runs it, and the CPU core, whose engine loop fills it.  Plain C layout.
#pragma once

#define KVCM_FORWARD_MAX_GROUPS 4

// One call site of the run order (host array).
struct KvcmForwardLayer {
  const void* w_qkv; const void* w_o; const void* w_gate_up; const void* w_down;
  const void* norm1; const void* norm2;
  void* k_cache; void* v_cache;
  float eps1, eps2;
  int group, window, writes, num_pages;
};

struct KvcmForwardArgs {
  // the model (fixed for an engine)
  const KvcmForwardLayer* layers;                       // host memory
  const void* embed; const void* final_norm; const void* lm_head;
  const float* inv_freq;
  // the step: the batch's integer arrays on the device
  const int* tokens; const int* positions; const int* row_seq; const int* seq_q_start; const int* seq_q_len;
  const int* seq_ctx_len; const int* tile_seq; const int* tile_q0; const int* logit_rows;
  const int* group_tables[KVCM_FORWARD_MAX_GROUPS]; const int* group_slots[KVCM_FORWARD_MAX_GROUPS];
  // buffers of the caller, sized for the step: x [T,H] float; h, proj [T,H]; qkv [T,QKV]; attn [T,nh*hd];
  // gate_up [T,2I]; act [T,I]; h_last [L,H]; logits [L,V] float; attn_scratch floats; a library workspace;
  // norm_partials: ceil(H/16)*16 floats, or null = every norm is a launch of its own (with it, a step
  // of at most 8 rows adds the residual and takes the norms inside its products)
  float* x; void* h; void* qkv; void* attn; void* proj; void* gate_up; void* act; void* h_last; float* logits;
  // rope_table: rows x hd floats, or null = every layer's rotary kernel computes its angles itself
  float* attn_scratch; void* lib_workspace; float* norm_partials; float* rope_table;
  long long attn_scratch_floats, lib_workspace_bytes, norm_partials_floats, rope_table_floats;
  int num_layers, f32, H, I, nh, nkv, hd, V, block_size, max_blocks, sm_count;
  int rows, seqs, decode_seqs, prefill_tiles, tile_rows, max_decode_ctx, num_logits, reserved;
  float final_eps, scale;
};

