// Turns "these requests, these portions" into the integer arrays one step of the model needs,
// packed into ONE host buffer so that a step costs one host-to-device copy (as the reference's
// forward does, src/model/llama.cpp:65-81; arrays as its ForwardBatch, src/model/llama.h:15-33).
//
// Rows are laid out with single-token entries (decodes) first and longer portions after them,
// so that the two attention kernels each take one contiguous range of rows.  Arrays:
//   tokens[T] positions[T] row_seq[T]          per row
//   slot_mapping[G][T]                          per group and row: page*B + offset, -1 = skip
//   seq_q_start[S] seq_q_len[S] seq_ctx_len[S] seq_state_slot[S]   per entry (ctx = start + n)
//   logit_rows[L]                               rows whose logits are wanted, in the caller's order
//   tile_seq[NT] tile_q0[NT]                    prefill work items: entry and first local row
//   block_tables[G][S][max_blocks]              page tables, -1 where no page is held
// Padding (decode steps replayed from a captured graph need fixed shapes): rows and entries up
// to pad_rows / pad_seqs are filled with slot -1, context 0, token 0; logit_rows is filled up to
// pad_logit_rows with row 0 (those logits are computed and ignored).
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "sequence.h"

namespace kvcm {

struct BatchEntry {
  const Sequence* seq = nullptr;
  int start = 0;               // first position of the portion
  int num_tokens = 0;
  std::vector<int32_t> want;   // places inside the portion whose logits are wanted
};

struct BatchLayout {
  int rows = 0, seqs = 0, logit_rows = 0, groups = 0, max_blocks = 0;
  int real_rows = 0, real_seqs = 0;       // before padding
  int decode_seqs = 0;                    // entries [0, decode_seqs) are single rows
  int prefill_rows = 0, prefill_tiles = 0, tile_rows = 0;
  int max_ctx = 0, max_decode_ctx = 0, max_q_len = 0;
  // offsets into the packed buffer, in int32 units
  int64_t off_tokens = 0, off_positions = 0, off_row_seq = 0, off_slot_mapping = 0;
  int64_t off_seq_q_start = 0, off_seq_q_len = 0, off_seq_ctx_len = 0, off_seq_state_slot = 0;
  int64_t off_logit_rows = 0, off_tile_seq = 0, off_tile_q0 = 0, off_block_tables = 0;
  int64_t total_ints = 0;
  std::vector<int32_t> entry_order;       // sorted position -> index in the caller's list
};

class BatchBuilder {
 public:
  BatchBuilder(int block_size, int max_blocks_per_seq, int num_groups, int tile_rows);
  // Upper bound of the packed size for a step of at most these counts.
  int64_t capacity_for(int rows, int seqs, int logit_rows) const;
  // Fills `out` (capacity in int32s).  Throws std::invalid_argument / std::runtime_error when an
  // entry is inconsistent (no page for a position, portion outside the token list, ...).
  BatchLayout build(const std::vector<BatchEntry>& entries, int32_t* out, int64_t capacity,
                    int pad_rows = 0, int pad_seqs = 0, int pad_logit_rows = 0) const;

 private:
  int block_size_, max_blocks_, groups_, tile_rows_;
};

}  // namespace kvcm
