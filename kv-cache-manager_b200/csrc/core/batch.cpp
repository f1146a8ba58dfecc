#include "batch.h"

#include <algorithm>
#include <numeric>
#include <stdexcept>
#include <string>

namespace kvcm {

namespace {
int64_t round4(int64_t n) { return (n + 3) & ~int64_t(3); }   // keep every array 16-byte aligned
}

BatchBuilder::BatchBuilder(int block_size, int max_blocks_per_seq, int num_groups, int tile_rows)
    : block_size_(block_size), max_blocks_(max_blocks_per_seq), groups_(num_groups),
      tile_rows_(tile_rows) {
  if (block_size <= 0 || max_blocks_per_seq <= 0 || num_groups <= 0 || tile_rows <= 0)
    throw std::invalid_argument("BatchBuilder: sizes must be positive");
}

int64_t BatchBuilder::capacity_for(int rows, int seqs, int logit_rows) const {
  const int64_t tiles = rows / tile_rows_ + seqs + 1;
  return round4(rows) * (3 + groups_) + round4(seqs) * 4 + round4(logit_rows) + round4(tiles) * 2 +
         round4(int64_t(groups_) * seqs * max_blocks_) + 64;
}

BatchLayout BatchBuilder::build(const std::vector<BatchEntry>& entries, int32_t* out,
                                int64_t capacity, int pad_rows, int pad_seqs,
                                int pad_logit_rows) const {
  BatchLayout L;
  const int n_entries = static_cast<int>(entries.size());
  L.entry_order.resize(n_entries);
  std::iota(L.entry_order.begin(), L.entry_order.end(), 0);
  std::stable_sort(L.entry_order.begin(), L.entry_order.end(), [&](int a, int b) {
    return (entries[a].num_tokens == 1) > (entries[b].num_tokens == 1);
  });

  int rows = 0, wanted = 0, tiles = 0;
  for (int e = 0; e < n_entries; ++e) {
    const BatchEntry& en = entries[e];
    if (!en.seq) throw std::invalid_argument("batch: entry without a request");
    const Sequence& s = *en.seq;
    if (en.num_tokens <= 0 || en.start < 0 || en.start + en.num_tokens > s.length())
      throw std::invalid_argument("batch: request " + std::to_string(s.id) + " portion [" +
                                  std::to_string(en.start) + ", " + std::to_string(en.start + en.num_tokens) +
                                  ") lies outside its " + std::to_string(s.length()) + " tokens");
    if (static_cast<int>(s.tables.size()) != groups_)
      throw std::invalid_argument("batch: request " + std::to_string(s.id) + " has no page tables");
    if ((en.start + en.num_tokens + block_size_ - 1) / block_size_ > max_blocks_)
      throw std::invalid_argument("batch: request " + std::to_string(s.id) + " exceeds max_seq_len");
    for (int w : en.want)
      if (w < 0 || w >= en.num_tokens)
        throw std::invalid_argument("batch: wanted place " + std::to_string(w) + " outside a portion of " +
                                    std::to_string(en.num_tokens) + " tokens");
    rows += en.num_tokens;
    wanted += static_cast<int>(en.want.size());
    if (en.num_tokens == 1) ++L.decode_seqs;
    else tiles += (en.num_tokens + tile_rows_ - 1) / tile_rows_;
  }
  L.real_rows = rows;
  L.real_seqs = n_entries;
  L.rows = std::max(rows, pad_rows);
  L.seqs = std::max(n_entries, pad_seqs);
  if ((L.rows > rows || L.seqs > n_entries) && L.decode_seqs != n_entries)
    throw std::invalid_argument("batch: padding is only defined for steps of single-row entries");
  if (L.rows - rows != L.seqs - n_entries && (pad_rows || pad_seqs))
    throw std::invalid_argument("batch: padding is for single-row entries (pad_rows - rows must equal pad_seqs - entries)");
  L.logit_rows = std::max(wanted, pad_logit_rows);
  L.groups = groups_;
  L.max_blocks = max_blocks_;
  L.tile_rows = tile_rows_;
  L.prefill_tiles = tiles;
  L.prefill_rows = rows - L.decode_seqs;

  int64_t at = 0;
  auto take = [&](int64_t n) { const int64_t o = at; at += round4(n); return o; };
  L.off_tokens = take(L.rows);
  L.off_positions = take(L.rows);
  L.off_row_seq = take(L.rows);
  L.off_slot_mapping = take(int64_t(groups_) * L.rows);
  L.off_seq_q_start = take(L.seqs);
  L.off_seq_q_len = take(L.seqs);
  L.off_seq_ctx_len = take(L.seqs);
  L.off_seq_state_slot = take(L.seqs);
  L.off_logit_rows = take(L.logit_rows);
  L.off_tile_seq = take(tiles);
  L.off_tile_q0 = take(tiles);
  L.off_block_tables = take(int64_t(groups_) * L.seqs * max_blocks_);
  L.total_ints = at;
  if (at > capacity)
    throw std::runtime_error("batch: step needs " + std::to_string(at) + " ints, buffer holds " +
                             std::to_string(capacity));
  std::fill(out, out + at, 0);
  std::fill(out + L.off_slot_mapping, out + L.off_slot_mapping + int64_t(groups_) * L.rows, -1);
  std::fill(out + L.off_seq_state_slot, out + L.off_seq_state_slot + L.seqs, -1);
  std::fill(out + L.off_block_tables, out + L.off_block_tables + int64_t(groups_) * L.seqs * max_blocks_, -1);

  std::vector<int> q_start_of(n_entries, 0);   // by caller index
  int row = 0, tile = 0;
  for (int si = 0; si < n_entries; ++si) {
    const int e = L.entry_order[si];
    const BatchEntry& en = entries[e];
    const Sequence& s = *en.seq;
    const int end = en.start + en.num_tokens;
    q_start_of[e] = row;
    out[L.off_seq_q_start + si] = row;
    out[L.off_seq_q_len + si] = en.num_tokens;
    out[L.off_seq_ctx_len + si] = end;
    out[L.off_seq_state_slot + si] = s.state_slot;
    L.max_ctx = std::max(L.max_ctx, end);
    L.max_q_len = std::max(L.max_q_len, en.num_tokens);
    if (en.num_tokens == 1) L.max_decode_ctx = std::max(L.max_decode_ctx, end);
    for (int g = 0; g < groups_; ++g) {
      const auto& table = s.tables[g];
      int32_t* dst = out + L.off_block_tables + (int64_t(g) * L.seqs + si) * max_blocks_;
      const int held = std::min<int>(static_cast<int>(table.size()), max_blocks_);
      std::copy(table.begin(), table.begin() + held, dst);
      int32_t* slots = out + L.off_slot_mapping + int64_t(g) * L.rows + row;
      for (int j = 0; j < en.num_tokens; ++j) {
        const int pos = en.start + j;
        const int page = pos / block_size_;
        if (page >= static_cast<int>(table.size()) || table[page] < 0)
          throw std::runtime_error("batch: request " + std::to_string(s.id) + " holds no page for position " +
                                   std::to_string(pos) + " in group " + std::to_string(g));
        slots[j] = table[page] * block_size_ + pos % block_size_;
      }
    }
    for (int j = 0; j < en.num_tokens; ++j) {
      out[L.off_tokens + row + j] = s.tokens[en.start + j];
      out[L.off_positions + row + j] = en.start + j;
      out[L.off_row_seq + row + j] = si;
    }
    if (en.num_tokens > 1)
      for (int q0 = 0; q0 < en.num_tokens; q0 += tile_rows_, ++tile) {
        out[L.off_tile_seq + tile] = si;
        out[L.off_tile_q0 + tile] = q0;
      }
    row += en.num_tokens;
  }
  // Padding entries: one row each, context 0, nothing written, nothing read.
  for (int si = n_entries; si < L.seqs; ++si, ++row) {
    out[L.off_seq_q_start + si] = row;
    out[L.off_seq_q_len + si] = 1;
    out[L.off_row_seq + row] = si;
    out[L.off_positions + row] = -1;          // context = position + 1 = 0 keys
  }
  int lr = 0;
  for (int e = 0; e < n_entries; ++e)
    for (int w : entries[e].want) out[L.off_logit_rows + lr++] = q_start_of[e] + w;
  return L;
}

}  // namespace kvcm
