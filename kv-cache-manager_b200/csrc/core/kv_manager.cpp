#include "kv_manager.h"

#include <algorithm>
#include <stdexcept>

#include "paged_manager.h"

namespace kvcm {

KVManager::KVManager(int num_blocks, int block_size, int max_seq_len,
                     std::vector<LayerGroupSpec> groups)
    : num_blocks_(num_blocks), block_size_(block_size), max_seq_len_(max_seq_len),
      groups_(std::move(groups)) {
  if (block_size_ <= 0) throw std::invalid_argument("KVManager: block_size must be positive");
  if (num_blocks_ < 0) throw std::invalid_argument("KVManager: num_blocks must not be negative");
  if (groups_.empty()) throw std::invalid_argument("KVManager: at least one layer group is needed");
  for (const auto& g : groups_)
    if (g.window < 0) throw std::invalid_argument("KVManager: negative window");
}

void KVManager::start_tables(Sequence& seq) const {
  for (const auto& t : seq.tables)
    if (!t.empty()) throw std::logic_error("admit: request " + std::to_string(seq.id) + " already holds pages");
  seq.tables.assign(groups_.size(), {});
  seq.window_freed.assign(groups_.size(), 0);
  seq.page_hashes.clear();
  seq.cached_tokens = 0;
  seq.num_computed = 0;
}

// Fill of every physical page = the largest fill among the requests that share it
// (accounting as the reference's KVManager::stats, src/core/kv_manager.cpp:11-39).
KVStats KVManager::stats(const std::vector<const Sequence*>& live) const {
  KVStats s;
  s.num_blocks = num_blocks_;
  s.block_size = block_size_;
  s.blocks_in_use = blocks_in_use(0);
  s.blocks_cached_free = blocks_cached_free();
  s.allocated_slots = static_cast<int64_t>(s.blocks_in_use) * block_size_;
  s.num_seqs = static_cast<int>(live.size());
  s.prefix = prefix_stats();
  std::vector<int> fill(num_blocks_, -1);
  for (const Sequence* q : live) {
    if (q->tables.empty()) continue;
    const auto& table = q->tables[0];
    s.block_table_entries += static_cast<int64_t>(table.size());
    for (size_t i = 0; i < table.size(); ++i) {
      if (table[i] < 0) continue;
      const int held = std::clamp(q->num_computed - static_cast<int>(i) * block_size_, 0, block_size_);
      fill[table[i]] = std::max(fill[table[i]], held);
    }
  }
  for (int f : fill) {
    if (f < 0) continue;
    s.used_slots += f;
    if (f == 0) s.reserved_unused_slots += block_size_;
    else s.tail_waste_slots += block_size_ - f;
  }
  return s;
}

std::unique_ptr<KVManager> make_kv_manager(const KVManagerConfig& c) {
  if (c.policy == "paged") {
    const int spare = c.watermark_blocks >= 0 ? c.watermark_blocks
                                              : static_cast<int>(c.watermark_frac * c.num_blocks);
    return std::make_unique<PagedManager>(c.num_blocks, c.block_size, c.max_seq_len,
                                          c.prefix_caching, spare, c.groups);
  }
  if (c.policy == "contiguous")
    return std::make_unique<ContiguousManager>(c.num_blocks, c.block_size, c.max_seq_len, c.groups);
  throw std::invalid_argument("unknown KV policy '" + c.policy + "' (paged | contiguous)");
}

StateSlots::StateSlots(int num_slots) : taken_(std::max(num_slots, 0), 0) {
  for (int i = num_slots - 1; i >= 0; --i) free_.push_back(i);
}

int StateSlots::take() {
  if (free_.empty()) return -1;
  const int s = free_.back();
  free_.pop_back();
  taken_[s] = 1;
  return s;
}

void StateSlots::give_back(int slot) {
  if (slot < 0 || slot >= num_slots() || !taken_[slot])
    throw std::logic_error("StateSlots: slot " + std::to_string(slot) + " is not taken");
  taken_[slot] = 0;
  free_.push_back(slot);
}

}  // namespace kvcm
