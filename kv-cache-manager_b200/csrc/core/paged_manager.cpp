#include "paged_manager.h"

#include <algorithm>
#include <stdexcept>

#include "hash.h"

namespace kvcm {

PagedManager::PagedManager(int num_blocks, int block_size, int max_seq_len, bool prefix_caching,
                           int watermark_blocks, std::vector<LayerGroupSpec> groups)
    : KVManager(num_blocks, block_size, max_seq_len, std::move(groups)),
      watermark_(watermark_blocks) {
  if (prefix_caching && (groups_.size() != 1 || groups_[0].window != 0))
    throw std::invalid_argument(
        "prefix caching needs a single layer group that keeps every key (no window)");
  for (size_t g = 0; g < groups_.size(); ++g)
    pools_.push_back(std::make_unique<Pool>(num_blocks, block_size, prefix_caching));
}

bool PagedManager::can_admit(const Sequence& seq) const {
  const int n = seq.length();
  if (n > max_seq_len_) return false;
  int parked_hits = 0;
  const int hits = pools_[0]->cache.count_match(seq.tokens.data(), shareable_pages(seq), &parked_hits);
  for (size_t g = 0; g < pools_.size(); ++g) {
    const int need = pages_for(n) - (g == 0 ? hits : 0);
    const int available = pools_[g]->cache.num_available() - (g == 0 ? parked_hits : 0);
    if (need > available - watermark_) return false;
  }
  return true;
}

void PagedManager::admit(Sequence& seq) {
  start_tables(seq);
  const int hits = pools_[0]->cache.match_and_acquire(seq.tokens.data(), shareable_pages(seq),
                                                      seq.tables[0], seq.page_hashes);
  seq.cached_tokens = hits * block_size_;
  seq.num_computed = seq.cached_tokens;
  seq.prefill_tokens_saved += seq.cached_tokens;
}

bool PagedManager::ensure(Sequence& seq, int upto) {
  if (seq.tables.size() != pools_.size()) throw std::logic_error("ensure: request was not admitted");
  const size_t need = static_cast<size_t>(pages_for(upto));
  for (size_t g = 0; g < pools_.size(); ++g) {
    auto& table = seq.tables[g];
    while (table.size() < need) {
      const int id = pools_[g]->cache.allocate();
      if (id < 0) return false;
      table.push_back(id);
    }
  }
  return true;
}

void PagedManager::commit(Sequence& seq) {
  PrefixCache& cache = pools_[0]->cache;
  if (cache.enabled()) {
    // Pages completed by the step just run.  Registered only now, so that a second request of
    // the same step cannot hit a page that is still being written (docs/design.md:52-55 of the
    // reference gives the same reason).
    const int full = seq.num_computed / block_size_;
    for (int b = static_cast<int>(seq.page_hashes.size()); b < full; ++b) {
      const uint64_t parent = b ? seq.page_hashes[b - 1] : 0;
      const int32_t* page_tokens = seq.tokens.data() + static_cast<size_t>(b) * block_size_;
      const uint64_t h = page_hash(parent, page_tokens, block_size_);
      cache.insert(seq.tables[0][b], parent, h, page_tokens);
      seq.page_hashes.push_back(h);
    }
  }
  for (size_t g = 0; g < pools_.size(); ++g) {
    const int w = groups_[g].window;
    if (w <= 0) continue;
    // The next query sits at position >= num_computed and reads keys t > position - w, so every
    // key below num_computed - w + 1 is dead; a page is given back once all its keys are.
    const int first_live = std::max(0, seq.num_computed - w + 1);
    const int dead_pages = std::min<int>(first_live / block_size_, seq.tables[g].size());
    for (int i = seq.window_freed[g]; i < dead_pages; ++i) {
      pools_[g]->cache.release(seq.tables[g][i]);
      seq.tables[g][i] = -1;
    }
    seq.window_freed[g] = std::max(seq.window_freed[g], dead_pages);
  }
}

void PagedManager::release(Sequence& seq) {
  // Tail first, so that the end of a shared prefix is recycled before its head.
  for (size_t g = 0; g < seq.tables.size(); ++g) {
    auto& table = seq.tables[g];
    for (auto it = table.rbegin(); it != table.rend(); ++it)
      if (*it >= 0) pools_[g]->cache.release(*it);
    table.clear();
  }
  std::fill(seq.window_freed.begin(), seq.window_freed.end(), 0);
  seq.page_hashes.clear();
  seq.num_computed = 0;
}

// ------------------------------------------------------------------------------ contiguous

ContiguousManager::ContiguousManager(int num_blocks, int block_size, int max_seq_len,
                                     std::vector<LayerGroupSpec> groups)
    : KVManager(num_blocks, block_size, max_seq_len, std::move(groups)),
      reserve_(pages_for(max_seq_len)), free_pages_(num_blocks) {
  if (num_blocks > 0) extents_.push_back({0, num_blocks});
}

int ContiguousManager::first_fit() const {
  for (size_t i = 0; i < extents_.size(); ++i)
    if (extents_[i].count >= reserve_) return static_cast<int>(i);
  return -1;
}

bool ContiguousManager::can_admit(const Sequence& seq) const {
  return seq.length() <= max_seq_len_ && first_fit() >= 0;
}

void ContiguousManager::admit(Sequence& seq) {
  start_tables(seq);
  const int at = first_fit();
  if (at < 0) throw std::runtime_error("admit: no run of " + std::to_string(reserve_) +
                                       " consecutive pages (ask can_admit first)");
  const int start = extents_[at].start;
  if (extents_[at].count == reserve_) {
    extents_.erase(extents_.begin() + at);
  } else {
    extents_[at].start += reserve_;
    extents_[at].count -= reserve_;
  }
  free_pages_ -= reserve_;
  // Every group has its own pool of the same size; the reservation covers the same ids in each.
  for (auto& table : seq.tables) {
    table.resize(reserve_);
    for (int i = 0; i < reserve_; ++i) table[i] = start + i;
  }
}

bool ContiguousManager::ensure(Sequence& seq, int upto) {
  if (seq.tables.empty() || seq.tables[0].empty()) throw std::logic_error("ensure: request was not admitted");
  return upto <= reserve_ * block_size_;
}

void ContiguousManager::release(Sequence& seq) {
  if (!seq.tables.empty() && !seq.tables[0].empty()) {
    Extent back{seq.tables[0].front(), static_cast<int>(seq.tables[0].size())};
    free_pages_ += back.count;
    auto next = std::lower_bound(extents_.begin(), extents_.end(), back.start,
                                 [](const Extent& e, int s) { return e.start < s; });
    if (next != extents_.end() && next->start == back.start + back.count) {
      back.count += next->count;
      next = extents_.erase(next);
    }
    if (next != extents_.begin() && (next - 1)->start + (next - 1)->count == back.start) {
      (next - 1)->count += back.count;
    } else {
      extents_.insert(next, back);
    }
  }
  for (auto& table : seq.tables) table.clear();
  std::fill(seq.window_freed.begin(), seq.window_freed.end(), 0);
  seq.num_computed = 0;
}

}  // namespace kvcm
