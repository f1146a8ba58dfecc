#include "prefix_cache.h"

#include <algorithm>

#include "hash.h"

namespace kvcm {

PrefixCache::PrefixCache(BlockAllocator& alloc, int block_size, bool enabled)
    : alloc_(alloc), block_size_(block_size), enabled_(enabled), meta_(alloc.num_blocks()) {
  if (enabled_) stored_tokens_.assign(static_cast<size_t>(alloc.num_blocks()) * block_size, 0);
}

void PrefixCache::park(int id) {
  PageMeta& m = meta_[id];
  m.parked = true;
  m.prev = newest_;
  m.next = -1;
  if (newest_ >= 0) meta_[newest_].next = id; else oldest_ = id;
  newest_ = id;
  ++parked_count_;
}

void PrefixCache::unpark(int id) {
  PageMeta& m = meta_[id];
  if (m.prev >= 0) meta_[m.prev].next = m.next; else oldest_ = m.next;
  if (m.next >= 0) meta_[m.next].prev = m.prev; else newest_ = m.prev;
  m.prev = m.next = -1;
  m.parked = false;
  --parked_count_;
}

void PrefixCache::recycle_oldest() {
  const int id = oldest_;
  unpark(id);
  index_.erase(meta_[id].hash);
  meta_[id].registered = false;
  ++stats_.evictions;
  alloc_.push_free(id);
}

int PrefixCache::allocate() {
  if (alloc_.num_free() == 0 && parked_count_ > 0) recycle_oldest();
  return alloc_.allocate();
}

void PrefixCache::release(int id) {
  if (!alloc_.decref(id)) return;          // other holders remain
  if (meta_[id].registered) park(id); else alloc_.push_free(id);
}

int PrefixCache::find(uint64_t parent, uint64_t hash, const int32_t* tokens) const {
  const auto hit = index_.find(hash);
  if (hit == index_.end()) return -1;
  const int id = hit->second;
  if (meta_[id].parent != parent) return -1;
  const int32_t* kept = &stored_tokens_[static_cast<size_t>(id) * block_size_];
  return std::equal(kept, kept + block_size_, tokens) ? id : -1;
}

int PrefixCache::count_match(const int32_t* tokens, int num_blocks, int* parked_hits) const {
  int hits = 0, parked = 0;
  uint64_t parent = 0;
  for (int b = 0; enabled_ && b < num_blocks; ++b, ++hits) {
    const int32_t* page_tokens = tokens + static_cast<size_t>(b) * block_size_;
    const uint64_t h = page_hash(parent, page_tokens, block_size_);
    const int id = find(parent, h, page_tokens);
    if (id < 0) break;
    parked += meta_[id].parked ? 1 : 0;
    parent = h;
  }
  if (parked_hits) *parked_hits = parked;
  return hits;
}

int PrefixCache::match_and_acquire(const int32_t* tokens, int num_blocks,
                                   std::vector<int32_t>& pages, std::vector<uint64_t>& hashes) {
  if (!enabled_) return 0;
  stats_.queried_blocks += num_blocks;
  int hits = 0;
  uint64_t parent = 0;
  for (int b = 0; b < num_blocks; ++b, ++hits) {
    const int32_t* page_tokens = tokens + static_cast<size_t>(b) * block_size_;
    const uint64_t h = page_hash(parent, page_tokens, block_size_);
    const int id = find(parent, h, page_tokens);
    if (id < 0) break;
    if (meta_[id].parked) {
      unpark(id);
      alloc_.revive(id);
    } else {
      alloc_.incref(id);
    }
    pages.push_back(id);
    hashes.push_back(h);
    parent = h;
  }
  stats_.hit_blocks += hits;
  return hits;
}

bool PrefixCache::insert(int page, uint64_t parent_hash, uint64_t hash, const int32_t* tokens) {
  if (!enabled_ || meta_.at(page).registered) return false;
  if (!index_.emplace(hash, page).second) {
    ++stats_.duplicate_inserts;
    return false;
  }
  PageMeta& m = meta_[page];
  m.hash = hash;
  m.parent = parent_hash;
  m.registered = true;
  std::copy(tokens, tokens + block_size_, &stored_tokens_[static_cast<size_t>(page) * block_size_]);
  ++stats_.inserted_blocks;
  return true;
}

std::vector<int> PrefixCache::lru_order() const {
  std::vector<int> order;
  for (int id = oldest_; id >= 0; id = meta_[id].next) order.push_back(id);
  return order;
}

}  // namespace kvcm
