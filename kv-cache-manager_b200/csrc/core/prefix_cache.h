// Reuse of full pages between requests that start with the same tokens.
//
//  * identity of page i of a request = chain hash h_i (hash.h); only full pages have one;
//  * a page registered under a hash stays findable when its last holder lets go: it is parked
//    on an LRU ring instead of the free stack and recycled only when the free stack is empty;
//  * a lookup is confirmed against the stored parent hash and the stored token ids, so a
//    64-bit collision cannot alias two different prefixes.
// Same policy as the reference's PrefixCache (src/core/prefix_cache.cpp:10-119).  The LRU is an
// index-linked ring over page ids (no node allocation per operation).
#pragma once
#include <cstdint>
#include <unordered_map>
#include <vector>

#include "block_allocator.h"

namespace kvcm {

struct PrefixCacheStats {
  int64_t queried_blocks = 0;     // full prompt pages offered for lookup
  int64_t hit_blocks = 0;
  int64_t inserted_blocks = 0;
  int64_t evictions = 0;
  int64_t duplicate_inserts = 0;  // equal content computed by two requests at the same time
};

class PrefixCache {
 public:
  PrefixCache(BlockAllocator& alloc, int block_size, bool enabled);

  bool enabled() const { return enabled_; }

  // A writable page: the free stack first, else the least recently parked page is recycled.
  int allocate();
  // Drops one reference; at zero a registered page is parked, an unregistered one is freed.
  void release(int id);

  // Walks the first `num_blocks` full pages of `tokens`, takes a reference on every leading hit
  // and appends (page id, hash).  Stops at the first miss.  Returns the number of hits.
  int match_and_acquire(const int32_t* tokens, int num_blocks, std::vector<int32_t>& pages,
                        std::vector<uint64_t>& hashes);
  // The same walk without side effects; *parked_hits counts hits that sit on the LRU ring
  // (taking them shrinks what allocate() can still recycle).
  int count_match(const int32_t* tokens, int num_blocks, int* parked_hits) const;
  // Registers a computed full page.  False if the page already has a hash or the hash is taken
  // (the page then stays private and is freed normally).
  bool insert(int page, uint64_t parent_hash, uint64_t hash, const int32_t* tokens);

  int num_available() const { return alloc_.num_free() + parked_count_; }
  int num_cached_free() const { return parked_count_; }
  int num_hashed() const { return static_cast<int>(index_.size()); }
  bool is_hashed(int id) const { return meta_.at(id).registered; }
  const PrefixCacheStats& stats() const { return stats_; }
  std::vector<int> lru_order() const;   // parked page ids, oldest first

 private:
  struct PageMeta {
    uint64_t hash = 0, parent = 0;
    int32_t prev = -1, next = -1;   // LRU ring links, valid while parked
    bool registered = false, parked = false;
  };
  int find(uint64_t parent, uint64_t hash, const int32_t* tokens) const;
  void park(int id);
  void unpark(int id);
  void recycle_oldest();

  BlockAllocator& alloc_;
  const int block_size_;
  const bool enabled_;
  std::unordered_map<uint64_t, int32_t> index_;
  std::vector<PageMeta> meta_;
  std::vector<int32_t> stored_tokens_;   // [num_blocks * block_size] when enabled
  int32_t oldest_ = -1, newest_ = -1;
  int parked_count_ = 0;
  PrefixCacheStats stats_;
};

}  // namespace kvcm
