// Pages on demand: a request holds ceil(len / B) pages per group (fewer once a window has
// passed some), so the only waste is the unfilled tail of its last page.  Optional reuse of
// equal prefixes through the PrefixCache.  Policy after the reference's PagedManager
// (src/core/paged_manager.cpp:9-66).
#pragma once
#include <memory>

#include "kv_manager.h"

namespace kvcm {

class PagedManager : public KVManager {
 public:
  PagedManager(int num_blocks, int block_size, int max_seq_len, bool prefix_caching,
               int watermark_blocks = 0, std::vector<LayerGroupSpec> groups = {LayerGroupSpec{}});
  std::string name() const override { return pools_[0]->cache.enabled() ? "paged+prefix" : "paged"; }

  bool can_admit(const Sequence& seq) const override;
  void admit(Sequence& seq) override;
  bool ensure(Sequence& seq, int upto) override;
  void commit(Sequence& seq) override;
  void release(Sequence& seq) override;

  int blocks_in_use(int g = 0) const override { return num_blocks_ - pools_.at(g)->cache.num_available(); }
  int blocks_cached_free() const override { return pools_[0]->cache.num_cached_free(); }
  PrefixCacheStats prefix_stats() const override { return pools_[0]->cache.stats(); }

  const BlockAllocator& allocator(int g = 0) const { return pools_.at(g)->alloc; }
  const PrefixCache& cache(int g = 0) const { return pools_.at(g)->cache; }

 private:
  struct Pool {
    BlockAllocator alloc;
    PrefixCache cache;
    Pool(int n, int block_size, bool prefix) : alloc(n), cache(alloc, block_size, prefix) {}
  };
  // Leading full pages that may be shared.  The last token is always computed (its logits are
  // needed), so the page that holds it is never taken from the cache.
  int shareable_pages(const Sequence& s) const { return (s.length() - 1) / block_size_; }
  std::vector<std::unique_ptr<Pool>> pools_;
  int watermark_;
};

// Baseline policy: a request reserves ceil(max_seq_len / B) *consecutive* pages at admission, as
// an engine with one maximum-length buffer per request would.  Same tables, same kernels.
// First fit over free extents, coalescing on release (src/core/contiguous_manager.cpp:7-66).
class ContiguousManager : public KVManager {
 public:
  ContiguousManager(int num_blocks, int block_size, int max_seq_len,
                    std::vector<LayerGroupSpec> groups = {LayerGroupSpec{}});
  std::string name() const override { return "contiguous"; }

  bool can_admit(const Sequence& seq) const override;
  void admit(Sequence& seq) override;
  bool ensure(Sequence& seq, int upto) override;
  void commit(Sequence&) override {}
  void release(Sequence& seq) override;
  int blocks_in_use(int = 0) const override { return num_blocks_ - free_pages_; }

  int reserve_blocks() const { return reserve_; }
  int num_free_extents() const { return static_cast<int>(extents_.size()); }

 private:
  struct Extent { int start, count; };
  int first_fit() const;               // index into extents_, or -1
  int reserve_;
  int free_pages_;
  std::vector<Extent> extents_;        // free runs, sorted by start, never adjacent
};

}  // namespace kvcm
