// The allocation-policy interface: everything above it (scheduler, engine, replay) and below
// it (kernels, page pools) is the same for every policy.  After the reference's KVManager
// (src/core/kv_manager.h:32-62), with two changes that chunked prefill and layer groups need:
//
//  * pages are taken per portion: ensure(seq, upto) makes room for tokens [0, upto), so a
//    request that is prefetched in portions holds only the pages its computed part needs
//    (the reference's admit()+append_slot() always cover the whole token list);
//  * a request has one page table per *layer group*.  A group is a set of layers with the
//    same cache needs: all keys (window 0) or only the last `window` keys, in which case
//    commit() gives back the pages that the window has passed.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "prefix_cache.h"
#include "sequence.h"

namespace kvcm {

struct LayerGroupSpec {
  int window = 0;        // 0: every key is kept; w > 0: only keys of the last w positions
};

struct KVStats {
  int num_blocks = 0, block_size = 0;
  int blocks_in_use = 0;              // referenced pages (a reserved extent counts as in use)
  int blocks_cached_free = 0;         // unreferenced pages kept for prefix hits
  int64_t allocated_slots = 0;        // blocks_in_use * block_size
  int64_t used_slots = 0;             // distinct physical slots that hold a token
  int64_t tail_waste_slots = 0;       // empty slots inside partly filled pages
  int64_t reserved_unused_slots = 0;  // slots of wholly empty reserved pages (contiguous)
  int64_t block_table_entries = 0;
  int num_seqs = 0;
  PrefixCacheStats prefix;
  double fragmentation() const {
    return allocated_slots ? double(allocated_slots - used_slots) / double(allocated_slots) : 0.0;
  }
};

class KVManager {
 public:
  virtual ~KVManager() = default;
  virtual std::string name() const = 0;
  int block_size() const { return block_size_; }
  int num_blocks() const { return num_blocks_; }
  int max_seq_len() const { return max_seq_len_; }
  int num_groups() const { return static_cast<int>(groups_.size()); }
  const LayerGroupSpec& group(int g) const { return groups_.at(g); }

  // Could the request (all of seq.tokens) be admitted right now?
  virtual bool can_admit(const Sequence& seq) const = 0;
  // Starts the request's tables; applies prefix hits and sets num_computed to the cached count.
  virtual void admit(Sequence& seq) = 0;
  // Room for tokens [0, upto) in every group.  False: out of pages (nothing is rolled back;
  // pages taken so far stay in the tables and are used by a later call or given back by release).
  virtual bool ensure(Sequence& seq, int upto) = 0;
  // After a step: newly full pages become reusable prefixes; windows give back passed pages.
  virtual void commit(Sequence& seq) = 0;
  virtual void release(Sequence& seq) = 0;

  virtual int blocks_in_use(int g = 0) const = 0;
  virtual int blocks_cached_free() const { return 0; }
  virtual PrefixCacheStats prefix_stats() const { return {}; }

  KVStats stats(const std::vector<const Sequence*>& live) const;   // group 0

 protected:
  KVManager(int num_blocks, int block_size, int max_seq_len, std::vector<LayerGroupSpec> groups);
  int pages_for(int tokens) const { return (tokens + block_size_ - 1) / block_size_; }
  void start_tables(Sequence& seq) const;
  int num_blocks_, block_size_, max_seq_len_;
  std::vector<LayerGroupSpec> groups_;
};

struct KVManagerConfig {
  std::string policy = "paged";   // "paged" | "contiguous"
  int num_blocks = 1024;          // per group
  int block_size = 16;
  int max_seq_len = 2048;
  bool prefix_caching = false;
  int watermark_blocks = -1;      // paged: pages kept spare at admission (-1: watermark_frac)
  double watermark_frac = 0.01;
  std::vector<LayerGroupSpec> groups = {LayerGroupSpec{}};
};

std::unique_ptr<KVManager> make_kv_manager(const KVManagerConfig& cfg);

// Fixed-size per-request state: a request takes one slot at admission and gives it back when
// it finishes or is preempted.  Device slabs [num_slots, ...] are indexed by the slot.
class StateSlots {
 public:
  explicit StateSlots(int num_slots);
  int take();                 // -1 when every slot is taken
  void give_back(int slot);   // throws std::logic_error when the slot is not taken
  int num_slots() const { return static_cast<int>(taken_.size()); }
  int num_taken() const { return num_slots() - static_cast<int>(free_.size()); }
  bool is_taken(int slot) const { return taken_.at(slot) != 0; }
 private:
  std::vector<int32_t> free_;
  std::vector<uint8_t> taken_;
};

}  // namespace kvcm
