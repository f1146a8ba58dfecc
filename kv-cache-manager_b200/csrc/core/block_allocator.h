// Physical page ids of one pool with reference counts.  A page is in exactly one of three
// states: FREE (on the free stack), HELD (refcount >= 1) or PARKED (refcount 0, kept off the
// free stack by its owner, e.g. the prefix cache's LRU list).  Misuse throws std::logic_error.
// Behaviour matches the reference's allocator (src/core/block_allocator.cpp:7-46): LIFO reuse,
// ids 0,1,2,... handed out first.
#pragma once
#include <cstdint>
#include <vector>

namespace kvcm {

class BlockAllocator {
 public:
  explicit BlockAllocator(int num_blocks);

  int allocate();            // FREE -> HELD(1); -1 when no page is free
  void free(int id);         // drop one reference; at zero the page becomes FREE
  void incref(int id);       // HELD(n) -> HELD(n+1)
  bool decref(int id);       // HELD(n) -> HELD(n-1), or PARKED when it reaches zero (returns true)
  void push_free(int id);    // PARKED -> FREE
  void revive(int id);       // PARKED -> HELD(1)

  int refcount(int id) const { return refs_.at(id); }
  bool is_free(int id) const { return state_.at(id) == kFree; }
  int num_free() const { return static_cast<int>(stack_.size()); }
  int num_blocks() const { return static_cast<int>(refs_.size()); }

 private:
  enum : uint8_t { kFree = 0, kHeld = 1, kParked = 2 };
  void check_id(int id, const char* what) const;
  std::vector<int32_t> stack_;
  std::vector<int32_t> refs_;
  std::vector<uint8_t> state_;
};

}  // namespace kvcm
