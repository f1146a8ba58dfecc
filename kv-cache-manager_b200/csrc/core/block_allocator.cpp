#include "block_allocator.h"

#include <stdexcept>
#include <string>

namespace kvcm {

BlockAllocator::BlockAllocator(int num_blocks) {
  if (num_blocks < 0) throw std::invalid_argument("BlockAllocator: negative pool size");
  refs_.assign(num_blocks, 0);
  state_.assign(num_blocks, kFree);
  stack_.resize(num_blocks);
  for (int i = 0; i < num_blocks; ++i) stack_[i] = num_blocks - 1 - i;   // top of stack = id 0
}

void BlockAllocator::check_id(int id, const char* what) const {
  if (id < 0 || id >= num_blocks())
    throw std::logic_error(std::string(what) + ": page id " + std::to_string(id) +
                           " outside pool of " + std::to_string(num_blocks()));
}

int BlockAllocator::allocate() {
  if (stack_.empty()) return -1;
  const int id = stack_.back();
  stack_.pop_back();
  state_[id] = kHeld;
  refs_[id] = 1;
  return id;
}

void BlockAllocator::incref(int id) {
  check_id(id, "incref");
  if (state_[id] != kHeld) throw std::logic_error("incref: page " + std::to_string(id) + " is not held");
  ++refs_[id];
}

bool BlockAllocator::decref(int id) {
  check_id(id, "decref");
  if (state_[id] != kHeld) throw std::logic_error("decref: page " + std::to_string(id) + " has no reference");
  if (--refs_[id] > 0) return false;
  state_[id] = kParked;
  return true;
}

void BlockAllocator::push_free(int id) {
  check_id(id, "push_free");
  if (state_[id] != kParked)
    throw std::logic_error("push_free: page " + std::to_string(id) +
                           (state_[id] == kFree ? " is already free" : " is still referenced"));
  state_[id] = kFree;
  stack_.push_back(id);
}

void BlockAllocator::revive(int id) {
  check_id(id, "revive");
  if (state_[id] != kParked) throw std::logic_error("revive: page " + std::to_string(id) + " is not parked");
  state_[id] = kHeld;
  refs_[id] = 1;
}

void BlockAllocator::free(int id) {
  if (decref(id)) push_free(id);
}

}  // namespace kvcm
