// Continuous batching above one step function: first come first served, a token budget per
// step, prompts cut into portions under that budget, preemption by recomputation when pages
// run out.  Queues, gates and counters follow the reference's Scheduler
// (src/core/scheduler.cpp:25-105); cutting prompts into portions is new here (the reference
// always schedules a prompt whole, scheduler.cpp:68-69).
//
// What happens when pages run out:
//  * a running request that cannot get the pages of its next portion evicts the YOUNGEST
//    running request (possibly itself): its pages and state slot go back, its tokens stay, and
//    it returns to the FRONT of the waiting queue to be computed again from its first token;
//  * no request is admitted in a step that had to evict;
//  * a waiting request that does not fit while nothing is running can never fit: it is
//    rejected (finished without a token).  While something is running it waits (strict order,
//    nothing overtakes it).
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <vector>

#include "kv_manager.h"
#include "sequence.h"

namespace kvcm {

struct SchedulerConfig {
  int max_num_seqs = 256;          // cap on running requests (= number of state slots)
  int max_batched_tokens = 4096;   // cap on rows per step, prompt portions and decodes together
  int prefill_chunk = 0;           // cap on one request's portion (0: the budget alone decides)
  bool chunked_prefill = true;     // false: a prompt is scheduled whole or not at all
  int eos_token_id = -1;           // >= 0: a request also ends when it samples this token
};

// One request's share of a step: compute tokens [start, start + num_tokens).
struct ScheduledSeq {
  std::shared_ptr<Sequence> seq;   // shared with the queues (and with Python wrappers)
  int start;
  int num_tokens;
  bool is_prefill;     // the portion lies (at least partly) inside the prompt
  bool wants_logits;   // the portion ends at the request's last token: a token is sampled
};

struct SchedulerCounters {
  int64_t steps = 0, preemptions = 0, admissions = 0, admission_blocked_steps = 0, rejected = 0;
  int64_t prefill_tokens = 0, decode_tokens = 0, prefill_tokens_saved = 0, batch_size_sum = 0;
  int max_running = 0;
};

class Scheduler {
 public:
  Scheduler(KVManager& kv, SchedulerConfig cfg);

  void add(std::shared_ptr<Sequence> seq);
  const std::vector<ScheduledSeq>& schedule(double now);
  // One sampled token for every plan entry with wants_logits, in plan order.
  void update(const std::vector<int32_t>& sampled, double now);
  std::vector<std::shared_ptr<Sequence>> take_finished();

  bool idle() const { return waiting_.empty() && running_.empty(); }
  size_t num_waiting() const { return waiting_.size(); }
  size_t num_running() const { return running_.size(); }
  const std::vector<ScheduledSeq>& plan() const { return plan_; }
  std::vector<const Sequence*> live() const;
  const std::deque<std::shared_ptr<Sequence>>& running() const { return running_; }
  const SchedulerCounters& counters() const { return ctr_; }
  void reset_counters() { ctr_ = {}; }
  KVManager& kv() { return kv_; }
  const StateSlots& slots() const { return slots_; }
  const SchedulerConfig& config() const { return cfg_; }

 private:
  int portion(const Sequence& s, int budget, bool plan_empty) const;
  void evict_youngest();

  KVManager& kv_;
  SchedulerConfig cfg_;
  StateSlots slots_;
  std::deque<std::shared_ptr<Sequence>> waiting_;
  std::deque<std::shared_ptr<Sequence>> running_;   // admission order: back = youngest
  std::vector<std::shared_ptr<Sequence>> finished_;
  std::vector<ScheduledSeq> plan_;
  SchedulerCounters ctr_;
};

}  // namespace kvcm
