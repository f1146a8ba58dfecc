#include "scheduler.h"

#include <algorithm>
#include <stdexcept>

namespace kvcm {

Scheduler::Scheduler(KVManager& kv, SchedulerConfig cfg)
    : kv_(kv), cfg_(cfg), slots_(cfg.max_num_seqs) {
  if (cfg_.max_num_seqs <= 0) throw std::invalid_argument("Scheduler: max_num_seqs must be positive");
  if (cfg_.max_batched_tokens <= 0) throw std::invalid_argument("Scheduler: max_batched_tokens must be positive");
}

void Scheduler::add(std::shared_ptr<Sequence> seq) {
  if (!seq || seq->tokens.empty()) throw std::invalid_argument("Scheduler::add: a request needs at least one token");
  if (seq->prompt_len <= 0) seq->prompt_len = seq->length();
  waiting_.push_back(std::move(seq));
}

std::vector<const Sequence*> Scheduler::live() const {
  std::vector<const Sequence*> v;
  for (const auto& s : running_) v.push_back(s.get());
  return v;
}

// How many of the request's outstanding tokens this step takes, given what is left of the
// budget.  0 = none this step.
int Scheduler::portion(const Sequence& s, int budget, bool plan_empty) const {
  const int outstanding = s.length() - s.num_computed;
  if (outstanding <= 0) return 0;
  if (!cfg_.chunked_prefill) {
    // Whole or nothing; a prompt larger than the budget is still taken when it is alone
    // (the reference's gate, scheduler.cpp:53).
    return (outstanding <= budget || plan_empty) ? outstanding : 0;
  }
  int n = std::min(outstanding, budget);
  if (cfg_.prefill_chunk > 0 && outstanding > 1) n = std::min(n, cfg_.prefill_chunk);
  return std::max(n, 0);
}

void Scheduler::evict_youngest() {
  std::shared_ptr<Sequence> victim = std::move(running_.back());
  running_.pop_back();
  kv_.release(*victim);                       // keys and values dropped, tokens kept
  if (victim->state_slot >= 0) { slots_.give_back(victim->state_slot); victim->state_slot = -1; }
  ++victim->num_preemptions;
  ++ctr_.preemptions;
  waiting_.push_front(std::move(victim));
}

const std::vector<ScheduledSeq>& Scheduler::schedule(double now) {
  plan_.clear();
  int budget = cfg_.max_batched_tokens;
  bool evicted = false;

  // 1) Requests that are already running, oldest first: the next decode token, or the next
  //    portion of a prompt that is not finished yet.
  for (size_t i = 0; i < running_.size();) {
    Sequence& s = *running_[i];
    const int n = portion(s, budget, plan_.empty());
    if (n == 0) { ++i; continue; }            // no budget left for it in this step
    if (kv_.ensure(s, s.num_computed + n)) {
      const bool in_prompt = s.num_computed < s.prompt_len;
      plan_.push_back({running_[i], s.num_computed, n, in_prompt, s.num_computed + n == s.length()});
      budget -= n;
      if (in_prompt) { ctr_.prefill_tokens += n; s.prefill_tokens_computed += n; }
      else ctr_.decode_tokens += n;
      ++i;
      continue;
    }
    evicted = true;
    const bool self = (i + 1 == running_.size());
    evict_youngest();
    if (self) break;                          // the asker was the youngest: it left
  }

  // 2) New requests in arrival order while they fit.
  bool blocked = false;
  while (!evicted && !waiting_.empty() && static_cast<int>(running_.size()) < cfg_.max_num_seqs &&
         budget > 0) {
    Sequence& head = *waiting_.front();
    if (!cfg_.chunked_prefill && head.length() > budget && !plan_.empty()) break;
    if (!kv_.can_admit(head)) {
      if (running_.empty()) {                 // larger than the pool or than max_seq_len
        head.finished = now;
        head.rejected = true;
        ++ctr_.rejected;
        finished_.push_back(std::move(waiting_.front()));
        waiting_.pop_front();
        continue;
      }
      blocked = true;
      break;
    }
    kv_.admit(head);
    const int n = portion(head, budget, plan_.empty());
    if (n == 0 || !kv_.ensure(head, head.num_computed + n)) {
      kv_.release(head);                      // raced with the watermark: try again next step
      blocked = true;
      break;
    }
    head.state_slot = slots_.take();
    if (head.admitted < 0) head.admitted = now;
    plan_.push_back({waiting_.front(), head.num_computed, n, true, head.num_computed + n == head.length()});
    budget -= n;
    ctr_.prefill_tokens += n;
    ctr_.prefill_tokens_saved += head.cached_tokens;
    head.prefill_tokens_computed += n;
    ++ctr_.admissions;
    running_.push_back(std::move(waiting_.front()));
    waiting_.pop_front();
  }
  if (blocked) ++ctr_.admission_blocked_steps;

  ++ctr_.steps;
  ctr_.batch_size_sum += static_cast<int64_t>(running_.size());
  ctr_.max_running = std::max(ctr_.max_running, static_cast<int>(running_.size()));
  return plan_;
}

void Scheduler::update(const std::vector<int32_t>& sampled, double now) {
  size_t next = 0;
  for (const ScheduledSeq& p : plan_) {
    Sequence& s = *p.seq;
    s.num_computed = p.start + p.num_tokens;
    kv_.commit(s);
    if (!p.wants_logits) continue;
    if (next >= sampled.size()) throw std::invalid_argument("Scheduler::update: too few sampled tokens");
    const int32_t tok = sampled[next++];
    s.tokens.push_back(tok);
    if (s.first_token < 0) s.first_token = now;
    if (s.reached_limit() || s.length() >= kv_.max_seq_len() ||
        (cfg_.eos_token_id >= 0 && tok == cfg_.eos_token_id))
      s.finished = now;
  }
  if (next != sampled.size()) throw std::invalid_argument("Scheduler::update: too many sampled tokens");
  for (auto it = running_.begin(); it != running_.end();) {
    if ((*it)->finished >= 0) {
      kv_.release(**it);
      if ((*it)->state_slot >= 0) { slots_.give_back((*it)->state_slot); (*it)->state_slot = -1; }
      finished_.push_back(std::move(*it));
      it = running_.erase(it);
    } else {
      ++it;
    }
  }
  plan_.clear();
}

std::vector<std::shared_ptr<Sequence>> Scheduler::take_finished() {
  std::vector<std::shared_ptr<Sequence>> out;
  out.swap(finished_);
  return out;
}

}  // namespace kvcm
