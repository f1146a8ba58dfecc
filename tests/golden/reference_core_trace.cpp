// Drives the REFERENCE's CPU core (src/core/*.cpp: block allocator, prefix cache, paged and
// contiguous managers, scheduler) with a script of operations read from standard input and prints
// one line of JSON per operation.  tests/golden/make_core_traces.py compiles this file against the
// reference's sources and stores what it prints; tests/test_reference_core.py replays the same
// scripts through this repository's own core and expects the same lines.
//
// Script (one operation per line, integers separated by blanks):
//   manager <paged|contiguous> <num_blocks> <block_size> <max_seq_len> <prefix 0|1> <watermark>
//   sched <max_num_seqs> <max_batched_tokens>
//   new <id> <n> <token>*n          a sequence outside the scheduler
//   can <id> | admit <id> | grow <id> <token> | commit <id> <num_computed> | release <id> | stats
//   add <id> <max_new_tokens> <n> <token>*n     a request for the scheduler
//   step                             schedule(); update() with token = next_token(id, length)
//   counters
#include <cstdio>
#include <iostream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "core/kv_manager.h"
#include "core/scheduler.h"
#include "core/sequence.h"

using namespace kvp;

static int next_token(int id, int length) { return (id * 7919 + length * 104729) % 1000 + 3; }

template <class T>
static std::string list(const std::vector<T>& v) {
  std::ostringstream o;
  o << "[";
  for (size_t i = 0; i < v.size(); ++i) o << (i ? "," : "") << v[i];
  o << "]";
  return o.str();
}

int main() {
  std::unique_ptr<KVManager> kv;
  std::unique_ptr<Scheduler> sched;
  std::map<int, std::unique_ptr<Sequence>> seqs;   // manager-level sequences
  std::map<int, bool> admitted;
  std::string line;
  while (std::getline(std::cin, line)) {
    std::istringstream in(line);
    std::string op;
    if (!(in >> op)) continue;
    if (op == "manager") {
      KVManagerConfig c;
      int prefix = 0;
      in >> c.policy >> c.num_blocks >> c.block_size >> c.max_seq_len >> prefix >> c.watermark_blocks;
      c.prefix_caching = prefix != 0;
      sched.reset();
      seqs.clear();
      admitted.clear();
      kv = make_kv_manager(c);
      std::printf("{\"op\":\"manager\"}\n");
    } else if (op == "sched") {
      SchedulerConfig c;
      in >> c.max_num_seqs >> c.max_batched_tokens;
      sched = std::make_unique<Scheduler>(*kv, c);
      std::printf("{\"op\":\"sched\"}\n");
    } else if (op == "new") {
      int id, n;
      in >> id >> n;
      auto s = std::make_unique<Sequence>();
      s->id = id;
      s->tokens.resize(n);
      for (int& t : s->tokens) in >> t;
      s->prompt_len = n;
      seqs[id] = std::move(s);
      admitted[id] = false;
      std::printf("{\"op\":\"new\",\"id\":%d}\n", id);
    } else if (op == "can") {
      int id;
      in >> id;
      std::printf("{\"op\":\"can\",\"id\":%d,\"ok\":%d}\n", id, kv->can_admit(*seqs[id]) ? 1 : 0);
    } else if (op == "admit") {
      int id;
      in >> id;
      Sequence& s = *seqs[id];
      kv->admit(s);
      admitted[id] = true;
      std::printf("{\"op\":\"admit\",\"id\":%d,\"table\":%s,\"num_computed\":%d,\"cached\":%d}\n", id,
                  list(s.block_table).c_str(), s.num_computed, s.cached_tokens);
    } else if (op == "grow") {
      int id, tok;
      in >> id >> tok;
      Sequence& s = *seqs[id];
      s.tokens.push_back(tok);
      const bool ok = kv->append_slot(s);
      std::printf("{\"op\":\"grow\",\"id\":%d,\"ok\":%d,\"table\":%s}\n", id, ok ? 1 : 0,
                  list(s.block_table).c_str());
    } else if (op == "commit") {
      int id, nc;
      in >> id >> nc;
      Sequence& s = *seqs[id];
      s.num_computed = nc;
      kv->commit(s);
      std::printf("{\"op\":\"commit\",\"id\":%d,\"hashes\":%d}\n", id, static_cast<int>(s.block_hashes.size()));
    } else if (op == "release") {
      int id;
      in >> id;
      kv->release(*seqs[id]);
      admitted[id] = false;
      std::printf("{\"op\":\"release\",\"id\":%d}\n", id);
    } else if (op == "stats") {
      std::vector<const Sequence*> live;
      if (sched) live = sched->live();
      else for (auto& kvp_ : seqs) if (admitted[kvp_.first]) live.push_back(kvp_.second.get());
      const KVStats s = kv->stats(live);
      std::printf("{\"op\":\"stats\",\"in_use\":%d,\"cached_free\":%d,\"allocated\":%lld,\"used\":%lld,"
                  "\"tail_waste\":%lld,\"reserved_unused\":%lld,\"entries\":%lld,\"seqs\":%d,"
                  "\"queried\":%lld,\"hits\":%lld,\"inserted\":%lld,\"evictions\":%lld,\"duplicates\":%lld}\n",
                  s.blocks_in_use, s.blocks_cached_free, (long long)s.allocated_slots, (long long)s.used_slots,
                  (long long)s.tail_waste_slots, (long long)s.reserved_unused_slots,
                  (long long)s.block_table_entries, s.num_seqs, (long long)s.prefix.queried_blocks,
                  (long long)s.prefix.hit_blocks, (long long)s.prefix.inserted_blocks,
                  (long long)s.prefix.evictions, (long long)s.prefix.duplicate_inserts);
    } else if (op == "add") {
      int id, max_new, n;
      in >> id >> max_new >> n;
      auto s = std::make_unique<Sequence>();
      s->id = id;
      s->tokens.resize(n);
      for (int& t : s->tokens) in >> t;
      s->prompt_len = n;
      s->max_new_tokens = max_new;
      sched->add(std::move(s));
      std::printf("{\"op\":\"add\",\"id\":%d}\n", id);
    } else if (op == "step") {
      const auto& plan = sched->schedule(0.0);
      std::ostringstream o;
      std::vector<int32_t> next;
      o << "[";
      for (size_t i = 0; i < plan.size(); ++i) {
        const ScheduledSeq& p = plan[i];
        o << (i ? "," : "") << "[" << p.seq->id << "," << p.start << "," << p.num_tokens << ","
          << (p.is_prefill ? 1 : 0) << "," << list(p.seq->block_table) << "]";
        next.push_back(next_token(p.seq->id, static_cast<int>(p.seq->tokens.size())));
      }
      o << "]";
      sched->update(next, 1.0);
      std::vector<int> done;
      for (auto& f : sched->take_finished()) done.push_back(f->first_token < 0 ? -f->id - 1 : f->id);
      std::printf("{\"op\":\"step\",\"plan\":%s,\"finished\":%s,\"running\":%d,\"waiting\":%d}\n",
                  o.str().c_str(), list(done).c_str(), (int)sched->num_running(), (int)sched->num_waiting());
    } else if (op == "counters") {
      const SchedulerCounters& c = sched->counters();
      std::printf("{\"op\":\"counters\",\"steps\":%lld,\"preemptions\":%lld,\"admissions\":%lld,"
                  "\"blocked\":%lld,\"rejected\":%lld,\"prefill\":%lld,\"decode\":%lld,\"saved\":%lld,"
                  "\"batch_sum\":%lld,\"max_running\":%d}\n",
                  (long long)c.steps, (long long)c.preemptions, (long long)c.admissions,
                  (long long)c.admission_blocked_steps, (long long)c.rejected, (long long)c.prefill_tokens,
                  (long long)c.decode_tokens, (long long)c.prefill_tokens_saved, (long long)c.batch_size_sum,
                  c.max_running);
    } else {
      std::fprintf(stderr, "unknown operation: %s\n", op.c_str());
      return 2;
    }
  }
  return 0;
}
