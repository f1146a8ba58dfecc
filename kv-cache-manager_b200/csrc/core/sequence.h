// One request as the host sees it.  `tokens` = prompt followed by what was generated; the
// keys and values of tokens [0, num_computed) are in the cache.  A step computes a portion
// [num_computed, num_computed + n); a decode step is the case n == 1 at the end of `tokens`.
// Fields follow the reference's Sequence (src/core/sequence.h:10-30), plus one page table per
// layer group, the fixed-size state slot and the sampling parameters.
#pragma once
#include <cstdint>
#include <vector>

namespace kvcm {

struct SamplingParams {
  float temperature = 0.f;   // 0: greedy
  uint64_t seed = 0;         // mixed with the request id and the position of the drawn token
};

struct Sequence {
  int64_t id = 0;
  std::vector<int32_t> tokens;
  int prompt_len = 0;
  int max_new_tokens = 0;
  int num_computed = 0;

  // tables[g][i] = physical page of logical page i in layer group g; -1 once a sliding
  // window has passed the page and it was given back.
  std::vector<std::vector<int32_t>> tables;
  std::vector<int32_t> window_freed;      // per group: leading logical pages already given back
  std::vector<uint64_t> page_hashes;      // chain hashes of the leading full pages (prefix cache)
  int cached_tokens = 0;                  // tokens skipped at the last admission (prefix hits)
  int state_slot = -1;                    // index into the per-request fixed-size state slabs

  SamplingParams sampling;

  double arrival = 0, admitted = -1, first_token = -1, finished = -1;
  bool rejected = false;
  int num_preemptions = 0;
  int64_t prefill_tokens_computed = 0;
  int64_t prefill_tokens_saved = 0;

  int length() const { return static_cast<int>(tokens.size()); }
  int num_generated() const { return length() - prompt_len; }
  bool reached_limit() const { return num_generated() >= max_new_tokens; }
};

}  // namespace kvcm
