// Teacher-forced logits of the REFERENCE engine: loads a weight file in the reference's format,
// calls its Engine::score (src/engine/engine.cpp:92-108: one whole-sequence pass through the paged
// path, every row's logits in fp32) on the token ids of a text file and writes the logits of the
// last `keep` rows as little-endian floats.  Compiled against the reference's own headers and its
// static libraries by tests/golden/make_reference_logits.py; nothing of this repository is linked.
//
//   reference_score_dump WEIGHTS TOKENS.txt OUT.f32 KEEP_ROWS [BLOCK_SIZE]
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <vector>

#include "engine/engine.h"

int main(int argc, char** argv) {
  if (argc < 5) { std::fprintf(stderr, "usage: %s weights tokens.txt out.f32 keep [block_size]\n", argv[0]); return 2; }
  try {
    std::vector<int32_t> tokens;
    std::ifstream tf(argv[2]);
    for (int t; tf >> t;) tokens.push_back(t);
    const size_t keep = std::strtoul(argv[4], nullptr, 10);
    kvp::LlamaWeights weights(argv[1]);
    kvp::EngineConfig ec;
    ec.kv.policy = "paged";
    ec.kv.block_size = argc > 5 ? std::atoi(argv[5]) : 16;
    ec.kv.max_seq_len = 1024;
    ec.kv.num_blocks = 256;
    ec.kv.watermark_blocks = 0;
    ec.sched.max_num_seqs = 4;
    ec.sched.max_batched_tokens = 1024;
    ec.max_logit_rows = 1024;
    kvp::Engine eng(weights, ec);
    std::vector<float> logits;
    eng.score(tokens, logits);
    const size_t vocab = weights.config().vocab, rows = tokens.size();
    const size_t first = rows > keep ? rows - keep : 0;
    FILE* f = std::fopen(argv[3], "wb");
    if (!f) { std::fprintf(stderr, "cannot write %s\n", argv[3]); return 1; }
    std::fwrite(logits.data() + first * vocab, sizeof(float), (rows - first) * vocab, f);
    std::fclose(f);
    std::printf("rows %zu kept %zu vocab %zu\n", rows, rows - first, vocab);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
