"""Configurations drawn at random (head sizes in steps of 16 up to 256, any number of heads and
groups, widths and vocabularies that are no power of two, tied or untied output head, pages of 8 to
128) through a mixed schedule of portions and single tokens, in float32 and bfloat16, against the
plain implementation.  The seeds are fixed, so the drawn configurations are the same every run."""
import itertools
import random

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


def draw(seed: int):
    rng = random.Random(1000 + seed)
    nkv = rng.choice([1, 2, 3, 5])
    cfg = dict(vocab_size=rng.choice([97, 256, 300, 1000, 1031]), hidden_size=rng.choice([40, 72, 100, 136, 200, 264, 520]),
               intermediate_size=rng.choice([56, 100, 172, 344, 600]), num_hidden_layers=rng.choice([1, 2, 3]),
               num_attention_heads=nkv * rng.choice([1, 2, 3, 4, 7]), num_key_value_heads=nkv,
               head_dim=rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256]),
               max_position_embeddings=rng.choice([256, 700]), rope_theta=rng.choice([1e4, 5e5, 1e6]),
               rms_norm_eps=rng.choice([1e-5, 1e-6, 3e-6]), tie_word_embeddings=rng.random() < 0.5)
    block = rng.choice([8, 16, 32, 64, 128])
    lens = [rng.randint(1, 40), rng.randint(41, 130), rng.randint(100, cfg["max_position_embeddings"] - 1)]
    return cfg, block, lens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration_in_a_mixed_schedule(seed, dtype, tmp_path):
    import kvcm
    cfgd, block, lens = draw(seed)
    what = f"{cfgd} pages of {block}"
    folder = str(tmp_path / "model")
    kvcm.write_random_model(folder, kvcm.LlamaConfig(architecture="LlamaForCausalLM", **cfgd), seed,
                            helpers.TORCH_DT[dtype], norm_jitter=0.1)
    pc, w = P.read_model_folder(folder)
    toks = [helpers.random_tokens(n, cfgd["vocab_size"], 50 + i) for i, n in enumerate(lens)]
    ref = [P.llama_forward(pc, w, t, None if dtype == "float32" else torch.bfloat16) for t in toks]
    r = helpers.Replayer(folder, dtype, sum(helpers.roundup(n, max(64, block)) for n in lens), block)
    fed, live = [0] * len(lens), list(range(len(lens)))
    sizes = itertools.cycle([9, 2, 33, 1, 4, 70, 1, 1, 17, 200, 1, 129])
    step = 0
    while live:
        entries, where, ended = [], [], []
        for i in list(live):
            if (step + i) % 4 == 3 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            k = min(next(sizes), lens[i] - fed[i])
            entries.append(dict(id=f"r{i}", tokens=toks[i][fed[i]:fed[i] + k], want=list(range(k))))
            where += [(i, fed[i] + j) for j in range(k)]
            fed[i] += k
            if fed[i] == lens[i]:
                ended.append(f"r{i}")
                live.remove(i)
        if entries:
            got = r.step(entries, ended)
            helpers.assert_logits_close(got, torch.stack([ref[i][p] for i, p in where]), dtype, f"{what}, step {step}")
        step += 1
    assert r.kv.blocks_in_use() == 0
