"""The kernels at the sizes they are tuned for, inside the engine: two layers of the TinyLlama-1.1B
shape (hidden 2048, 32 query heads on 4 KV heads of 64, feed-forward 5632; a vocabulary that is no
power of two) with random weights.  The bfloat16 engine (tcgen05 attention and gated product for
long portions, the streaming products with fused epilogues and the clustered decode attention for
single tokens, the library products and unfused kernels of larger decode batches) against the plain
implementation in float64 on the CPU with the same roundings of stored tensors, and against this
engine's own true 32-bit path: whole at the full context of 2,048 tokens, in portions, token by
token, mixed, and in decode batches of 24 and 64."""
import math

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engines():
    import kvcm
    from kvcm.config import LlamaConfig
    from kvcm.engine import model_from_tensors
    from kvcm.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=4100, hidden_size=2048, intermediate_size=5632,
                      num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    t16 = dict(random_tensors(cfg, 7, torch.bfloat16, device="cuda:0", norm_jitter=0.1))
    t32 = {k: v.float() for k, v in t16.items()}
    out = {}
    for dtype, t in (("bfloat16", t16), ("float32", t32)):
        spec = model_from_tensors(cfg, dict(t), dtype, "cuda:0")
        out[dtype] = lambda spec=spec, dtype=dtype, max_live=4, max_tokens=4096: helpers.Replayer(
            None, dtype, max_tokens, 16, spec=spec, max_live=max_live)
    # the plain implementation on the same (bfloat16-rounded) weights, in float64 on the CPU
    w = {k: v.double().cpu() for k, v in t16.items()}
    cj = cfg.to_json_dict()
    memo = {}

    def plain(tokens, storage=torch.bfloat16):
        key = (tuple(tokens), storage)
        if key not in memo:
            memo[key] = P.llama_forward(cj, w, list(tokens), storage)
        return memo[key]
    out["plain"] = plain
    return cfg, out


def _rms_max(d):
    return d.pow(2).mean().sqrt().item(), d.abs().max().item()


def near_plain(got, rounded, exact, what):
    """The bfloat16 engine against the plain implementation in float64, at the same places.
    ``exact`` rounds nothing; ``rounded`` rounds every stored tensor to bfloat16 where the
    reference's kernels round to their storage type, so ``rounded - exact`` is what the reference's
    own arithmetic loses at this shape (about 1 % of the logits' standard deviation in the root mean
    square), and that is the yardstick: the engine may lose as much (10 % more in the root mean square,
    30 % more at the worst element, whose size varies from sample to sample), and it stays as close
    to ``rounded`` as two evaluations that share no rounding at all would (sqrt 2 of the yardstick).
    A real fault (a missed or wrong key, a stale page, a wrong tile) moves whole rows by the order of
    the standard deviation itself."""
    got, rounded, exact = got.double().cpu(), rounded.double().cpu(), exact.double().cpu()
    assert got.shape == exact.shape and torch.isfinite(got).all(), what
    ref_rms, ref_max = _rms_max(rounded - exact)
    rms, worst = _rms_max(got - exact)
    assert rms <= 1.1 * ref_rms and worst <= 1.3 * ref_max, \
        f"{what}: from the exact logits rms {rms:.5f}, max {worst:.5f} (the reference's arithmetic: {ref_rms:.5f}, {ref_max:.5f})"
    rms, worst = _rms_max(got - rounded)
    assert rms <= math.sqrt(2.0) * ref_rms and worst <= math.sqrt(2.0) * 1.3 * ref_max, \
        f"{what}: from the rounded logits rms {rms:.5f}, max {worst:.5f} (the reference's arithmetic: {ref_rms:.5f}, {ref_max:.5f})"


def same_cut(got, other, rounded, exact, what):
    """Two ways of cutting the same work in bfloat16: what differs are roundings the paths do not
    share (other kernels, other orders of summation, the norm applied before or after a product), so
    they are no further apart than two evaluations that share no rounding at all: sqrt 2 of what
    the reference's arithmetic loses at these places (see near_plain)."""
    got, other = got.double().cpu(), other.double().cpu()
    assert torch.isfinite(got).all(), what
    ref_rms, ref_max = _rms_max(rounded.double().cpu() - exact.double().cpu())
    rms, worst = _rms_max(got - other)
    assert rms <= math.sqrt(2.0) * ref_rms and worst <= math.sqrt(2.0) * 1.3 * ref_max, \
        f"{what}: apart by rms {rms:.5f}, max {worst:.5f} (the reference's arithmetic: {ref_rms:.5f}, {ref_max:.5f})"


def near_float32(got, ref, what):
    """bfloat16 against the true 32-bit path, which rounds no activation: about twenty tensors on the
    way to a logit are rounded with a relative error of 2^-9 / sqrt(3) each, which the attention's
    rounded probabilities and two residual layers roughly double: about 1 % of the logits' standard
    deviation in the root mean square, five times that at the worst of ~10^5 elements.  A real fault
    (a missed or wrong key, a stale page, a wrong tile) moves whole rows by the order of that
    deviation itself."""
    got, ref = got.double(), ref.double()
    assert torch.isfinite(got).all(), what
    std = ref.std().item()
    d = got - ref
    rms, worst = d.pow(2).mean().sqrt().item(), d.abs().max().item()
    assert rms <= 0.02 * std and worst <= 0.1 * std, f"{what}: rms {rms / std:.4f}, max {worst / std:.4f} of std"


def test_whole_portions_and_token_by_token(engines):
    cfg, make = engines
    n = 2048                                                         # the benchmark's full context
    toks = helpers.random_tokens(n, cfg.vocab_size, 3)
    want = [0, 1, 63, 64, 127, 128, 129, 700, 1023, 1024, 1535, 1536] + list(range(n - 64, n))
    plain = make["plain"](toks)[want]
    ref = make["float32"]().step([dict(id="a", tokens=toks, want=want)])
    helpers.assert_logits_close(ref, make["plain"](toks, None)[want], "float32",
                                "true 32-bit path, whole prompt of 2,048")
    whole = make["bfloat16"]().step([dict(id="a", tokens=toks, want=want)])
    exact = make["plain"](toks, None)[want]
    near_plain(whole, plain, exact, "whole prompt of 2,048 tokens")
    near_float32(whole, ref, "whole prompt")
    r = make["bfloat16"]()
    got, at = [], 0
    for k in (700, 2, 300, 466, 548):                              # 2016 tokens in portions ...
        w = [p - at for p in want if at <= p < at + k]
        o = r.step([dict(id="a", tokens=toks[at:at + k], want=w)])
        if w:
            got.append(o)
        at += k
    assert at == n - 32
    for t in range(at, n):                                           # ... the last 32 one by one
        got.append(r.step([dict(id="a", tokens=toks[t:t + 1], want=[0])]))
    near_plain(torch.cat(got), plain, exact, "portions, then token by token")
    near_float32(torch.cat(got), ref, "portions, then token by token")
    same_cut(torch.cat(got), whole, plain, exact, "portions, then token by token, against the whole prompt")
    from kvcm.kernels import library as K
    assert K.attention_tcgen05_error() == 0 and K.tcgen05_error() == 0 and K.stream_error() == 0


def test_mixed_batch(engines):
    """Three requests: portions of one beside single tokens of the others, in one step each."""
    cfg, make = engines
    seqs = [helpers.random_tokens(n, cfg.vocab_size, 10 + i) for i, n in enumerate((400, 333, 150))]
    refs, alone = [], []
    for s in seqs:
        w = list(range(len(s) - 20, len(s)))
        refs.append(make["float32"]().step([dict(id="x", tokens=s, want=w)]))
        alone.append(make["bfloat16"]().step([dict(id="x", tokens=s, want=w)]))
    r = make["bfloat16"]()
    # everything but the last 20 tokens of each request first, in two steps
    r.step([dict(id=f"r{i}", tokens=s[:len(s) - 20 - 7 * i], want=[]) for i, s in enumerate(seqs)])
    fed = [len(s) - 20 - 7 * i for i, s in enumerate(seqs)]
    got = [[] for _ in seqs]
    while any(f < len(s) for f, s in zip(fed, seqs)):
        entries = []
        for i, s in enumerate(seqs):
            if fed[i] >= len(s):
                continue
            k = 1 if i != 1 else min(5, len(s) - fed[i])           # request 1 goes on in portions of five
            k = min(k, len(s) - fed[i])
            w = [p - fed[i] for p in range(len(s) - 20, len(s)) if fed[i] <= p < fed[i] + k]
            entries.append((i, dict(id=f"r{i}", tokens=s[fed[i]:fed[i] + k], want=w)))
            fed[i] += k
        out = r.step([e for _, e in entries])
        at = 0
        for i, e in entries:
            n = len(e["want"])
            if n:
                got[i].append(out[at:at + n])
            at += n
    for i in range(3):
        rounded, exact = make["plain"](seqs[i])[-20:], make["plain"](seqs[i], None)[-20:]
        near_plain(torch.cat(got[i]), rounded, exact, f"mixed, request {i}, against the plain implementation")
        near_float32(torch.cat(got[i]), refs[i], f"mixed, request {i}")
        same_cut(torch.cat(got[i]), alone[i], rounded, exact, f"mixed, request {i}, against the request alone")


def greedy_or_near_tie(prompts, run_a, run_b, plain, n):
    """Every token of both runs is the plain implementation's greedy choice, or within a near-tie of
    it.  The two runs need not agree to the bit (a padded batch and the batch itself take other
    context partitions, and larger ones other library kernels), so where they part ways, the plain
    logits must show a near-tie at that very place."""
    for p, a, b in zip(prompts, run_a, run_b):
        assert len(a) == n and len(b) == n
        for o in ((a,) if a == b else (a, b)):
            logits = plain(list(p) + list(o))
            margin = 0.08 * logits.std().item()
            for k, tok in enumerate(o):
                row = logits[len(p) - 1 + k]
                assert row.max().item() - row[tok].item() <= margin, (len(p), k, tok)
        if a != b:
            k = next(i for i in range(n) if a[i] != b[i])
            row = plain(list(p) + list(a))[len(p) - 1 + k]
            top = row.topk(2).values
            assert (top[0] - top[1]).item() <= 0.08 * row.std().item(), f"runs part ways at a clear choice (token {k})"


@pytest.mark.parametrize("batch", [24, 64])
def test_decode_batches_beyond_the_streaming_kernels(engines, batch):
    """Decode steps of 24 and 64 requests: more rows than the weight-streaming products take, so the
    library products, the separate rotary / cache-write and activation kernels and another plan of
    context partitions run.  Contexts differ from request to request (pages and tiles end in
    different places); every request's logits are held against the plain implementation."""
    cfg, make = engines
    lens = [33 + (37 * i) % 190 for i in range(batch)]
    seqs = [helpers.random_tokens(n + 3, cfg.vocab_size, 500 + i) for i, n in enumerate(lens)]
    r = make["bfloat16"](max_live=batch, max_tokens=batch * 256)
    for lo in range(0, batch, 8):                                    # the prompts, eight requests a step
        r.step([dict(id=f"r{i}", tokens=seqs[i][:lens[i]], want=[]) for i in range(lo, min(lo + 8, batch))])
    outs = []
    for t in range(3):                                               # three decode steps of the whole batch
        outs.append(r.step([dict(id=f"r{i}", tokens=[seqs[i][lens[i] + t]], want=[0]) for i in range(batch)]))
    for t in range(3):
        ref = torch.stack([make["plain"](seqs[i])[lens[i] + t] for i in range(batch)])
        exact = torch.stack([make["plain"](seqs[i], None)[lens[i] + t] for i in range(batch)])
        near_plain(outs[t], ref, exact, f"decode step {t} of {batch} requests")


def test_decode_graphs_give_the_tokens_of_eager_steps(engines):
    """Greedy generation through the engine at this shape with CUDA graphs (padded batch buckets,
    context buckets, dependent launches inside the graph) and without: the plain implementation's
    greedy tokens in both runs, and the same tokens unless the choice is a near-tie (the context
    bucket of a graph splits the keys into other partitions than the context itself)."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    from kvcm.engine import model_from_tensors
    from kvcm.weights import random_tensors
    cfg, make = engines
    spec = model_from_tensors(cfg, dict(random_tensors(cfg, 7, torch.bfloat16, device="cuda:0", norm_jitter=0.1)),
                              "bfloat16", "cuda:0")
    prompts = [helpers.random_tokens(n, cfg.vocab_size, 20 + i) for i, n in enumerate((300, 150, 700))]
    outs = {}
    for graphs in (True, False):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=160, block_size=16, max_seq_len=1024, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=4, max_batched_tokens=1024), dtype="bfloat16",
                          cuda_graphs=graphs)
        eng = kvcm.Engine(spec, ec)
        outs[graphs] = kvcm.generate(eng, prompts, 24)
        assert (eng.graphs is not None) == graphs
        if graphs:
            assert eng.graphs.replays > 0
        assert eng.kv.blocks_in_use() == 0
    greedy_or_near_tie(prompts, outs[True], outs[False], make["plain"], 24)


def test_graph_buckets_are_crossed_while_portions_are_in_flight(engines):
    """Eleven requests arrive one after another while earlier ones decode: prompts are cut into
    portions of at most 96 tokens, so for many steps a portion runs beside the decode rows (those
    steps run eagerly), and in between the decode-only steps grow from one request to eleven, over
    the graph buckets 1, 2, 4, 8 and 16.  With graphs and without, every token is the plain
    implementation's greedy choice unless that choice is a near-tie."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    from kvcm.engine import model_from_tensors
    from kvcm.weights import random_tensors
    cfg, make = engines
    spec = model_from_tensors(cfg, dict(random_tensors(cfg, 7, torch.bfloat16, device="cuda:0", norm_jitter=0.1)),
                              "bfloat16", "cuda:0")
    prompts = [helpers.random_tokens(60 + 23 * i, cfg.vocab_size, 700 + i) for i in range(11)]
    outs, seen = {}, {}
    for graphs in (True, False):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=400, block_size=16, max_seq_len=512, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=16, max_batched_tokens=96), dtype="bfloat16",
                          cuda_graphs=graphs)
        eng = kvcm.Engine(spec, ec)
        ids, done, mixed, step = [], {}, 0, 0
        while len(ids) < len(prompts) or not eng.idle():
            if step % 3 == 0 and len(ids) < len(prompts):
                ids.append(eng.add_request(prompts[len(ids)], max_new_tokens=40))
            info = eng.step()
            mixed += int(info.prefill_tokens > 0 and info.decode_seqs > 0)
            for f in eng.take_finished():
                done[f.id] = f.generated()
            step += 1
        outs[graphs] = [done[i] for i in ids]
        seen[graphs] = (mixed, sorted({k[0] for k in eng.graphs.captured}) if eng.graphs else [])
    assert seen[True][0] >= 8 and set(seen[True][1]) >= {1, 2, 4, 8, 16}, seen[True]
    greedy_or_near_tie(prompts, outs[True], outs[False], make["plain"], 40)
