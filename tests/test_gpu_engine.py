"""Generation through the Python entry point (scheduler, chunked prefill, sampling, decode
graphs) against the plain implementation, and the engine's invariances: batch vs alone, paged vs
contiguous, prefix cache on vs off, with and without preemption, with and without CUDA graphs."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


def make_engine(folder, dtype, name, **over):
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    kv = KVManagerConfig(num_blocks=over.pop("num_blocks", 128), block_size=helpers.TINY[name]["block_size"],
                         max_seq_len=over.pop("max_seq_len", 256), policy=over.pop("policy", "paged"),
                         prefix_caching=over.pop("prefix", False), watermark_blocks=over.pop("watermark", 0))
    sc = SchedulerConfig(max_num_seqs=over.pop("max_num_seqs", 8),
                         max_batched_tokens=over.pop("max_batched_tokens", 256),
                         prefill_chunk=over.pop("prefill_chunk", 0),
                         chunked_prefill=over.pop("chunked_prefill", True))
    cfg = EngineConfig(kv=kv, sched=sc, dtype=dtype, **over)
    return kvcm.Engine.from_folder(folder, cfg)


def run(engine, prompts, max_new, temperature=0.0, seed=None):
    import kvcm
    return kvcm.generate(engine, prompts, max_new, temperature, seed)


def margin(dtype, ref_logits):
    return 2e-4 if dtype == "float32" else 0.04 * ref_logits.std().item()


def check_greedy(folder, dtype, prompts, outs):
    """Every generated token must be the plain implementation's argmax on the engine's own
    prefix, or within the dtype's tolerance of it (a near-tie)."""
    cfg, w = P.read_model_folder(folder)
    storage = None if dtype == "float32" else torch.bfloat16
    for p, o in zip(prompts, outs):
        logits = P.llama_forward(cfg, w, list(p) + list(o), storage)
        m = margin(dtype, logits)
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= m, \
                f"token {k} = {tok}: plain prefers {P.greedy_pick(row)} by {row.max().item() - row[tok].item():.3e}"


PROMPTS_A = [5, 17, 33, 64]
PROMPTS_B = [1, 7, 40, 100, 150, 200]


def prompts(name, lengths):
    v = helpers.TINY[name]["cfg"]["vocab_size"]
    return [helpers.random_tokens(n, v, 500 + i) for i, n in enumerate(lengths)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(dtype, model_folders):
    folder = model_folders("tiny-a", dtype)
    ps = prompts("tiny-a", PROMPTS_A)
    eng = make_engine(folder, dtype, "tiny-a")
    outs = run(eng, ps, 16)
    assert [len(o) for o in outs] == [16] * 4
    check_greedy(folder, dtype, ps, outs)
    assert eng.kv.blocks_in_use() == 0
    assert eng.graphs.replays > 0                       # decode steps went through captured graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_tiny_b_chunked_and_mixed(dtype, model_folders):
    from kvcm.sampling import uniform_for
    folder = model_folders("tiny-b", dtype)
    ps = prompts("tiny-b", PROMPTS_B)
    eng = make_engine(folder, dtype, "tiny-b", num_blocks=256, max_seq_len=256, prefill_chunk=24,
                      max_batched_tokens=64, sampling_seed=1234)
    infos = []
    ids = [eng.add_request(p, 24, temperature=0.8) for p in ps]
    done = {}
    while not eng.idle():
        infos.append(eng.step())
        for f in eng.take_finished():
            done[f.id] = f
    assert any(i.prefill_tokens and i.decode_seqs for i in infos), "portions must run beside decodes"
    assert max(i.rows for i in infos) <= 64
    cfg, w = P.read_model_folder(folder)
    storage = None if dtype == "float32" else torch.bfloat16
    for rid, p in zip(ids, ps):
        o = done[rid].generated()
        assert len(o) == 24
        logits = P.llama_forward(cfg, w, list(p) + o, storage)
        m = 1e-4 if dtype == "float32" else 0.02
        for k, tok in enumerate(o):
            probs = P.temperature_probs(logits[len(p) - 1 + k], 0.8)
            c = torch.cumsum(probs, 0)
            u = uniform_for(1234, rid, len(p) + k)
            lo = float(c[tok - 1]) if tok else 0.0
            assert lo - m <= u <= float(c[tok]) + m, f"request {rid} token {k}: u={u} outside [{lo}, {float(c[tok])}]"
    # the same requests alone, unchunked, in another order: the same tokens (the draw depends on
    # seed, request id and position only)
    eng2 = make_engine(folder, dtype, "tiny-b", num_blocks=256, max_seq_len=256, sampling_seed=1234,
                       chunked_prefill=False, max_batched_tokens=256)
    for rid, p in reversed(list(zip(ids, ps))):
        eng2.add_request(p, 24, temperature=0.8, request_id=rid)
        eng2.run_until_idle()
        f = eng2.take_finished()[0]
        if dtype == "float32":
            assert f.generated() == done[rid].generated()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_invariances_of_generation(dtype, model_folders):
    name = "tiny-a"
    folder = model_folders(name, dtype)
    ps = prompts(name, [5, 17, 33, 64, 40, 40])
    ps[5] = ps[4][:32] + ps[5][32:]                        # shares two full pages with request 4
    base = run(make_engine(folder, dtype, name), ps, 16)
    check_greedy(folder, dtype, ps, base)
    variants = {
        "alone": [run(make_engine(folder, dtype, name), [p], 16)[0] for p in ps],
        "contiguous": run(make_engine(folder, dtype, name, policy="contiguous", num_blocks=128, max_seq_len=128), ps, 16),
        "prefix cache": run(make_engine(folder, dtype, name, prefix=True), ps, 16),
        "no graphs": run(make_engine(folder, dtype, name, cuda_graphs=False), ps, 16),
        "small portions": run(make_engine(folder, dtype, name, prefill_chunk=5, max_batched_tokens=24), ps, 16),
    }
    for what, outs in variants.items():
        if dtype == "float32":
            assert outs == base, what
        else:
            check_greedy(folder, dtype, ps, outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_on_the_gpu_gives_the_same_tokens(dtype, model_folders):
    name = "tiny-a"
    folder = model_folders(name, dtype)
    ps = prompts(name, [30, 30, 30, 30, 30, 30])
    roomy = make_engine(folder, dtype, name)
    want = run(roomy, ps, 40)
    tight = make_engine(folder, dtype, name, num_blocks=14, max_seq_len=96)    # 14 pages of 16: not enough
    got = run(tight, ps, 40)
    assert tight.sched.counters().preemptions > 0, "the pool must be small enough to evict"
    assert tight.kv.blocks_in_use() == 0 and tight.sched.slots_taken() == 0
    if dtype == "float32":
        assert got == want
    else:
        check_greedy(folder, dtype, ps, got)


def test_prefix_cache_saves_prompt_tokens(model_folders):
    name, dtype = "tiny-a", "bfloat16"
    folder = model_folders(name, dtype)
    v = helpers.TINY[name]["cfg"]["vocab_size"]
    shared = helpers.random_tokens(48, v, 9)
    ps = [shared + helpers.random_tokens(10, v, 20 + i) for i in range(3)]
    eng = make_engine(folder, dtype, name, prefix=True)
    outs = [run(eng, [p], 4)[0] for p in ps]                # one after the other: pages are registered
    assert eng.sched.counters().prefill_tokens_saved == 2 * 48
    check_greedy(folder, dtype, ps, outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_score_returns_every_position(dtype, model_folders):
    name = "tiny-b"
    folder = model_folders(name, dtype)
    toks = helpers.random_tokens(77, helpers.TINY[name]["cfg"]["vocab_size"], 3)
    eng = make_engine(folder, dtype, name)
    cfg, w = P.read_model_folder(folder)
    ref = P.llama_forward(cfg, w, toks, None if dtype == "float32" else torch.bfloat16)
    helpers.assert_logits_close(eng.score(toks), ref, dtype, "score")
    assert eng.kv.blocks_in_use() == 0
    with pytest.raises(RuntimeError):
        make_engine(folder, dtype, name, prefix=True).score(toks)


def test_native_products_only(model_folders):
    """``gemm='native'``: no library product anywhere (streaming kernel up to 16 rows, split-K
    tcgen05 up to 255, tiled tcgen05 from 256): whole-sequence logits and greedy generation with
    portions of every size class."""
    name, dtype = "tiny-b", "bfloat16"
    folder = model_folders(name, dtype)
    import kvcm.parts.linear as L
    calls = []
    real_mm = torch.mm
    try:
        torch.mm = lambda *a, **k: calls.append(1) or real_mm(*a, **k)
        eng = make_engine(folder, dtype, name, gemm="native", max_seq_len=512, num_blocks=256,
                          max_batched_tokens=512)
        toks = helpers.random_tokens(300, helpers.TINY[name]["cfg"]["vocab_size"], 4)     # 300 rows: tiled tcgen05
        cfg, w = P.read_model_folder(folder)
        ref = P.llama_forward(cfg, w, toks, torch.bfloat16)
        helpers.assert_logits_close(eng.score(toks), ref, dtype, "score, native products")
        ps = prompts(name, [1, 7, 40, 100, 150])                                         # split-K and streaming sizes
        outs = run(eng, ps, 12)
        check_greedy(folder, dtype, ps, outs)
    finally:
        torch.mm = real_mm
    assert not calls, "a library product ran in native mode"
    from kvcm.kernels import library as K
    assert K.splitk_error() == 0 and K.tcgen05_error() == 0 and K.stream_error() == 0


def test_rejects_bad_requests_and_cpu_device(model_folders):
    folder = model_folders("tiny-a", "bfloat16")
    eng = make_engine(folder, "bfloat16", "tiny-a", max_seq_len=64)
    with pytest.raises(ValueError):
        eng.add_request([], 4)
    with pytest.raises(ValueError):
        eng.add_request([999999], 4)
    eng.add_request([1] * 100, 4)                          # longer than max_seq_len
    eng.run_until_idle()
    assert eng.take_finished()[0].rejected
    with pytest.raises(Exception):
        make_engine(folder, "bfloat16", "tiny-a", device="cpu")
