"""The engine against the plain implementation under every way of cutting the work, in float32
and in bfloat16: each request alone and whole; most of it in one step and the last 32 tokens one
by one; portions of changing size down to two tokens; and mixed, up to four live requests,
portions of some beside decoded tokens of others, with so few pages that they are used again.
In-process through the step function, and through ``bin/trace_run`` as a user runs it."""
import itertools

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny-a": [5, 17, 33, 64, 100], "tiny-b": [1, 7, 40, 100, 150, 200], "tiny-c": [3, 70, 130, 250, 193],
           "tiny-d": [2, 65, 129, 255, 200]}
CASES = [(n, d) for n in ("tiny-a", "tiny-b") for d in ("float32", "bfloat16")] + [("tiny-c", "bfloat16"), ("tiny-d", "bfloat16")]


@pytest.fixture(scope="module")
def oracle(model_folders):
    """(name, dtype, request index) -> plain logits [len, vocab] of the whole request."""
    cache = {}

    def get(name, dtype, i):
        key = (name, dtype, i)
        if key not in cache:
            cfg, w = P.read_model_folder(model_folders(name, dtype))
            toks = tokens_of(name, i)
            cache[key] = P.llama_forward(cfg, w, toks, None if dtype == "float32" else torch.bfloat16)
        return cache[key]
    return get


def tokens_of(name, i):
    return helpers.random_tokens(LENGTHS[name][i], helpers.TINY[name]["cfg"]["vocab_size"], 100 + i)


def replayer(model_folders, name, dtype, max_tokens, **kw):
    return helpers.Replayer(model_folders(name, dtype), dtype, max_tokens,
                            helpers.TINY[name]["block_size"], **kw)


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(name, dtype, model_folders, oracle):
    r = replayer(model_folders, name, dtype, 256)
    for i in range(len(LENGTHS[name])):
        toks = tokens_of(name, i)
        got = r.step([dict(id=f"r{i}", tokens=toks, want=list(range(len(toks))))], end=[f"r{i}"])
        helpers.assert_logits_close(got, oracle(name, dtype, i), dtype, f"{name} whole request {i}")
    assert r.kv.blocks_in_use() == 0
    assert r.stray_writes() == []          # pages that were never handed out are still zero


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_last_32_tokens_one_by_one(name, dtype, model_folders, oracle):
    r = replayer(model_folders, name, dtype, 256)
    for i, n in enumerate(LENGTHS[name]):
        if n < 34:
            continue
        toks = tokens_of(name, i)
        head = n - 32
        outs = [r.step([dict(id="x", tokens=toks[:head], want=list(range(head)))])]
        for t in range(head, n):
            outs.append(r.step([dict(id="x", tokens=[toks[t]], want=[0])], end=["x"] if t == n - 1 else []))
        got = torch.cat(outs)
        ref = oracle(name, dtype, i)
        helpers.assert_logits_close(got[:head], ref[:head], dtype, f"{name} request {i} prefill")
        helpers.assert_logits_close(got[head:], ref[head:], dtype, f"{name} request {i} decode")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size_down_to_two_tokens(name, dtype, model_folders, oracle):
    r = replayer(model_folders, name, dtype, 256)
    sizes = itertools.cycle([7, 2, 13, 2, 5, 31, 3, 2, 17])
    for i, n in enumerate(LENGTHS[name]):
        toks = tokens_of(name, i)
        outs, at = [], 0
        while at < n:
            k = min(next(sizes), n - at)
            outs.append(r.step([dict(id="x", tokens=toks[at:at + k], want=list(range(k)))],
                               end=["x"] if at + k == n else []))
            at += k
        helpers.assert_logits_close(torch.cat(outs), oracle(name, dtype, i), dtype,
                                    f"{name} request {i} in portions")


def mixed_trace(name):
    """A schedule with up to four live requests: portions of some beside single tokens of others.
    Returns (steps, place of every wanted row: (request, position))."""
    n_req = len(LENGTHS[name])
    toks = [tokens_of(name, i) for i in range(n_req)]
    fed = [0] * n_req
    sizes = itertools.cycle([9, 2, 21, 4, 2, 14])
    waiting = list(range(n_req))
    live, steps, places = [], [], []
    step_no = 0
    while waiting or live:
        while waiting and len(live) < 4 and (step_no % 2 == 0 or not live):
            live.append(waiting.pop(0))
        entries, ended, where = [], [], []
        for j, i in enumerate(list(live)):
            n = len(toks[i])
            left = n - fed[i]
            # the last 6 tokens of every request go one by one (decode rows beside portions)
            k = 1 if left <= 6 else min(next(sizes), left - 6)
            if (step_no + j) % 5 == 4 and len(live) > 1:
                continue                                   # left out of this step, goes on later
            entries.append(dict(id=f"r{i}", tokens=toks[i][fed[i]:fed[i] + k], want=list(range(k))))
            where += [(i, fed[i] + w) for w in range(k)]
            fed[i] += k
            if fed[i] == n:
                ended.append(f"r{i}")
                live.remove(i)
        steps.append(dict(step=step_no, entries=entries, end=ended))
        places.append(where)
        step_no += 1
    return steps, places


def mixed_pool_tokens(name):
    """The most tokens live at any time, each request's count rounded up to a multiple of 64."""
    steps, _ = mixed_trace(name)
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(helpers.roundup(v, 64) for v in held.values()))
        for rid in s["end"]:
            held.pop(rid)
    return peak


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_pages_used_again(name, dtype, model_folders, oracle):
    steps, places = mixed_trace(name)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(any(len(e["tokens"]) == 1 for e in s["entries"]) and any(len(e["tokens"]) > 1 for e in s["entries"])
               for s in steps), "the trace must mix portions and single tokens"
    r = replayer(model_folders, name, dtype, mixed_pool_tokens(name))
    for s, where in zip(steps, places):
        got = r.step(s["entries"], s["end"])
        ref = torch.stack([oracle(name, dtype, i)[pos] for i, pos in where])
        helpers.assert_logits_close(got, ref, dtype, f"{name} mixed step {s['step']}")
    assert len(set(r.pages_seen)) <= r.kv.num_blocks()
    assert any(len(owners) > 1 for owners in r.page_owners.values()), "no page was used again"
    assert r.stray_writes() == []
    total_pages = sum(helpers.roundup(n, r.runner.block_size) // r.runner.block_size for n in LENGTHS[name])
    assert total_pages > r.kv.num_blocks(), "the pool must be too small to hold every request at once"
    assert r.kv.blocks_in_use() == 0


@pytest.mark.parametrize("name,dtype", CASES)
def test_trace_tool_as_a_user_runs_it(name, dtype, model_folders, oracle, tmp_path):
    steps, places = mixed_trace(name)
    out = helpers.run_trace_tool(model_folders(name, dtype), dtype, steps, mixed_pool_tokens(name),
                                 str(tmp_path), ["--block-size", str(helpers.TINY[name]["block_size"])])
    for s, where in zip(steps, places):
        ref = torch.stack([oracle(name, dtype, i)[pos] for i, pos in where])
        helpers.assert_logits_close(torch.from_numpy(out[s["step"]]), ref, dtype,
                                    f"{name} trace_run step {s['step']}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_tool_default_page_size_and_steps_without_wants(dtype, model_folders, oracle, tmp_path):
    name = "tiny-a"
    toks = tokens_of(name, 3)
    steps = [dict(step=0, entries=[dict(id="a", tokens=toks[:40], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=toks[40:], want=[0, 23])], end=["a"]),
             dict(step=2, entries=[dict(id="b", tokens=toks[:3], want=[2])], end=["b"])]
    out = helpers.run_trace_tool(model_folders(name, dtype), dtype, steps, 64, str(tmp_path))
    ref = oracle(name, dtype, 3)
    assert sorted(out) == [1, 2]
    helpers.assert_logits_close(torch.from_numpy(out[1]), ref[[40, 63]], dtype, "wants in a later portion")
    helpers.assert_logits_close(torch.from_numpy(out[2]), ref[[2]], dtype, "pages of a used again by b")


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(name, dtype, model_folders, oracle):
    """Positions 0, 1, 2: one key, no history, the first slot of the first page."""
    r = replayer(model_folders, name, dtype, 64)
    i = 2
    toks = tokens_of(name, i)
    outs = [r.step([dict(id="x", tokens=[toks[t]], want=[0])]) for t in range(3)]
    helpers.assert_logits_close(torch.cat(outs), oracle(name, dtype, i)[:3], dtype, f"{name} first tokens")


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding(name, dtype, model_folders, oracle):
    """Every token after the first decoded one by one, across many page edges."""
    r = replayer(model_folders, name, dtype, 256)
    i = len(LENGTHS[name]) - 1
    toks = tokens_of(name, i)
    outs = [r.step([dict(id="x", tokens=[t], want=[0])]) for t in toks]
    helpers.assert_logits_close(torch.cat(outs), oracle(name, dtype, i), dtype, f"{name} long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuts_agree_bit_for_bit_with_plain_kernels(dtype, model_folders):
    """With the plain kernels every row is computed by the same sums whatever the batch, so two
    ways of cutting give equal bits; a difference here is a fault of the cache or the batch."""
    name = "tiny-b"
    opts = {"attention": "plain", "gemm": "plain"}
    toks = tokens_of(name, 3)
    a = replayer(model_folders, name, dtype, 128, options=opts)
    whole = a.step([dict(id="x", tokens=toks, want=list(range(len(toks))))])
    b = replayer(model_folders, name, dtype, 128, options=opts)
    parts, at = [], 0
    for k in itertools.cycle([5, 2, 1, 19]):
        k = min(k, len(toks) - at)
        parts.append(b.step([dict(id="x", tokens=toks[at:at + k], want=list(range(k)))]))
        at += k
        if at == len(toks):
            break
    assert torch.equal(torch.cat(parts), whole)


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_tcgen05_products_inside_the_engine(name, model_folders, oracle):
    """The same requests with every many-row product forced onto the tcgen05 kernel."""
    dtype = "bfloat16"
    r = replayer(model_folders, name, dtype, 256, options={"gemm": "tcgen05"})
    for i in (3, len(LENGTHS[name]) - 1):
        toks = tokens_of(name, i)
        got = r.step([dict(id="x", tokens=toks, want=list(range(len(toks))))], end=["x"])
        helpers.assert_logits_close(got, oracle(name, dtype, i), dtype, f"{name} request {i} through tcgen05")
    from kvcm.kernels import library as K
    assert K.tcgen05_error() == 0


def test_trace_tool_refuses_with_one_line(model_folders, tmp_path):
    """What the tool cannot run ends it with a message that names the step and the request, not
    with a stack trace: a portion beyond the pool, a wanted place outside the portion, no tokens, a
    token beyond the vocabulary."""
    import json
    import os
    import subprocess
    import sys
    folder = model_folders("tiny-a", "bfloat16")
    toks = tokens_of("tiny-a", 4)
    cases = [([dict(step=3, entries=[dict(id="a", tokens=toks[:100], want=[99])], end=[])], "does not fit the cache"),
             ([dict(step=3, entries=[dict(id="a", tokens=toks[:10], want=[10])], end=[])], "wants place 10"),
             ([dict(step=3, entries=[dict(id="a", tokens=[], want=[])], end=[])], "brings no tokens"),
             ([dict(step=3, entries=[dict(id="a", tokens=[256], want=[0])], end=[])], "outside the vocabulary")]
    for steps, message in cases:
        p = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", folder,
                            "--dtype", "bfloat16", "--out", str(tmp_path), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), text=True,
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=600)
        assert p.returncode != 0 and "done 3" not in p.stdout
        last = [l for l in p.stderr.splitlines() if l.strip()][-1]
        assert last.startswith("trace_run: step 3:") and message in last, p.stderr[-1500:]


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_under_the_contiguous_policy(name, dtype, model_folders, oracle):
    """The mixed schedule again with the contiguous policy (every request reserves its longest
    length as one run of pages): right against the plain implementation, and equal bit for bit to
    the paged run -- the kernels are the same, only the page numbers differ."""
    steps, places = mixed_trace(name)
    block = helpers.TINY[name]["block_size"]
    longest = helpers.roundup(max(LENGTHS[name]), block)
    paged = replayer(model_folders, name, dtype, mixed_pool_tokens(name))
    contiguous = replayer(model_folders, name, dtype, 4 * longest, policy="contiguous", max_seq_len=longest)
    assert contiguous.kv.name() == "contiguous"
    for s, where in zip(steps, places):
        a = paged.step(s["entries"], s["end"])
        b = contiguous.step(s["entries"], s["end"])
        ref = torch.stack([oracle(name, dtype, i)[pos] for i, pos in where])
        helpers.assert_logits_close(b, ref, dtype, f"{name} contiguous, mixed step {s['step']}")
        assert torch.equal(a, b), f"{name} step {s['step']}: paged and contiguous differ"
        for e in s["entries"]:
            if e["id"] in contiguous.live:
                t = contiguous.live[e["id"]].table(0)
                assert t == list(range(t[0], t[0] + len(t))) and len(t) == longest // block
    assert contiguous.kv.blocks_in_use() == 0


@pytest.mark.parametrize("name,dtype", [("tiny-b", "float32"), ("tiny-b", "bfloat16"), ("tiny-c", "bfloat16"),
                                        ("tiny-d", "bfloat16")])
def test_prefix_cache_hits_at_the_logit_level(name, dtype, model_folders):
    """With prefix caching a new request takes over the pages of an earlier one that hold the same
    tokens, and computes only the rest.  Checked on logits, not on greedy tokens: a shared page that
    is slightly wrong moves them.  Request b shares 67 tokens with a; its first portion ends in the
    middle of a page, the next ones start there; a is still live meanwhile (the pages are held
    twice) and goes on afterwards; c arrives after both have ended and hits the parked pages."""
    block = helpers.TINY[name]["block_size"]
    vocab = helpers.TINY[name]["cfg"]["vocab_size"]
    cfg, w = P.read_model_folder(model_folders(name, dtype))
    storage = None if dtype == "float32" else torch.bfloat16
    ta = helpers.random_tokens(101, vocab, 7)
    tb = ta[:67] + helpers.random_tokens(53, vocab, 8)
    tc = tb[:90] + helpers.random_tokens(20, vocab, 9)
    ra, rb, rc = (P.llama_forward(cfg, w, t, storage) for t in (ta, tb, tc))
    r = replayer(model_folders, name, dtype, 512, prefix_caching=True)
    got = r.step([dict(id="a", tokens=ta[:100], want=list(range(100)))])
    helpers.assert_logits_close(got, ra[:100], dtype, "request a")
    # b: its first portion of 70 tokens; the pages of a that match (whole pages, and never the page
    # with the portion's last token) are taken over
    hit = min(67 // block, (70 - 1) // block) * block
    assert hit >= 32
    with pytest.raises(Exception, match="taken over from the prefix cache"):
        r.step([dict(id="b", tokens=tb[:70], want=[0])])
    assert "b" not in r.live                                   # a refused request is not taken
    got = r.step([dict(id="b", tokens=tb[:70], want=list(range(hit, 70)))])
    assert r.session.cached_tokens_last == {"b": hit}
    assert r.live["b"].table(0)[:hit // block] == r.live["a"].table(0)[:hit // block]     # the same pages
    helpers.assert_logits_close(got, rb[hit:70], dtype, "b after a prefix hit")
    outs, at = [], 70
    for k in (2, 13, 1, 1, len(tb) - 87):
        outs.append(r.step([dict(id="b", tokens=tb[at:at + k], want=list(range(k)))]))
        at += k
    assert at == len(tb)
    helpers.assert_logits_close(torch.cat(outs), rb[70:], dtype, "b in portions that start inside a page")
    # a goes on: its shared pages are what they were
    got = r.step([dict(id="a", tokens=ta[100:], want=[0])], end=["a", "b"])
    helpers.assert_logits_close(got, ra[100:], dtype, "a after b read its pages")
    assert r.kv.blocks_in_use() == 0 and r.kv.blocks_cached_free() > 0
    # c: both are gone, their pages are parked; c finds 90 tokens of b among them
    hit_c = min(90 // block, (len(tc) - 1) // block) * block
    got = r.step([dict(id="c", tokens=tc, want=list(range(hit_c, len(tc))))], end=["c"])
    assert r.session.cached_tokens_last == {"c": hit_c} and hit_c >= 64
    helpers.assert_logits_close(got, rc[hit_c:], dtype, "c after hitting parked pages")
    st = r.kv.prefix_stats()
    assert st.hit_blocks >= (hit + hit_c) // block


def test_trace_tool_with_policy_and_prefix_flags(model_folders, tmp_path):
    """``bin/trace_run --policy contiguous`` and ``--prefix`` as a user runs them."""
    name, dtype = "tiny-b", "bfloat16"
    block = helpers.TINY[name]["block_size"]
    vocab = helpers.TINY[name]["cfg"]["vocab_size"]
    cfg, w = P.read_model_folder(model_folders(name, dtype))
    ta = helpers.random_tokens(60, vocab, 17)
    tb = ta[:41] + helpers.random_tokens(30, vocab, 18)
    ra, rb = (P.llama_forward(cfg, w, t, torch.bfloat16) for t in (ta, tb))
    hit = (41 // block) * block
    steps = [dict(step=0, entries=[dict(id="a", tokens=ta, want=[59])], end=[]),
             dict(step=1, entries=[dict(id="b", tokens=tb[:50], want=list(range(hit, 50)))], end=["a"]),
             dict(step=2, entries=[dict(id="b", tokens=tb[50:], want=list(range(21)))], end=["b"])]
    out = helpers.run_trace_tool(model_folders(name, dtype), dtype, steps, 256, str(tmp_path / "p"),
                                 ["--block-size", str(block), "--prefix"])
    helpers.assert_logits_close(torch.from_numpy(out[0]), ra[[59]], dtype, "trace_run --prefix, a")
    helpers.assert_logits_close(torch.from_numpy(out[1]), rb[hit:50], dtype, "trace_run --prefix, b after a hit")
    helpers.assert_logits_close(torch.from_numpy(out[2]), rb[50:], dtype, "trace_run --prefix, b goes on")
    steps = [dict(step=0, entries=[dict(id="a", tokens=ta, want=[59])], end=[]),
             dict(step=1, entries=[dict(id="b", tokens=tb, want=[70])], end=["a", "b"])]
    out = helpers.run_trace_tool(model_folders(name, dtype), dtype, steps, 256, str(tmp_path / "c"),
                                 ["--block-size", str(block), "--policy", "contiguous", "--max-seq-len", "96"])
    helpers.assert_logits_close(torch.from_numpy(out[0]), ra[[59]], dtype, "trace_run --policy contiguous, a")
    helpers.assert_logits_close(torch.from_numpy(out[1]), rb[[70]], dtype, "trace_run --policy contiguous, b")
