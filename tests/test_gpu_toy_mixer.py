"""A toy architecture defined HERE, outside the package: layers with different mixers (attention
with a window, and a toy mixer with fixed-size state of its own), a layer that runs twice, and a
call site that reads another site's cache.  It is registered, built from a config.json, given
random weights, stepped in portions and decoded, and generated from through the engine, without
a change to the package's files.  A plain whole-sequence implementation of the toy model, also
here, is the oracle.  The toy parts stand for nothing but themselves."""
import json
import math
import os
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


def register_toy():
    import kvcm
    from kvcm.config import ModelConfig, register_architecture
    from kvcm.models.spec import ModelSpec, TensorBinding
    from kvcm.parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall, Linear, Mixer,
                            StateSpec)
    from kvcm.parts.embedding import Embedding, LMHead

    class DecayingSum(Mixer):
        """y_t = W (s_t / (t + 1)),  s_t = decay * s_{t-1} + h_t.  State per request: s (float32 [hidden]).
        Written with torch ops that read step data on the host: it is a test's toy, not a kernel of
        the engine, and says so (``capturable = False``: no CUDA graphs with it)."""

        capturable = False

        def __init__(self, hidden: int, decay: float) -> None:
            super().__init__()
            self.hidden, self.decay = hidden, decay
            self.proj = self.add_child("proj", Linear(hidden, hidden))

        def state_spec(self):
            return StateSpec((self.hidden,), torch.float32)

        def forward(self, h, ctx, site):
            out = torch.empty_like(h)
            starts, lens = ctx.seq_q_start.tolist(), ctx.seq_q_len.tolist()
            slots, pos = ctx.seq_state_slot.tolist(), ctx.positions.tolist()
            for q0, n, slot in zip(starts, lens, slots):
                if slot < 0:
                    continue
                s = site.state[slot]
                for r in range(q0, q0 + n):
                    s = self.decay * s + h[r].float()
                    out[r] = (s / (pos[r] + 1)).to(h.dtype)
                site.state[slot] = s
            return self.proj.forward(out, ctx)

    if "decaying_sum" not in MIXERS.names():
        MIXERS.register("decaying_sum", DecayingSum)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab: int = 0
        width: int = 0
        ffn: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        window: int = 0
        decay: float = 0.5
        eps: float = 1e-5
        theta: float = 10000.0

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyMixedForTests", **{k: d[k] for k in
                       ("vocab", "width", "ffn", "heads", "kv_heads", "head_dim", "window", "decay", "eps", "theta")})

        def to_json_dict(self):
            d = {k: getattr(self, k) for k in ("vocab", "width", "ffn", "heads", "kv_heads", "head_dim",
                                               "window", "decay", "eps", "theta")}
            d["architectures"] = [self.architecture]
            return d

    def build(cfg):
        H = cfg.width
        emb = Embedding(cfg.vocab, H)
        bind = [TensorBinding(emb, "weight", [("emb.weight", (cfg.vocab, H))])]
        blocks = []
        # layer 0: windowed attention; layer 1: the toy state mixer; layer 2: full attention
        kinds = [("attention", dict(window=cfg.window)), ("decaying_sum", {}), ("attention", dict(window=0))]
        for l, (kind, extra) in enumerate(kinds):
            if kind == "attention":
                pos = POSITION_ENCODINGS.build("rope", head_dim=cfg.head_dim, theta=cfg.theta)
                mixer = MIXERS.build("attention", hidden=H, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads,
                                     head_dim=cfg.head_dim, position=pos, **extra)
                q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
                bind += [TensorBinding(mixer.qkv, "weight", [(f"l{l}.q", (q, H)), (f"l{l}.k", (kv, H)), (f"l{l}.v", (kv, H))]),
                         TensorBinding(mixer.o, "weight", [(f"l{l}.o", (H, q))])]
            else:
                mixer = MIXERS.build("decaying_sum", hidden=H, decay=cfg.decay)
                bind.append(TensorBinding(mixer.proj, "weight", [(f"l{l}.proj", (H, H))]))
            ffn = FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=cfg.ffn)
            n1, n2 = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps), NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
            blocks.append(BLOCKS.build("pre_norm", norm1=n1, mixer=mixer, norm2=n2, ffn=ffn))
            bind += [TensorBinding(n1, "weight", [(f"l{l}.n1", (H,))]), TensorBinding(n2, "weight", [(f"l{l}.n2", (H,))]),
                     TensorBinding(ffn.gate_up, "weight", [(f"l{l}.gate", (cfg.ffn, H)), (f"l{l}.up", (cfg.ffn, H))]),
                     TensorBinding(ffn.down, "weight", [(f"l{l}.down", (H, cfg.ffn))])]
        fin = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
        head = LMHead(H, cfg.vocab)
        bind += [TensorBinding(fin, "weight", [("final.weight", (H,))]),
                 TensorBinding(head, "weight", [("head.weight", (cfg.vocab, H))], tie_to=bind[0], tied=True)]
        # run order: layer 0, layer 1, layer 2, layer 1 AGAIN (its own state), then layer 2's weights
        # once more reading the cache that the first run of layer 2 wrote
        order = [LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(1), LayerCall(2, cache_of=2)]
        return ModelSpec(cfg, emb, blocks, order, fin, head, bind)

    register_architecture("ToyMixedForTests", ToyConfig, build, replace=True)
    return ToyConfig


def plain_toy(cfg, w, tokens):
    """Whole sequence, float64, no cache."""
    n = len(tokens)
    pos = torch.arange(n)
    x = P.embedding(w["emb.weight"], tokens)
    c = dict(nh=cfg["heads"], nkv=cfg["kv_heads"], hd=cfg["head_dim"], theta=cfg["theta"])

    def attn(l, h, window):
        return P.attention_block(h, w[f"l{l}.q"], w[f"l{l}.k"], w[f"l{l}.v"], w[f"l{l}.o"], pos, c, window or None)

    def toy(l, h):
        s = torch.zeros(cfg["width"], dtype=torch.float64)
        out = torch.zeros_like(h)
        for t in range(n):
            s = cfg["decay"] * s + h[t]
            out[t] = s / (t + 1)
        return out @ w[f"l{l}.proj"].T

    def layer(l, x, mix):
        x = x + mix(l, P.rmsnorm(x, w[f"l{l}.n1"], cfg["eps"]))
        return x + P.gated_mlp(P.rmsnorm(x, w[f"l{l}.n2"], cfg["eps"]), w[f"l{l}.gate"], w[f"l{l}.up"], w[f"l{l}.down"])

    x = layer(0, x, lambda l, h: attn(l, h, cfg["window"]))
    x = layer(1, x, toy)
    x = layer(2, x, lambda l, h: attn(l, h, 0))
    x = layer(1, x, toy)
    # the fifth call site reads the keys and values that the first run of layer 2 wrote: those came
    # from ITS input, so this site's own k/v are never used; only its queries are its own.
    x = layer_reading_cache(cfg, w, x, pos, c, kv_input=None)
    return P.rmsnorm(x, w["final.weight"], cfg["eps"]) @ w["emb.weight"].T


_cached_kv = {}


def layer_reading_cache(cfg, w, x, pos, c, kv_input):
    n = x.shape[0]
    h = P.rmsnorm(x, w["l2.n1"], cfg["eps"])
    q = P.rope_rotate_half((h @ w["l2.q"].T).reshape(n, c["nh"], c["hd"]), pos, c["theta"])
    k, v = _cached_kv["k"], _cached_kv["v"]
    a = P.attention_causal(q, k, v, 1.0 / math.sqrt(c["hd"])) @ w["l2.o"].T
    x = x + a
    return x + P.gated_mlp(P.rmsnorm(x, w["l2.n2"], cfg["eps"]), w["l2.gate"], w["l2.up"], w["l2.down"])


def plain_toy_logits(cfg, w, tokens):
    """Runs plain_toy, capturing the k/v of the first run of layer 2 for the site that shares them."""
    n = len(tokens)
    pos = torch.arange(n)
    c = dict(nh=cfg["heads"], nkv=cfg["kv_heads"], hd=cfg["head_dim"], theta=cfg["theta"])
    orig = P.attention_block

    def spy(h, wq, wk, wv, wo, positions, cc, window=None, storage=None):
        if wq is w["l2.q"]:
            _cached_kv["k"] = P.rope_rotate_half((h @ wk.T).reshape(n, c["nkv"], c["hd"]), pos, c["theta"])
            _cached_kv["v"] = (h @ wv.T).reshape(n, c["nkv"], c["hd"])
        return orig(h, wq, wk, wv, wo, positions, cc, window, storage)
    P.attention_block = spy
    try:
        return plain_toy(cfg, w, tokens)
    finally:
        P.attention_block = orig


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    import kvcm
    ToyConfig = register_toy()
    cfg = ToyConfig(architecture="ToyMixedForTests", vocab=130, width=48, ffn=72, heads=3, kv_heads=1,
                    head_dim=16, window=10, decay=0.7, eps=1e-5, theta=10000.0)
    folder = str(tmp_path_factory.mktemp("toy"))
    kvcm.write_random_model(folder, cfg, seed=5, dtype=torch.float32, norm_jitter=0.1)
    assert kvcm.load_config(folder) == cfg                       # the registry finds it by name
    from safetensors import safe_open
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    return folder, json.load(open(os.path.join(folder, "config.json"))), w


def test_toy_model_layout(toy):
    folder, cfg, w = toy
    r = helpers.Replayer(folder, "float32", 128, 8)
    plan = r.runner.plan
    assert len(r.spec.order) == 5 and len(r.spec.blocks) == 3
    assert len(plan.groups) == 2 and sorted(plan.windows) == [0, 10]       # windowed and full attention: two groups
    assert plan.site_group[0] != plan.site_group[2] and plan.site_group[4] == plan.site_group[2]
    assert plan.site_layer[4] == plan.site_layer[2] and not plan.site_writes[4] and plan.site_writes[2]
    assert [s is not None for s in plan.site_state] == [False, True, False, True, False]
    sites = r.runner.pools.sites
    assert sites[1].state.data_ptr() != sites[3].state.data_ptr()            # a layer run twice: two states
    assert sites[4].k.data_ptr() == sites[2].k.data_ptr()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_stepped_in_portions_and_decoded(toy, dtype):
    folder, cfg, w = toy
    toks = helpers.random_tokens(60, cfg["vocab"], 8)
    ref = plain_toy_logits(cfg, w, toks)
    r = helpers.Replayer(folder, dtype, 128, 8)
    outs, at = [], 0
    for k in (7, 2, 13, 1, 1, 20, 2, 14):                                    # portions and single tokens
        outs.append(r.step([dict(id="x", tokens=toks[at:at + k], want=list(range(k)))]))
        at += k
    assert at == len(toks)
    got = torch.cat(outs)
    if dtype == "float32":
        helpers.assert_logits_close(got, ref, "float32", "toy model in portions")
    else:
        assert (got.double() - ref).abs().max().item() <= 0.06 * ref.std().item()   # weights stored in 32 bits stay so
    seq = r.live["x"]
    assert seq.table(r.runner.plan.windows.index(10))[:5] == [-1] * 5        # the window gave pages back
    assert all(p >= 0 for p in seq.table(r.runner.plan.windows.index(0)))
    # a second request beside the first, then the first one's slot used again after it ends
    toks2 = helpers.random_tokens(25, cfg["vocab"], 9)
    ref2 = plain_toy_logits(cfg, w, toks2)
    a = r.step([dict(id="y", tokens=toks2[:24], want=list(range(24)))], end=["x"])
    b = r.step([dict(id="y", tokens=toks2[24:], want=[0]), dict(id="z", tokens=toks[:9], want=list(range(9)))])
    tol_dtype = "float32"
    if dtype == "float32":
        helpers.assert_logits_close(torch.cat([a, b[:1]]), ref2, tol_dtype, "second request")
        helpers.assert_logits_close(b[1:], ref[:9], tol_dtype, "state slot used again starts from zero")


def test_toy_model_generates_through_the_engine(toy):
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder, cfg, w = toy
    ec = EngineConfig(kv=KVManagerConfig(num_blocks=24, block_size=8, max_seq_len=96, watermark_blocks=0),
                      sched=SchedulerConfig(max_num_seqs=3, max_batched_tokens=16), dtype="float32")
    eng = kvcm.Engine.from_folder(folder, ec)
    prompts = [helpers.random_tokens(n, cfg["vocab"], 30 + i) for i, n in enumerate([20, 5, 33, 12, 9])]
    outs = kvcm.generate(eng, prompts, 10)
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        logits = plain_toy_logits(cfg, w, list(p) + list(o))
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= 2e-4, (k, tok, P.greedy_pick(row))
    assert eng.graphs is None                                    # a part that is not capturable: no graphs
    assert eng.kv.blocks_in_use(0) == 0 and eng.kv.blocks_in_use(1) == 0 and eng.sched.slots_taken() == 0
    with pytest.raises(ValueError, match="prefix caching"):
        kvcm.Engine.from_folder(folder, EngineConfig(kv=KVManagerConfig(num_blocks=24, block_size=8, max_seq_len=96,
                                                                        prefix_caching=True), dtype="float32"))


# ------------------------------------------------------------------------------------------------
# A second toy: a mixer with state of its own that CAN be recorded into CUDA graphs (device-side
# tensor operations only, nothing read on the host).  Decode steps are then replayed from graphs,
# and the step in which a graph is recorded must still advance the state exactly once.

def register_capturable_toy():
    from kvcm.config import ModelConfig, register_architecture
    from kvcm.models.spec import ModelSpec, TensorBinding
    from kvcm.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall, Linear, Mixer, StateSpec
    from kvcm.parts.embedding import Embedding, LMHead

    class RunningMean(Mixer):
        """y_t = W (s_t / (t + 1)),  s_t = s_{t-1} + h_t.  State per request: s (float32 [hidden])."""

        def __init__(self, hidden: int) -> None:
            super().__init__()
            self.hidden = hidden
            self.proj = self.add_child("proj", Linear(hidden, hidden))

        def state_spec(self):
            return StateSpec((self.hidden,), torch.float32)

        def forward(self, h, ctx, site):
            hf = h.float()
            seq = ctx.row_seq.long()
            slot = ctx.seq_state_slot.long()
            valid = slot >= 0                                          # padding entries hold no slot
            slot_c = slot.clamp(min=0)
            c = torch.cumsum(hf, 0)
            start = ctx.seq_q_start.long()[seq]
            before = torch.where((start > 0)[:, None], c[(start - 1).clamp(min=0)], torch.zeros_like(c))
            old = site.state[slot_c] * valid[:, None]
            s = old[seq] + (c - before)                                # the sum up to and including each row
            out = (s / (ctx.positions.float()[:, None] + 1).clamp(min=1)).to(h.dtype)
            last = (ctx.seq_q_start + ctx.seq_q_len - 1).long()
            site.state.index_add_(0, slot_c, (s[last] - old) * valid[:, None])
            return self.proj.forward(out, ctx)

    if "running_mean" not in MIXERS.names():
        MIXERS.register("running_mean", RunningMean)

    @dataclass(frozen=True)
    class CapToyConfig(ModelConfig):
        vocab: int = 0
        width: int = 0
        ffn: int = 0
        heads: int = 0
        head_dim: int = 0
        eps: float = 1e-5

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyCapturableForTests",
                       **{k: d[k] for k in ("vocab", "width", "ffn", "heads", "head_dim", "eps")})

        def to_json_dict(self):
            d = {k: getattr(self, k) for k in ("vocab", "width", "ffn", "heads", "head_dim", "eps")}
            d["architectures"] = [self.architecture]
            return d

    def build(cfg):
        H = cfg.width
        emb = Embedding(cfg.vocab, H)
        bind = [TensorBinding(emb, "weight", [("emb.weight", (cfg.vocab, H))])]
        blocks = []
        for l, kind in enumerate(["attention", "running_mean"]):
            if kind == "attention":
                pos = POSITION_ENCODINGS.build("rope", head_dim=cfg.head_dim, theta=10000.0)
                mixer = MIXERS.build("attention", hidden=H, num_heads=cfg.heads, num_kv_heads=cfg.heads,
                                     head_dim=cfg.head_dim, position=pos)
                q = cfg.heads * cfg.head_dim
                bind += [TensorBinding(mixer.qkv, "weight", [(f"l{l}.q", (q, H)), (f"l{l}.k", (q, H)), (f"l{l}.v", (q, H))]),
                         TensorBinding(mixer.o, "weight", [(f"l{l}.o", (H, q))])]
            else:
                mixer = MIXERS.build("running_mean", hidden=H)
                bind.append(TensorBinding(mixer.proj, "weight", [(f"l{l}.proj", (H, H))]))
            ffn = FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=cfg.ffn)
            n1, n2 = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps), NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
            blocks.append(BLOCKS.build("pre_norm", norm1=n1, mixer=mixer, norm2=n2, ffn=ffn))
            bind += [TensorBinding(n1, "weight", [(f"l{l}.n1", (H,))]), TensorBinding(n2, "weight", [(f"l{l}.n2", (H,))]),
                     TensorBinding(ffn.gate_up, "weight", [(f"l{l}.gate", (cfg.ffn, H)), (f"l{l}.up", (cfg.ffn, H))]),
                     TensorBinding(ffn.down, "weight", [(f"l{l}.down", (H, cfg.ffn))])]
        fin = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
        head = LMHead(H, cfg.vocab)
        bind += [TensorBinding(fin, "weight", [("final.weight", (H,))]),
                 TensorBinding(head, "weight", [("head.weight", (cfg.vocab, H))], tie_to=bind[0], tied=True)]
        return ModelSpec(cfg, emb, blocks, [LayerCall(0), LayerCall(1)], fin, head, bind)

    register_architecture("ToyCapturableForTests", CapToyConfig, build, replace=True)
    return CapToyConfig


def plain_capturable_toy(cfg, w, tokens):
    n = len(tokens)
    pos = torch.arange(n)
    c = dict(nh=cfg["heads"], nkv=cfg["heads"], hd=cfg["head_dim"], theta=10000.0)
    x = P.embedding(w["emb.weight"], tokens)

    def layer(l, x, mix):
        x = x + mix(P.rmsnorm(x, w[f"l{l}.n1"], cfg["eps"]))
        return x + P.gated_mlp(P.rmsnorm(x, w[f"l{l}.n2"], cfg["eps"]), w[f"l{l}.gate"], w[f"l{l}.up"], w[f"l{l}.down"])

    x = layer(0, x, lambda h: P.attention_block(h, w["l0.q"], w["l0.k"], w["l0.v"], w["l0.o"], pos, c))
    x = layer(1, x, lambda h: (torch.cumsum(h, 0) / (pos.double()[:, None] + 1)) @ w["l1.proj"].T)
    return P.rmsnorm(x, w["final.weight"], cfg["eps"]) @ w["emb.weight"].T


def test_stateful_mixer_under_cuda_graphs_advances_once_per_step(tmp_path):
    """Greedy generation with decode steps replayed from CUDA graphs, against the plain
    implementation and against the same engine without graphs.  Requests of several lengths make
    several (batch, context) shapes, so graphs are recorded in the middle of generation: a recorded
    step that ran twice would add its input to the state twice."""
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    CapToyConfig = register_capturable_toy()
    cfg = CapToyConfig(architecture="ToyCapturableForTests", vocab=150, width=40, ffn=64, heads=2, head_dim=16, eps=1e-5)
    folder = str(tmp_path / "captoy")
    kvcm.write_random_model(folder, cfg, seed=11, dtype=torch.float32, norm_jitter=0.1)
    cj = json.load(open(os.path.join(folder, "config.json")))
    from safetensors import safe_open
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).double()
    prompts = [helpers.random_tokens(n, cfg.vocab, 60 + i) for i, n in enumerate([6, 19, 3, 30, 11])]

    def run(graphs):
        ec = EngineConfig(kv=KVManagerConfig(num_blocks=64, block_size=8, max_seq_len=128, watermark_blocks=0),
                          sched=SchedulerConfig(max_num_seqs=4, max_batched_tokens=32), dtype="float32",
                          cuda_graphs=graphs)
        eng = kvcm.Engine.from_folder(folder, ec)
        outs = kvcm.generate(eng, prompts, 24)
        return eng, outs

    eng, outs = run(True)
    assert eng.graphs is not None and eng.graphs.replays > 20 and len(eng.graphs.captured) >= 2
    for p, o in zip(prompts, outs):
        assert len(o) == 24
        logits = plain_capturable_toy(cj, w, list(p) + list(o))
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= 2e-4, (len(p), k, tok, P.greedy_pick(row))
    eng2, outs2 = run(False)
    assert eng2.graphs is None and outs2 == outs
