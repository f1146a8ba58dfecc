"""More toy parts defined HERE, outside the package: a feed-forward with routing (every row goes
through the one expert its router picks) and a position encoding of its own (rotary with stretched
positions), next to the package's interleaved, partial rotary encoding in another layer.  They are
registered, built from a config.json, given random weights, stepped in portions, decoded and
generated from through the engine, without a change to the package's files.  A plain
whole-sequence implementation of the toy model, also here, is the oracle.  The toy parts stand
for nothing but themselves."""
import json
import math
import os
from dataclasses import dataclass

import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

F = torch.float64


def register_toy():
    from kvcm.config import ModelConfig, register_architecture
    from kvcm.models.spec import ModelSpec, TensorBinding
    from kvcm.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, FeedForward, LayerCall, Linear
    from kvcm.parts.embedding import Embedding, LMHead
    from kvcm.parts.rope import RotaryEmbedding

    class StretchedRotary(RotaryEmbedding):
        """Rotary encoding of positions divided by ``stretch``: only the frequency table differs, the
        engine's rotary kernels take it as it is."""

        def __init__(self, head_dim: int, theta: float, stretch: float) -> None:
            super().__init__(head_dim, theta)
            self.stretch = float(stretch)

        def frequency_table(self) -> torch.Tensor:
            return (super().frequency_table().double() / self.stretch).float()

    class TopOneExperts(FeedForward):
        """y[row] = expert_e(h[row]) with e = argmax of the row's router logits (float32).  The rows
        are sorted to their experts on the host: a test's toy, not a kernel of the engine
        (``capturable = False``: no CUDA graphs with it)."""

        capturable = False

        def __init__(self, hidden: int, intermediate: int, experts: int) -> None:
            super().__init__()
            self.router = self.add_child("router", Linear(hidden, experts))
            self.experts = [self.add_child(f"expert{e}", FEED_FORWARDS.build("gated_mlp", hidden=hidden,
                                                                             intermediate=intermediate))
                            for e in range(experts)]

        def forward(self, h, ctx):
            logits = h.float() @ self.router.param("weight").float().T
            choice = logits.argmax(dim=-1)
            y = torch.zeros_like(h)
            for e, expert in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y[rows] = expert.forward(h[rows].contiguous(), ctx)
            return y

    if "stretched_rope" not in POSITION_ENCODINGS.names():
        POSITION_ENCODINGS.register("stretched_rope", StretchedRotary)
    if "top1_experts" not in FEED_FORWARDS.names():
        FEED_FORWARDS.register("top1_experts", TopOneExperts)

    keys = ("vocab", "width", "ffn", "experts", "heads", "kv_heads", "head_dim", "rotary_dim", "stretch", "eps", "theta")

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab: int = 0
        width: int = 0
        ffn: int = 0
        experts: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        rotary_dim: int = 0
        stretch: float = 1.0
        eps: float = 1e-5
        theta: float = 10000.0

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyRoutedForTests", **{k: d[k] for k in keys})

        def to_json_dict(self):
            d = {k: getattr(self, k) for k in keys}
            d["architectures"] = [self.architecture]
            return d

    def build(cfg):
        H = cfg.width
        emb = Embedding(cfg.vocab, H)
        bind = [TensorBinding(emb, "weight", [("emb.weight", (cfg.vocab, H))])]
        blocks = []
        q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for l in range(2):
            if l == 0:      # the test's own position encoding and its routed feed-forward
                pos = POSITION_ENCODINGS.build("stretched_rope", head_dim=cfg.head_dim, theta=cfg.theta, stretch=cfg.stretch)
                ffn = FEED_FORWARDS.build("top1_experts", hidden=H, intermediate=cfg.ffn, experts=cfg.experts)
                bind.append(TensorBinding(ffn.router, "weight", [(f"l{l}.router", (cfg.experts, H))]))
                for e, ex in enumerate(ffn.experts):
                    bind += [TensorBinding(ex.gate_up, "weight", [(f"l{l}.e{e}.gate", (cfg.ffn, H)), (f"l{l}.e{e}.up", (cfg.ffn, H))]),
                             TensorBinding(ex.down, "weight", [(f"l{l}.e{e}.down", (H, cfg.ffn))])]
            else:           # the package's rotary encoding, interleaved pairs over a part of the head
                pos = POSITION_ENCODINGS.build("rope", head_dim=cfg.head_dim, theta=cfg.theta, rotary_dim=cfg.rotary_dim,
                                               pairing="interleaved")
                ffn = FEED_FORWARDS.build("gated_mlp", hidden=H, intermediate=cfg.ffn)
                bind += [TensorBinding(ffn.gate_up, "weight", [(f"l{l}.gate", (cfg.ffn, H)), (f"l{l}.up", (cfg.ffn, H))]),
                         TensorBinding(ffn.down, "weight", [(f"l{l}.down", (H, cfg.ffn))])]
            mixer = MIXERS.build("attention", hidden=H, num_heads=cfg.heads, num_kv_heads=cfg.kv_heads,
                                 head_dim=cfg.head_dim, position=pos)
            n1, n2 = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps), NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
            blocks.append(BLOCKS.build("pre_norm", norm1=n1, mixer=mixer, norm2=n2, ffn=ffn))
            bind += [TensorBinding(mixer.qkv, "weight", [(f"l{l}.q", (q, H)), (f"l{l}.k", (kv, H)), (f"l{l}.v", (kv, H))]),
                     TensorBinding(mixer.o, "weight", [(f"l{l}.o", (H, q))]),
                     TensorBinding(n1, "weight", [(f"l{l}.n1", (H,))]), TensorBinding(n2, "weight", [(f"l{l}.n2", (H,))])]
        fin = NORMS.build("rmsnorm", hidden=H, eps=cfg.eps)
        head = LMHead(H, cfg.vocab)
        bind += [TensorBinding(fin, "weight", [("final.weight", (H,))]),
                 TensorBinding(head, "weight", [("head.weight", (cfg.vocab, H))])]
        return ModelSpec(cfg, emb, blocks, [LayerCall(0), LayerCall(1)], fin, head, bind)

    register_architecture("ToyRoutedForTests", ToyConfig, build, replace=True)
    return ToyConfig


# ------------------------------------------------------------------------------------ the oracle

def rotate(x, positions, inv_freq, rotary_dim, interleaved):
    """x [n, heads, hd]: the first ``rotary_dim`` elements of every head rotated in pairs (j, j + half)
    or (2j, 2j + 1) by position * inv_freq[j]; the angle is formed in float32 as the kernels do."""
    half = rotary_dim // 2
    ang = (positions.float()[:, None] * inv_freq.float()[None, :]).double()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2], out[..., 1:rotary_dim:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:rotary_dim]
        out[..., :half], out[..., half:rotary_dim] = a * c - b * s, b * c + a * s
    return out


def plain_toy(cfg, w, tokens):
    """Whole sequence, float64, no cache.  Returns (logits, expert chosen by every row)."""
    n = len(tokens)
    pos = torch.arange(n)
    nh, nkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    x = P.embedding(w["emb.weight"], tokens)
    base = (1.0 / torch.pow(torch.tensor(cfg["theta"], dtype=F), 2.0 * torch.arange(hd // 2, dtype=F) / hd)).float()
    part = (1.0 / torch.pow(torch.tensor(cfg["theta"], dtype=F),
                            2.0 * torch.arange(cfg["rotary_dim"] // 2, dtype=F) / cfg["rotary_dim"])).float()
    chosen = None
    for l in range(2):
        h = P.rmsnorm(x, w[f"l{l}.n1"], cfg["eps"])
        q = (h @ w[f"l{l}.q"].T).reshape(n, nh, hd)
        k = (h @ w[f"l{l}.k"].T).reshape(n, nkv, hd)
        v = (h @ w[f"l{l}.v"].T).reshape(n, nkv, hd)
        if l == 0:
            inv = (base.double() / cfg["stretch"]).float()
            q, k = rotate(q, pos, inv, hd, False), rotate(k, pos, inv, hd, False)
        else:
            q, k = rotate(q, pos, part, cfg["rotary_dim"], True), rotate(k, pos, part, cfg["rotary_dim"], True)
        x = x + P.attention_causal(q, k, v, 1.0 / math.sqrt(hd)) @ w[f"l{l}.o"].T
        h = P.rmsnorm(x, w[f"l{l}.n2"], cfg["eps"])
        if l == 0:
            chosen = (h @ w["l0.router"].T).argmax(dim=-1)
            y = torch.zeros_like(h)
            for e in range(cfg["experts"]):
                rows = (chosen == e).nonzero().flatten()
                y[rows] = P.gated_mlp(h[rows], w[f"l0.e{e}.gate"], w[f"l0.e{e}.up"], w[f"l0.e{e}.down"])
            x = x + y
        else:
            x = x + P.gated_mlp(h, w["l1.gate"], w["l1.up"], w["l1.down"])
    return P.rmsnorm(x, w["final.weight"], cfg["eps"]) @ w["head.weight"].T, chosen


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    import kvcm
    ToyConfig = register_toy()
    cfg = ToyConfig(architecture="ToyRoutedForTests", vocab=150, width=40, ffn=56, experts=3, heads=4, kv_heads=2,
                    head_dim=16, rotary_dim=8, stretch=4.0, eps=3e-6, theta=5000.0)
    folder = str(tmp_path_factory.mktemp("toy_routed"))
    kvcm.write_random_model(folder, cfg, seed=11, dtype=torch.float32, norm_jitter=0.1)
    assert kvcm.load_config(folder) == cfg
    from safetensors import safe_open
    from safetensors.torch import save_file
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).clone()           # (the tensors map the file that is written again below)
    w["l0.router"] = w["l0.router"] * 40.0           # wide gaps between router logits: the choice is no near-tie
    save_file(w, os.path.join(folder, "model.safetensors"))
    return folder, json.load(open(os.path.join(folder, "config.json"))), {k: v.double() for k, v in w.items()}


def test_toy_parts_are_what_the_model_is_built_from(toy):
    folder, cfg, w = toy
    r = helpers.Replayer(folder, "float32", 128, 8)
    b0, b1 = r.spec.blocks
    assert type(b0.ffn).__name__ == "TopOneExperts" and len(b0.ffn.experts) == 3
    assert type(b0.mixer.position).__name__ == "StretchedRotary" and type(b1.mixer.position).__name__ == "RotaryEmbedding"
    assert b1.mixer.position.interleaved and b1.mixer.position.rotary_dim == 8
    assert b1.mixer.position.inv_freq.shape == (4,)
    base = 1.0 / torch.pow(torch.tensor(5000.0, dtype=F), 2.0 * torch.arange(8, dtype=F) / 16)
    assert torch.allclose(b0.mixer.position.inv_freq.cpu().double(), base / 4.0, rtol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_stepped_in_portions_and_decoded(toy, dtype):
    folder, cfg, w = toy
    toks = helpers.random_tokens(70, cfg["vocab"], 21)
    ref, chosen = plain_toy(cfg, w, toks)
    assert len(set(chosen.tolist())) == cfg["experts"], "the sequence must visit every expert"
    r = helpers.Replayer(folder, dtype, 128, 8)
    outs, at = [], 0
    for k in (9, 2, 17, 1, 1, 23, 2, 15):                                    # portions and single tokens
        outs.append(r.step([dict(id="x", tokens=toks[at:at + k], want=list(range(k)))]))
        at += k
    assert at == len(toks)
    got = torch.cat(outs)
    if dtype == "float32":
        helpers.assert_logits_close(got, ref, "float32", "toy parts in portions")
    else:
        assert (got.double().cpu() - ref).abs().max().item() <= 0.06 * ref.std().item()   # weights stored in 32 bits stay so
    whole = helpers.Replayer(folder, dtype, 128, 8).step([dict(id="w", tokens=toks, want=list(range(len(toks))))])
    if dtype == "float32":
        helpers.assert_logits_close(whole, ref, "float32", "toy parts, whole sequence")


def test_toy_parts_generate_through_the_engine(toy):
    import kvcm
    from kvcm.config import EngineConfig, KVManagerConfig, SchedulerConfig
    folder, cfg, w = toy
    ec = EngineConfig(kv=KVManagerConfig(num_blocks=24, block_size=8, max_seq_len=96, watermark_blocks=0),
                      sched=SchedulerConfig(max_num_seqs=3, max_batched_tokens=16), dtype="float32")
    eng = kvcm.Engine.from_folder(folder, ec)
    prompts = [helpers.random_tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate([18, 4, 31, 11])]
    outs = kvcm.generate(eng, prompts, 8)
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        logits, _ = plain_toy(cfg, w, list(p) + list(o))
        for k, tok in enumerate(o):
            row = logits[len(p) - 1 + k]
            assert row.max().item() - row[tok].item() <= 2e-4, (k, tok, P.greedy_pick(row))
    assert eng.graphs is None                                    # a part that is not capturable: no graphs
    assert eng.kv.blocks_in_use() == 0
