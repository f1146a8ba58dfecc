"""Test helpers: the two tiny configurations, model folders, replay drivers, tolerances.

tiny-A and tiny-B (and tiny-C, tiny-D for the head sizes of the tcgen05 attention kernel) differ in every size and option: layers 2/3, hidden 64/96, query heads 4/3,
KV heads 2/1 (group 2/3), head_dim 16/32, FFN 172/256 (172 is no multiple of 16), vocabulary
256/384, rope_theta 1e4/5e5, rms_norm_eps 1e-5/1e-6, max positions 128/256, untied/tied output
head, page size 16/8, norm weights 1 / 1+N(0,0.1), seeds 0/1.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TINY = {
    "tiny-a": dict(cfg=dict(vocab_size=256, hidden_size=64, intermediate_size=172, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                            max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-5,
                            tie_word_embeddings=False),
                   block_size=16, seed=0, norm_jitter=0.0),
    "tiny-b": dict(cfg=dict(vocab_size=384, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
                            num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                            max_position_embeddings=256, rope_theta=500000.0, rms_norm_eps=1e-6,
                            tie_word_embeddings=True),
                   block_size=8, seed=1, norm_jitter=0.1),
    # heads of 64 (the width the tcgen05 attention kernel takes), three query heads on one KV head,
    # a width that is no multiple of the head size
    "tiny-c": dict(cfg=dict(vocab_size=320, hidden_size=136, intermediate_size=344, num_hidden_layers=2,
                            num_attention_heads=3, num_key_value_heads=1, head_dim=64,
                            max_position_embeddings=512, rope_theta=250000.0, rms_norm_eps=2e-6,
                            tie_word_embeddings=False),
                   block_size=16, seed=2, norm_jitter=0.05),
    # heads of 128 (the other width of the tcgen05 attention kernel: operands as two 64-wide blocks),
    # pages of 32
    "tiny-d": dict(cfg=dict(vocab_size=288, hidden_size=264, intermediate_size=520, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                            max_position_embeddings=512, rope_theta=1000000.0, rms_norm_eps=3e-6,
                            tie_word_embeddings=True),
                   block_size=32, seed=3, norm_jitter=0.05),
}

TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tiny_config(name: str):
    import kvcm
    return kvcm.LlamaConfig(architecture="LlamaForCausalLM", **TINY[name]["cfg"])


def write_tiny(name: str, dtype: str, folder: str) -> str:
    import kvcm
    t = TINY[name]
    return kvcm.write_random_model(folder, tiny_config(name), t["seed"], TORCH_DT[dtype],
                                   norm_jitter=t["norm_jitter"])


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------ tolerances
# Fixed once, from the arithmetic, not from what passes:
#  * float32 engine vs the float64 plain implementation: only the order of float32 sums differs:
#    |d| <= 1e-4 * max(1, |logit|).
#  * bfloat16 engine vs the plain implementation run with the same bfloat16 roundings of stored
#    tensors: what remains are roundings the emulation does not share (probabilities rounded for
#    the tensor-core P*V, other summation orders flipping a last bit).  Unit roundoff 2^-9, a few
#    dozen roundings on the path to a logit, maximum over ~10^4 elements: below 4 % of the
#    logits' standard deviation.  A real fault (a missed or wrong key, a stale page) moves
#    logits by the order of that deviation itself.
def assert_logits_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    d = (got - ref).abs()
    if dtype == "float32":
        bound = 1e-4 * torch.clamp(ref.abs(), min=1.0)
        worst = (d - bound).max().item()
        assert worst <= 0, f"{what}: float32 logits differ by {d.max().item():.3e} (bound 1e-4 rel)"
    else:
        tol = 0.04 * ref.std().item()
        where = int(d.max(dim=-1).values.argmax()) if d.dim() == 2 else 0
        assert d.max().item() <= tol, (f"{what}: bfloat16 logits differ by {d.max().item():.3e} > {tol:.3e} "
                                       f"(first at row {first_bad_row(d, tol)}, worst row {where})")


def first_bad_row(d: torch.Tensor, tol: float) -> int:
    if d.dim() != 2:
        return 0
    bad = (d.max(dim=-1).values > tol).nonzero()
    return int(bad[0]) if bad.numel() else -1


# ------------------------------------------------------------------------- in-process replay

class Replayer:
    """The replay driver of ``bin/trace_run`` (``kvcm.engine.replay.ReplaySession``) inside the test
    process, with a record of which pages every request held."""

    def __init__(self, folder: str, dtype: str, max_tokens: int, block_size: int, options=None,
                 spec=None, max_live: int = 8, policy: str = "paged", prefix_caching: bool = False,
                 max_seq_len: int = 0) -> None:
        from kvcm.cache import core
        from kvcm.engine import load_model
        from kvcm.engine.replay import ReplaySession
        self.core = core
        self.spec = spec if spec is not None else load_model(folder, dtype, "cuda:0")
        self.session = ReplaySession(self.spec, dtype, max_tokens, block_size=block_size, max_live=max_live,
                                     policy=policy, prefix_caching=prefix_caching, max_seq_len=max_seq_len,
                                     options=options or {})
        self.runner, self.kv, self.slots, self.live = (self.session.runner, self.session.kv, self.session.slots,
                                                       self.session.live)
        self.pages_seen: List[int] = []
        self.page_owners: Dict[int, set] = {}

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[torch.Tensor]:
        out = self.session.step(entries, ())
        for e in entries:
            seq = self.live[e["id"]]
            self.pages_seen.extend(p for p in seq.table(0) if p >= 0)
            for p in seq.table(0):
                if p >= 0:
                    self.page_owners.setdefault(p, set()).add(seq.id)
        torch.cuda.synchronize()
        for rid in end:
            self.session.release(rid)
        return None if out is None else out.float().cpu()

    def stray_writes(self) -> List[int]:
        """Pages of the first layer group that no request ever held and that are no longer all
        zero (pools start zero-filled): a kernel wrote through a wrong page number or slot."""
        pools = self.runner.pools
        never = sorted(set(range(self.kv.num_blocks())) - set(self.pages_seen))
        bad = []
        for page in never:
            if any(bool(t[:, page].count_nonzero()) for t in (pools.k[0], pools.v[0])):
                bad.append(page)
        return bad


def run_trace_tool(folder: str, dtype: str, steps: List[dict], max_tokens: int, out_dir: str,
                   extra: Sequence[str] = ()) -> Dict[int, np.ndarray]:
    """Runs bin/trace_run as a user would and returns {step: float32 [wanted, vocab]}."""
    cfg = json.load(open(os.path.join(folder, "config.json")))
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens), *extra],
                       input=text, text=True, stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=900)
    assert p.returncode == 0, f"trace_run exit {p.returncode}\n{p.stderr[-3000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], p.stdout[-2000:]
    out = {}
    for s in steps:
        f = os.path.join(out_dir, f"{s['step']}.f32")
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        if wanted:
            a = np.fromfile(f, dtype="<f4")
            out[s["step"]] = a.reshape(wanted, cfg["vocab_size"])
        else:
            assert not os.path.exists(f)
    return out


def roundup(n: int, m: int) -> int:
    return (n + m - 1) // m * m
