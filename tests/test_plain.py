"""Checks of the plain implementation itself (no GPU): each part against a second, even plainer
statement of its formula, and properties that hold by construction."""
import math

import pytest
import torch

import helpers
import plain_llama as P


def test_rmsnorm_formula():
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.randn(12, dtype=torch.float64)
    got = P.rmsnorm(x, w, 1e-5)
    for r in range(5):
        ms = sum(float(v) ** 2 for v in x[r]) / 12
        for i in range(12):
            assert abs(float(got[r, i]) - float(w[i]) * float(x[r, i]) / math.sqrt(ms + 1e-5)) < 1e-12


def test_rope_is_a_rotation_by_position_times_frequency():
    hd, theta = 8, 10000.0
    x = torch.randn(6, 2, hd, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 7, 100, 1999])
    y = P.rope_rotate_half(x, pos, theta)
    assert torch.allclose(y[0], x[0])                              # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))          # rotations keep lengths
    for t in range(6):
        for j in range(hd // 2):
            ang = float(pos[t]) / theta ** (2 * j / hd)
            a, b = float(x[t, 1, j]), float(x[t, 1, j + hd // 2])  # pairs (j, j + hd/2)
            assert abs(float(y[t, 1, j]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-9
            assert abs(float(y[t, 1, j + hd // 2]) - (b * math.cos(ang) + a * math.sin(ang))) < 1e-9


def test_rope_scores_depend_on_the_distance_only():
    hd = 16
    q, k = torch.randn(1, 1, hd, dtype=torch.float64), torch.randn(1, 1, hd, dtype=torch.float64)
    def score(m, n):
        return float((P.rope_rotate_half(q, torch.tensor([m]), 1e4) *
                      P.rope_rotate_half(k, torch.tensor([n]), 1e4)).sum())
    assert abs(score(5, 3) - score(105, 103)) < 1e-9
    assert abs(score(5, 3) - score(6, 3)) > 1e-6


def brute_attention(q, k, v, scale, window=None):
    n, nh, hd = q.shape
    G = nh // k.shape[1]
    out = torch.zeros(n, nh, hd, dtype=torch.float64)
    for r in range(n):
        lo = 0 if window is None else max(0, r - window + 1)
        for h in range(nh):
            s = [scale * float(q[r, h] @ k[t, h // G]) for t in range(lo, r + 1)]
            m = max(s)
            p = [math.exp(x - m) for x in s]
            for i, t in enumerate(range(lo, r + 1)):
                out[r, h] += p[i] / sum(p) * v[t, h // G]
    return out.reshape(n, nh * hd)


@pytest.mark.parametrize("nh,nkv,window", [(4, 2, None), (3, 1, None), (4, 4, 3), (6, 2, 1)])
def test_attention_against_loops(nh, nkv, window):
    n, hd = 9, 4
    q = torch.randn(n, nh, hd, dtype=torch.float64)
    k = torch.randn(n, nkv, hd, dtype=torch.float64)
    v = torch.randn(n, nkv, hd, dtype=torch.float64)
    got = P.attention_causal(q, k, v, 0.5, window)
    assert torch.allclose(got, brute_attention(q, k, v, 0.5, window), atol=1e-12)


def test_silu_and_gated_mlp():
    g, u = torch.randn(3, 7, dtype=torch.float64), torch.randn(3, 7, dtype=torch.float64)
    assert torch.allclose(P.silu_mul(g, u), g * torch.sigmoid(g) * u)
    h = torch.randn(3, 5, dtype=torch.float64)
    wg, wu, wd = (torch.randn(7, 5, dtype=torch.float64), torch.randn(7, 5, dtype=torch.float64),
                  torch.randn(5, 7, dtype=torch.float64))
    want = ((h @ wg.T) * torch.sigmoid(h @ wg.T) * (h @ wu.T)) @ wd.T
    assert torch.allclose(P.gated_mlp(h, wg, wu, wd), want)


def test_storage_rounding_is_applied_where_the_reference_rounds():
    x = torch.randn(4, 16, dtype=torch.float64)
    w = 1 + 0.1 * torch.randn(16, dtype=torch.float64)
    y = P.rmsnorm(x, w.to(torch.bfloat16).double(), 1e-5, torch.bfloat16)
    assert torch.equal(y, y.to(torch.bfloat16).double())           # result is representable
    assert not torch.equal(y, P.rmsnorm(x, w.to(torch.bfloat16).double(), 1e-5))


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_logits_do_not_depend_on_later_tokens(name, model_folders):
    cfg, w = P.read_model_folder(model_folders(name, "float32"))
    toks = helpers.random_tokens(24, cfg["vocab_size"], 11)
    full = P.llama_forward(cfg, w, toks)
    assert full.shape == (24, cfg["vocab_size"])
    part = P.llama_forward(cfg, w, toks[:10])
    assert torch.allclose(full[:10], part, atol=1e-12)
    changed = list(toks); changed[15] = (changed[15] + 1) % cfg["vocab_size"]
    other = P.llama_forward(cfg, w, changed)
    assert torch.allclose(full[:15], other[:15], atol=1e-12)
    assert not torch.allclose(full[15:], other[15:], atol=1e-6)


def test_tied_head_uses_the_embedding(model_folders):
    cfg, w = P.read_model_folder(model_folders("tiny-b", "float32"))
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    assert P.llama_forward(cfg, w, [1, 2, 3]).shape == (3, cfg["vocab_size"])


def test_greedy_picks_the_lowest_index_among_equals():
    assert P.greedy_pick(torch.tensor([0.0, 3.0, 3.0, 1.0])) == 1
    assert P.greedy_pick(torch.tensor([5.0, 3.0, 5.0])) == 0
    assert P.greedy_pick(torch.tensor([-1.0, -2.0, -0.5])) == 2


def test_temperature_sampling_pieces():
    row = torch.tensor([1.0, 2.0, 3.0, 0.0])
    p = P.temperature_probs(row, 0.8)
    assert abs(float(p.sum()) - 1) < 1e-12 and float(p[2]) > float(p[1]) > float(p[0])
    assert P.inverse_cdf_pick(p, 0.0) == 0
    assert P.inverse_cdf_pick(p, 0.999999) == 3
    c = torch.cumsum(p, 0)
    assert P.inverse_cdf_pick(p, float(c[1]) + 1e-9) == 2
    from kvcm.sampling import uniform_for
    us = [uniform_for(7, rid, pos) for rid in range(20) for pos in range(50)]
    assert all(0 <= u < 1 for u in us) and len(set(us)) > 990
    assert abs(sum(us) / len(us) - 0.5) < 0.05
    assert uniform_for(7, 3, 9) == uniform_for(7, 3, 9) != uniform_for(8, 3, 9)
