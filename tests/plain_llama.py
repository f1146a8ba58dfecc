"""Plain, slow implementation of the Llama dense decoder: the oracle of this test suite.

It restates the reference's formulas; each function below cites the lines whose arithmetic it
restates.  The reference's own model code is CUDA + cuBLAS (``src/model/llama.cpp``,
``src/cuda/*.cu``) and cannot be imported or run on a CPU, but it was run once on a B200, built
unmodified, on three small random models: its logits lie under ``tests/golden/`` with the scripts
that made them, and ``tests/test_reference_logits.py`` holds this file to them (largest difference
0.0016 where the reference's own published error is 0.0148).  Whole sequences, no cache, no
batching, one function per part, float64 by default.  It shares no code with the product package: the model folder is read with the
``safetensors`` library and ``json``, never with the package's own loader.

``storage`` (optional): a torch dtype to which every tensor that the reference keeps in 16 bits
between kernels (h, qkv, attn, proj, gate_up, act: ``src/model/llama.h:75-81``) is rounded, so
that a bfloat16 engine is compared with the same roundings instead of with a looser bound.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F = torch.float64


def _rt(x: torch.Tensor, storage: Optional[torch.dtype]) -> torch.Tensor:
    """Round-trip through the storage dtype (no-op for None)."""
    return x if storage is None else x.to(storage).to(x.dtype)


def read_model_folder(folder: str):
    """config.json as a dict and every tensor of model.safetensors as float64."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k).to(F)
    return cfg, tensors


# ---------------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """x[t,:] = float(embed[token[t],:]), no scaling (``src/cuda/kernels.cu:27-32``)."""
    return table[torch.tensor(tokens, dtype=torch.long)].to(F)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """inv = 1/sqrt(mean(x^2) + eps); out = w * round(x * inv)
    (``src/cuda/kernels.cu:36-49``: the normalised value is rounded to the storage type before
    the multiplication by the weight, and the product is rounded again)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return _rt(weight * _rt(x * inv, storage), storage)


def rope_rotate_half(x: torch.Tensor, positions: torch.Tensor, theta: float,
                     storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """Rotate-half pairing (j, j + hd/2) on the last axis of x = [n, heads, hd]
    (``src/cuda/kernels.cu:51-70``): f_j = 1/theta^(2j/hd); a' = a cos - b sin; b' = b cos + a sin.
    The reference forms f_j, the angle and the rotation in float32 (``:60-62``)."""
    hd = x.shape[-1]
    half = hd // 2
    j = torch.arange(half, dtype=F)
    inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=F), 2.0 * j / hd)
    ang = positions.to(F)[:, None] * inv_freq[None, :]            # [n, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return _rt(torch.cat([a * c - b * s, b * c + a * s], dim=-1), storage)


def attention_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None,
                     storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """q [n, nh, hd], k/v [n, nkv, hd] -> [n, nh*hd].

    Query head h reads KV head h // G (``src/cuda/paged_attention.cu:80-86``: head = kvh*G+g).
    Row r sees keys t <= r: the causal mask is the loop bound ``ctx = pos+1`` (``:71-75``).
    s_t = sum_d (q_d*scale) k_td; p = exp(s - max); o = (sum_t p_t v_t) / sum p
    (``:94-113`` scores, ``:116-131`` softmax, ``:134-182`` PV and division).
    ``window`` w keeps only keys t > r - w (not in the reference: parts of this engine take it
    as a parameter; None = all keys)."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    G = nh // nkv
    out = torch.zeros(n, nh, hd, dtype=F)
    idx = torch.arange(n)
    mask = idx[None, :] <= idx[:, None]
    if window is not None:
        mask &= idx[None, :] > (idx[:, None] - window)
    for h in range(nh):
        kvh = h // G
        s = (q[:, h, :] * scale) @ k[:, kvh, :].T                 # [n, n]
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        out[:, h, :] = (p @ v[:, kvh, :]) / p.sum(dim=-1, keepdim=True)
    return _rt(out.reshape(n, nh * hd), storage)


def silu_mul(gate: torch.Tensor, up: torch.Tensor,
             storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """act = round(round(silu(g)) * u), silu(g) = g / (1 + exp(-g))
    (``src/cuda/kernels.cu:72-82``: silu is rounded before the product)."""
    return _rt(_rt(gate / (1.0 + torch.exp(-gate)), storage) * up, storage)


def gated_mlp(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
              storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """down( silu(h Wg^T) * (h Wu^T) ) (``src/model/llama.cpp:120-122``; gate = first I columns of
    the fused product, up = the next I)."""
    g = _rt(h @ w_gate.T, storage)
    u = _rt(h @ w_up.T, storage)
    return _rt(silu_mul(g, u, storage) @ w_down.T, storage)


def attention_block(h: torch.Tensor, wq, wk, wv, wo, positions, cfg,
                    window: Optional[int] = None,
                    storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """QKV projection, rotary on q and k, causal GQA attention, output projection
    (``src/model/llama.cpp:108-116``; scale = 1/sqrt(hd), ``:100``)."""
    n = h.shape[0]
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    q = _rt(h @ wq.T, storage).reshape(n, nh, hd)
    k = _rt(h @ wk.T, storage).reshape(n, nkv, hd)
    v = _rt(h @ wv.T, storage).reshape(n, nkv, hd)
    q = rope_rotate_half(q, positions, cfg["theta"], storage)
    k = rope_rotate_half(k, positions, cfg["theta"], storage)
    a = attention_causal(q, k, v, 1.0 / math.sqrt(hd), window, storage)
    return _rt(a @ wo.T, storage)


# ---------------------------------------------------------------------------------- model

def sizes_from_config(c: dict) -> dict:
    """The keys the reference's export reads (``tools/export_weights.py:59-67``)."""
    nh = c["num_attention_heads"]
    return {
        "V": c["vocab_size"], "H": c["hidden_size"], "I": c["intermediate_size"],
        "L": c["num_hidden_layers"], "nh": nh, "nkv": c.get("num_key_value_heads") or nh,
        "hd": c.get("head_dim") or c["hidden_size"] // nh,
        "theta": float(c.get("rope_theta", 10000.0)), "eps": float(c["rms_norm_eps"]),
        "tied": bool(c.get("tie_word_embeddings", False)),
    }


def llama_forward(cfg_json: dict, w: Dict[str, torch.Tensor], tokens: List[int],
                  storage: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits [n, V] (float64) at every position of one whole sequence.

    Order of operations as ``src/model/llama.cpp:84-128``: embedding; per layer
    norm -> attention -> residual -> norm -> MLP -> residual with the residual stream kept
    unrounded (fp32 in the reference, ``src/model/llama.h:74``); final norm; lm_head without
    bias, which falls back to the embedding table when tied
    (``tools/export_weights.py:82``)."""
    c = sizes_from_config(cfg_json)
    n = len(tokens)
    pos = torch.arange(n)
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(c["L"]):
        p = f"model.layers.{l}."
        h = rmsnorm(x, w[p + "input_layernorm.weight"], c["eps"], storage)
        x = x + attention_block(h, w[p + "self_attn.q_proj.weight"],
                                w[p + "self_attn.k_proj.weight"],
                                w[p + "self_attn.v_proj.weight"],
                                w[p + "self_attn.o_proj.weight"], pos, c, None, storage)
        h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["eps"], storage)
        x = x + gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"], storage)
    h = rmsnorm(x, w["model.norm.weight"], c["eps"], storage)
    lm = w.get("lm_head.weight")
    if lm is None or c["tied"]:
        lm = w["model.embed_tokens.weight"]
    return h @ lm.T


# ------------------------------------------------------------------------------- sampling

def greedy_pick(logits_row: torch.Tensor) -> int:
    """Lowest index among the maxima (``src/cuda/kernels.cu:90-119``)."""
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def greedy_generate(cfg_json: dict, w: Dict[str, torch.Tensor], prompt: List[int],
                    steps: int, storage: Optional[torch.dtype] = None):
    """Recomputes the whole sequence for every new token.  Returns (tokens, last-row logits per
    step) so that a caller can tell a near-tie from a fault."""
    toks = list(prompt)
    rows = []
    for _ in range(steps):
        row = llama_forward(cfg_json, w, toks, storage)[-1]
        rows.append(row)
        toks.append(greedy_pick(row))
    return toks[len(prompt):], rows


def temperature_probs(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """softmax(logits / T) (not in the reference, which is greedy only:
    ``docs/design.md:264``)."""
    z = logits_row.to(F) / temperature
    p = torch.exp(z - z.max())
    return p / p.sum()


def inverse_cdf_pick(probs: torch.Tensor, u: float) -> int:
    """The first index whose cumulative probability exceeds u * total."""
    c = torch.cumsum(probs, 0)
    i = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=c.dtype), right=True))
    return min(i, probs.numel() - 1)
