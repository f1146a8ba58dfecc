"""The small random models whose logits the reference engine computed for tests/golden/.

Everything here is integer arithmetic plus a few IEEE multiplications, so that the same weights
come out on every machine and library version: element i of tensor `name` is the sum of the four
16-bit fields of a 64-bit mix of (seed, name, i), centred and scaled to a standard deviation of
0.02 (an Irwin-Hall bell curve), then rounded to float16 -- the storage type of the reference.

Shapes are ones the reference's kernels take (src/cuda/paged_attention.cu:321-326,369-371: head
sizes 64 and 128, groups of 1, 4 and 8 query heads to a KV head; hidden == heads * head_dim,
src/model/weights.h:23) and are otherwise as odd as they may be.
"""
from __future__ import annotations

import struct
import zlib
from typing import Dict, List

import numpy as np

MODELS = {
    # head_dim 64, eight query heads on one KV head
    "hd64_g8": dict(cfg=dict(vocab_size=1000, hidden_size=512, intermediate_size=1368, num_hidden_layers=2,
                             num_attention_heads=8, num_key_value_heads=1, head_dim=64,
                             max_position_embeddings=1024, rope_theta=10000.0, rms_norm_eps=1e-5,
                             tie_word_embeddings=False),
                    seed=101, tokens=300, keep=48, block_size=16),
    # head_dim 128, four query heads on one KV head, three layers
    "hd128_g4": dict(cfg=dict(vocab_size=776, hidden_size=512, intermediate_size=1000, num_hidden_layers=3,
                              num_attention_heads=4, num_key_value_heads=1, head_dim=128,
                              max_position_embeddings=1024, rope_theta=500000.0, rms_norm_eps=1e-6,
                              tie_word_embeddings=False),
                     seed=102, tokens=150, keep=48, block_size=8),
    # head_dim 128, every query head with a KV head of its own
    "hd128_g1": dict(cfg=dict(vocab_size=520, hidden_size=256, intermediate_size=520, num_hidden_layers=2,
                              num_attention_heads=2, num_key_value_heads=2, head_dim=128,
                              max_position_embeddings=1024, rope_theta=10000.0, rms_norm_eps=1e-5,
                              tie_word_embeddings=False),
                     seed=103, tokens=90, keep=48, block_size=32),
}

_M = (1 << 64) - 1


def _mix(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays (wrap-around arithmetic)."""
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & np.uint64(_M)
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & np.uint64(_M)
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & np.uint64(_M)
    return x ^ (x >> np.uint64(31))


def bell(seed: int, name: str, n: int, std: float = 0.02) -> np.ndarray:
    """n float16 values of standard deviation `std`, a pure function of (seed, name, index)."""
    with np.errstate(over="ignore"):
        key = np.uint64((seed * 0x100000001B3 + zlib.crc32(name.encode())) & _M)
        h = _mix(np.arange(n, dtype=np.uint64) ^ _mix(np.full(1, key, dtype=np.uint64))[0])
    s = np.zeros(n, dtype=np.int64)
    for k in range(4):
        s += ((h >> np.uint64(16 * k)) & np.uint64(0xFFFF)).astype(np.int64)
    # sum of four uniforms on [0, 65535]: mean 131070, standard deviation 65535 / sqrt(3)
    x = (s - 131070).astype(np.float64) * (std * 1.7320508075688772 / 65535.0)
    return x.astype(np.float16)


def token_ids(seed: int, n: int, vocab: int) -> List[int]:
    with np.errstate(over="ignore"):
        h = _mix(np.arange(n, dtype=np.uint64) ^ np.uint64(seed * 7919 + 17))
    return [int(v) for v in (h % np.uint64(vocab - 3)) + np.uint64(3)]


def tensors(name: str) -> Dict[str, np.ndarray]:
    """HF-named float16 tensors of one golden model; norm weights are 1 + a bell curve of 0.1."""
    m = MODELS[name]
    c, seed = m["cfg"], m["seed"]
    V, H, I = c["vocab_size"], c["hidden_size"], c["intermediate_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    out: Dict[str, np.ndarray] = {}

    def mat(key, rows, cols):
        out[key] = bell(seed, key, rows * cols).reshape(rows, cols)

    def norm(key):
        out[key] = (1.0 + bell(seed, key, H, 0.1).astype(np.float64)).astype(np.float16)

    mat("model.embed_tokens.weight", V, H)
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        norm(p + "input_layernorm.weight")
        mat(p + "self_attn.q_proj.weight", nh * hd, H)
        mat(p + "self_attn.k_proj.weight", nkv * hd, H)
        mat(p + "self_attn.v_proj.weight", nkv * hd, H)
        mat(p + "self_attn.o_proj.weight", H, nh * hd)
        norm(p + "post_attention_layernorm.weight")
        mat(p + "mlp.gate_proj.weight", I, H)
        mat(p + "mlp.up_proj.weight", I, H)
        mat(p + "mlp.down_proj.weight", H, I)
    norm("model.norm.weight")
    mat("lm_head.weight", V, H)
    return out


def write_reference_weight_file(name: str, path: str) -> None:
    """The reference's own weight format: 64-byte header (src/model/weights.cpp:24-40), then flat
    fp16 tensors in the order of src/model/weights.cpp:69-82 with q, k, v rows and gate, up rows
    concatenated as tools/export_weights.py:73-79 does."""
    m = MODELS[name]
    c = m["cfg"]
    t = tensors(name)
    hdr = b"KVPW" + struct.pack("<9i", 1, c["vocab_size"], c["hidden_size"], c["intermediate_size"],
                                c["num_hidden_layers"], c["num_attention_heads"], c["num_key_value_heads"],
                                c["head_dim"], c["max_position_embeddings"]) \
        + struct.pack("<2f", c["rope_theta"], c["rms_norm_eps"])
    hdr += b"\0" * (64 - len(hdr))
    with open(path, "wb") as f:
        f.write(hdr)
        f.write(t["model.embed_tokens.weight"].tobytes())
        for l in range(c["num_hidden_layers"]):
            p = f"model.layers.{l}."
            f.write(t[p + "input_layernorm.weight"].tobytes())
            for k in ("q_proj", "k_proj", "v_proj"):
                f.write(t[p + f"self_attn.{k}.weight"].tobytes())
            f.write(t[p + "self_attn.o_proj.weight"].tobytes())
            f.write(t[p + "post_attention_layernorm.weight"].tobytes())
            f.write(t[p + "mlp.gate_proj.weight"].tobytes())
            f.write(t[p + "mlp.up_proj.weight"].tobytes())
            f.write(t[p + "mlp.down_proj.weight"].tobytes())
        f.write(t["model.norm.weight"].tobytes())
        f.write(t["lm_head.weight"].tobytes())
