"""What the command-line tools share: building an engine from the reference's flag names."""
from __future__ import annotations

import os
import tempfile


def engine_config_from_args(a):
    """Flags as the reference's kvbench (``src/main_bench.cpp:24-42``) plus this engine's own."""
    from ..config import EngineConfig, KVManagerConfig, SchedulerConfig, canonical_dtype
    kv = KVManagerConfig(policy=a.str("policy", "paged"), block_size=a.i32("block-size", 16),
                         max_seq_len=a.i32("max-seq-len", 2048), prefix_caching=a.flag("prefix"),
                         num_blocks=a.i32("num-blocks", 0), watermark_blocks=a.i32("watermark", -1))
    sc = SchedulerConfig(max_num_seqs=a.i32("max-num-seqs", 256),
                         max_batched_tokens=a.i32("max-batched-tokens", 4096),
                         prefill_chunk=a.i32("prefill-chunk", 0),
                         chunked_prefill=not a.flag("no-chunked-prefill"))
    return EngineConfig(kv=kv, pool_gb=a.f64("pool-gb", 1.0), sched=sc,
                        dtype=canonical_dtype(a.str("dtype", "bfloat16")), attn=a.str("attn", "auto"), gemm=a.str("gemm", "auto"),
                        sampling_seed=a.i64("sampling-seed", 0), cuda_graphs=not a.flag("no-graphs"))


PRESETS = {
    # name: (config.json keys of a Llama dense decoder, seed, norm jitter)
    "tiny-a": (dict(vocab_size=256, hidden_size=64, intermediate_size=172, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=128,
                    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False), 0, 0.0),
    "tiny-b": (dict(vocab_size=384, hidden_size=96, intermediate_size=256, num_hidden_layers=3,
                    num_attention_heads=3, num_key_value_heads=1, head_dim=32, max_position_embeddings=256,
                    rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True), 1, 0.1),
    "tiny-c": (dict(vocab_size=320, hidden_size=136, intermediate_size=344, num_hidden_layers=2,
                    num_attention_heads=3, num_key_value_heads=1, head_dim=64, max_position_embeddings=512,
                    rope_theta=250000.0, rms_norm_eps=2e-6, tie_word_embeddings=False), 2, 0.05),
    "tinyllama-1.1b": (dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                            num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                            max_position_embeddings=2048, rope_theta=10000.0, rms_norm_eps=1e-5,
                            tie_word_embeddings=False), 0, 0.0),
    "llama-2-7b": (dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                        num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                        max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-5,
                        tie_word_embeddings=False), 0, 0.0),
    "llama-3-8b": (dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                        num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                        max_position_embeddings=8192, rope_theta=500000.0, rms_norm_eps=1e-5,
                        tie_word_embeddings=False), 0, 0.0),
}


def load_model_from_args(a, dtype: str, device: str = "cuda:0", stored_as: str = ""):
    """``--model DIR`` (config.json + model.safetensors) or ``--preset NAME [--random-seed S]``
    (random weights of a named shape, generated on the device).  ``stored_as``: the random weights
    are rounded to that type first, as if read from a checkpoint stored in it (a float32 model with
    the very values of the bfloat16 one)."""
    import torch
    from ..config import LlamaConfig
    from ..engine import load_model, model_from_tensors, torch_dtype
    from ..weights import random_tensors
    folder = a.str("model", "")
    preset = a.str("preset", "")
    if folder:
        return load_model(folder, dtype, device)
    if not preset:
        raise SystemExit("give --model DIR or --preset NAME (" + ", ".join(PRESETS) + ")")
    if preset not in PRESETS:
        raise SystemExit(f"unknown preset '{preset}'; known: {', '.join(PRESETS)}")
    keys, seed, jitter = PRESETS[preset]
    cfg = LlamaConfig(architecture="LlamaForCausalLM", **keys)
    seed = a.i64("random-seed", seed)
    tensors = dict(random_tensors(cfg, seed, torch_dtype(stored_as or dtype), device=device, norm_jitter=jitter))
    if stored_as and stored_as != dtype:
        tensors = {k: v.to(torch_dtype(dtype)) for k, v in tensors.items()}
    return model_from_tensors(cfg, tensors, dtype, device)
