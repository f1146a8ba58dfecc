"""Configuration and registry (no GPU)."""
import json
import os

import pytest

import kvcm
from kvcm.config import (ConfigError, LlamaConfig, canonical_dtype, config_from_dict, load_config,
                         registered_architectures)
import helpers


def base_dict(**over):
    d = dict(architectures=["LlamaForCausalLM"], **helpers.TINY["tiny-a"]["cfg"])
    d.update(over)
    return d


def test_registry_has_the_architecture():
    assert "LlamaForCausalLM" in registered_architectures()


def test_round_trip_through_json(tmp_path):
    cfg = helpers.tiny_config("tiny-b")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg.to_json_dict(), f)
    assert load_config(str(tmp_path)) == cfg


def test_every_size_comes_from_the_json():
    a, b = helpers.tiny_config("tiny-a"), helpers.tiny_config("tiny-b")
    for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
              "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
              "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.qkv_dim == (4 + 2 * 2) * 16 and b.qkv_dim == (3 + 2) * 32


def test_defaults_follow_the_reference():
    d = base_dict()
    del d["num_key_value_heads"], d["head_dim"], d["rope_theta"]
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads       # MHA when the key is absent
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0


def test_head_dim_need_not_be_hidden_over_heads():
    cfg = config_from_dict(base_dict(head_dim=32))
    assert cfg.q_dim == 4 * 32 != cfg.hidden_size


def test_nested_rope_parameters():
    d = base_dict()
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert config_from_dict(d).rope_theta == 12345.0


@pytest.mark.parametrize("change, word", [
    (dict(architectures=["NoSuchModel"]), "unknown architecture"),
    (dict(architectures=[]), "architectures"),
    (dict(vocab_size=None), "vocab_size"),
    (dict(hidden_size="64"), "hidden_size"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 8.0}), "rope scaling"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(sliding_window=128), "sliding_window"),
    (dict(head_dim=15), "even"),
    (dict(rms_norm_eps=0.0), "rms_norm_eps"),
])
def test_bad_configs_are_refused_with_the_key_named(change, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(base_dict(**change))
    assert word in str(e.value)


def test_missing_or_broken_config_file(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))


def test_dtype_names():
    assert canonical_dtype("bf16") == canonical_dtype("bfloat16") == "bfloat16"
    assert canonical_dtype("fp32") == canonical_dtype("float32") == "float32"
    with pytest.raises(ValueError):
        canonical_dtype("fp8")


def test_second_architecture_can_be_registered_without_touching_the_package():
    from kvcm.config import register_architecture, get_architecture
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class ToyConfig(kvcm.config.ModelConfig):
        width: int = 8

        @classmethod
        def from_json_dict(cls, d):
            return cls(architecture="ToyForTests", width=d["width"])

    register_architecture("ToyForTests", ToyConfig, lambda cfg: None, replace=True)
    cfg = config_from_dict({"architectures": ["ToyForTests"], "width": 24})
    assert cfg.width == 24 and get_architecture("ToyForTests").config_cls is ToyConfig
    with pytest.raises(ValueError):
        register_architecture("ToyForTests", ToyConfig, lambda cfg: None)
