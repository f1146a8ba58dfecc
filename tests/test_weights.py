"""Weights: container I/O, loading by name, the one error that lists everything (no GPU)."""
import json
import os
import struct

import pytest
import torch

import kvcm
from kvcm.config import get_architecture, load_config
from kvcm.weights import (SafetensorsError, SafetensorsFile, WeightError, load_from_tensors,
                          load_weights, random_tensors, target_dtype, write_safetensors)
import helpers


def test_writer_is_read_by_the_safetensors_library_and_back(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
         "c": torch.arange(6, dtype=torch.int64).reshape(2, 3), "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, list(t.items()), {"k": "v"})
    with safe_open(p, framework="pt") as f:
        assert sorted(f.keys()) == sorted(t)
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
    q = str(tmp_path / "y.safetensors")
    save_file(t, q)
    mine = SafetensorsFile(q)
    for k in t:
        assert torch.equal(mine.tensor(k), t[k]) and mine.info(k) == (t[k].dtype, tuple(t[k].shape))


def test_truncated_and_corrupt_files(tmp_path):
    p = str(tmp_path / "model.safetensors")
    write_safetensors(p, [("a", torch.randn(64, 64))])
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:-100])
    with pytest.raises(SafetensorsError, match="truncated|outside"):
        SafetensorsFile(p)
    open(p, "wb").write(blob[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10) + b"not json!!")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        load_weights(None, str(tmp_path / "nowhere"), "cpu", torch.float32)


def test_random_model_folder_loads_and_fuses(tmp_path):
    folder = helpers.write_tiny("tiny-a", "bfloat16", str(tmp_path))
    cfg = load_config(folder)
    spec = get_architecture(cfg.architecture).build(cfg)
    load_weights(spec, folder, "cpu", torch.bfloat16)
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    mixer = spec.blocks[1].mixer
    w = mixer.qkv.param("weight")
    assert w.dtype == torch.bfloat16 and w.shape == (cfg.qkv_dim, cfg.hidden_size)
    q = f.tensor("model.layers.1.self_attn.q_proj.weight")
    k = f.tensor("model.layers.1.self_attn.k_proj.weight")
    v = f.tensor("model.layers.1.self_attn.v_proj.weight")
    assert torch.equal(w, torch.cat([q, k, v], 0))              # q rows, then k, then v
    gu = spec.blocks[0].ffn.gate_up.param("weight")
    assert torch.equal(gu[:cfg.intermediate_size], f.tensor("model.layers.0.mlp.gate_proj.weight"))
    assert torch.equal(gu[cfg.intermediate_size:], f.tensor("model.layers.0.mlp.up_proj.weight"))
    assert spec.lm_head.param("weight").data_ptr() != spec.embedding.param("weight").data_ptr()


def test_tied_head_aliases_the_embedding(tmp_path):
    folder = helpers.write_tiny("tiny-b", "float32", str(tmp_path))
    names = SafetensorsFile(os.path.join(folder, "model.safetensors")).names()
    assert "lm_head.weight" not in names
    cfg = load_config(folder)
    spec = get_architecture(cfg.architecture).build(cfg)
    load_weights(spec, folder, "cpu", torch.float32)
    assert spec.lm_head.param("weight").data_ptr() == spec.embedding.param("weight").data_ptr()


def test_untied_config_without_head_falls_back_to_the_embedding():
    cfg = helpers.tiny_config("tiny-a")
    t = dict(random_tensors(cfg, 0, torch.float32))
    del t["lm_head.weight"]
    spec = get_architecture(cfg.architecture).build(cfg)
    load_from_tensors(spec, t, "cpu", torch.float32)
    assert spec.lm_head.param("weight").data_ptr() == spec.embedding.param("weight").data_ptr()


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    cfg = helpers.tiny_config("tiny-a")
    t = dict(random_tensors(cfg, 0, torch.float32))
    del t["model.layers.0.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(5, 64)
    t["model.layers.9.bogus.weight"] = torch.zeros(1)
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # harmless: ignored
    spec = get_architecture(cfg.architecture).build(cfg)
    with pytest.raises(WeightError) as e:
        load_from_tensors(spec, t, "cpu", torch.float32)
    err = e.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.bogus.weight"]
    assert len(err.wrong_shape) == 1 and "k_proj" in err.wrong_shape[0] and "[5, 64]" in err.wrong_shape[0]
    msg = str(err)
    for word in ("missing tensors (2)", "wrong shapes (1)", "unexpected tensors (1)", "bogus", "up_proj"):
        assert word in msg


def test_dtype_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(torch.bfloat16, bf) == bf and target_dtype(torch.float16, bf) == bf
    assert target_dtype(torch.float32, bf) == f32           # stored in 32 bits: stays so
    assert target_dtype(torch.int64, bf) == torch.int32     # integer tables
    assert target_dtype(torch.bfloat16, f32) == f32 and target_dtype(torch.float32, f32) == f32
    cfg = helpers.tiny_config("tiny-a")
    t = dict(random_tensors(cfg, 0, torch.bfloat16))
    t["model.norm.weight"] = t["model.norm.weight"].float()
    spec = get_architecture(cfg.architecture).build(cfg)
    load_from_tensors(spec, t, "cpu", bf)
    assert spec.final_norm.param("weight").dtype == f32
    assert spec.blocks[0].norm1.param("weight").dtype == bf


def test_random_weights_depend_on_seed_and_name_only():
    cfg = helpers.tiny_config("tiny-a")
    a = dict(random_tensors(cfg, 3, torch.float32))
    b = dict(reversed(list(random_tensors(cfg, 3, torch.float32))))
    c = dict(random_tensors(cfg, 4, torch.float32))
    for k in a:
        assert torch.equal(a[k], b[k])
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert torch.all(a["model.norm.weight"] == 1)
    w = a["model.layers.0.mlp.down_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    j = dict(random_tensors(cfg, 3, torch.float32, norm_jitter=0.1))["model.norm.weight"]
    assert 0.03 < (j - 1).std().item() < 0.2


def test_reader_in_the_core_keeps_the_map_alive_and_reports_header_faults(tmp_path):
    """The C++ reader: metadata, header order, a tensor view that outlives its file object, escapes
    in names, and one message per kind of header fault."""
    import gc
    p = str(tmp_path / "m.safetensors")
    a, b = torch.randn(5, 3), torch.arange(4, dtype=torch.int32)
    write_safetensors(p, [("layer \"0\".wé", a), ("b", b), ("empty", torch.empty(0, 7))], {"format": "pt"})
    f = SafetensorsFile(p)
    assert f.names() == ["layer \"0\".wé", "b", "empty"] and f.metadata == {"format": "pt"}
    view = f.tensor("layer \"0\".wé")
    assert f.tensor("empty").shape == (0, 7) and f.info("b") == (torch.int32, (4,))
    f.close()
    del f
    gc.collect()
    assert torch.equal(view, a)                               # the map lives while a view of it does

    def header_file(header: str, data: bytes = b"") -> str:
        q = str(tmp_path / "h.safetensors")
        blob = header.encode()
        open(q, "wb").write(struct.pack("<Q", len(blob)) + blob + data)
        return q
    for header, data, message in [
            ('{"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}', b"\0" * 4, "outside the data section"),
            ('{"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}', b"\0" * 8, "needs 12"),
            ('{"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}', b"\0" * 8, "bad header entry"),
            ('{"a": {"dtype": "F32", "shape": [2]}}', b"\0" * 8, "bad header entry"),
            ('{"a": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}', b"\0" * 8, "bad header entry"),
            ('{"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, '
             '"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}', b"\0" * 8, "appears twice"),
            # 2^32 * 2^32 * 2 wraps round to 0 in 64 bits, and 0 * 4 bytes would "fit" an empty range
            ('{"a": {"dtype": "F32", "shape": [4294967296, 4294967296, 2], "data_offsets": [0, 0]}}', b"",
             "does not fit"),
            # 2^30 * 2^30 * 16 = 2^64 wraps round to 0 as well
            ('{"a": {"dtype": "F32", "shape": [1073741824, 1073741824, 16], "data_offsets": [0, 0]}}', b"",
             "does not fit"),
            ('[1, 2]', b"", "JSON object"),
            ('{"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},}', b"\0" * 8, "not valid JSON")]:
        with pytest.raises(SafetensorsError, match=message):
            SafetensorsFile(header_file(header, data))
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(str(tmp_path / "absent.safetensors"))


def test_model_folder_in_shards_through_the_index_file(tmp_path):
    """A model folder without model.safetensors but with model.safetensors.index.json and two
    shards loads like the single file; a tensor that the index promises but no shard holds is
    reported as missing, by name."""
    import json
    import kvcm
    from kvcm.weights.loader import load_weights
    cfg = helpers.tiny_config("tiny-a")
    tensors = list(random_tensors(cfg, 0, torch.float32))
    folder = tmp_path / "sharded"
    folder.mkdir()
    with open(folder / "config.json", "w") as f:
        json.dump(cfg.to_json_dict(), f)
    half = len(tensors) // 2
    shards = {"model-00001-of-00002.safetensors": tensors[:half], "model-00002-of-00002.safetensors": tensors[half:]}
    weight_map = {}
    for name, items in shards.items():
        write_safetensors(str(folder / name), items)
        weight_map.update({k: name for k, _ in items})
    with open(folder / "model.safetensors.index.json", "w") as f:
        json.dump({"metadata": {"total_size": 0}, "weight_map": weight_map}, f)
    spec = get_architecture(cfg.architecture).build(cfg)
    load_weights(spec, str(folder), "cpu", torch.float32)
    want = dict(tensors)
    assert torch.equal(spec.embedding.param("weight"), want["model.embed_tokens.weight"])
    assert torch.equal(spec.blocks[1].ffn.down.param("weight"), want["model.layers.1.mlp.down_proj.weight"])
    assert torch.equal(spec.final_norm.param("weight"), want["model.norm.weight"])
    # the second shard loses a tensor
    write_safetensors(str(folder / "model-00002-of-00002.safetensors"),
                      [(k, v) for k, v in tensors[half:] if k != "model.norm.weight"])
    spec = get_architecture(cfg.architecture).build(cfg)
    with pytest.raises(WeightError) as e:
        load_weights(spec, str(folder), "cpu", torch.float32)
    assert e.value.missing == ["model.norm.weight"]
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        load_weights(get_architecture(cfg.architecture).build(cfg), str(tmp_path), "cpu", torch.float32)
