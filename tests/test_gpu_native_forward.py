"""The forward pass launched from C++ (``csrc/cuda/step_forward.cu``) against the same step run part
by part from Python: the same kernels in the same order, so equal bits wherever no library product
is involved (everything in float32; bfloat16 steps of a handful of rows), and agreement within the
plain implementation's tolerance elsewhere.  And: which models take the native loop."""
import time

import pytest
import torch

import helpers
import plain_llama as P
from test_gpu_replay import LENGTHS, mixed_pool_tokens, mixed_trace, tokens_of

pytestmark = pytest.mark.gpu


def pair(model_folders, name, dtype, max_tokens, fuse_norms=False):
    block = helpers.TINY[name]["block_size"]
    native = helpers.Replayer(model_folders(name, dtype), dtype, max_tokens, block, options={"fuse_norms": fuse_norms})
    parts = helpers.Replayer(model_folders(name, dtype), dtype, max_tokens, block, options={"native_forward": False})
    assert native.runner.native is not None and parts.runner.native is None
    return native, parts


@pytest.mark.parametrize("name", ["tiny-a", "tiny-b"])
def test_float32_steps_give_equal_bits(name, model_folders):
    steps, _ = mixed_trace(name)
    native, parts = pair(model_folders, name, "float32", mixed_pool_tokens(name))
    for s in steps:
        a, b = native.step(s["entries"], s["end"]), parts.step(s["entries"], s["end"])
        assert torch.equal(a, b), f"{name} step {s['step']}"
    assert native.runner.native.calls == len(steps)


@pytest.mark.parametrize("name", ["tiny-b", "tiny-c", "tiny-d"])
def test_bfloat16_steps(name, model_folders):
    """Decode steps (up to eight single rows: this engine's kernels only) bit for bit while every norm
    is a launch of its own; with the norms riding in the products (the default: fewer launches, the
    normed row rounded once instead of twice) within the tolerance of the replay tests, like the mixed
    schedule, whose longer portions take library products."""
    from kvcm.kernels import library as K
    dtype = "bfloat16"
    native, parts = pair(model_folders, name, dtype, 1024)
    riding, _ = pair(model_folders, name, dtype, 1024, fuse_norms=True)
    cfg, w = P.read_model_folder(model_folders(name, dtype))
    oracle = {i: P.llama_forward(cfg, w, tokens_of(name, i), torch.bfloat16) for i in range(len(LENGTHS[name]))}
    toks = [tokens_of(name, i) for i in range(4)]
    for r in (native, parts, riding):
        r.step([dict(id=f"r{i}", tokens=t[:-3], want=[]) for i, t in enumerate(toks) if len(t) > 3])
    live = [i for i, t in enumerate(toks) if len(t) > 3]
    for k in (3, 2, 1):
        entries = [dict(id=f"r{i}", tokens=[toks[i][-k]], want=[0]) for i in live]
        n0 = K.launch_count()
        separate = native.step(entries)
        n1 = K.launch_count()
        together = riding.step(entries)
        n2 = K.launch_count()
        assert torch.equal(separate, parts.step(entries)), f"{name} decode step"
        ref = torch.stack([oracle[i][len(toks[i]) - k] for i in live])
        helpers.assert_logits_close(together, ref, dtype, f"{name} decode step, norms in the products")
        assert (n1 - n0) - (n2 - n1) >= cfg["num_hidden_layers"], "norms ride in the products: fewer launches"
    steps, places = mixed_trace(name)
    native, parts = pair(model_folders, name, dtype, mixed_pool_tokens(name), fuse_norms=True)
    for s, where in zip(steps, places):
        a, b = native.step(s["entries"], s["end"]), parts.step(s["entries"], s["end"])
        ref = torch.stack([oracle[i][pos] for i, pos in where])
        helpers.assert_logits_close(a, ref, dtype, f"{name} native, mixed step {s['step']}")
        helpers.assert_logits_close(b, ref, dtype, f"{name} part by part, mixed step {s['step']}")


def test_forcing_options_and_other_parts_run_part_by_part(model_folders):
    name = "tiny-c"
    block = helpers.TINY[name]["block_size"]
    forced = helpers.Replayer(model_folders(name, "bfloat16"), "bfloat16", 256, block, options={"gemm": "tcgen05"})
    assert forced.runner.native is not None
    toks = tokens_of(name, 1)
    forced.step([dict(id="x", tokens=toks, want=[0])])
    assert forced.runner.native.calls == 0                     # the option is honoured by the parts themselves


def test_host_time_of_a_prefill_step(model_folders):
    """What the native loop is for: launching a prefill step of 2,048 rows and eight layers of the
    benchmark shape takes the host about half the time the part-by-part path needs (what remains is
    the launches themselves, the tensor maps of the attention kernel and the library's own set-up)."""
    from kvcm.config import LlamaConfig
    from kvcm.engine import model_from_tensors
    from kvcm.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=4100, hidden_size=2048, intermediate_size=5632,
                      num_hidden_layers=8, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                      max_position_embeddings=4096, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    spec = model_from_tensors(cfg, dict(random_tensors(cfg, 7, torch.bfloat16, device="cuda:0")), "bfloat16", "cuda:0")
    toks = helpers.random_tokens(2048, cfg.vocab_size, 3)
    host = {}
    for native in (True, False):
        r = helpers.Replayer(None, "bfloat16", 4096, 16, spec=spec, max_live=2,
                             options={} if native else {"native_forward": False})
        best = 1e9
        for rep in range(4):
            s = r.session
            seq_entries = [dict(id=f"p{rep}", tokens=toks, want=[2047])]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = s.step(seq_entries, [f"p{rep}"])
            t1 = time.perf_counter()
            torch.cuda.synchronize()
            best = min(best, t1 - t0)
        host[native] = best
    assert host[True] < 0.8 * host[False], host
