"""The kernels that the Llama-3-8B and Llama-2-7B shapes take and the TinyLlama shape does not,
inside the engine: two layers of hidden size 4,096 with 32 query heads on 8 (or 32) KV heads of 128
and a feed-forward of 14,336 (or 11,008) (heads of 128 in the tcgen05 prefill attention and in decode attention, the gate/up product
with its activation on pairs of SMs, the library's product for the 14,336-wide down projection of a
decode step, a rotary base of 500,000), against the plain implementation in float64 on the CPU."""
import pytest
import torch

import helpers
import plain_llama as P
from test_gpu_big_shape import near_float32, near_plain, same_cut

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv_heads,ffn,theta", [(8, 14336, 500000.0),       # Llama-3-8B
                                                (32, 11008, 10000.0)])       # Llama-2-7B: every query head its own KV head
def test_whole_prompt_then_token_by_token_at_the_8b_shape(kv_heads, ffn, theta):
    from kvcm.config import LlamaConfig
    from kvcm.engine import model_from_tensors
    from kvcm.kernels import library as K
    from kvcm.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=4100, hidden_size=4096, intermediate_size=ffn,
                      num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=kv_heads, head_dim=128,
                      max_position_embeddings=8192, rope_theta=theta, rms_norm_eps=1e-5, tie_word_embeddings=False)
    t16 = dict(random_tensors(cfg, 11, torch.bfloat16, device="cuda:0", norm_jitter=0.1))
    spec16 = model_from_tensors(cfg, dict(t16), "bfloat16", "cuda:0")
    spec32 = model_from_tensors(cfg, {k: v.float() for k, v in t16.items()}, "float32", "cuda:0")
    w = {k: v.double().cpu() for k, v in t16.items()}
    cj = cfg.to_json_dict()
    n = 600
    toks = helpers.random_tokens(n, cfg.vocab_size, 5)
    want = [0, 1, 63, 64, 127, 128, 255, 256, 300, 511, 512] + list(range(n - 24, n))
    exact = P.llama_forward(cj, w, toks, None)[want]
    rounded = P.llama_forward(cj, w, toks, torch.bfloat16)[want]
    ref = helpers.Replayer(None, "float32", 1024, 16, spec=spec32, max_live=2).step([dict(id="a", tokens=toks, want=want)])
    helpers.assert_logits_close(ref, exact, "float32", "true 32-bit path at the 8B shape")
    whole = helpers.Replayer(None, "bfloat16", 1024, 16, spec=spec16, max_live=2).step([dict(id="a", tokens=toks, want=want)])
    near_plain(whole, rounded, exact, "whole prompt of 600 tokens")
    near_float32(whole, ref, "whole prompt of 600 tokens")
    r = helpers.Replayer(None, "bfloat16", 1024, 16, spec=spec16, max_live=2)
    early = [p for p in want if p < n - 24]
    got = [r.step([dict(id="a", tokens=toks[:n - 24], want=early)])]
    for t in range(n - 24, n):                                      # the last 24 tokens one by one
        got.append(r.step([dict(id="a", tokens=toks[t:t + 1], want=[0])]))
    got = torch.cat(got)
    near_plain(got, rounded, exact, "most of the prompt, then token by token")
    same_cut(got, whole, rounded, exact, "token by token against the whole prompt")
    assert K.attention_tcgen05_error() == 0 and K.tcgen05_error() == 0 and K.stream_error() == 0 and K.pair_error() == 0
    assert r.stray_writes() == []                                   # pages never handed out are still zero
