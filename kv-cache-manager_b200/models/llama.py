"""The Llama dense decoder assembled from parts (registered as ``LlamaForCausalLM``).

Layer = pre-norm block of RMSNorm -> grouped-query attention with rotate-half rotary encoding ->
RMSNorm -> SiLU-gated MLP; final RMSNorm; output head, tied to the embedding when the config
says so or the checkpoint has no ``lm_head.weight``.  Structure and tensor names after the
reference (``src/model/llama.cpp:84-128``, ``tools/export_weights.py:69-82``): q,k,v rows are
fused into one matrix and gate,up rows into another at load, as its export does.
"""
from __future__ import annotations

from typing import List

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LayerCall
from ..parts.embedding import Embedding, LMHead
from .spec import ModelSpec, TensorBinding


def layer_plan(cfg: LlamaConfig) -> List[dict]:
    """Which parts each layer is made of.  Every layer of this architecture is alike; the list
    form is what lets another architecture vary mixers and feed-forwards by layer."""
    return [dict(block="pre_norm", norm="rmsnorm", mixer="attention", position="rope",
                 feed_forward="gated_mlp") for _ in range(cfg.num_hidden_layers)]


def build_llama(cfg: LlamaConfig, norm_init=("ones",)) -> ModelSpec:
    H, I = cfg.hidden_size, cfg.intermediate_size
    nh, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    embedding = Embedding(cfg.vocab_size, H)
    bindings = [TensorBinding(embedding, "weight",
                              [("model.embed_tokens.weight", (cfg.vocab_size, H))])]
    embed_binding = bindings[0]
    blocks = []
    for l, plan in enumerate(layer_plan(cfg)):
        position = POSITION_ENCODINGS.build(plan["position"], head_dim=hd, theta=cfg.rope_theta)
        mixer = MIXERS.build(plan["mixer"], hidden=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                             position=position)
        ffn = FEED_FORWARDS.build(plan["feed_forward"], hidden=H, intermediate=I,
                                  activation=cfg.hidden_act)
        norm1 = NORMS.build(plan["norm"], hidden=H, eps=cfg.rms_norm_eps, init=norm_init)
        norm2 = NORMS.build(plan["norm"], hidden=H, eps=cfg.rms_norm_eps, init=norm_init)
        block = BLOCKS.build(plan["block"], norm1=norm1, mixer=mixer, norm2=norm2, ffn=ffn)
        blocks.append(block)
        p = f"model.layers.{l}."
        bindings += [
            TensorBinding(norm1, "weight", [(p + "input_layernorm.weight", (H,))]),
            TensorBinding(mixer.qkv, "weight", [(p + "self_attn.q_proj.weight", (nh * hd, H)),
                                                (p + "self_attn.k_proj.weight", (nkv * hd, H)),
                                                (p + "self_attn.v_proj.weight", (nkv * hd, H))]),
            TensorBinding(mixer.o, "weight", [(p + "self_attn.o_proj.weight", (H, nh * hd))]),
            TensorBinding(norm2, "weight", [(p + "post_attention_layernorm.weight", (H,))]),
            TensorBinding(ffn.gate_up, "weight", [(p + "mlp.gate_proj.weight", (I, H)),
                                                  (p + "mlp.up_proj.weight", (I, H))]),
            TensorBinding(ffn.down, "weight", [(p + "mlp.down_proj.weight", (H, I))]),
        ]
    final_norm = NORMS.build("rmsnorm", hidden=H, eps=cfg.rms_norm_eps, init=norm_init)
    bindings.append(TensorBinding(final_norm, "weight", [("model.norm.weight", (H,))]))
    lm_head = LMHead(H, cfg.vocab_size)
    bindings.append(TensorBinding(lm_head, "weight", [("lm_head.weight", (cfg.vocab_size, H))],
                                  tie_to=embed_binding, tied=cfg.tie_word_embeddings))
    order = [LayerCall(l) for l in range(cfg.num_hidden_layers)]
    return ModelSpec(cfg, embedding, blocks, order, final_norm, lm_head, bindings,
                     ignorable=("rotary_emb.inv_freq",))


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama, replace=True)
