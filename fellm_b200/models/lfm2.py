"""Lfm2ForCausalLM: how the LFM2 ShortConv hybrid is put together from parts.

Per block (crates/fellm-model/src/graph.rs:1650-1777): h = x + Mixer(RMSNorm(x; operator_norm)),
out = h + SwiGLU(RMSNorm(h; ffn_norm)); the mixer of layer i is a gated short convolution or GQA
attention with per-head QK RMSNorm and rotary positions, as layer_types says
(probe.rs:340-363 infers the same from tensor names).  Final RMSNorm, then the head, which is the
embedding matrix when tie_word_embeddings (graph.rs:29-39).

Tensor names are those of the safetensors folder this engine reads and writes:
model.embed_tokens, model.layers.{i}.operator_norm / ffn_norm / conv.{in_proj,conv,out_proj} /
self_attn.{q_proj,k_proj,v_proj,out_proj,q_layernorm,k_layernorm} / feed_forward.{w1,w3,w2},
model.embedding_norm, lm_head.  (FeLLM reads GGUF names blk.N.shortconv.in_proj ... instead:
graph.rs:1790-1801,2014-2039,2260-2271.)
"""
from __future__ import annotations

from ..config.lfm2 import Lfm2Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

NAME = "Lfm2ForCausalLM"


def build_spec(cfg: Lfm2Config) -> ModelSpec:
    d = cfg.hidden_size
    position = PartSpec.make("rope", rot_dim=cfg.head_dim, theta=cfg.rope_theta, pairing=cfg.rope_pairing)
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        p = f"model.layers.{i}."
        if kind == "conv":
            mixer = PartSpec.make("shortconv", prefix=p + "conv.", size=d, taps=cfg.conv_L_cache,
                                  bias=cfg.conv_bias)
        else:
            mixer = PartSpec.make(
                "attention", prefix=p + "self_attn.",
                names={"q_norm.weight": p + "self_attn.q_layernorm.weight",
                       "k_norm.weight": p + "self_attn.k_layernorm.weight"},
                size=d, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, qk_norm=True, norm_eps=cfg.norm_eps, position=position, window=None)
        ffn = PartSpec.make("swiglu", prefix=p + "feed_forward.",
                            names={"gate.weight": p + "feed_forward.w1.weight",
                                   "up.weight": p + "feed_forward.w3.weight",
                                   "down.weight": p + "feed_forward.w2.weight"},
                            size=d, ff=cfg.ff_dim)
        layers.append(LayerSpec(
            norm1=PartSpec.make("rmsnorm", prefix=p + "operator_norm.", size=d, eps=cfg.norm_eps),
            mixer=mixer,
            norm2=PartSpec.make("rmsnorm", prefix=p + "ffn_norm.", size=d, eps=cfg.norm_eps),
            ffn=ffn))
    return ModelSpec(
        architecture=NAME, hidden_size=d, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        embedding=PartSpec.make("table", prefix="model.embed_tokens.", vocab=cfg.vocab_size, size=d),
        layers=layers,
        final_norm=PartSpec.make("rmsnorm", prefix="model.embedding_norm.", size=d, eps=cfg.norm_eps),
        head=PartSpec.make("linear", prefix="lm_head.", vocab=cfg.vocab_size, size=d,
                           tied=cfg.tie_word_embeddings))


register_architecture(NAME, Lfm2Config.from_dict, build_spec)
