"""The Llama-3 dense decoder as a registry entry: configuration -> model spec.

Pre-norm blocks of GQA attention with rotate-half RoPE (llama3 frequency scaling) and a
SwiGLU feed-forward, RMSNorm everywhere, head tied to the embedding when the file has
no `lm_head.weight` (crates/infer-worker/src/models/llama3.rs:14-24,
crates/infer-worker/src/models/decoder.rs:214-410).  Tensor names are those the
reference reads (crates/infer-worker/src/models/decoder.rs:237-331).
"""
from __future__ import annotations

import math

from ..config.model_config import LlamaConfig
from ..config.registry import ArchitectureFamily, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def llama_model_spec(cfg: LlamaConfig) -> ModelSpec:
    rope = PartSpec("rope", {
        "head_dim": cfg.head_dim,
        "rotary_dim": cfg.head_dim,
        "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
    })
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        # crates/infer-worker/src/models/decoder.rs:276
        "scale": 1.0 / math.sqrt(cfg.head_dim),
        "window": None,
        "position": rope,
    })
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                              "intermediate_size": cfg.intermediate_size})
    layers = tuple(
        LayerSpec(mixer=mixer, mixer_norm=norm, ffn=ffn, ffn_norm=norm,
                  names={"mixer": f"model.layers.{i}.self_attn.",
                         "mixer_norm": f"model.layers.{i}.input_layernorm.",
                         "ffn": f"model.layers.{i}.mlp.",
                         "ffn_norm": f"model.layers.{i}.post_attention_layernorm."})
        for i in range(cfg.num_hidden_layers))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        run_order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        embed_name="model.embed_tokens.",
        final_norm_name="model.norm.",
        head_name="lm_head.",
        tie_head=cfg.tie_word_embeddings,
        eos_token_ids=cfg.eos_token_ids,
    )


LLAMA = ArchitectureFamily(name="llama", parse_config=LlamaConfig.from_dict,
                           model_spec=llama_model_spec)
register_architecture(["llama", "LlamaForCausalLM"], LLAMA)
