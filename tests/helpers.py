"""Shared by the tests: tiny configurations that differ in every size and option, model
folders with weights that make faults show, and the plain implementation's logits."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import torch

import plain_llama

# Two configurations from the benchmark description plus a third whose head size is
# neither a power of two nor hidden/heads.  They differ in layers, width, heads and
# groups, head size, feed-forward width, vocabulary, theta, scaling, eps and tying.
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2,
              hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              intermediate_size=192, vocab_size=256, rope_theta=10000.0, rope_scaling=None,
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128)
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=3,
              hidden_size=96, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
              intermediate_size=272, vocab_size=391, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                high_freq_factor=4.0, original_max_position_embeddings=64),
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512)
TINY_C = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=1,
              hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              intermediate_size=104, vocab_size=130, rope_theta=30000.0,
              rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0,
                                high_freq_factor=2.0, original_max_position_embeddings=32),
              rms_norm_eps=3e-6, tie_word_embeddings=True, max_position_embeddings=256)
# Three more whose head sizes are 64 and 128: the attention kernels that serve the benchmark
# shapes (keys and values fetched by TMA for decoding, tcgen05 for prompt portions) take only
# those, so whole-model comparisons reach them through these.  D: groups of 4 (tcgen05 prompt
# attention, TMA decode); E: groups of 3 (rows of a tile do not fill it evenly); F: one kv head,
# heads*head_dim != hidden.
TINY_D = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2,
              hidden_size=256, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
              intermediate_size=512, vocab_size=1000, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0,
                                high_freq_factor=4.0, original_max_position_embeddings=256),
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024)
TINY_E = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2,
              hidden_size=384, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
              intermediate_size=520, vocab_size=777, rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                high_freq_factor=4.0, original_max_position_embeddings=128),
              rms_norm_eps=2e-6, tie_word_embeddings=False, max_position_embeddings=1024)
TINY_F = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=3,
              hidden_size=192, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
              intermediate_size=328, vocab_size=515, rope_theta=10000.0, rope_scaling=None,
              rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024)
# B with the feed-forward width and vocabulary that are powers of two times three (256, 384),
# beside the odd ones above
TINY_BS = dict(TINY_B, intermediate_size=256, vocab_size=384)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F, "Bs": TINY_BS}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Names and shapes of a Llama checkpoint, written out here so that the tests do not
    lean on the framework's own list."""
    d, inter, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = cfg.get("head_dim") or d // cfg["num_attention_heads"]
    q, kv = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    s = {"model.embed_tokens.weight": (v, d), "model.norm.weight": (d,)}
    if not cfg.get("tie_word_embeddings"):
        s["lm_head.weight"] = (v, d)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (d,)
        s[p + "post_attention_layernorm.weight"] = (d,)
        s[p + "self_attn.q_proj.weight"] = (q, d)
        s[p + "self_attn.k_proj.weight"] = (kv, d)
        s[p + "self_attn.v_proj.weight"] = (kv, d)
        s[p + "self_attn.o_proj.weight"] = (d, q)
        s[p + "mlp.gate_proj.weight"] = (inter, d)
        s[p + "mlp.up_proj.weight"] = (inter, d)
        s[p + "mlp.down_proj.weight"] = (d, inter)
    return s


def sharp_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Weights of size 1/sqrt(fan_in) (q and k twice that) and norm weights spread around
    1, so that activations are O(1), attention is peaked rather than flat and every
    multiply matters.  Stored in bf16 so that both engine precisions see the same values."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif "embed_tokens" in name:
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if "q_proj" in name or "k_proj" in name:
                t = t * 2.0
        out[name] = t.to(dtype)
    return out


def write_model(folder: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def make_sharp_model(folder: str, name: str, seed: int = 0, dtype=torch.bfloat16) -> str:
    return write_model(folder, TINY[name], sharp_weights(TINY[name], seed, dtype))


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Plain:
    """The plain implementation over one model folder, with per-sequence memo."""

    def __init__(self, folder: str):
        self.cfg, self.w = plain_llama.read_model_folder(folder)
        self._memo = {}

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = plain_llama.forward_logits(self.cfg, self.w, list(ids))
        return self._memo[key]


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| over max |ref|: the measure every logits comparison uses."""
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
