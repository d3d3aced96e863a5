"""Typed configuration of the Llama-3 dense decoder, read from config.json's own keys.

RustInfer parses config.json into a flat `HfConfig` that holds every family's optional
fields and lowers it to `LoadConfig` (crates/infer-worker/src/bin/worker_main.rs:56-126,
389-449).  Here one architecture has one typed record; every size and constant that
config.json gives is a field, and code reads the field.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """config.json lacks a key, or holds a value the engine cannot run."""


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency rescaling (crates/infer-worker/src/models/loader.rs:30-35)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> Dict[str, Any]:
        return {"rope_type": "llama3", "factor": self.factor,
                "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


def _need(d: Mapping[str, Any], key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    try:
        return kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: key '{key}' = {d[key]!r} is not {kind.__name__}")


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    eos_token_ids: Tuple[int, ...]
    architecture: str = "LlamaForCausalLM"
    model_type: str = "llama"

    # -- derived sizes (crates/infer-worker/src/domain/model.rs:12-49) ----------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None
                  ) -> "LlamaConfig":
        """Defaults follow crates/infer-worker/src/bin/worker_main.rs:173-181, 389-449:
        head_dim = hidden/heads, eps 1e-5, theta 10000, max positions 4096;
        num_key_value_heads has no fallback; rope_scaling counts only when its
        rope_type is "llama3" and all four numbers are present (:393-404)."""
        hidden = _need(d, "hidden_size")
        heads = _need(d, "num_attention_heads")
        kv_heads = _need(d, "num_key_value_heads")
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive")
        head_dim = int(d["head_dim"]) if d.get("head_dim") else hidden // heads
        scaling = None
        rs = d.get("rope_scaling")
        if isinstance(rs, Mapping) and rs.get("rope_type", rs.get("type")) == "llama3":
            keys = ("factor", "low_freq_factor", "high_freq_factor",
                    "original_max_position_embeddings")
            if all(rs.get(k) is not None for k in keys):
                scaling = RopeScaling(float(rs["factor"]), float(rs["low_freq_factor"]),
                                      float(rs["high_freq_factor"]),
                                      int(rs["original_max_position_embeddings"]))
        vocab = _need(d, "vocab_size")
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size"),
            num_hidden_layers=_need(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=vocab,
            max_position_embeddings=int(d.get("max_position_embeddings") or 4096),
            rms_norm_eps=float(d.get("rms_norm_eps") or 1e-5),
            rope_theta=float(d.get("rope_theta") or 10000.0),
            rope_scaling=scaling,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            eos_token_ids=_eos_ids(d, generation, vocab),
            architecture=str((d.get("architectures") or ["LlamaForCausalLM"])[0]),
            model_type=str(d.get("model_type") or "llama"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "vocab_size",
                     "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if not self.rope_theta > 0.0:
            raise ConfigError("config.json: rope_theta must be positive")
        rs = self.rope_scaling
        if rs is not None:
            if rs.factor <= 0 or rs.high_freq_factor == rs.low_freq_factor or rs.low_freq_factor <= 0:
                raise ConfigError("config.json: rope_scaling needs factor > 0 and "
                                  "0 < low_freq_factor != high_freq_factor")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _eos_ids(cfg: Mapping[str, Any], generation: Optional[Mapping[str, Any]], vocab: int
             ) -> Tuple[int, ...]:
    """generation_config.json first, then config.json; an int or a list
    (crates/infer-worker/src/bin/worker_main.rs:327-373).  The reference falls back to
    Llama 3's three stop ids when neither file has the key; a model whose files name no
    stop id stops on none here, so that no id stands in code."""
    for src in (generation, cfg):
        if not src:
            continue
        e = src.get("eos_token_id")
        if isinstance(e, bool):
            continue
        if isinstance(e, int):
            return (int(e),)
        if isinstance(e, (list, tuple)):
            ids = tuple(int(x) for x in e if isinstance(x, int) and not isinstance(x, bool))
            if ids:
                return ids
    return ()


def read_config_json(folder: str) -> Tuple[Dict[str, Any], Optional[Dict[str, Any]]]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path) as f:
        try:
            cfg = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})")
    gen = None
    gpath = os.path.join(folder, "generation_config.json")
    if os.path.isfile(gpath):
        try:
            with open(gpath) as f:
                gen = json.load(f)
        except json.JSONDecodeError:
            gen = None
    return cfg, gen
