"""The run file: one TOML with the engine's options, in RustInfer's names and meanings
(crates/infer-protocol/src/config.rs:55-262; example run_llama1b.toml:5-36).  Unknown
keys are refused, every key has a default, ranges are checked (:281-344).  Keys of the
reference that belong to its HTTP server, its process split or tensor parallelism are
accepted and ignored, so that a reference run file loads; `model_type` never stands
here, it always comes from config.json.

Added for this engine: `dtype`, a `[sampling]` table (temperature, top_k, top_p, min_p,
seed, max_tokens), `[[request]]` tables (`prompt_ids` or `random_len`) and a
`[random_weights]` table (`config`, `seed`, `std`) that builds the model folder first.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

try:
    import tomllib
except ModuleNotFoundError:                                    # pragma: no cover
    tomllib = None

DEFAULT_CAPTURE_SIZES = [1, 2, 4, 8, 16, 24, 32, 40, 48, 56, 64]

# keys of the reference's file that configure parts this engine does not have
_IGNORED = {"model_name", "cluster_id", "host", "port", "request_timeout_secs", "batch_wait_ms",
            "enable_prefix_caching", "mode", "worker_id", "log_level", "tensor_parallel_size",
            "tp_operation_timeout_secs", "tp_startup_timeout_secs", "worker_heartbeat_timeout_secs",
            "max_inflight_requests", "max_prefill_seqs_per_iter", "prefill_sjf", "cuda_memory"}


class RunConfigError(ValueError):
    pass


@dataclass
class RunConfig:
    model: str = ""
    device: str = "cuda:0"
    dtype: str = "bfloat16"
    max_batch_tokens: int = 8192
    max_batch_seqs: int = 32
    max_model_len: int = 4096
    paged_block_size: int = 16           # the reference's default is 1 (token slots); pages here
    chunked_prefill_size: int = 0        # 0 => whole prompts
    mem_fraction_static: float = 0.9
    num_blocks: int = 0                  # 0 => sized from free memory
    ignore_eos: bool = False
    capture_sizes: List[int] = field(default_factory=lambda: list(DEFAULT_CAPTURE_SIZES))
    sampling: Dict[str, Any] = field(default_factory=dict)
    requests: List[Dict[str, Any]] = field(default_factory=list)
    random_weights: Optional[Dict[str, Any]] = None

    def validate(self) -> None:
        if not self.model and not self.random_weights:
            raise RunConfigError("`model` (a folder with config.json and safetensors) is required")
        for k in ("max_batch_tokens", "max_batch_seqs", "max_model_len", "paged_block_size"):
            if int(getattr(self, k)) <= 0:
                raise RunConfigError(f"`{k}` must be positive")
        if self.chunked_prefill_size < 0 or self.num_blocks < 0:
            raise RunConfigError("`chunked_prefill_size` and `num_blocks` must not be negative")
        if not 0.0 < self.mem_fraction_static <= 1.0:
            raise RunConfigError("`mem_fraction_static` must lie in (0, 1]")
        if self.dtype not in ("bfloat16", "bf16", "float32", "fp32"):
            raise RunConfigError("`dtype` must be bfloat16 or float32")
        if any(int(c) <= 0 for c in self.capture_sizes):
            raise RunConfigError("`capture_sizes` must be positive batch sizes")
        if not str(self.device).startswith("cuda"):
            raise RunConfigError("`device` must be a CUDA device; there is no CPU path")

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RunConfig":
        known = set(cls.__dataclass_fields__) | {"request"}
        unknown = sorted(set(d) - known - _IGNORED)
        if unknown:
            raise RunConfigError(f"unknown keys in the run file: {', '.join(unknown)}")
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        if "request" in d:
            kw["requests"] = list(d["request"])
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, path: str) -> "RunConfig":
        if tomllib is None:
            raise RunConfigError("this Python has no tomllib")
        with open(path, "rb") as f:
            try:
                d = tomllib.load(f)
            except tomllib.TOMLDecodeError as e:
                raise RunConfigError(f"{path}: {e}")
        cfg = cls.from_dict(d)
        base = os.path.dirname(os.path.abspath(path))
        if cfg.model and not os.path.isabs(cfg.model):
            cfg.model = os.path.normpath(os.path.join(base, cfg.model))
        # paths in the run file are relative to the run file, not to where the program was started
        rw = cfg.random_weights
        if rw and rw.get("config") and not os.path.isabs(str(rw["config"])):
            cfg.random_weights = dict(rw, config=os.path.normpath(os.path.join(base, str(rw["config"]))))
        return cfg
