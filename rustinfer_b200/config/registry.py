"""One registry from an architecture's name to the code that builds it.

RustInfer maps config.json's `model_type` / `architectures[0]` to an internal type by
substring and dispatches with a `match` (crates/infer-protocol/src/config.rs:437-492,
crates/infer-worker/src/bin/worker_main.rs:778-855).  Here an architecture is an
`ArchitectureFamily` value registered under its names; adding one is one call to
`register_architecture` and touches no other file.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

from ..parts.spec import ModelSpec
from .model_config import ConfigError


@dataclass(frozen=True)
class ArchitectureFamily:
    """`parse_config(config.json dict, generation_config dict|None)` -> typed config;
    `model_spec(typed config)` -> ModelSpec (parts, their numbers, run order, names)."""
    name: str
    parse_config: Callable[[Mapping[str, Any], Optional[Mapping[str, Any]]], Any]
    model_spec: Callable[[Any], ModelSpec]


_BY_NAME: Dict[str, ArchitectureFamily] = {}


def register_architecture(names, family: ArchitectureFamily) -> None:
    for n in names:
        _BY_NAME[n.lower()] = family


def supported_architectures() -> List[str]:
    return sorted(_BY_NAME)


def resolve_architecture(cfg: Mapping[str, Any]) -> ArchitectureFamily:
    """`architectures[0]` and `model_type` are looked up by exact (case-folded) name;
    an unknown model is an error that lists what is supported."""
    hints: List[str] = []
    archs = cfg.get("architectures")
    if isinstance(archs, (list, tuple)) and archs and isinstance(archs[0], str):
        hints.append(archs[0])
    if isinstance(cfg.get("model_type"), str):
        hints.append(cfg["model_type"])
    for h in hints:
        fam = _BY_NAME.get(h.lower())
        if fam is not None:
            return fam
    shown = ", ".join(repr(h) for h in hints) or "<missing model_type/architectures>"
    raise ConfigError(f"unsupported model {shown}; supported: {', '.join(supported_architectures())}")


def load_model_description(folder: str) -> Tuple[ArchitectureFamily, Any, ModelSpec]:
    """config.json of `folder` -> (family, typed config, model spec)."""
    from .model_config import read_config_json
    cfg, gen = read_config_json(folder)
    fam = resolve_architecture(cfg)
    typed = fam.parse_config(cfg, gen)
    spec = fam.model_spec(typed)
    spec.validate()
    return fam, typed, spec
