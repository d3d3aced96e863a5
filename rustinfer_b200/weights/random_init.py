"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

RustInfer has only the primitive (`Tensor::randn`, crates/infer-core/src/tensor.rs:554-566)
and no such mode.  Every tensor gets its own generator seeded from (seed, tensor name), so
a tensor's values do not depend on which other tensors the model has.  Matrices are
N(0, std); norm weights are 1, or 1 + N(0, norm_std) when `norm_std` > 0 so that the
multiply is exercised.  The head is left out of the file when the configuration ties it.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _generator(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(config: Mapping[str, Any], seed: int, std: float = 0.02, norm_std: float = 0.0,
                   dtype: str = "bfloat16") -> Dict[str, torch.Tensor]:
    from ..models.decoder import Decoder
    fam = resolve_architecture(config)
    spec = fam.model_spec(fam.parse_config(config, None))
    decls = Decoder(spec).param_decls()
    store = _STORE[dtype]
    out: Dict[str, torch.Tensor] = {}
    for name, d in decls.items():
        if d.optional:                   # a tied head is not stored
            continue
        g = _generator(seed, name)
        if d.init == "ones":
            t = torch.ones(d.shape, dtype=torch.float32)
            if norm_std > 0:
                t += torch.randn(d.shape, generator=g, dtype=torch.float32) * norm_std
        else:
            t = torch.randn(d.shape, generator=g, dtype=torch.float32) * std
        out[name] = t.to(store)
    return out


def write_random_model(folder: str, config: Mapping[str, Any], seed: int, std: float = 0.02,
                       norm_std: float = 0.0, dtype: str = "bfloat16") -> str:
    """`config` is a config.json dict (the architecture's own keys).  Returns `folder`."""
    os.makedirs(folder, exist_ok=True)
    fam = resolve_architecture(config)
    typed = fam.parse_config(config, None)            # validates, fills defaults
    cfg_out = typed.to_dict() if hasattr(typed, "to_dict") else dict(config)
    cfg_out["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg_out, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(config, seed, std, norm_std, dtype))
    return folder
