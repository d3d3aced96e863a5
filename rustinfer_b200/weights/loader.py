"""Weights by tensor name, from safetensors to the device.

The model declares every tensor it owns (name -> shape); the file is checked against
that list before anything is read, and everything wrong is reported at once: missing
tensors, tensors the model does not know, and wrong shapes.  RustInfer reports the first
missing tensor or shape only and ignores extras
(crates/infer-worker/src/models/loader.rs:191-201,1038-1052).

Precision: a bfloat16 engine keeps bf16 tensors as they are, turns fp16 into bf16, and
leaves what the file stores in 32-bit in 32-bit; integer tables become int32.  A float32
engine widens every float tensor to fp32 (exact for bf16 and fp16).
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..parts.base import ParamDecl
from .safetensors_io import SafetensorsReader


class WeightError(ValueError):
    def __init__(self, folder: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"weights in {folder} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


# Buffers that some exporters of Llama checkpoints write beside the weights; they are derived
# from the configuration, no model declares them, and a file that has them is not at fault.
# Anything else the model does not know stays an error.
IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


def check_against(reader: SafetensorsReader, decls: Mapping[str, ParamDecl], folder: str) -> None:
    have = set(n for n in reader.names() if not n.endswith(IGNORED_SUFFIXES))
    missing = sorted(n for n, d in decls.items() if n not in have and not d.optional)
    unexpected = sorted(have - set(decls))
    wrong = [f"{n}: expected {list(decls[n].shape)}, got {list(reader.shape(n))}"
             for n in sorted(have & set(decls)) if tuple(reader.shape(n)) != tuple(decls[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(folder, missing, unexpected, wrong)


def target_dtype(stored: torch.dtype, engine: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(folder: str, decls: Mapping[str, ParamDecl], engine_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    reader = SafetensorsReader(folder)
    check_against(reader, decls, folder)
    out: Dict[str, torch.Tensor] = {}
    for name in decls:
        if name not in reader:
            continue
        t = reader.tensor(name)
        out[name] = t.to(device=device, dtype=target_dtype(t.dtype, engine_dtype)).contiguous()
    return out
