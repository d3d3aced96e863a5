"""How a layer's parts are arranged.  "pre_norm": the stream h is only ever changed by
adding what a sublayer returned, and that add is fused into the next norm:

    x = mixer_norm(h += pending);  pending = mixer(x)
    x = ffn_norm(h += pending);    pending = ffn(x)

(crates/infer-worker/src/components/decoder_block.rs:13-32 over
crates/infer-core/src/component.rs:8-27).  h is fp32; pending is in the activation dtype.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from .base import FEED_FORWARDS, MIXERS, NORMS, BuildContext, FeedForward, Mixer, Norm, StepContext
from .spec import LayerSpec


@dataclass
class Hidden:
    stream: torch.Tensor                # [T, hidden] fp32
    pending: Optional[torch.Tensor]     # [T, hidden] activation dtype, not yet added


class Block:
    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer: Mixer = MIXERS.build(spec.mixer)
        self.mixer_norm: Optional[Norm] = NORMS.build(spec.mixer_norm) if spec.mixer_norm else None
        self.ffn: Optional[FeedForward] = FEED_FORWARDS.build(spec.ffn) if spec.ffn else None
        self.ffn_norm: Optional[Norm] = NORMS.build(spec.ffn_norm) if spec.ffn_norm else None
        self.extra_norms: Dict[str, Norm] = {role: NORMS.build(ps) for role, ps in spec.extra_norms.items()}
        fn = ARRANGEMENTS.get(spec.arrangement)
        if fn is None:
            raise KeyError(f"no block arrangement '{spec.arrangement}'; known: {sorted(ARRANGEMENTS)}")
        self._run = fn
        missing = [r for r in self.roles() if r not in spec.names]
        if missing:
            raise KeyError(f"layer names no tensor prefix for {missing}")

    def roles(self):
        """role -> part, for every part the layer has."""
        named = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "ffn": self.ffn, "ffn_norm": self.ffn_norm}
        named.update(self.extra_norms)
        return {role: part for role, part in named.items() if part is not None}

    def prepare(self, ctx: BuildContext) -> None:
        for part in self.roles().values():
            part.prepare(ctx)

    @property
    def graph_safe(self) -> bool:
        return self.mixer.graph_safe and (self.ffn is None or self.ffn.graph_safe)

    def forward(self, hidden: Hidden, step: StepContext, cache) -> None:
        self._run(self, hidden, step, cache)


def _pre_norm(block: Block, hidden: Hidden, step: StepContext, cache) -> None:
    if block.mixer_norm is None or block.ffn is None or block.ffn_norm is None:
        raise ValueError("the pre_norm arrangement wants a mixer, a feed-forward and a norm before each")
    # a part that declares `adds_to_residual` may add its output into the stream itself
    # (inside its last product's epilogue) and return None; otherwise the add rides on the
    # next norm
    x = block.mixer_norm.add_norm(hidden.stream, hidden.pending)
    if getattr(block.mixer, "adds_to_residual", False):
        hidden.pending = block.mixer.forward(x, step, cache, residual=hidden.stream)
    else:
        hidden.pending = block.mixer.forward(x, step, cache)
    x = block.ffn_norm.add_norm(hidden.stream, hidden.pending)
    if getattr(block.ffn, "adds_to_residual", False):
        hidden.pending = block.ffn.forward(x, step, residual=hidden.stream)
    else:
        hidden.pending = block.ffn.forward(x, step)


ARRANGEMENTS: Dict[str, Callable] = {"pre_norm": _pre_norm}


def register_arrangement(name: str, fn: Callable) -> None:
    ARRANGEMENTS[name] = fn
