"""The data that describes a model: which part stands where, with which numbers.

A model is a tuple of `LayerSpec` plus a run order.  Each layer names its mixer,
feed-forward and norms by the *kind* under which the part is registered and hands
them their sizes and constants as `params`; nothing in a part refers to the model
it sits in.  Layers may differ from one another, and the run order is data too: it
may name a layer twice, or let a layer read the cache another layer wrote.

RustInfer wires its decoder in code (crates/infer-worker/src/models/decoder.rs:214-410
builds `Embed`, N x `DecoderBlock{Attention, DenseFfn}`, the final `RmsNorm` and
`LmHead`); here the same wiring is a value that a configuration produces.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _freeze(value: Any) -> Any:
    if isinstance(value, Mapping):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(v) for v in value)
    return value


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by registered `kind`, with its parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def key(self) -> Tuple:
        """Hashable identity: two specs with the same key may share tables."""
        return (self.kind, _freeze(self.params))


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts it has, how they are arranged, and the tensor-name prefix of
    each (`names[role] + local_name` is the tensor's name in the file).  Only the mixer is
    required: a block of one sublayer has no feed-forward, a block whose sublayers share a
    norm names one, and norms beyond the two usual ones (after a sublayer, say) go by a role
    of their own in `extra_norms`.  What the arrangement does with them is its business."""
    mixer: PartSpec
    mixer_norm: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    names: Mapping[str, str] = field(default_factory=dict)   # role -> prefix; roles: mixer, mixer_norm, ffn, ffn_norm, extras
    arrangement: str = "pre_norm"
    extra_norms: Mapping[str, PartSpec] = field(default_factory=dict)   # role -> norm


@dataclass(frozen=True)
class RunEntry:
    """One stop of the run order: run `layer`; `cache_of` names the layer whose cache
    it reads and writes (None: its own).  A layer that reads another layer's cache
    does not write keys of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    embed_name: str                     # prefix of the embedding table
    final_norm_name: str
    head_name: str
    tie_head: bool                      # config says the head is the embedding table
    eos_token_ids: Tuple[int, ...] = ()
    # the stem and the tail, chosen like every other part; None: a plain token embedding and a
    # linear head of the model's sizes
    embed: Optional[PartSpec] = None
    head: Optional[PartSpec] = None

    def embed_spec(self) -> PartSpec:
        return self.embed or PartSpec("token_embedding", {"vocab_size": self.vocab_size,
                                                          "hidden_size": self.hidden_size})

    def head_spec(self) -> PartSpec:
        return self.head or PartSpec("linear_head", {"vocab_size": self.vocab_size,
                                                     "hidden_size": self.hidden_size, "tied": self.tie_head})

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("a model needs at least one layer")
        for e in self.run_order:
            if not 0 <= e.layer < n:
                raise ValueError(f"run order names layer {e.layer}, model has {n}")
            if e.cache_of is not None and not 0 <= e.cache_of < n:
                raise ValueError(f"run order reads cache of layer {e.cache_of}, model has {n}")
