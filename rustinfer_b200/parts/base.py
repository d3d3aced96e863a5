"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from the `params` of its `PartSpec` alone and knows nothing of the
model around it.  It declares the tensors it owns (`param_decls`), receives them
(`load`), and runs on what the step hands it.  New kinds are added by registering a
class; no file of the framework changes.

    Mixer          forward(x[T,hidden], step, cache) -> delta[T,hidden]
                   cache_need() -> PagedKV | FixedState | None
    FeedForward    forward(x[T,hidden], step) -> delta[T,hidden]
    Norm           add_norm(h_fp32[T,hidden], delta|None, rows|None) -> normed
    PositionEncoding   prepare(ctx) builds whatever tables the mixer's kernel reads

RustInfer's counterparts are the `Component` impls under
crates/infer-worker/src/components/ (attention.rs, ffn_dense.rs, norm.rs) driven through
`Hidden{stream, pending}` (crates/infer-core/src/component.rs:8-27).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple, Type, Union

import torch

from .spec import PartSpec


# ------------------------------------------------------------------ declarations
@dataclass(frozen=True)
class ParamDecl:
    """A tensor a part owns: its shape, how the random-weights mode fills it
    ("normal": N(0, std); "ones": 1, or 1 + N(0, std) when norms are perturbed)."""
    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every token (or of the last `window` tokens) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, one slot per live request."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


CacheNeed = Union[PagedKV, FixedState]


@dataclass
class BuildContext:
    """What a part may know of the engine it is built into."""
    device: torch.device
    dtype: torch.dtype                  # activation and cache dtype: bfloat16 or float32
    max_model_len: int                  # positions a request can reach
    page_size: int
    shared: Dict[Any, Any] = field(default_factory=dict)   # tables and scratch shared between layers
    max_batch_seqs: int = 64            # most entries a step can bring
    num_sms: int = 148


# ------------------------------------------------------------- per-step information
@dataclass
class GroupStep:
    """Page tables of one cache group for the entries of this step (device, int32)."""
    block_table: torch.Tensor           # [entries, max_pages]
    slot_of_token: torch.Tensor         # [tokens] page*page_size + offset


@dataclass
class HostEntry:
    request_id: Any
    slot: int                           # state slot of the request
    q_len: int
    pos0: int                           # position of the entry's first token


@dataclass
class StepContext:
    """Everything a part may read about the batch it runs on.  Device tensors are int32
    and live in buffers whose addresses do not change between steps of one bucket."""
    num_tokens: int
    num_entries: int
    token_ids: torch.Tensor             # [tokens]
    positions: torch.Tensor             # [tokens]
    cu_q: torch.Tensor                  # [entries + 1]
    kv_len: torch.Tensor                # [entries] length after this step
    state_slots: torch.Tensor           # [entries]
    groups: List[GroupStep]
    tiles: Dict[int, Tuple[torch.Tensor, torch.Tensor]]   # tokens per tile -> (tile_entry, tile_q0), all entries
    entries: List[HostEntry]            # host mirror, for parts that are not graph-safe
    max_q_len: int
    max_kv_len: int                     # an upper bound of kv_len (exact in eager steps)
    decode_only: bool
    # entries of one token (decoding) and tiles over the other entries, for kernels that
    # treat the two differently
    decode_entries: Optional[torch.Tensor] = None          # [num_decode] entry indices
    num_decode: int = 0
    prefill_tiles: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)


@dataclass
class PagedLayerCache:
    kv: torch.Tensor                    # [pages, 2, kv heads, page, head_dim]
    group: int                          # index into StepContext.groups
    writes: bool = True                 # False: the layer reads a cache another one wrote


@dataclass
class StateLayerCache:
    state: torch.Tensor                 # [slots, *shape]; row = StepContext.state_slots[entry]


# ---------------------------------------------------------------------------- parts
class Part:
    def __init__(self, params: Mapping[str, Any]):
        self.params = dict(params)

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {}

    def prepare(self, ctx: BuildContext) -> None:
        """Build tables on the device; called once before `load`."""
        self.ctx = ctx

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the declared tensors (already on the device, dtype per the loader)."""


class Norm(Part):
    def add_norm(self, h: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    graph_safe = True                   # forward reads only device tensors of the step
    attention_tile_rows: Tuple[int, ...] = ()   # tile lists over all entries the step must prepare
    prefill_tile_rows: Tuple[int, ...] = ()     # tile lists over the entries of more than one token

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, x: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = True

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


# ----------------------------------------------------------------------- registries
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Type[Part]] = {}

    def register(self, kind: str) -> Callable[[Type[Part]], Type[Part]]:
        def deco(cls):
            self._kinds[kind] = cls
            return cls
        return deco

    def build(self, spec: PartSpec) -> Part:
        cls = self._kinds.get(spec.kind)
        if cls is None:
            raise KeyError(f"no {self.what} registered as '{spec.kind}'; known: {sorted(self._kinds)}")
        return cls(spec.params)

    def kinds(self) -> List[str]:
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
