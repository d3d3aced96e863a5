"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from the `params` of its `PartSpec` alone and knows nothing of the
model around it.  It declares the tensors it owns (`param_decls`), receives them
(`load`), and runs on what the step hands it.  New kinds are added by registering a
class; no file of the framework changes.

    Embedding      forward(step, h_fp32[T,hidden]) fills the stream for the step's tokens (the stem)
    Mixer          forward(x[T,hidden], step, cache) -> delta[T,hidden]
                   cache_need() -> PagedKV | FixedState | None
                   step_indices() -> the int32 arrays it wants made for every step
    FeedForward    forward(x[T,hidden], step) -> delta[T,hidden]
    Norm           add_norm(h_fp32[T,hidden], delta|None, rows|None) -> normed
    PositionEncoding   prepare(ctx) builds whatever tables the mixer's kernel reads
    Head           forward(normed[R,hidden]) -> fp32 logits [R,vocab] (the tail)

RustInfer's counterparts are the `Component` impls under
crates/infer-worker/src/components/ (attention.rs, ffn_dense.rs, norm.rs) driven through
`Hidden{stream, pending}` (crates/infer-core/src/component.rs:8-27).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, List, Mapping, Optional, Sequence, Tuple, Type, Union

import numpy as np
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
    num_sms: int = 0                    # streaming multiprocessors; 0: asked of the device

    def __post_init__(self):
        if self.num_sms <= 0:
            from ..ops import library
            self.num_sms = library.num_sms(self.device) if self.device.type == "cuda" else 1


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
class StepShape:
    """The batch of a step as the host knows it before anything runs (int64 arrays, one
    element per entry): what an index array may be computed from."""
    q_lens: np.ndarray                  # tokens each entry brings
    pos0: np.ndarray                    # position of each entry's first token
    cu_q: np.ndarray                    # [entries + 1] running sum of q_lens
    kv_len: np.ndarray                  # pos0 + q_lens
    slots: np.ndarray                   # state slot of each entry


@dataclass(frozen=True)
class StepIndex:
    """An index array (or a few that belong together) a part wants on the device for every
    step, made on the host from the step's shape and uploaded with the step's other indices.
    Parts that declare the same `key` share one copy.

    `build(shape)` returns a tuple of integer arrays; `capacity(max_tokens, max_entries)` an
    upper bound of their total length, for the staging buffer.  In a captured step of single
    tokens the arrays must have the same lengths whenever the number of rows is the same
    (they live at fixed addresses); `depends_on_positions` says whether they must be made
    anew at every replay or once per bucket."""
    key: Hashable
    build: Callable[[StepShape], Tuple[np.ndarray, ...]]
    capacity: Callable[[int, int], int]
    depends_on_positions: bool = False


def single_token_entries() -> StepIndex:
    """The entries that bring exactly one token (decoding), as a list of entry numbers."""
    return StepIndex(("single_token_entries",),
                     lambda sh: (np.flatnonzero(sh.q_lens == 1),),
                     lambda max_tokens, max_entries: max_entries + 4)


def token_tiles(rows: int, skip_single_token: bool) -> StepIndex:
    """Every entry's tokens cut into tiles of `rows` tokens: (entry of the tile, first token of
    the tile within its entry).  With `skip_single_token`, entries of one token get no tile."""
    def build(sh: StepShape):
        n_tiles = (sh.q_lens + rows - 1) // rows
        if skip_single_token:
            n_tiles = np.where(sh.q_lens == 1, 0, n_tiles)
        entry = np.repeat(np.arange(sh.q_lens.size), n_tiles)
        first = np.zeros(sh.q_lens.size, dtype=np.int64)
        np.cumsum(n_tiles[:-1], out=first[1:])
        return entry, (np.arange(int(n_tiles.sum())) - first[entry]) * rows
    return StepIndex(("token_tiles", rows, skip_single_token), build,
                     lambda max_tokens, max_entries: 2 * (max_tokens // rows + max_entries + 8))


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
    entries: List[HostEntry]            # host mirror, for parts that are not graph-safe
    max_q_len: int
    max_kv_len: int                     # an upper bound of kv_len (exact in eager steps)
    decode_only: bool
    # what the model's parts declared through `step_indices()`: key -> tuple of device tensors
    indices: Dict[Hashable, Tuple[torch.Tensor, ...]] = field(default_factory=dict)

    def index(self, need: "StepIndex") -> Tuple[torch.Tensor, ...]:
        try:
            return self.indices[need.key]
        except KeyError:
            raise KeyError(f"the step was built without the index arrays {need.key!r}; the part that reads "
                           f"them must return them from step_indices()") from None


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


class Embedding(Part):
    """The stem: turns the step's token ids (and, if it wants, positions) into the fp32 stream."""

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        """Fill h [step.num_tokens, hidden] (fp32)."""
        raise NotImplementedError

    def shared_table(self) -> Optional[torch.Tensor]:
        """A [vocab, hidden] matrix a head may use as its weight when the file has none of its own."""
        return None


class Head(Part):
    """The tail: logits of rows that the final norm has already normed."""
    shared: Optional[torch.Tensor] = None

    def offer_shared(self, table: Optional[torch.Tensor]) -> None:
        """Called before `load` with the matrix the embedding offers to share (or None); a
        head whose optional weight is absent from the file may use it."""
        self.shared = table

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        """normed [R, hidden] -> fp32 logits [R, vocab]."""
        raise NotImplementedError


class Mixer(Part):
    graph_safe = True                   # in steps of single tokens, forward reads only device tensors

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def step_indices(self) -> Sequence[StepIndex]:
        """Index arrays the step builder must make for this part (see `StepIndex`)."""
        return ()

    def forward(self, x: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = True

    def step_indices(self) -> Sequence[StepIndex]:
        return ()

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


EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")

register_embedding = EMBEDDINGS.register
register_head = HEADS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
