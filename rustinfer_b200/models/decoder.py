"""A decoder put together from a `ModelSpec`: the stem (an embedding part), the blocks in
their run order, final norm over the wanted rows, the tail (a head part).  It owns no sizes of its own; everything comes
from the spec (crates/infer-worker/src/models/decoder.rs:57-200 is the reference's
`Decoder` with `embed / decode_layers / finalize`).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts import attention, ffn, norm, rope, stem_tail  # noqa: F401  (registers the built-in parts)
from ..parts.base import EMBEDDINGS, HEADS, NORMS, BuildContext, CacheNeed, ParamDecl, StepContext, StepIndex
from ..parts.block import Block, Hidden
from ..parts.spec import ModelSpec


class Decoder:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks: List[Block] = [Block(ls) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embed = EMBEDDINGS.build(spec.embed_spec())
        self.head = HEADS.build(spec.head_spec())
        self.chained = None
        for i, e in enumerate(spec.run_order):
            mixer = self.blocks[e.layer].mixer
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if getattr(mixer, "own_kv", False):
                    raise ValueError(f"run entry {i} reads another entry's cache but its mixer projects keys of its own")

    # ------------------------------------------------------------------ declarations
    def param_decls(self) -> Dict[str, ParamDecl]:
        """Full tensor name -> declaration, for the loader and the random-weights mode."""
        s = self.spec
        decls: Dict[str, ParamDecl] = {}
        for prefix, part in ((s.embed_name, self.embed), (s.head_name, self.head),
                             (s.final_norm_name, self.final_norm)):
            for name, d in part.param_decls().items():
                decls[prefix + name] = d
        for block, ls in zip(self.blocks, s.layers):
            for role, part in block.roles().items():
                for name, d in part.param_decls().items():
                    decls[ls.names[role] + name] = d
        return decls

    def cache_needs(self) -> List[Tuple[int, Optional[CacheNeed], Optional[int]]]:
        """Per run entry: (layer, what its mixer keeps between steps, entry whose cache it reads)."""
        return [(e.layer, self.blocks[e.layer].mixer.cache_need(), e.cache_of) for e in self.spec.run_order]

    def step_indices(self) -> List[StepIndex]:
        """The index arrays the model's parts want made for every step, each key once."""
        seen: Dict = {}
        for b in self.blocks:
            for part in (b.mixer, b.ffn):
                if part is None:
                    continue
                for need in part.step_indices():
                    seen.setdefault(need.key, need)
        return list(seen.values())

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks)

    # ------------------------------------------------------------------------- build
    def prepare(self, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.embed.prepare(ctx)
        for b in self.blocks:
            b.prepare(ctx)
        self.final_norm.prepare(ctx)
        self.head.prepare(ctx)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        pick = lambda prefix, part: {n: tensors[prefix + n] for n in part.param_decls() if prefix + n in tensors}
        self.embed.load(pick(s.embed_name, self.embed))
        # a head without a weight of its own in the file takes what the embedding offers to share
        # (crates/infer-worker/src/models/decoder.rs:245-262)
        self.head.offer_shared(self.embed.shared_table())
        self.head.load(pick(s.head_name, self.head))
        self.final_norm.load({n: tensors[s.final_norm_name + n] for n in self.final_norm.param_decls()})
        for block, ls in zip(self.blocks, s.layers):
            for role, part in block.roles().items():
                part.load({n: tensors[ls.names[role] + n] for n in part.param_decls()
                           if ls.names[role] + n in tensors})
        # few-token steps of a decoder of the usual shape run their products chained
        from .chained_decoder import ChainedDecoder
        self.chained = ChainedDecoder.build(self)

    # --------------------------------------------------------------------------- run
    def forward(self, step: StepContext, caches: List, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the tokens of `step`; returns fp32 logits [rows, vocab] at `logit_rows`
        (token indices, int32, device), or None when no logits are wanted."""
        s = self.spec
        if self.chained is not None and self.chained.takes(step):
            return self.chained.forward(step, caches, logit_rows)
        h = torch.empty((step.num_tokens, s.hidden_size), dtype=torch.float32, device=self.ctx.device)
        self.embed.forward(step, h)
        hidden = Hidden(h, None)
        for i, e in enumerate(s.run_order):
            self.blocks[e.layer].forward(hidden, step, caches[i])
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        n = self.final_norm.add_norm(hidden.stream, hidden.pending, rows=logit_rows)
        return self.head.forward(n)
