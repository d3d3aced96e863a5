"""A decoder put together from a `ModelSpec`: embedding, the blocks in their run order,
final norm over the wanted rows, head.  It owns no sizes of its own; everything comes
from the spec (crates/infer-worker/src/models/decoder.rs:57-200 is the reference's
`Decoder` with `embed / decode_layers / finalize`).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..parts import attention, ffn, norm, rope  # noqa: F401  (registers the built-in parts)
from ..parts.base import NORMS, BuildContext, CacheNeed, ParamDecl, StepContext
from ..parts.block import Block, Hidden
from ..parts.linear import Linear
from ..parts.spec import ModelSpec


class Decoder:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks: List[Block] = [Block(ls) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embed_table: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self.head_is_tied = False
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
        decls: Dict[str, ParamDecl] = {
            s.embed_name + "weight": ParamDecl((s.vocab_size, s.hidden_size)),
            s.head_name + "weight": ParamDecl((s.vocab_size, s.hidden_size), optional=s.tie_head),
        }
        for name, d in self.final_norm.param_decls().items():
            decls[s.final_norm_name + name] = d
        for block, ls in zip(self.blocks, s.layers):
            for role, part in block.roles().items():
                for name, d in part.param_decls().items():
                    decls[ls.names[role] + name] = d
        return decls

    def cache_needs(self) -> List[Tuple[int, Optional[CacheNeed], Optional[int]]]:
        """Per run entry: (layer, what its mixer keeps between steps, entry whose cache it reads)."""
        return [(e.layer, self.blocks[e.layer].mixer.cache_need(), e.cache_of) for e in self.spec.run_order]

    def attention_tile_rows(self) -> Tuple[int, ...]:
        rows = set()
        for b in self.blocks:
            rows.update(b.mixer.attention_tile_rows)
        return tuple(sorted(rows))

    def prefill_tile_rows(self) -> Tuple[int, ...]:
        rows = set()
        for b in self.blocks:
            rows.update(b.mixer.prefill_tile_rows)
        return tuple(sorted(rows))

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks)

    # ------------------------------------------------------------------------- build
    def prepare(self, ctx: BuildContext) -> None:
        self.ctx = ctx
        for b in self.blocks:
            b.prepare(ctx)
        self.final_norm.prepare(ctx)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed_table = tensors[s.embed_name + "weight"].contiguous()
        head = tensors.get(s.head_name + "weight")
        # the head is the embedding table when the file has no head of its own
        # (crates/infer-worker/src/models/decoder.rs:245-262)
        self.head_is_tied = head is None
        self.head = Linear(self.embed_table if head is None else head, self.ctx.num_sms)
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
        K.embed_gather(step.token_ids[: step.num_tokens], self.embed_table, h)
        hidden = Hidden(h, None)
        for i, e in enumerate(s.run_order):
            self.blocks[e.layer].forward(hidden, step, caches[i])
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        n = self.final_norm.add_norm(hidden.stream, hidden.pending, rows=logit_rows)
        return self.head(n, out_dtype=torch.float32)
