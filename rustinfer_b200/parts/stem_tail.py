"""The stem and the tail of a decoder as parts of their own: the embedding that starts the
residual stream and the head that turns normed rows into logits.

`token_embedding`: h[t, :] = E[ids[t], :], no scaling, no position table
(crates/infer-worker/src/components/embed.rs:78-81).  `linear_head`: logits = n W^T in fp32;
when the file has no weight for it, it takes the matrix the embedding offers to share, as
the reference ties the head to the embedding table when `lm_head.weight` is absent
(crates/infer-worker/src/models/decoder.rs:245-262).  An embedding multiplier, learned
positions or a soft cap on the logits would be other kinds registered beside these.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Embedding, Head, ParamDecl, StepContext, register_embedding, register_head
from .linear import Linear


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.table: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors["weight"].contiguous()

    def shared_table(self) -> Optional[torch.Tensor]:
        return self.table

    def forward(self, step: StepContext, h: torch.Tensor) -> None:
        K.embed_gather(step.token_ids[: step.num_tokens], self.table, h)


@register_head("linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, tied (the configuration says the head is the embedding
    table: the file need not have a weight for it)."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.tied = bool(params.get("tied", False))
        self.linear: Optional[Linear] = None
        self.is_tied = False

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.vocab, self.hidden), optional=self.tied)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors.get("weight")
        self.is_tied = w is None
        if w is None:
            shared = self.shared
            if shared is None or tuple(shared.shape) != (self.vocab, self.hidden):
                raise ValueError("the head has no weight of its own and the embedding offers none of its shape")
            w = shared
        self.linear = Linear(w, self.ctx.num_sms)

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        return self.linear(normed, out_dtype=torch.float32)
