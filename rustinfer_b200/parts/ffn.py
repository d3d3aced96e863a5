"""Dense SwiGLU feed-forward: down( silu(gate(x)) * up(x) )
(crates/infer-worker/src/components/ffn_dense.rs:26-33,76-115).  gate and up are fused by
rows into one matrix, gate rows first (crates/infer-worker/src/models/loader.rs:543-571)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import FeedForward, ParamDecl, StepContext, register_feed_forward
from .linear import Linear


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"gate_proj.weight": ParamDecl((self.inter, self.hidden)),
                "up_proj.weight": ParamDecl((self.inter, self.hidden)),
                "down_proj.weight": ParamDecl((self.hidden, self.inter))}

    adds_to_residual = True

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        sms = self.ctx.num_sms
        # bf16: rows alternate gate_j, up_j so that the product's epilogue can form
        # silu(gate) * up; fp32: gate rows first, then up rows, for the separate kernel
        self.paired = dt == torch.bfloat16 and self.hidden % 8 == 0 and g.is_cuda
        if self.paired:
            self.gate_up = Linear(torch.stack([g.to(dt), u.to(dt)], dim=1).reshape(2 * self.inter, self.hidden), sms)
        else:
            self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0), sms)
        self.down = Linear(tensors["down_proj.weight"], sms)

    def forward(self, x: torch.Tensor, step: StepContext, residual: Optional[torch.Tensor] = None):
        """Returns the sublayer's output, or None when it was added into `residual`."""
        m = self.gate_up.silu_pairs(x) if self.paired else None
        if m is None:
            gu = self.gate_up(x, out_dtype=self.ctx.dtype)
            if self.paired:                               # the fused path refused this input
                gu = torch.cat([gu[:, 0::2], gu[:, 1::2]], dim=1).contiguous()
            m = torch.empty((x.shape[0], self.inter), dtype=self.ctx.dtype, device=x.device)
            K.silu_mul(gu, m)
        if residual is not None and self.down.add_into(m, residual):
            return None
        return self.down(m, out_dtype=self.ctx.dtype)
