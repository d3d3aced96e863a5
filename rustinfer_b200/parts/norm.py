"""RMSNorm fused with the residual add: y = x * w / sqrt(mean(x^2) + eps), the weight
multiplying directly (crates/infer-worker/src/components/norm.rs:10-27,
crates/infer-backend-cuda/src/kernels/rmsnorm/rmsnorm.cu:52-113).  Sum of squares, the
scale and the residual sum are fp32."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels as K
from .base import Norm, ParamDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.size,), init="ones")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def add_norm(self, h, delta, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=h.device)
        K.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out
