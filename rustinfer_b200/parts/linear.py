"""y = x W^T with W stored [out, in], no bias
(crates/infer-worker/src/components/linear.rs:14-34,172-212, dense variant only).

bf16 weights go through the library matrix product, as RustInfer's bf16 GEMMs go through
cuBLASLt (crates/infer-backend-cuda/src/kernels/matmul/matmul.cu:131-650), with fp32
accumulation.  fp32 weights go through this engine's exact fp32 kernel; a weight the file
stores in 32-bit keeps that precision even in a bfloat16 engine.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels as K


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x [M, in] -> [M, out] in `out_dtype` (default: x's dtype)."""
        out_dtype = out_dtype or x.dtype
        w = self.weight
        if w.dtype == torch.float32:
            xf = x if x.dtype == torch.float32 else x.float()
            if xf.stride(-1) != 1:
                xf = xf.contiguous()
            out = torch.empty((x.shape[0], self.out_features), dtype=torch.float32, device=x.device)
            K.gemm_f32(xf, w, out)
            return out if out_dtype == torch.float32 else out.to(out_dtype)
        if x.dtype != w.dtype:
            x = x.to(w.dtype)
        if out_dtype == w.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
