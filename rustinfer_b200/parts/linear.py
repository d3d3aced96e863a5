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
    def __init__(self, weight: torch.Tensor, num_sms: Optional[int] = None):
        if weight.dim() != 2:
            raise ValueError("a linear weight is a matrix [out, in]")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.num_sms = num_sms          # None: the kernel front asks the device
        # bf16 weights whose rows are 16-byte multiples run on this engine's tcgen05 kernel
        self.tensor_core = (self.weight.dtype == torch.bfloat16 and self.weight.is_cuda
                            and self.in_features % 8 == 0)

    def _own(self, x: torch.Tensor) -> bool:
        return self.tensor_core and x.dtype == torch.bfloat16 and x.is_contiguous() and x.data_ptr() % 16 == 0

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
        if self._own(x) and out_dtype in (torch.bfloat16, torch.float32):
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
            K.gemm_tc(x, w, out, K.EPI_BF16 if out_dtype == torch.bfloat16 else K.EPI_F32, num_sms=self.num_sms)
            return out
        if out_dtype == w.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> bool:
        """residual (fp32 [M, out]) += x W^T inside the product's epilogue; False if this
        weight cannot take that path (the caller then adds the product itself)."""
        if not self._own(x) or residual.dtype != torch.float32 or not residual.is_contiguous():
            return False
        K.gemm_tc(x, self.weight, residual, K.EPI_RESIDUAL, num_sms=self.num_sms)
        return True

    def silu_pairs(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """For a weight whose rows alternate gate_j, up_j: silu(gate) * up, [M, out/2], fused
        into the product's epilogue; None if this weight cannot take that path."""
        if not self._own(x) or self.out_features % 2:
            return None
        out = torch.empty((x.shape[0], self.out_features // 2), dtype=torch.bfloat16, device=x.device)
        K.gemm_tc(x, self.weight, out, K.EPI_SILU, num_sms=self.num_sms)
        return out
