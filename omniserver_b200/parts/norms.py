"""Norm parts. RMSNorm with the residual add folded in, as the reference runs it
(omniserve/model/qwen2_llm.py:39-56, omniserve/kernels/fused_ops.py:21-57)."""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .. import ops
from .base import Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    """y = r / sqrt(mean(r^2) + eps) * weight with r = residual + x, statistics in fp32."""

    def __init__(self, dim: int, eps: float, prefix: str, weight_name: str = "weight"):
        self.dim = int(dim)
        self.eps = float(eps)
        self.prefix = prefix
        self._weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", (self._weight_name,), ((self.dim,),), init="ones")]

    def forward_add(self, x, residual, out_dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        return ops.kernels().add_rmsnorm(x, residual, self.weight, self.eps, out_dtype)

    def forward_add_rows(self, x, residual, rows, out_dtype) -> torch.Tensor:
        return ops.kernels().add_rmsnorm_rows(x, residual, self.weight, self.eps, rows, out_dtype)

    def rms_operands(self):
        return self.weight, self.eps

    def fused_linear(self, x, residual, linear, out_dtype):
        k = ops.kernels()
        if (out_dtype == torch.bfloat16 and k.fuse_norm_linear_decode
                and k.can_stream_linear(x, linear.weight, linear.bias, self.weight) and k.prefer_norm_inside(x)):
            return k.stream_linear(x, linear.weight, linear.bias, norm=(residual, self.weight, self.eps))
        return None


register_norm("rmsnorm", RMSNorm)
