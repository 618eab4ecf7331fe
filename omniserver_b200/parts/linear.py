"""Dense projection y = x W^T (+ b): the product kernels are chosen by operand type and row count."""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops
from .base import ParamSpec


class Linear:
    """A weight [N, K] (+ optional bias [N]) possibly concatenated from several checkpoint tensors."""

    def __init__(self, attr: str, in_features: int, out_features: Sequence[int], sources: Sequence[str],
                 bias: bool = False):
        self.attr = attr
        self.in_features = int(in_features)
        self.out_splits = tuple(int(o) for o in out_features)
        self.sources = tuple(sources)
        self.has_bias = bool(bias)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.attr + "_weight", tuple(s + ".weight" for s in self.sources),
                           tuple((o, self.in_features) for o in self.out_splits))]
        if self.has_bias:
            specs.append(ParamSpec(self.attr + "_bias", tuple(s + ".bias" for s in self.sources),
                                   tuple((o,) for o in self.out_splits)))
        return specs

    def bind(self, tensors) -> None:
        self.weight = tensors[self.attr + "_weight"]
        if self.has_bias:
            self.bias = tensors[self.attr + "_bias"]

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.kernels().linear(x, self.weight, self.bias, out_dtype)
