"""Feed-forward parts. SwiGLU: down( silu(gate(x)) * up(x) ), no biases
(omniserve/model/qwen2_llm.py:116-134; gate and up fused into one product, gate first,
omniserve/model/qwen2_llm.py:215-216)."""

from __future__ import annotations

from typing import Any, List

import torch

from .. import ops
from .base import FeedForward, ParamSpec, register_feed_forward
from .linear import Linear


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.prefix = prefix
        self.gate_up = Linear("gate_up", hidden_size, (intermediate_size, intermediate_size), ("gate_proj", "up_proj"))
        self.down = Linear("down", intermediate_size, (hidden_size,), ("down_proj",))

    def param_specs(self) -> List[ParamSpec]:
        return self.gate_up.param_specs() + self.down.param_specs()

    def bind(self, tensors) -> None:
        self.gate_up.bind(tensors)
        self.down.bind(tensors)

    def forward(self, ctx: Any, x: torch.Tensor) -> torch.Tensor:
        m = ops.kernels().gate_up_silu(x, self.gate_up.weight, ctx.act_dtype)
        return self.down(m, ctx.act_dtype)

    def forward_prenorm(self, ctx: Any, x: torch.Tensor, residual, norm):
        # a few rows (a decode step): norm, both projections and the activation as one kernel, if the
        # norm is one that the kernel computes and the rows are few and short enough for that form to be the faster
        k = ops.kernels()
        rms = norm.rms_operands()
        if (rms is not None and k.can_stream_ffn(x, rms[0], self.gate_up.weight, self.down.weight)
                and k.prefer_stream_ffn(x, self.gate_up.weight)):
            return k.stream_ffn(x, residual, rms[0], rms[1], self.gate_up.weight, self.down.weight)
        return super().forward_prenorm(ctx, x, residual, norm)


register_feed_forward("swiglu", SwiGLU)
