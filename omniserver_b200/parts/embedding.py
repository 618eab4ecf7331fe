"""Token embedding and the LM head.

Lookup with overwritten rows: omniserve/model/qwen2_llm.py:164, omniserve/runners/multimodal.py:123-126.
Head: logits = h W^T without bias, W the embedding table when tied (omniserve/model/qwen2_llm.py:167-168,190).
Logits come out in fp32.
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch

from .. import ops
from .base import ParamSpec, Part


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, prefix: str = "embed_tokens."):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.prefix = prefix
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weight", ("weight",), ((self.vocab_size, self.hidden_size),))]

    def forward(self, ctx: Any) -> torch.Tensor:
        k = ops.kernels()
        x = k.embed_lookup(self.weight, ctx.token_ids, ctx.act_dtype, getattr(ctx, "token_src", None),
                           getattr(ctx, "last_token", None))
        if ctx.override_rows is not None:
            k.scatter_rows(x, ctx.override_rows, ctx.override_vals)
        return x


class LMHead(Part):
    """Untied heads own ``lm_head.weight`` (outside the decoder's prefix); tied ones borrow the table."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[TokenEmbedding] = None,
                 prefix: str = "lm_head.", absolute: bool = True):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tied_to = tied_to
        self.prefix = prefix
        self.absolute_prefix = absolute  # name is not under the decoder's prefix
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        if self.tied_to is not None:
            return []
        return [ParamSpec("weight", ("weight",), ((self.vocab_size, self.hidden_size),))]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        w = self.tied_to.weight if self.tied_to is not None else self.weight
        return ops.kernels().linear(h, w, None, torch.float32)
