"""Blocks: how a layer arranges its norms, mixer and feed-forward.

PreNormBlock is the reference's DecoderLayer (omniserve/model/qwen2_llm.py:137-157): the
residual stream is carried between layers and each add is folded into the next norm;
there is no explicit x = x + f(x).
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import torch

from .base import Block, CacheBinding, FeedForward, Mixer, Norm, Part, register_block


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def forward(self, ctx: Any, x: torch.Tensor, residual: Optional[torch.Tensor], binding: CacheBinding
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        # each norm is handed to the part behind it, which may take it into its first projection's kernel
        a, residual = self.mixer.forward_prenorm(ctx, x, residual, self.mixer_norm, binding)
        m, residual = self.ffn.forward_prenorm(ctx, a, residual, self.ffn_norm)
        return m, residual


register_block("prenorm", PreNormBlock)
