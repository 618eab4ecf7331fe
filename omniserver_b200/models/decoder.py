"""Runs a ModelSpec: builds the parts, tells the loader which tensors they own, tells the cache
manager what each run of a layer needs, and steps a batch of tokens through the schedule.

The forward pass follows omniserve/model/qwen2_llm.py:179-190: embed, layers with the residual
carried between them, final norm folded with the last add, head at the wanted rows only.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..parts import base as pb
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheBinding, KVCacheNeed, ParamSpec, Part, StateNeed
from ..parts.embedding import LMHead, TokenEmbedding
from .spec import ModelSpec


@dataclass
class EntryNeeds:
    """What one schedule entry asks of the cache manager."""

    kv: Optional[KVCacheNeed]
    states: List[StateNeed]
    cache_of: Optional[int]


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embed = TokenEmbedding(spec.vocab_size, spec.hidden_size, prefix=spec.embed_prefix)
        self.positions: Dict[pb.PartSpec, pb.PositionEncoding] = {}
        self.blocks: List[pb.Block] = []
        for ls in spec.layers:
            pos = None
            if ls.position is not None:
                if ls.position not in self.positions:
                    self.positions[ls.position] = POSITIONS.build(ls.position)
                pos = self.positions[ls.position]
            mixer = MIXERS.build(ls.mixer, prefix=ls.prefix + ls.mixer_prefix, position=pos)
            ffn = FEED_FORWARDS.build(ls.feed_forward, prefix=ls.prefix + ls.ffn_prefix)
            n1 = NORMS.build(ls.mixer_norm, prefix=ls.prefix + ls.mixer_norm_prefix)
            n2 = NORMS.build(ls.ffn_norm, prefix=ls.prefix + ls.ffn_norm_prefix)
            self.blocks.append(BLOCKS.build(pb.PartSpec(ls.block), mixer_norm=n1, mixer=mixer, ffn_norm=n2, ffn=ffn))
        self.final_norm = NORMS.build(spec.final_norm, prefix=spec.final_norm_prefix)
        self.head = LMHead(spec.vocab_size, spec.hidden_size,
                           tied_to=self.embed if spec.tie_word_embeddings else None, prefix=spec.head_prefix)
        for i, e in enumerate(spec.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.blocks)} layers")
            if e.cache_of is not None and not (0 <= e.cache_of < i):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
            if e.cache_of is not None and spec.schedule[e.cache_of].cache_of is not None:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which owns none")
        self.bindings: List[CacheBinding] = []
        self.shared_state: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ weights
    def parts(self) -> List[Tuple[Part, bool]]:
        """(part, name is absolute) for every part with tensors."""
        out: List[Tuple[Part, bool]] = [(self.embed, False)]
        for b in self.blocks:
            out += [(p, False) for p in b.parts()]
        out.append((self.final_norm, False))
        out.append((self.head, True))
        return out

    # ------------------------------------------------------------------ cache
    def entry_needs(self) -> List[EntryNeeds]:
        needs = []
        for e in self.spec.schedule:
            mixer = self.blocks[e.layer].mixer
            kv = None
            states: List[StateNeed] = []
            for n in mixer.cache_needs():
                if isinstance(n, KVCacheNeed):
                    if kv is not None:
                        raise ValueError("a mixer may ask for one paged key/value cache")
                    kv = n
                elif isinstance(n, StateNeed):
                    states.append(n)
                else:
                    raise TypeError(f"unknown cache need {n!r}")
            needs.append(EntryNeeds(kv, states, e.cache_of))
        return needs

    def shared_state_needs(self) -> List[StateNeed]:
        out: Dict[str, StateNeed] = {}
        for pos in self.positions.values():
            for n in pos.state_needs():
                out[n.name] = n
        return list(out.values())

    # ------------------------------------------------------------------ positions (the encodings' own business)
    @property
    def position_columns(self) -> int:
        """Rows of integers per token that requests may give with their prompts: what the model's position
        encodings take (encodings that take some must agree on how many)."""
        cols = {p.position_columns for p in self.positions.values() if p.position_columns}
        if len(cols) > 1:
            raise ValueError(f"the model's position encodings take different numbers of position columns: {sorted(cols)}")
        return cols.pop() if cols else 0

    def request_state(self, given: Optional[Any], num_prompt_tokens: int) -> Dict[str, Any]:
        """State rows (field name -> values) of a request that takes its slot, from every position encoding."""
        rows: Dict[str, Any] = {}
        for pos in self.positions.values():
            rows.update(pos.request_state(given if pos.position_columns else None, num_prompt_tokens))
        return rows

    def positions_for(self, given: Optional[Any], num_prompt_tokens: int, start: int, stop: int) -> Optional[Any]:
        """The position columns to send with tokens [start, stop) of a request, or None (see PositionEncoding)."""
        if given is None:
            return None
        out = None
        for pos in self.positions.values():
            if pos.position_columns:
                p = pos.positions_for(given, num_prompt_tokens, start, stop)
                if p is not None:
                    out = p
        return out

    def attach_cache(self, bindings: List[CacheBinding], shared_state: Dict[str, torch.Tensor]) -> None:
        if len(bindings) != len(self.spec.schedule):
            raise ValueError("one cache binding per schedule entry is needed")
        self.bindings = bindings
        self.shared_state = shared_state

    # ------------------------------------------------------------------ step
    def forward(self, ctx: Any) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns fp32 logits [R, vocab] at ctx.logit_rows."""
        ctx.bind_model(self)
        x = self.embed.forward(ctx)
        residual = None
        for i, e in enumerate(self.spec.schedule):
            x, residual = self.blocks[e.layer].forward(ctx, x, residual, self.bindings[i])
        if getattr(ctx, "advance_state", True):
            for pos in self.positions.values():
                pos.finish_step(ctx, self.shared_state)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        h = self.final_norm.forward_add_rows(x, residual, ctx.logit_rows, ctx.act_dtype)
        return self.head.forward(h)
