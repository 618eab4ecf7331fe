"""Position encodings.

MRope: rotary encoding whose frequency bands are driven by three position axes
(t, h, w).  Angles: omniserve/model/qwen2_llm.py:169-177; which axis drives which band:
omniserve/model/qwen2_llm.py:64-69 (the section list doubled, band i -> axis i mod 3).
Prompt positions are given with the request (omniserve/model/positions.py:17-58 builds
them for images); a token without given positions sits at cursor + rope_delta on all
axes (omniserve/models/qwen2_vl.py:108-112), both kept in the request's state slot.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .base import PositionEncoding, RotaryOperands, StateNeed, register_position_encoding

ROPE_STATE = "rope_cursor"  # per-request state row: (cursor, rope_delta), int32


class MRope(PositionEncoding):
    position_columns = 3    # (t, h, w)

    def __init__(self, head_dim: int, theta: float, sections: Sequence[int], rot_dim: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rot_dim = int(rot_dim) if rot_dim is not None else self.head_dim
        self.theta = float(theta)
        self.sections = tuple(int(s) for s in sections)
        half = self.rot_dim // 2
        if self.rot_dim % 2 or self.rot_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rot_dim} must be even and at most head_dim {self.head_dim}")
        if sum(self.sections) != half or len(self.sections) != 3:
            raise ValueError(f"mrope sections {self.sections} must be three numbers summing to {half}")
        # inv_freq[j] = theta^(-2j/rot), computed in float32 as the reference does
        self._inv_freq_cpu = 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2).float() / self.rot_dim))
        axis: List[int] = []
        for a, n in enumerate(self.sections):
            axis += [a] * n
        self._axis_cpu = torch.tensor(axis, dtype=torch.int32)
        self._dev: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}

    def key(self) -> Tuple:
        return ("mrope", self.head_dim, self.rot_dim, self.theta, self.sections)

    def state_needs(self) -> List[StateNeed]:
        return [StateNeed(ROPE_STATE, (2,), torch.int32, shared=True)]

    def _consts(self, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
        k = str(device)
        if k not in self._dev:
            self._dev[k] = (self._inv_freq_cpu.to(device), self._axis_cpu.to(device))
        return self._dev[k]

    @staticmethod
    def rope_delta(given: Optional[Any], num_prompt_tokens: int) -> int:
        """The next text position is max + 1 (omniserve/model/positions.py:57): the offset between a
        token's index in the request and its position once the prompt is over."""
        return 0 if given is None else int(np.asarray(given).max()) + 1 - int(num_prompt_tokens)

    def request_state(self, given: Optional[Any], num_prompt_tokens: int) -> Dict[str, Sequence[int]]:
        return {ROPE_STATE: [0, self.rope_delta(given, num_prompt_tokens)]}

    def positions_for(self, given: Optional[Any], num_prompt_tokens: int, start: int, stop: int) -> Optional[Any]:
        # tokens after the prompt sit at index + rope_delta on all axes (omniserve/models/qwen2_vl.py:108-112);
        # the kernel finds that from the state row, so columns are sent only for spans that touch the prompt
        n = int(num_prompt_tokens)
        if given is None or start >= n:
            return None
        given = np.asarray(given)
        head = given[:, start:min(stop, n)]
        if stop <= n:
            return head
        tail = np.arange(n, stop, dtype=np.int64) + self.rope_delta(given, n)
        return np.concatenate([head, np.broadcast_to(tail, (3, stop - n))], axis=1)

    def prepare(self, ctx: Any, state: Dict[str, torch.Tensor]) -> RotaryOperands:
        inv_freq, axis_of = self._consts(ctx.device)
        cos, sin = ops.kernels().rope_tables(ctx.positions, ctx.pos_mode, ctx.tok_seq, ctx.cu_q, ctx.state_slot,
                                             state[ROPE_STATE], inv_freq, axis_of)
        return RotaryOperands(cos, sin, self.rot_dim)

    def rotary(self, tables: RotaryOperands) -> RotaryOperands:
        return tables

    def finish_step(self, ctx: Any, state: Dict[str, torch.Tensor]) -> None:
        ops.kernels().advance_cursor(state[ROPE_STATE], ctx.state_slot, ctx.cu_q)


register_position_encoding("mrope", MRope)
