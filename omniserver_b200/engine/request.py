"""Requests and the engine's per-request state.

Names and meanings follow omniserve/request.py:21-115.  Differences: a prompt is token ids (the
tokenizer is outside the engine); a request may carry positions for its prompt, as many columns per
token as the model's position encoding takes, and rows of embeddings that replace looked-up ones (what
the reference computes from images, omniserve/runners/multimodal.py:123-127); ``top_p`` is accepted
only at 1.0, since the reference declares it and never reads it (omniserve/request.py:32,
omniserve/runners/multimodal.py:374-379).  A generated token may stand in a sequence before its value
is known on the host (``PENDING_TOKEN``), so the end of a request is decided on places filled and on
the newest known value.
"""

from __future__ import annotations

import enum
import itertools
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence as Seq

import numpy as np
import torch

_counter = itertools.count()

#: stands in ``Sequence.output_token_ids`` for a token that has been sampled on the device but not read yet
PENDING_TOKEN = -1


class Status(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"
    ABORTED = "aborted"


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 0.0      # 0 means greedy
    top_p: float = 1.0
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None    # None: the engine's seed
    ignore_eos: bool = False      # do not add the model's eos id to the stop ids

    def __post_init__(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_p != 1.0:
            raise ValueError("top_p other than 1.0 is not supported")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


@dataclass
class Request:
    """What a user submits. ``prompt`` is a list of token ids.

    ``positions``: optional int array [columns, len(prompt)], what the model's position encoding takes
    (three rows (t, h, w) for Qwen2-VL); absent means text positions.  ``embed_rows``/``embed_values``:
    prompt places whose embedding is given.
    """

    prompt: Seq[int]
    sampling: SamplingParams = field(default_factory=SamplingParams)
    request_id: str = field(default_factory=lambda: f"req-{next(_counter)}")
    arrival_t: float = field(default_factory=time.perf_counter)
    positions: Optional[np.ndarray] = None
    embed_rows: Optional[Seq[int]] = None
    embed_values: Optional[torch.Tensor] = None


@dataclass(eq=False)
class Sequence:
    """Mutable per-request state inside the engine (omniserve/request.py:50-115). A sequence is equal to itself
    only: the scheduler looks sequences up in its lists every step, and a field-by-field comparison (prompts of
    thousands of tokens) of 64 running requests cost a millisecond a step."""

    request: Request
    prompt_token_ids: List[int] = field(default_factory=list)
    output_token_ids: List[int] = field(default_factory=list)
    status: Status = Status.WAITING
    num_computed: int = 0          # tokens of prompt + outputs already in the cache
    scheduled: int = 0             # tokens the scheduler handed out for the running step
    prompt_positions: Optional[np.ndarray] = None    # what came with the prompt; the position encoding reads it
    finish_reason: Optional[str] = None              # "stop" or "length" once the request has ended by itself
    num_streamed: int = 0
    num_preemptions: int = 0
    admit_order: int = -1
    first_token_t: Optional[float] = None
    finish_t: Optional[float] = None

    def __post_init__(self) -> None:
        if not self.prompt_token_ids:
            self.prompt_token_ids = [int(t) for t in self.request.prompt]
        if not self.prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        p = self.request.positions
        if p is not None:
            p = np.asarray(p, dtype=np.int64)
            if p.ndim != 2 or p.shape[1] != len(self.prompt_token_ids):
                raise ValueError(f"positions must be [columns, {len(self.prompt_token_ids)}], got {p.shape}")
            self.prompt_positions = p

    # -- identity and sizes (omniserve/request.py:77-96)
    @property
    def request_id(self) -> str:
        return self.request.request_id

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def total_len(self) -> int:
        return self.num_prompt_tokens + self.num_output_tokens

    @property
    def num_prefilled(self) -> int:
        return min(self.num_computed, self.num_prompt_tokens)

    @property
    def remaining(self) -> int:
        """Tokens not yet in the cache (the last one yields the next token's logits)."""
        return self.total_len - self.num_computed

    @property
    def is_decoding(self) -> bool:
        return self.remaining == 1 and self.num_output_tokens > 0

    def token_at(self, i: int) -> int:
        n = self.num_prompt_tokens
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    def tokens(self, start: int, stop: int) -> List[int]:
        n = self.num_prompt_tokens
        if stop <= n:
            return self.prompt_token_ids[start:stop]
        if start >= n:
            return self.output_token_ids[start - n:stop - n]
        return self.prompt_token_ids[start:] + self.output_token_ids[:stop - n]

    def last_token_id(self) -> int:
        return self.output_token_ids[-1] if self.output_token_ids else self.prompt_token_ids[-1]

    # -- generation (the names of omniserve/request.py:98-115)
    def append_token(self, token_id: int) -> None:
        """A new place of the output: a token id, or PENDING_TOKEN while the value is still on the device."""
        if self.first_token_t is None:
            self.first_token_t = time.perf_counter()
        self.output_token_ids.append(int(token_id))

    def stop_reason(self) -> Optional[str]:
        """Why the request is over, if it is: "stop", the newest place holds a known value that is one of
        its stop ids; "length", max_new_tokens places are filled (known or pending)."""
        outs = self.output_token_ids
        sp = self.request.sampling
        if outs and outs[-1] != PENDING_TOKEN and outs[-1] in sp.stop_token_ids:
            return "stop"
        return "length" if len(outs) >= sp.max_new_tokens else None

    def maybe_finish(self) -> bool:
        why = self.stop_reason()
        if why is not None:
            self.finish_reason = why
            self.status = Status.FINISHED
            self.finish_t = time.perf_counter()
        return why is not None
