"""Greedy and temperature sampling over the step's fp32 logits rows.

Greedy: argmax (omniserve/runners/multimodal.py:306-310).  Temperature: softmax(logits / T) and
one draw (omniserve/runners/multimodal.py:378-379); the draw here is the inverse CDF at a uniform
from ``rng.uniform``.  One kernel launch and one device-to-host copy per step for all rows.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from . import rng


class SampleHandle:
    """Tokens that are being sampled on the device; ``result()`` waits for them and returns a list."""

    def __init__(self, ids: Optional[torch.Tensor], n: int, host: Optional[torch.Tensor] = None):
        self.n = n
        self._ids = ids
        self._host = None
        self._event = None
        if ids is not None and ids.is_cuda:
            self._host = host if host is not None else torch.empty(n, dtype=torch.int32, pin_memory=True)
            self._host.copy_(ids, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()

    def result(self) -> List[int]:
        if self.n == 0:
            return []
        if self._event is not None:
            self._event.synchronize()
            return self._host.tolist()
        return self._ids.tolist()


class Sampler:
    RING, RING_WIDTH = 4, 1024

    def __init__(self, seed: int = 0):
        self.seed = int(seed)
        self._ring: Optional[torch.Tensor] = None    # pinned landing places for the tokens, used in turn
        self._turn = 0

    def _landing(self, n: int, device: torch.device) -> Optional[torch.Tensor]:
        """A pinned buffer for n tokens; a handle has to be read before RING - 1 more have been made."""
        if device.type != "cuda" or n > self.RING_WIDTH:
            return None
        if self._ring is None:
            with torch.inference_mode(False):
                self._ring = torch.empty((self.RING, self.RING_WIDTH), dtype=torch.int32, pin_memory=True)
        self._turn = (self._turn + 1) % self.RING
        return self._ring[self._turn, :n]

    def sample(self, logits: torch.Tensor, seqs: Sequence) -> List[int]:
        """One token per row of ``logits`` [R, V]; row i belongs to seqs[i]."""
        return self.sample_async(logits, seqs).result()

    def sample_async(self, logits: torch.Tensor, seqs: Optional[Sequence], keep: Optional[torch.Tensor] = None,
                     keep_at: Optional[torch.Tensor] = None) -> SampleHandle:
        """Launches the sampling of one token per row and the copy to the host; does not wait.
        ``seqs`` None: every row greedy. ``keep``/``keep_at``: row i's token is also stored at
        ``keep[keep_at[i]]`` on the device."""
        R = logits.shape[0]
        if R == 0:
            return SampleHandle(None, 0)
        if seqs is not None and R != len(seqs):
            raise ValueError("one logits row per sequence is needed")
        k = ops.kernels()
        if seqs is None or all(s.request.sampling.greedy for s in seqs):
            ids = k.sample(logits, None, None, keep, keep_at)
        else:
            temps, us = [], []
            for s in seqs:
                sp = s.request.sampling
                temps.append(float(sp.temperature))
                seed = self.seed if sp.seed is None else sp.seed
                us.append(rng.uniform(seed, s.request_id, s.num_output_tokens))
            tu = torch.tensor([temps, us], dtype=torch.float32).to(logits.device, non_blocking=True)
            ids = k.sample(logits, tu[0].contiguous(), tu[1].contiguous(), keep, keep_at)
        return SampleHandle(ids, R, self._landing(R, logits.device))
