"""Greedy and temperature sampling over the step's fp32 logits rows.

Greedy: argmax (omniserve/runners/multimodal.py:306-310).  Temperature: softmax(logits / T) and
one draw (omniserve/runners/multimodal.py:378-379); the draw here is the inverse CDF at a uniform
from ``rng.uniform``.  One kernel launch and one device-to-host copy per step for all rows.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from . import rng


class Sampler:
    def __init__(self, seed: int = 0):
        self.seed = int(seed)

    def sample(self, logits: torch.Tensor, seqs: Sequence) -> List[int]:
        """One token per row of ``logits`` [R, V]; row i belongs to seqs[i]."""
        R = logits.shape[0]
        if R == 0:
            return []
        if R != len(seqs):
            raise ValueError("one logits row per sequence is needed")
        k = ops.kernels()
        if all(s.request.sampling.greedy for s in seqs):
            ids = k.sample(logits, None, None)
        else:
            temps, us = [], []
            for s in seqs:
                sp = s.request.sampling
                temps.append(float(sp.temperature))
                seed = self.seed if sp.seed is None else sp.seed
                us.append(rng.uniform(seed, s.request_id, s.num_output_tokens))
            tu = torch.tensor([temps, us], dtype=torch.float32).to(logits.device, non_blocking=True)
            ids = k.sample(logits, tu[0].contiguous(), tu[1].contiguous())
        return ids.tolist()
