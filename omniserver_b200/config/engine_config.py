"""Engine-side settings (not read from the checkpoint)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {name!r}") from None


# Tokens per cache page. The prefill attention fetches a 128-key tile page by page with TMA boxes, at about 56 cycles a
# box and head-size atom: with 16-token pages the boxes of a tile's keys and values (32) take longer than its arithmetic;
# from 32 tokens on they do not (2,048-token prompt: 26.4 us with pages of 16, 23.6 with 32, 23.5 with 64), and decode
# steps time the same.
DEFAULT_PAGE_SIZE = 32


@dataclass
class EngineConfig:
    """dtype: bfloat16 is the serving path; float32 runs every product and sum in true 32-bit.

    The pool holds ``max_cache_tokens`` tokens per page group (rounded up to whole pages);
    ``max_requests`` bounds the live requests (state slots).
    """

    dtype: str = "bfloat16"
    page_size: int = DEFAULT_PAGE_SIZE
    max_cache_tokens: int = 8192
    max_requests: int = 64
    device: str = "cuda:0"
    check_device_errors: bool = True
    cuda_graphs: bool = True          # replay pure decode steps from CUDA graphs

    @property
    def torch_dtype(self) -> torch.dtype:
        return parse_dtype(self.dtype)
