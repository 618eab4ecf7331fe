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


@dataclass
class EngineConfig:
    """dtype: bfloat16 is the serving path; float32 runs every product and sum in true 32-bit.

    The pool holds ``max_cache_tokens`` tokens per page group (rounded up to whole pages);
    ``max_requests`` bounds the live requests (state slots).
    """

    dtype: str = "bfloat16"
    page_size: int = 16
    max_cache_tokens: int = 8192
    max_requests: int = 64
    device: str = "cuda:0"
    check_device_errors: bool = True
    cuda_graphs: bool = True          # replay pure decode steps from CUDA graphs

    @property
    def torch_dtype(self) -> torch.dtype:
        return parse_dtype(self.dtype)
