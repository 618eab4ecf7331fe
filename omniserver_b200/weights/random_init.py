"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration
and a seed, or fills a built model in place.

The reference has no such mode (its micro-benchmarks draw torch.randn ad hoc).  Every tensor is drawn
by its checkpoint name from (seed, name), in float32 on the CPU, so the values do not depend on
the order of generation or on which other tensors exist: matrices and biases ~ N(0, std^2), norm
weights 1 + N(0, norm_noise^2).
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import torch

from ..config.registry import resolve
from ..models.decoder import DecoderModel
from .loader import expected_tensors, target_dtype

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 62) - 1)


def draw(seed: int, name: str, shape, init: str, std: float, norm_noise: float) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(tensor_seed(seed, name))
    if init == "zeros":
        return torch.zeros(shape, dtype=torch.float32)
    if init == "ones":
        t = torch.ones(shape, dtype=torch.float32)
        if norm_noise > 0:
            t += torch.randn(shape, generator=g, dtype=torch.float32) * norm_noise
        return t
    return torch.randn(shape, generator=g, dtype=torch.float32) * std


def random_state_dict(model: DecoderModel, seed: int, std: float = 0.02, norm_noise: float = 0.0,
                      store_dtype: torch.dtype = torch.bfloat16, prefix: str = "model.") -> Dict[str, torch.Tensor]:
    sd: Dict[str, torch.Tensor] = {}
    for _part, ps, full in expected_tensors(model, prefix):
        for n, shape in zip(full, ps.shapes):
            t = draw(seed, n, shape, ps.init, std, norm_noise)
            sd[n] = t.to(torch.int32) if ps.kind == "int" else t.to(store_dtype)
    return sd


def write_random_model(config: dict, seed: int, out_dir: str, store_dtype: str = "bfloat16", std: float = 0.02,
                       norm_noise: float = 0.0) -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns out_dir."""
    from safetensors.torch import save_file
    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}")
    cfg, spec = resolve(config)
    model = DecoderModel(spec)
    os.makedirs(out_dir, exist_ok=True)
    cfg_out = dict(config)
    cfg_out.setdefault("torch_dtype", store_dtype)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg_out, f, indent=2)
    sd = random_state_dict(model, seed, std, norm_noise, _STORE[store_dtype])
    save_file(sd, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return out_dir


def fill_random(model: DecoderModel, seed: int, engine_dtype: torch.dtype, device, std: float = 0.02,
                norm_noise: float = 0.0, store_dtype: torch.dtype = torch.bfloat16, on_device: bool = False) -> None:
    """Binds random tensors to a built model without a folder.

    ``on_device`` draws with the device's generator (fast for large models; the values then differ
    from the CPU draw of ``write_random_model``).
    """
    by_part = {}
    for part, ps, full in expected_tensors(model, "model."):
        dt = target_dtype(store_dtype, ps.kind, engine_dtype)
        dest = torch.empty(ps.shape, dtype=dt, device=device)
        row = 0
        for n, shape in zip(full, ps.shapes):
            if on_device:
                g = torch.Generator(device=device)
                g.manual_seed(tensor_seed(seed, n))
                if ps.init == "ones":
                    t = torch.ones(shape, dtype=torch.float32, device=device)
                    if norm_noise > 0:
                        t += torch.randn(shape, generator=g, dtype=torch.float32, device=device) * norm_noise
                elif ps.init == "zeros":
                    t = torch.zeros(shape, dtype=torch.float32, device=device)
                else:
                    t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
            else:
                t = draw(seed, n, shape, ps.init, std, norm_noise)
            t = t.to(store_dtype)  # what a folder would hold
            dest[row:row + shape[0]].copy_(t.to(dt))
            row += shape[0]
        by_part.setdefault(id(part), (part, {}))[1][ps.attr] = dest
    for part, tensors in by_part.values():
        part.bind(tensors)
