"""Shared test helpers: tiny model folders in temporary directories, plain-implementation oracles."""

from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from plain import model as pm
from tiny_configs import ALL


def make_model_dir(tmp_path, name: str, store_dtype: str = "float32") -> str:
    from omniserver_b200.weights import write_random_model
    config, init = ALL[name]
    d = os.path.join(str(tmp_path), f"{name}_{store_dtype}")
    if not os.path.isdir(d):
        write_random_model(config, init["seed"], d, store_dtype=store_dtype, std=init["std"],
                           norm_noise=init["norm_noise"])
    return d


def plain_model(model_dir: str, dtype=torch.float32) -> Tuple[pm.PlainConfig, Dict[str, torch.Tensor]]:
    return pm.PlainConfig.from_dir(model_dir), pm.load_weights(model_dir, dtype)
