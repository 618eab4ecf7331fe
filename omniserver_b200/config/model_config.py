"""Typed model configuration read from a checkpoint's ``config.json``.

The reference engine never opens ``config.json``: it builds its model from a
dataclass of defaults (omniserve/model/qwen2_llm.py:25-36,
omniserve/models/qwen2_vl.py:50).  Here every size and constant comes from the
file; nothing about a particular checkpoint stands in code.  The keys are the
ones a Qwen2-VL checkpoint folder carries; the text-decoder keys may also sit
under ``text_config`` (a later layout of the same file).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine can run."""


_REQUIRED = (
    "hidden_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "intermediate_size",
    "vocab_size",
    "rms_norm_eps",
    "rope_theta",
)


@dataclass(frozen=True)
class Qwen2VLConfig:
    """Text decoder of Qwen2-VL (dense, GQA, biased q/k/v, M-RoPE, SwiGLU).

    Field meanings follow omniserve/model/qwen2_llm.py:25-36; names follow the
    keys of config.json.
    """

    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    mrope_section: Tuple[int, ...]
    tie_word_embeddings: bool
    max_position_embeddings: Optional[int] = None
    hidden_act: str = "silu"
    # window: layers with index >= max_window_layers attend to the last
    # ``sliding_window`` keys only when use_sliding_window is set.
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    image_token_id: Optional[int] = None
    vision_start_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer_idx: int) -> Optional[int]:
        """Window of keys layer ``layer_idx`` sees; None means all keys."""
        if not self.use_sliding_window or self.sliding_window is None:
            return None
        first = self.max_window_layers if self.max_window_layers is not None else 0
        return int(self.sliding_window) if layer_idx >= first else None

    # --------------------------------------------------------------- validation
    def validate(self) -> "Qwen2VLConfig":
        def need_pos(name: str) -> None:
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config: {name} must be a positive integer, got {v!r}")

        for n in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size"):
            need_pos(n)
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config: num_attention_heads ({self.num_attention_heads}) is not a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config: rms_norm_eps must be > 0, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config: rope_theta must be > 0, got {self.rope_theta!r}")
        if len(self.mrope_section) != 3 or any((not isinstance(s, int)) or s < 0 for s in self.mrope_section):
            raise ConfigError(
                f"config: rope_scaling.mrope_section must be three non-negative integers, got "
                f"{list(self.mrope_section)!r}")
        if sum(self.mrope_section) != self.head_dim // 2:
            raise ConfigError(
                f"config: sum(mrope_section)={sum(self.mrope_section)} must equal head_dim/2="
                f"{self.head_dim // 2}")
        if self.hidden_act != "silu":
            raise ConfigError(
                f"config: hidden_act {self.hidden_act!r} is not supported (the architecture's MLP is "
                f"SiLU-gated, omniserve/model/qwen2_llm.py:116-134)")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("config: use_sliding_window is set but sliding_window is not a positive integer")
        return self

    # --------------------------------------------------------------------- I/O
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2VLConfig":
        if not isinstance(d, dict):
            raise ConfigError("config.json must hold a JSON object")
        text = d.get("text_config") if isinstance(d.get("text_config"), dict) else {}

        def get(key: str, default: Any = None) -> Any:
            if key in text:
                return text[key]
            return d.get(key, default)

        archs = d.get("architectures")
        if not archs or not isinstance(archs, list):
            raise ConfigError("config: 'architectures' (a non-empty list) is missing")
        missing = [k for k in _REQUIRED if get(k) is None]
        if missing:
            raise ConfigError("config: missing required keys: " + ", ".join(missing))

        nh = get("num_attention_heads")
        hidden = get("hidden_size")
        head_dim = get("head_dim")
        if head_dim is None:
            if not isinstance(nh, int) or nh <= 0 or hidden % nh != 0:
                raise ConfigError(
                    f"config: head_dim is absent and hidden_size ({hidden}) is not a multiple of "
                    f"num_attention_heads ({nh})")
            head_dim = hidden // nh

        rope = get("rope_scaling") or get("rope_parameters") or {}
        section = rope.get("mrope_section") if isinstance(rope, dict) else None
        if section is None:
            # Plain rotary: all three axes carry the same index, so any split works;
            # give the whole band to the first axis (omniserve/models/base.py:55-56).
            section = [head_dim // 2, 0, 0]
        known = {
            "architectures", "text_config", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "vocab_size", "rms_norm_eps",
            "rope_theta", "rope_scaling", "rope_parameters", "tie_word_embeddings",
            "max_position_embeddings", "hidden_act", "use_sliding_window", "sliding_window",
            "max_window_layers", "eos_token_id", "bos_token_id", "image_token_id",
            "vision_start_token_id", "torch_dtype",
        }
        extra = {k: v for k, v in d.items() if k not in known}
        cfg = cls(
            architecture=str(archs[0]),
            hidden_size=hidden,
            num_hidden_layers=get("num_hidden_layers"),
            num_attention_heads=nh,
            num_key_value_heads=get("num_key_value_heads"),
            head_dim=head_dim,
            intermediate_size=get("intermediate_size"),
            vocab_size=get("vocab_size"),
            rms_norm_eps=float(get("rms_norm_eps")),
            rope_theta=float(get("rope_theta")),
            mrope_section=tuple(section) if isinstance(section, (list, tuple)) else (section,),
            tie_word_embeddings=bool(get("tie_word_embeddings", False)),
            max_position_embeddings=get("max_position_embeddings"),
            hidden_act=str(get("hidden_act", "silu")),
            use_sliding_window=bool(get("use_sliding_window", False)),
            sliding_window=get("sliding_window"),
            max_window_layers=get("max_window_layers"),
            eos_token_id=_first_int(get("eos_token_id")),
            bos_token_id=_first_int(get("bos_token_id")),
            image_token_id=get("image_token_id"),
            vision_start_token_id=get("vision_start_token_id"),
            torch_dtype=get("torch_dtype"),
            extra=extra,
        )
        return cfg.validate()

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen2VLConfig":
        with open(path, "r", encoding="utf-8") as f:
            try:
                d = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path}: not valid JSON ({e})") from e
        return cls.from_dict(d)

    def to_dict(self) -> Dict[str, Any]:
        """The config.json form (flat layout) of this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2_vl",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": {"type": "mrope", "mrope_section": list(self.mrope_section)},
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
        }
        for k in ("max_position_embeddings", "sliding_window", "max_window_layers", "eos_token_id",
                  "bos_token_id", "image_token_id", "vision_start_token_id", "torch_dtype"):
            v = getattr(self, k)
            if v is not None:
                d[k] = v
        return d


def _first_int(v: Any) -> Optional[int]:
    if isinstance(v, list):
        return int(v[0]) if v else None
    return None if v is None else int(v)


def read_config_dict(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
