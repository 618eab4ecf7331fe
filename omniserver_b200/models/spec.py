"""A model as data: its layers, the parts each is made of, and the order they run in."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts. ``prefix`` is the checkpoint prefix under the decoder's, e.g. "layers.3."."""

    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    position: Optional[PartSpec] = None
    block: str = "prenorm"
    mixer_prefix: str = "self_attn."
    ffn_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    ffn_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache_of``: index of the earlier schedule entry whose cache this run
    reads instead of owning (and writing) one; None means the run has a cache of its own."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embed_prefix: str = "embed_tokens."
    final_norm_prefix: str = "norm."
    head_prefix: str = "lm_head."
    #: checkpoint prefixes under which the decoder's tensors may sit (first match wins)
    decoder_prefixes: tuple = ("model.language_model.", "model.")
    #: tensors of the checkpoint that are not the decoder's and are skipped without complaint
    ignored_prefixes: tuple = ("visual.", "model.visual.")
    ignored_suffixes: tuple = ("rotary_emb.inv_freq",)
