"""Qwen2-VL's text decoder as a ModelSpec (the architecture of omniserve/model/qwen2_llm.py).

Every layer: RMSNorm -> grouped-query attention (biased q/k/v, unbiased o, M-RoPE) -> RMSNorm ->
SwiGLU, residual carried through (omniserve/model/qwen2_llm.py:137-157); final RMSNorm; head tied
to the embedding or its own.  Checkpoint names: omniserve/model/qwen2_llm.py:196-219.
"""

from __future__ import annotations

from ..config.model_config import Qwen2VLConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, ScheduleEntry


def qwen2_vl_spec(cfg: Qwen2VLConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("mrope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                  "sections": tuple(cfg.mrope_section)})
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qkv_bias": True, "out_bias": False, "window": cfg.layer_window(i)})
        layers.append(LayerSpec(prefix=f"layers.{i}.", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                                position=position))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)], final_norm=norm,
        tie_word_embeddings=cfg.tie_word_embeddings)


register_architecture("Qwen2VLForConditionalGeneration", Qwen2VLConfig.from_dict, qwen2_vl_spec)
