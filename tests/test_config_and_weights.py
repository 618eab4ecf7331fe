"""Configuration parsing and validation, the registry, and the weight loader's errors."""

import copy
import json
import os

import pytest
import torch

from tiny_configs import ALL, TINY_A, TINY_B, TINY_C


def test_config_reads_every_size_from_json():
    from omniserver_b200.config import resolve
    for name, (cfg_dict, _) in ALL.items():
        cfg, spec = resolve(cfg_dict)
        assert cfg.hidden_size == cfg_dict["hidden_size"]
        assert cfg.num_hidden_layers == cfg_dict["num_hidden_layers"] == len(spec.layers) == len(spec.schedule)
        assert cfg.head_dim == cfg_dict["head_dim"]
        assert tuple(cfg.mrope_section) == tuple(cfg_dict["rope_scaling"]["mrope_section"])
        assert cfg.rms_norm_eps == cfg_dict["rms_norm_eps"] and cfg.rope_theta == cfg_dict["rope_theta"]
        assert spec.tie_word_embeddings == cfg_dict["tie_word_embeddings"]
    cfg, spec = resolve(TINY_C)
    assert [cfg.layer_window(i) for i in range(4)] == [None, 20, 20, 20]
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 20, 20, 20]


def test_config_text_config_layout_and_head_dim_default():
    from omniserver_b200.config import resolve
    d = {k: v for k, v in TINY_A.items() if k in ("architectures", "tie_word_embeddings")}
    d["text_config"] = {k: v for k, v in TINY_A.items() if k not in d and k != "head_dim"}
    cfg, _ = resolve(d)
    assert cfg.head_dim == 64 // 4 and cfg.intermediate_size == 128


@pytest.mark.parametrize("patch,match", [
    ({"architectures": ["LlamaForCausalLM"]}, "unknown architecture"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"rope_scaling": {"type": "mrope", "mrope_section": [2, 3, 4]}}, "sum"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"hidden_size": None}, "missing required keys: hidden_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"head_dim": 15}, "head_dim"),
])
def test_config_errors(patch, match):
    from omniserver_b200.config import ConfigError, resolve
    d = copy.deepcopy(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=match):
        resolve(d)


def test_registry_lists_known_names():
    from omniserver_b200.config import known_architectures
    assert known_architectures() == ["Qwen2VLForConditionalGeneration"]


def _folder(tmp_path, cfg=TINY_B, **kw):
    from omniserver_b200.weights import write_random_model
    return write_random_model(cfg, 1, str(tmp_path / "m"), **kw)


def _rewrite(d, fn):
    from safetensors.torch import load_file, save_file
    p = os.path.join(d, "model.safetensors")
    sd = load_file(p)
    fn(sd)
    save_file(sd, p)


def _load(d, dtype=torch.float32):
    from omniserver_b200.config import resolve_dir
    from omniserver_b200.models import DecoderModel
    from omniserver_b200.weights import load_weights
    _, spec = resolve_dir(d)
    m = DecoderModel(spec)
    return m, load_weights(m, d, dtype, "cpu")


def test_random_folder_loads_and_is_reproducible(tmp_path):
    from safetensors.torch import load_file
    d = _folder(tmp_path, store_dtype="bfloat16")
    m, kept = _load(d, torch.bfloat16)
    assert set(kept.values()) == {torch.bfloat16}
    attn = m.blocks[0].mixer
    assert attn.qkv.weight.shape == (3 * 32 + 2 * 32, 96) and attn.qkv.bias.shape == (160,)
    sd = load_file(os.path.join(d, "model.safetensors"))
    assert torch.equal(attn.qkv.weight[96:128], sd["model.layers.0.self_attn.k_proj.weight"])
    assert torch.equal(m.blocks[2].ffn.gate_up.weight[200:], sd["model.layers.2.mlp.up_proj.weight"])
    assert torch.equal(m.head.weight, sd["lm_head.weight"])
    d2 = _folder(tmp_path / "again", store_dtype="bfloat16")
    sd2 = load_file(os.path.join(d2, "model.safetensors"))
    assert all(torch.equal(sd[k], sd2[k]) for k in sd)


def test_dtype_rules(tmp_path):
    d = _folder(tmp_path, store_dtype="bfloat16")
    _rewrite(d, lambda sd: sd.update({"model.norm.weight": sd["model.norm.weight"].float()}))
    m, kept = _load(d, torch.bfloat16)
    assert kept["model.norm.weight"] == torch.float32            # stored in 32-bit: stays so
    assert kept["model.layers.0.mlp.down_proj.weight"] == torch.bfloat16
    m, kept = _load(d, torch.float32)
    assert set(kept.values()) == {torch.float32}


def test_language_model_prefix_and_ignored_tensors(tmp_path):
    d = _folder(tmp_path)

    def rename(sd):
        for k in list(sd):
            if k.startswith("model."):
                sd["model.language_model." + k[len("model."):]] = sd.pop(k)
        sd["visual.blocks.0.attn.qkv.weight"] = torch.zeros(3, 3)
    _rewrite(d, rename)
    _load(d)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from omniserver_b200.weights import WeightsError
    d = _folder(tmp_path)

    def damage(sd):
        del sd["model.layers.1.input_layernorm.weight"]
        del sd["model.layers.0.self_attn.k_proj.bias"]
        sd["model.layers.0.self_attn.rotary.extra"] = torch.zeros(2)
        sd["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 199)
    _rewrite(d, damage)
    with pytest.raises(WeightsError) as ei:
        _load(d)
    e = ei.value
    assert e.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.input_layernorm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary.extra"]
    assert e.wrong_shape == [("model.layers.2.mlp.down_proj.weight", (96, 199), (96, 200))]
    msg = str(e)
    for s in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "file has [96, 199], model needs [96, 200]"):
        assert s in msg


def test_untied_head_is_required_and_tied_head_is_not(tmp_path):
    from omniserver_b200.weights import WeightsError
    d = _folder(tmp_path)
    _rewrite(d, lambda sd: sd.pop("lm_head.weight"))
    with pytest.raises(WeightsError, match="lm_head.weight"):
        _load(d)
    d2 = _folder(tmp_path / "tied", cfg=TINY_A)
    m, _ = _load(d2)
    assert m.head.tied_to is m.embed


def test_no_safetensors_file(tmp_path):
    from omniserver_b200.weights import WeightsError
    os.makedirs(tmp_path / "empty")
    with open(tmp_path / "empty" / "config.json", "w") as f:
        json.dump(TINY_A, f)
    with pytest.raises(WeightsError, match="no model\\*.safetensors"):
        _load(str(tmp_path / "empty"))
