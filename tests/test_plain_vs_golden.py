"""The plain implementation against the reference's own model code.

The stored logits were produced by omniserve's Qwen2LLM on the CPU (see tests/golden/make_golden.py
for how, and for the shims it needed); the weights are regenerated here from (configuration, seed)
and verified by checksum.
"""

import os
import tempfile

import pytest
import torch
from safetensors.torch import load_file

from plain import model as pm
from tiny_configs import ALL

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = [("tiny_a_text", "tiny_a"), ("tiny_b_image", "tiny_b"), ("tiny_b_text", "tiny_b"),
         ("tiny_b_image_decode", "tiny_b")]


@pytest.mark.parametrize("case,cfg_name", CASES)
def test_plain_matches_reference_logits(case, cfg_name, tmp_path):
    from omniserver_b200.weights import write_random_model
    gold = load_file(os.path.join(GOLDEN, f"{case}.safetensors"))
    config, init = ALL[cfg_name]
    d = str(tmp_path / cfg_name)
    write_random_model(config, init["seed"], d, store_dtype="float32", std=init["std"], norm_noise=init["norm_noise"])
    sd = load_file(os.path.join(d, "model.safetensors"))
    checksum = torch.tensor([float(sd[k].double().abs().sum()) for k in sorted(sd)], dtype=torch.float64)
    assert torch.allclose(checksum, gold["weights_checksum"], rtol=1e-12, atol=0), \
        "the regenerated weights differ from the ones the golden logits were made with"
    cfg = pm.PlainConfig.from_dir(d)
    w = pm.load_weights(d)
    rows = gold["override_rows"] if len(gold["override_rows"]) else None
    logits = pm.forward(cfg, w, gold["ids"].long(), gold["positions"].long(), rows, gold["override_vals"])
    err = (logits - gold["logits"]).abs().max().item()
    assert err < 2e-5, f"max abs logit difference {err}"
    assert torch.equal(logits.argmax(-1), gold["logits"].argmax(-1))


def test_image_span_positions_match_reference_positions():
    gold = load_file(os.path.join(GOLDEN, "tiny_b_image.safetensors"))
    pos, delta = pm.image_span_positions(64, 10, 1, 4, 6)
    assert torch.equal(pos.int(), gold["positions"])
    assert delta == int(gold["rope_delta"][0]) == -18


def test_positions_after_the_prompt_match_the_reference_decode_rule():
    """The six tokens after the 64-token prompt of the golden case got their positions from the reference
    adapter's decode rule (cache index + rope_delta on all axes); the plain implementation's extension of the
    prompt's positions gives the same columns."""
    gold = load_file(os.path.join(GOLDEN, "tiny_b_image_decode.safetensors"))
    prompt_pos, delta = pm.image_span_positions(64, 10, 1, 4, 6)
    assert delta == int(gold["rope_delta"][0])
    assert gold["positions"].shape == (3, 70)
    assert torch.equal(pm.extend_positions(prompt_pos, delta, 70).int(), gold["positions"])
    assert torch.equal(gold["positions"][:, 64:], (torch.arange(64, 70) + delta).int().expand(3, 6))
