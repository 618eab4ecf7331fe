"""Makes the golden outputs of the reference's own model code for two tiny random models.

    python tests/golden/make_golden.py --reference /path/to/omniserve-checkout

It imports ``omniserve.model.qwen2_llm`` and ``omniserve.model.positions`` from the given
checkout and runs ``Qwen2LLM`` whole-prompt, in float32, on the CPU.  The reference's forward
cannot run on a CPU as it is: its norm and activation wrappers launch Triton kernels, and its MLP
casts to fp16.  So this script replaces ``omniserve.kernels.fused_ops.{rms_norm, add_rms_norm,
silu_mul}`` by plain-torch restatements of those kernels' formulas (fused_ops.py:21-29, 43-57,
111-119) and sets ``down_proj.forward_prequant`` so that the fp16 cast (qwen2_llm.py:132-133) is
skipped.  Attention runs through the reference's own SDPA path with a causal mask
(qwen2_llm.py:105-112), positions through its own ``mrope_position_ids``.

The weights are drawn by this repository's random-weights mode from (configuration, seed); the
golden file keeps a checksum of them, the inputs and the reference's logits.  The test
``tests/test_plain_vs_golden.py`` regenerates the weights, checks the checksum and compares the
plain implementation with the stored logits.  Nothing of the reference is stored besides its outputs.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tiny_configs import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT  # noqa: E402


def shim_reference():
    import omniserve.kernels.fused_ops as fo

    def rms_norm(x, w, eps):
        xf = x.float()
        rstd = 1.0 / torch.sqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
        return (xf * rstd * w.float()).to(x.dtype)

    def add_rms_norm(x, residual, w, eps):
        r = (residual.float() + x.float()).to(residual.dtype)
        return rms_norm(r, w, eps), r

    def silu_mul(gu):
        n = gu.shape[-1] // 2
        g, u = gu[..., :n].float(), gu[..., n:].float()
        return ((g * torch.sigmoid(g)) * u).to(gu.dtype)

    fo.rms_norm, fo.add_rms_norm, fo.silu_mul = rms_norm, add_rms_norm, silu_mul


def weights_checksum(sd):
    return torch.tensor([float(sd[k].double().abs().sum()) for k in sorted(sd)], dtype=torch.float64)


def run_case(name, config, init, ids, grid, out_dir, decode_tail=0):
    """``decode_tail``: the last so many ids are tokens after the prompt; their positions come from the
    reference adapter's own decode rule (omniserve/models/qwen2_vl.py:108-112) at cache indices L .. L+tail-1."""
    from omniserve.model.positions import mrope_position_ids
    from omniserve.model.qwen2_llm import Qwen2Config, Qwen2LLM, load_from_hf
    from safetensors.torch import load_file, save_file

    from omniserver_b200.weights import write_random_model

    with tempfile.TemporaryDirectory() as d:
        write_random_model(config, init["seed"], d, store_dtype="float32", std=init["std"],
                           norm_noise=init["norm_noise"])
        sd = load_file(os.path.join(d, "model.safetensors"))
    rc = Qwen2Config(hidden_size=config["hidden_size"], num_layers=config["num_hidden_layers"],
                     num_heads=config["num_attention_heads"], num_kv_heads=config["num_key_value_heads"],
                     head_dim=config["head_dim"], intermediate_size=config["intermediate_size"],
                     vocab_size=config["vocab_size"], rms_norm_eps=config["rms_norm_eps"],
                     rope_theta=config["rope_theta"], mrope_section=config["rope_scaling"]["mrope_section"])
    m = Qwen2LLM(rc).float().eval()
    load_from_hf(m, sd)
    if not config["tie_word_embeddings"]:
        m.lm_head.weight = torch.nn.Parameter(sd["lm_head.weight"].clone())
    for layer in m.layers:
        layer.mlp.down_proj.forward_prequant = None  # skips the fp16 cast, never called

    tail_ids = ids[ids.shape[0] - decode_tail:] if decode_tail else ids[:0]
    ids = ids[:ids.shape[0] - decode_tail]
    L = ids.shape[0]
    override_rows = torch.zeros(0, dtype=torch.int32)
    override_vals = torch.zeros(0, config["hidden_size"])
    if grid is None:
        pos = torch.arange(L).view(1, 1, -1).expand(3, 1, -1)
        delta = 0
    else:
        pos, deltas = mrope_position_ids(ids[None], torch.tensor([grid]), image_token_id=config["image_token_id"],
                                         vision_start_token_id=config["vision_start_token_id"])
        delta = int(deltas.flatten()[0])
        override_rows = (ids == config["image_token_id"]).nonzero().flatten().to(torch.int32)
        g = torch.Generator().manual_seed(1234)
        override_vals = torch.randn(len(override_rows), config["hidden_size"], generator=g)
    if decode_tail:
        from omniserve.models.qwen2_vl import Qwen2VLAdapter
        # the adapter's method reads nothing of the adapter: called unbound, one "slot" per decoded token
        tail_pos = Qwen2VLAdapter.decode_positions(None, torch.arange(L, L + decode_tail),
                                                   torch.full((decode_tail,), delta))       # [3, tail, 1]
        pos = torch.cat([pos, tail_pos.reshape(3, 1, decode_tail)], dim=2)
        ids = torch.cat([ids, tail_ids])
        L = ids.shape[0]
    with torch.no_grad():
        emb = m.embed_tokens(ids[None]).clone()
        if len(override_rows):
            emb[0, override_rows.long()] = override_vals
        mask = torch.full((L, L), float("-inf")).triu(1)
        logits = m(emb, pos, mask, None)[0]
    save_file({
        "ids": ids.to(torch.int32), "positions": pos[:, 0, :].to(torch.int32).contiguous(),
        "rope_delta": torch.tensor([delta], dtype=torch.int32), "override_rows": override_rows,
        "override_vals": override_vals, "logits": logits.float().contiguous(),
        "weights_checksum": weights_checksum(sd),
    }, os.path.join(out_dir, f"{name}.safetensors"))
    print(f"{name}: L={L} delta={delta} logits {tuple(logits.shape)} max|logit| {float(logits.abs().max()):.4f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of an omniserve checkout (holds omniserve/)")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    shim_reference()
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(7)
    # A: text only, 33 tokens
    ids_a = torch.randint(0, 499, (33,), generator=g)
    run_case("tiny_a_text", TINY_A, TINY_A_INIT, ids_a, None, args.out)
    # B: 64 tokens with a 24-token image span (grid 1 x 8 x 12 merged by 2 -> 4 x 6) after 9 text tokens
    ids_b = torch.randint(0, 989, (64,), generator=g)
    ids_b[9] = TINY_B["vision_start_token_id"]
    ids_b[10:34] = TINY_B["image_token_id"]
    run_case("tiny_b_image", TINY_B, TINY_B_INIT, ids_b, (1, 8, 12), args.out)
    # B text only too (untied head, 1 kv head)
    ids_b2 = torch.randint(0, 989, (40,), generator=g)
    run_case("tiny_b_text", TINY_B, TINY_B_INIT, ids_b2, None, args.out)
    # B with the image span, followed by 6 tokens placed by the reference's decode rule (cursor + rope_delta)
    ids_b3 = torch.cat([ids_b, torch.randint(0, 989, (6,), generator=g)])
    run_case("tiny_b_image_decode", TINY_B, TINY_B_INIT, ids_b3, (1, 8, 12), args.out, decode_tail=6)


if __name__ == "__main__":
    main()
