"""Random tiny configurations of the architecture through the whole engine against the plain model: head sizes
in steps of 16, one to five kv heads with groups of one to eight, widths, intermediate sizes and vocabularies that
are no powers of two, windows, tied and untied heads, pages of 4 to 64 tokens; each with one of the replay families
(whole, tail, portions, mixed), in 32-bit and in bfloat16. The seeds are fixed: the same configurations every run."""

import os
import random

import pytest
import torch

import replay_cases as rc
from plain import model as pm
from test_replay_gpu import check

pytestmark = pytest.mark.gpu
ARCH = "Qwen2VLForConditionalGeneration"
FAMILIES = {"whole": rc.whole, "tail": rc.tail_decode, "portions": rc.portions, "mixed": rc.mixed}


def random_config(seed: int):
    rng = random.Random(seed)
    hd = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 64])
    nkv = rng.choice([1, 2, 3, 4, 5])
    nh = nkv * rng.choice([1, 2, 3, 4, 6, 7, 8])
    half = hd // 2
    a = rng.randint(1, half - 2)
    b = rng.randint(1, half - a - 1)
    window = rng.choice([None, None, 7, 20, 33])
    cfg = {"architectures": [ARCH], "model_type": "qwen2_vl",
           "hidden_size": rng.choice([64, 72, 80, 96, 128, 136, 200, 256, 384, 520]),
           "num_hidden_layers": rng.choice([1, 2, 3]), "num_attention_heads": nh, "num_key_value_heads": nkv,
           "head_dim": hd, "intermediate_size": rng.choice([64, 88, 128, 176, 200, 256, 384, 512, 640, 1000]),
           "vocab_size": rng.choice([257, 512, 777, 1000, 1531, 2048]),
           "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]), "rope_theta": rng.choice([1e4, 1e6, 5e4]),
           "rope_scaling": {"type": "mrope", "mrope_section": [a, b, half - a - b]},
           "tie_word_embeddings": rng.random() < 0.5, "hidden_act": "silu", "use_sliding_window": window is not None}
    if window is not None:
        cfg.update({"sliding_window": window, "max_window_layers": rng.choice([0, 1])})
    return cfg, rng.choice([4, 8, 16, 32, 64]), rng.choice(sorted(FAMILIES))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(100, 116))
def test_random_configuration_matches_plain(seed, dtype, tmp_path):
    from omniserver_b200 import EngineConfig, build_runner
    from omniserver_b200.replay import TraceReplayer
    from omniserver_b200.weights import write_random_model
    cfg, page_size, family = random_config(seed)
    d = os.path.join(str(tmp_path), "model")
    write_random_model(cfg, seed, d, store_dtype="float32" if dtype == "float32" else "bfloat16", std=0.03, norm_noise=0.1)
    pc, w = pm.PlainConfig.from_dir(d), pm.load_weights(d, torch.float32)
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate((5, 19, 40, 71, 100, 33))}
    steps = FAMILIES[family](reqs)
    pool = -(-rc.max_live_tokens(steps) // page_size) * page_size + page_size
    runner = build_runner(model_dir=d, engine_config=EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool,
                                                                  max_requests=8))
    runner.cache.poison_freed = True
    rp, outs = TraceReplayer(runner), {}
    with torch.inference_mode():
        for st in steps:
            lg = rp.run_step(st)
            if lg is not None:
                outs[st["step"]] = lg.float().cpu()
            runner.cache.check_invariants()
    assert not runner.cache.requests and all(p == 0 for p in runner.cache.pages_in_use())
    got = rc.collect(steps, outs)
    what = f"seed {seed}: {cfg} pages of {page_size}, {family}"
    for rid, toks in reqs.items():
        assert torch.isfinite(got[rid]).all(), what
        check(got[rid], pm.forward(pc, w, torch.tensor(toks)), dtype, f"{what} / {rid}")
