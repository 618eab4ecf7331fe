"""The engine's host logic (step function, cache manager, block tables, slot maps, state slots)
on a machine without a GPU: the kernels are replaced by their plain references from
tests/plain/kernels.py, everything else is the product's code.  The same replay families run on
the GPU in tests/test_replay_gpu.py."""

import pytest
import torch

import replay_cases as rc
from helpers import make_model_dir, plain_model
from plain import kernels as plain_kernels
from plain import model as pm


@pytest.fixture()
def cpu_kernels():
    k = plain_kernels.install()
    yield k
    plain_kernels.uninstall()


def _requests(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lens)}


def _runner(model_dir, max_tokens, page_size=16):
    from omniserver_b200 import EngineConfig, build_runner
    ec = EngineConfig(dtype="float32", page_size=page_size, max_cache_tokens=max_tokens, max_requests=8, device="cpu")
    return build_runner(model_dir=model_dir, engine_config=ec)


def _replay(runner, steps):
    from omniserver_b200.replay import TraceReplayer
    rp = TraceReplayer(runner)
    outs = {}
    for st in steps:
        lg = rp.run_step(st)
        if lg is not None:
            outs[st["step"]] = lg.clone()
        runner.cache.check_invariants()
    assert not runner.cache.requests
    assert all(p == 0 for p in runner.cache.pages_in_use())
    return outs


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_families_match_plain(name, family, tmp_path, cpu_kernels):
    d = make_model_dir(tmp_path, name)
    cfg, w = plain_model(d)
    reqs = _requests(cfg.V, [5, 17, 33, 70, 100, 41], seed=3)
    steps = {"whole": rc.whole, "tail": rc.tail_decode, "portions": rc.portions, "mixed": rc.mixed}[family](reqs)
    runner = _runner(d, rc.max_live_tokens(steps))
    got = rc.collect(steps, _replay(runner, steps))
    for rid, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        err = (got[rid] - want).abs().max().item()
        assert err < 5e-5, f"{family}/{rid}: max abs logit difference {err}"
