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


def test_decode_plan_equals_general_plan(tmp_path, cpu_kernels):
    """The vectorised plan of a pure decode step lays out the same metadata as the general one,
    also right at a page boundary (where a request needs a new page)."""
    import numpy as np
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_c")
    runner = _runner(d, 512)
    lens = {"a": 15, "b": 16, "c": 40, "d": 1}
    for rid, n in lens.items():
        runner.start_request(rid)
        runner.step([StepEntry(rid, list(range(1, n + 1)), [])])
    entries = [StepEntry(r, [7 + i], [0]) for i, r in enumerate(lens)]

    def undo(snapshot):
        for r, (tables, first_live) in snapshot.items():
            rc = runner.cache.requests[r]
            rc.reserved = 0
            for g, t in enumerate(tables):
                while len(rc.tables[g]) > len(t):
                    page = rc.tables[g][len(rc.tables[g]) - 1]
                    rc.tables[g]._n -= 1
                    if page >= 0:
                        runner.cache.groups[g].pool.free(page)
            rc.first_live = list(first_live)

    snap = {r: ([list(t) for t in runner.cache.requests[r].tables], list(runner.cache.requests[r].first_live)) for r in lens}
    p1 = runner._plan(entries, bt_round=4)
    undo(snap)
    p2 = runner._plan_decode(entries, bt_round=4)
    undo(snap)
    assert [n for n, _ in p1["segs"]] == [n for n, _ in p2["segs"]]
    for (n1, a1), (n2, a2) in zip(p1["segs"], p2["segs"]):
        assert np.array_equal(np.asarray(a1), np.asarray(a2)), n1
    for k in ("S", "T", "q_lens", "kv_lens", "bt_widths", "n_logit_rows", "n_decode"):
        assert p1[k] == p2[k], k
    runner.cache.check_invariants()


def _engine(model_dir, overlap, max_tokens=1024, page_size=16, **sched):
    from omniserver_b200 import LLMEngine, SchedulerConfig
    return LLMEngine(_runner(model_dir, max_tokens, page_size), SchedulerConfig(**sched), seed=5, overlap=overlap)


def _greedy_by_plain(cfg, w, prompt, n, stop=()):
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(pm.forward(cfg, w, torch.tensor(toks))[-1].argmax())
        toks.append(nxt)
        out.append(nxt)
        if nxt in stop:
            break
    return out


@pytest.mark.parametrize("name", ["tiny_a", "tiny_c"])
def test_overlapped_steps_give_the_same_tokens(name, tmp_path, cpu_kernels):
    """Launching step t+1 before the tokens of step t are read (they stay on the device for the
    embedding lookup) changes nothing: same tokens as step-by-step, as the plain model's greedy
    decoding, with requests that end at different lengths and others that arrive meanwhile."""
    from omniserver_b200 import Request, SamplingParams
    d = make_model_dir(tmp_path, name)
    cfg, w = plain_model(d)
    prompts = list(_requests(cfg.V, [9, 21, 4, 30], seed=8).values())
    lens = [12, 5, 9, 7]
    outs = {}
    for overlap in (False, True):
        eng = _engine(d, overlap, max_running=3, max_prefill_tokens=16)
        ids = [eng.add_request(Request(prompt=p, sampling=SamplingParams(max_new_tokens=n), request_id=f"q{i}"))
               for i, (p, n) in enumerate(zip(prompts[:3], lens))]
        got = {i: [] for i in ids}
        steps = 0
        while eng.has_unfinished():
            for dl in eng.step():
                got[dl.request_id] += dl.new_token_ids
            steps += 1
            if steps == 6:      # a late arrival: the engine leaves the overlapped mode to admit it
                ids.append(eng.add_request(Request(prompt=prompts[3], sampling=SamplingParams(max_new_tokens=lens[3]),
                                                   request_id="q3")))
                got["q3"] = []
            eng.runner.cache.check_invariants()
        assert all(p == 0 for p in eng.runner.cache.pages_in_use())
        assert all(-1 not in s.output_token_ids for s in eng.sequences())
        assert (eng.counters["overlapped_steps"] > 3) == overlap
        outs[overlap] = got
    assert outs[True] == outs[False]
    for i, (p, n) in enumerate(zip(prompts, lens)):
        assert outs[True][f"q{i}"] == _greedy_by_plain(cfg, w, p, n), f"request {i}"


def test_overlapped_steps_and_stop_tokens(tmp_path, cpu_kernels):
    """A stop token is seen one step late in the overlapped mode: the token computed meanwhile is
    dropped, the outputs end with the stop token, and the pages come back."""
    from omniserver_b200 import Request, SamplingParams
    d = make_model_dir(tmp_path, "tiny_b")
    cfg, w = plain_model(d)
    prompts = list(_requests(cfg.V, [7, 13], seed=2).values())
    free_run = [_greedy_by_plain(cfg, w, p, 10) for p in prompts]
    stops = [[free_run[0][3]], [free_run[1][6]]]           # the 4th and the 7th token end their requests
    want = [_greedy_by_plain(cfg, w, p, 10, stop=s) for p, s in zip(prompts, stops)]
    for overlap in (False, True):
        eng = _engine(d, overlap)
        ids = [eng.add_request(Request(prompt=p, sampling=SamplingParams(max_new_tokens=10, stop_token_ids=list(s))))
               for p, s in zip(prompts, stops)]
        outs = eng.run_until_complete()
        assert [outs[i] for i in ids] == want
        assert [s.output_token_ids for s in eng.sequences()] == want
        assert all(p == 0 for p in eng.runner.cache.pages_in_use())
