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


def test_a_bad_entry_leaves_the_cache_as_it_was(tmp_path, cpu_kernels):
    """A step with one bad entry (a token id outside the vocabulary, a wanted place outside the entry, positions
    of the wrong shape, an unknown request) raises before any page is taken: nothing stays reserved for the
    other requests of the batch, no page is lost, and the same requests step normally afterwards."""
    import numpy as np
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_a")
    cfg, w = plain_model(d)
    runner = _runner(d, 256)
    toks = _requests(cfg.V, [30, 20], seed=4)
    for rid in toks:
        runner.start_request(rid)
    runner.step([StepEntry("r0", toks["r0"][:10], []), StepEntry("r1", toks["r1"][:5], [])])
    held = runner.cache.pages_in_use()
    bad_steps = [
        [StepEntry("r0", toks["r0"][10:28], [0]), StepEntry("r1", [3, cfg.V, 5], [0])],
        [StepEntry("r0", toks["r0"][10:28], [0]), StepEntry("r1", [3, 4], [2])],
        [StepEntry("r0", toks["r0"][10:28], [0]), StepEntry("r1", [3, 4], [0], positions=np.zeros((2, 2), dtype=np.int64))],
    ]
    for entries in bad_steps:
        with pytest.raises(ValueError):
            runner.step(entries)
        runner.cache.check_invariants()
        assert all(rc.reserved == 0 for rc in runner.cache.requests.values())
        assert runner.cache.pages_in_use() == held
    with pytest.raises(KeyError):
        runner.step([StepEntry("r0", toks["r0"][10:28], [0]), StepEntry("nobody", [1], [0])])
    assert all(rc.reserved == 0 for rc in runner.cache.requests.values()) and runner.cache.pages_in_use() == held
    # the requests go on as if nothing had happened
    a = runner.step([StepEntry("r0", toks["r0"][10:], list(range(20))), StepEntry("r1", toks["r1"][5:], list(range(15)))])
    want0, want1 = pm.forward(cfg, w, torch.tensor(toks["r0"])), pm.forward(cfg, w, torch.tensor(toks["r1"]))
    assert (a[:20] - want0[10:]).abs().max() < 5e-5 and (a[20:] - want1[5:]).abs().max() < 5e-5


def test_a_step_that_fails_after_planning_gives_its_pages_back(tmp_path, cpu_kernels, monkeypatch):
    """When the forward pass itself raises, the pages the step took beyond the requests' cursors go back to the
    pool and nothing stays reserved."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_c")      # a window: tables with pages already given back
    cfg, _ = plain_model(d)
    runner = _runner(d, 512)
    toks = _requests(cfg.V, [90, 40], seed=6)
    for rid in toks:
        runner.start_request(rid)
    runner.step([StepEntry("r0", toks["r0"][:50], []), StepEntry("r1", toks["r1"][:7], [])])
    held = runner.cache.pages_in_use()
    tables = {r: [list(t) for t in rc.tables] for r, rc in runner.cache.requests.items()}

    def boom(ctx):
        raise RuntimeError("forward failed")
    monkeypatch.setattr(runner.model, "forward", boom)
    with pytest.raises(RuntimeError, match="forward failed"):
        runner.step([StepEntry("r0", toks["r0"][50:], [0]), StepEntry("r1", toks["r1"][7:], [0])])
    monkeypatch.undo()
    runner.cache.check_invariants()
    assert runner.cache.pages_in_use() == held
    assert {r: [list(t) for t in rc.tables] for r, rc in runner.cache.requests.items()} == tables
    assert all(rc.reserved == 0 for rc in runner.cache.requests.values())


def test_token_ids_and_positions_are_checked_when_a_request_is_added(tmp_path, cpu_kernels):
    import numpy as np
    from omniserver_b200 import Request
    d = make_model_dir(tmp_path, "tiny_a")
    cfg, _ = plain_model(d)
    eng = _engine(d, False)
    with pytest.raises(ValueError, match="token id"):
        eng.add_request(Request(prompt=[1, 2, cfg.V]))
    with pytest.raises(ValueError, match="positions"):
        eng.add_request(Request(prompt=[1, 2, 3], positions=np.zeros((2, 3), dtype=np.int64)))
    with pytest.raises(ValueError, match="embed"):
        eng.add_request(Request(prompt=[1, 2, 3], embed_rows=[1], embed_values=torch.zeros(1, cfg.H + 1)))
    assert not eng.has_unfinished()


@pytest.mark.parametrize("overlap", [False, True])
def test_preemption_of_a_request_with_given_positions_and_embeddings(overlap, tmp_path, cpu_kernels):
    """A request whose prompt carries positions (a 4 x 6 grid span) and given embedding rows is preempted while
    it decodes (the pool is too small for both requests) and recomputed from its prompt plus the tokens it
    had produced: the span's rows and positions are applied again, the generated tokens sit at index +
    delta, and the tokens equal the plain model's greedy decoding."""
    from omniserver_b200 import Request, SamplingParams
    d = make_model_dir(tmp_path, "tiny_b")
    cfg, w = plain_model(d)
    L, start, n_new = 40, 6, 14
    prompt = _requests(cfg.V, [L], seed=12)["r0"]
    pos, delta = pm.image_span_positions(L, start, 1, 4, 6)
    rows = list(range(start, start + 24))
    vals = torch.randn(24, cfg.H, generator=torch.Generator().manual_seed(3))
    other = _requests(cfg.V, [30], seed=13)["r0"]
    want_img = pm.generate(cfg, w, prompt, n_new, prompt_pos=pos, rope_delta=delta, override_rows=torch.tensor(rows),
                           override_vals=vals)
    want_txt = pm.generate(cfg, w, other, n_new)
    # 6 pages of 16 tokens: both prompts fit (3 + 2 pages), their decoding does not: 54 + 44 tokens need 7
    eng = _engine(d, overlap, max_tokens=96, max_running=2, max_prefill_per_step=2, max_prefill_tokens=64)
    a = eng.add_request(Request(prompt=other, sampling=SamplingParams(max_new_tokens=n_new)))
    b = eng.add_request(Request(prompt=prompt, positions=pos.numpy(), embed_rows=rows, embed_values=vals,
                                sampling=SamplingParams(max_new_tokens=n_new)))
    outs = eng.run_until_complete()
    seq_b = [s for s in eng.sequences() if s.request_id == b][0]
    assert eng.counters["preemptions"] >= 1 and seq_b.num_preemptions >= 1
    assert seq_b.num_output_tokens > 0
    assert outs[b] == want_img and outs[a] == want_txt
    eng.runner.cache.check_invariants()
    assert all(p == 0 for p in eng.runner.cache.pages_in_use())


def test_decode_splits_take_uneven_lengths_into_account():
    """One CTA per (request, kv head) when they fill the SMs and the lengths are alike; twice the splits when the
    longest request would otherwise set the time; never when the CTAs already come in several waves."""
    from omniserver_b200.ops import CudaKernels
    split = CudaKernels.decode_splits
    assert split(64, 2, 6, 2048, 148, max_splits=16)[1] == 1
    assert split(64, 2, 6, 2048, 148, max_splits=16, uneven=True)[1] == 2
    assert split(64, 2, 6, 512, 148, max_splits=16, uneven=True)[1] == 1        # short requests: the fixed part dominates
    assert split(64, 2, 6, 4352, 148, max_splits=16)[1] == 1
    chunk, n = split(64, 2, 6, 4352, 148, max_splits=16, uneven=True)
    assert n == 2 and chunk % 64 == 0 and chunk * n >= 4352
    assert split(64, 4, 7, 4352, 148, max_splits=16, uneven=True)[1] == 1       # 256 CTAs: two waves already
    assert split(8, 2, 6, 2048, 148, max_splits=16)[1] == 8
    assert split(8, 2, 6, 2048, 148, max_splits=16, uneven=True)[1] == 8


def test_prefill_units_list_every_row_tile_with_work_most_keys_first():
    from omniserver_b200.ops import CudaKernels
    u = CudaKernels.prefill_units([300, 1, 130, 1, 2], [300, 900, 700, 5, 259])
    # request 0: 3 tiles seeing 128, 256, 300 keys; request 2: 2 tiles seeing 698, 700; request 4: one tile seeing 259
    assert u.tolist() == [[2, 1], [2, 0], [0, 2], [4, 0], [0, 1], [0, 0]]
    assert CudaKernels.prefill_units([1, 1], [10, 20]).shape == (0, 2)


def test_decode_steps_share_graphs_of_power_of_two_batch_sizes():
    from omniserver_b200.engine.step import ModelRunner
    assert [ModelRunner._graph_bucket(n) for n in (1, 2, 3, 5, 8, 9, 17, 33, 63, 64, 65, 200)] == \
        [1, 2, 4, 8, 8, 16, 32, 64, 64, 64, 128, 256]
    assert ModelRunner.GRAPH_FILLERS >= 127


def test_spare_state_slots_are_not_counted_and_never_handed_to_requests():
    from omniserver_b200.cache.state_slots import OutOfSlots, StateSlots
    s = StateSlots(2, {}, "cpu", allocate=False, spare=2)
    assert s.num_free == 2
    a, b = s.alloc(), s.alloc()
    assert {a, b} == {0, 1} and s.num_free == 0
    with pytest.raises(OutOfSlots):
        s.alloc()
    x, y = s.alloc(spare=True), s.alloc(spare=True)
    assert {x, y} == {2, 3} and s.num_free == 0
    with pytest.raises(OutOfSlots):
        s.alloc(spare=True)
    s.free(x)
    assert s.num_free == 0 and s.alloc(spare=True) == x
    s.free(a)
    assert s.num_free == 1
    with pytest.raises(ValueError):
        s.free(a)
