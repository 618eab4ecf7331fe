"""Generation through the Python entry point against the plain implementation: greedy tokens under
several batchings, seeded temperature sampling, preemption when pages run out."""

import pytest
import torch

from helpers import make_model_dir, plain_model
from plain import model as pm

pytestmark = pytest.mark.gpu


def engine(model_dir, dtype="float32", max_tokens=2048, seed=0, **sched):
    from omniserver_b200 import EngineConfig, LLMEngine, SchedulerConfig
    return LLMEngine.from_model_dir(model_dir, EngineConfig(dtype=dtype, max_cache_tokens=max_tokens, max_requests=16),
                                    SchedulerConfig(**sched), seed=seed)


def prompts_for(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


@pytest.mark.parametrize("sched", [
    dict(max_running=8, max_prefill_per_step=8, max_prefill_tokens=8192),   # whole prompts packed
    dict(max_running=2, max_prefill_per_step=1, max_prefill_tokens=16),     # portions of 16 beside decodes
    dict(max_running=3, max_prefill_per_step=2, max_prefill_tokens=7),
])
def test_greedy_generation_matches_plain(sched, tmp_path):
    from omniserver_b200 import SamplingParams
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    prompts = prompts_for(cfg.V, (5, 17, 33))
    with torch.inference_mode():
        outs = engine(d, **sched).generate(prompts, SamplingParams(max_new_tokens=8))
    for p, o in zip(prompts, outs):
        assert o == pm.generate(cfg, w, p, 8)


def test_temperature_sampling_is_seeded_and_independent_of_batching(tmp_path):
    from omniserver_b200 import Request, SamplingParams
    from omniserver_b200.sampling import rng
    d = make_model_dir(tmp_path, "tiny_b", "float32")
    cfg, w = plain_model(d)
    prompts = prompts_for(cfg.V, (9, 40, 64, 100), seed=1)
    results = []
    for sched in (dict(max_running=4, max_prefill_per_step=4, max_prefill_tokens=4096),
                  dict(max_running=3, max_prefill_per_step=1, max_prefill_tokens=16)):
        with torch.inference_mode():
            eng = engine(d, seed=11, **sched)
            for i, p in enumerate(prompts):
                eng.add_request(Request(prompt=p, sampling=SamplingParams(max_new_tokens=12, temperature=0.8),
                                        request_id=f"q{i}"))
            results.append(eng.run_until_complete())
    assert results[0] == results[1]
    for i, p in enumerate(prompts):
        us = [rng.uniform(11, f"q{i}", k) for k in range(12)]
        want = pm.generate(cfg, w, p, 12, temperature=0.8, uniforms=us)
        got = results[0][f"q{i}"]
        # a draw that falls within float rounding of a CDF edge may pick the neighbour; then the
        # sequences part ways and only the tokens before it can be compared
        k = next((j for j in range(12) if got[j] != want[j]), 12)
        if k < 12:
            logits = pm.forward(cfg, w, torch.tensor(p + want[:k]))[-1]
            cdf = pm.temperature_cdf(logits, 0.8)
            edges = torch.cat([cdf[got[k] - 1:got[k] + 1], cdf[want[k] - 1:want[k] + 1]])
            assert (edges - us[k]).abs().min() < 1e-5, f"request {i}: token {k} differs away from a CDF edge"


def test_stop_token_and_max_new_tokens(tmp_path):
    from omniserver_b200 import Request, SamplingParams
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    p = prompts_for(cfg.V, (12,), seed=4)[0]
    ref = pm.generate(cfg, w, p, 10)
    stop = ref[3]
    cut = ref.index(stop) + 1
    with torch.inference_mode():
        eng = engine(d)
        rid = eng.add_request(Request(prompt=p, sampling=SamplingParams(max_new_tokens=10, stop_token_ids=[stop])))
        out = eng.run_until_complete()[rid]
    assert out == ref[:cut]
    assert all(x == 0 for x in eng.runner.cache.pages_in_use())


def test_running_out_of_pages_preempts_and_recomputes(tmp_path):
    """Four requests whose contexts together outgrow the pool: the one admitted last gives its pages
    back, waits, and is recomputed; every request still produces the plain implementation's tokens."""
    from omniserver_b200 import SamplingParams
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    prompts = prompts_for(cfg.V, (30, 28, 31, 29), seed=2)
    with torch.inference_mode():
        eng = engine(d, max_tokens=160, max_running=4, max_prefill_per_step=4, max_prefill_tokens=64)
        outs = eng.generate(prompts, SamplingParams(max_new_tokens=24))
    assert eng.stats()["preemptions"] > 0
    for p, o in zip(prompts, outs):
        assert o == pm.generate(cfg, w, p, 24)
    eng.runner.cache.check_invariants()
    assert all(x == 0 for x in eng.runner.cache.pages_in_use())


def near_argmax(cfg, w, prompt, out, rel=0.12, prompt_pos=None, rope_delta=0, override_rows=None, override_vals=None):
    """Every generated token is, for the plain model given the same prefix, the largest logit or within
    ``rel`` of the largest logit's size below it (twice the bound that the bfloat16 replay tests put on one
    logit's error: the winner's and the runner-up's may both be off). Returns the first place where that fails."""
    toks = list(prompt)
    for j, t in enumerate(out):
        pos = None if prompt_pos is None else pm.extend_positions(prompt_pos, rope_delta, len(toks))
        lg = pm.forward(cfg, w, torch.tensor(toks), pos, override_rows, override_vals)[-1]
        if lg[t] < lg.max() - rel * lg.abs().max():
            return j
        toks.append(t)
    return None


def test_bfloat16_generation_picks_the_plain_models_tokens(tmp_path):
    """bfloat16 through the entry point, portions beside decodes: every generated token must be the plain
    model's choice for the same prefix, up to bfloat16 rounding of the logits. With a vocabulary of 1,000 a
    token of a wrong key, page or position passes this with a chance of a few in a thousand."""
    from omniserver_b200 import SamplingParams
    d = make_model_dir(tmp_path, "tiny_b", "bfloat16")
    cfg, w = plain_model(d)
    prompts = prompts_for(cfg.V, (9, 40, 64), seed=3)
    with torch.inference_mode():
        outs = engine(d, dtype="bfloat16", max_running=4, max_prefill_per_step=2, max_prefill_tokens=32).generate(
            prompts, SamplingParams(max_new_tokens=10))
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 10
        bad = near_argmax(cfg, w, p, o)
        assert bad is None, f"prompt {i}: generated token {bad} ({o[bad]}) is not the plain model's choice"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_of_a_request_with_given_positions_and_embeddings(dtype, tmp_path):
    """A request whose prompt carries positions over a 4 x 6 grid and given embedding rows is preempted while it
    decodes and recomputed from its prompt plus the tokens it had produced: rows and positions are applied
    again across the border between prompt and generated tokens."""
    from omniserver_b200 import Request, SamplingParams
    d = make_model_dir(tmp_path, "tiny_b", dtype)
    cfg, w = plain_model(d)
    L, start, n_new = 40, 6, 14
    prompt = prompts_for(cfg.V, (L,), seed=12)[0]
    other = prompts_for(cfg.V, (30,), seed=13)[0]
    pos, delta = pm.image_span_positions(L, start, 1, 4, 6)
    rows = list(range(start, start + 24))
    vals = torch.randn(24, cfg.H, generator=torch.Generator().manual_seed(3))
    with torch.inference_mode():
        eng = engine(d, dtype=dtype, max_tokens=96, max_running=2, max_prefill_per_step=2, max_prefill_tokens=64)
        a = eng.add_request(Request(prompt=other, sampling=SamplingParams(max_new_tokens=n_new)))
        b = eng.add_request(Request(prompt=prompt, positions=pos.numpy(), embed_rows=rows, embed_values=vals,
                                    sampling=SamplingParams(max_new_tokens=n_new)))
        outs = eng.run_until_complete()
    assert eng.stats()["preemptions"] >= 1
    assert [s for s in eng.sequences() if s.request_id == b][0].num_preemptions >= 1
    fwd = dict(prompt_pos=pos, rope_delta=delta, override_rows=torch.tensor(rows), override_vals=vals)
    if dtype == "float32":
        assert outs[b] == pm.generate(cfg, w, prompt, n_new, **fwd)
        assert outs[a] == pm.generate(cfg, w, other, n_new)
    else:
        assert len(outs[b]) == n_new and near_argmax(cfg, w, prompt, outs[b], **fwd) is None
        assert len(outs[a]) == n_new and near_argmax(cfg, w, other, outs[a]) is None
    eng.runner.cache.check_invariants()
    assert all(x == 0 for x in eng.runner.cache.pages_in_use())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_and_step_by_step_engines_agree(dtype, tmp_path):
    """The engine launches a step before it has read the tokens of the one before (they stay on the
    device for the embedding lookup, also inside the CUDA graphs of decode steps). Same tokens as
    with a wait after every step; greedy and seeded temperature rows, a stop token, uneven lengths."""
    from omniserver_b200 import EngineConfig, LLMEngine, Request, SamplingParams, SchedulerConfig
    d = make_model_dir(tmp_path, "tiny_c", dtype)
    cfg, w = plain_model(d)
    prompts = prompts_for(cfg.V, (6, 19, 40, 11), seed=4)
    outs = {}
    for overlap in (False, True):
        with torch.inference_mode():
            eng = LLMEngine.from_model_dir(d, EngineConfig(dtype=dtype, max_cache_tokens=2048, max_requests=8),
                                           SchedulerConfig(max_running=4, max_prefill_per_step=4), seed=3)
            eng.overlap = overlap
            sps = [SamplingParams(max_new_tokens=40), SamplingParams(max_new_tokens=23, temperature=0.8, seed=9),
                   SamplingParams(max_new_tokens=31), SamplingParams(max_new_tokens=12, temperature=1.3)]
            if outs:
                sps[2].stop_token_ids = [outs[False][2][17]]      # ends the third request at its 18th token
            ids = [eng.add_request(Request(prompt=p, sampling=sp, request_id=f"o{i}")) for i, (p, sp) in
                   enumerate(zip(prompts, sps))]
            res = eng.run_until_complete()
            assert (eng.counters["overlapped_steps"] > 10) == overlap
            assert all(p == 0 for p in eng.runner.cache.pages_in_use())
        outs[overlap] = [res[i] for i in ids]
    want = [list(o) for o in outs[False]]
    first = want[2].index(want[2][17])                           # the stop token may have come earlier too
    want[2] = want[2][:first + 1]
    assert outs[True] == want
    if dtype == "float32":
        assert outs[False][0] == pm.generate(cfg, w, prompts[0], 40)


@pytest.mark.parametrize("seed,pool", [(s, p) for s in range(1, 7) for p in (96, 160, 4096)][::2] + [(2, 96)])
def test_random_traffic_matches_plain(seed, pool, tmp_path):
    """Requests of random lengths that arrive while others run, some ending on a stop token, some aborted, in a
    pool that forces preemptions (or none), batch sizes that need padding to the graphs' sizes, steps launched
    before the ones before are read: every request's greedy tokens are the plain model's; nothing is left in the
    cache."""
    import random
    from omniserver_b200 import EngineConfig, LLMEngine, Request, SamplingParams, SchedulerConfig
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    n_req = 14
    prompts = [torch.randint(0, cfg.V, (rnd.randint(1, 40),), generator=g).tolist() for _ in range(n_req)]
    new = [rnd.randint(1, 24) for _ in range(n_req)]
    arrive = sorted(rnd.randint(0, 30) for _ in range(n_req))
    want = [pm.generate(cfg, w, p, n) for p, n in zip(prompts, new)]
    stops = {}
    for i in range(n_req):
        if rnd.random() < 0.3 and len(want[i]) > 2:
            k = rnd.randrange(1, len(want[i]))
            stops[i] = want[i][k]
            want[i] = want[i][:want[i].index(stops[i]) + 1]
    aborted = {i for i in range(n_req) if rnd.random() < 0.15}
    with torch.inference_mode():
        eng = LLMEngine.from_model_dir(d, EngineConfig(dtype="float32", page_size=8, max_cache_tokens=pool, max_requests=16),
                                       SchedulerConfig(max_running=rnd.choice([3, 6, 11]), max_prefill_per_step=rnd.choice([1, 3]),
                                                       max_prefill_tokens=rnd.choice([8, 24, 64])), seed=seed)
        ids, got, step, nxt = {}, {}, 0, 0
        while nxt < n_req or eng.has_unfinished():
            while nxt < n_req and arrive[nxt] <= step:
                sp = SamplingParams(max_new_tokens=new[nxt], stop_token_ids=[stops[nxt]] if nxt in stops else [])
                ids[nxt] = eng.add_request(Request(prompt=prompts[nxt], sampling=sp, request_id=f"t{nxt}"))
                got[ids[nxt]] = []
                if nxt in aborted and rnd.random() < 0.5:
                    eng.abort(ids[nxt])                       # before it ever ran
                nxt += 1
            for dl in eng.step():
                got[dl.request_id].extend(dl.new_token_ids)
            for i in list(aborted):
                if i in ids and len(got[ids[i]]) >= 2:
                    eng.abort(ids[i])                         # while it decodes
                    aborted.discard(i)
                    want[i] = None
            step += 1
            assert step < 3000
            eng.runner.cache.check_invariants()
        from omniserver_b200 import ops
        ops.kernels().check_device_errors()
    for i in range(n_req):
        if want[i] is None or i in aborted:
            continue       # aborted: whatever it produced before is a prefix
        assert got[ids[i]] == want[i], (i, got[ids[i]], want[i])
    if pool == 96:
        assert eng.stats()["preemptions"] >= 1
    assert all(x == 0 for x in eng.runner.cache.pages_in_use()) and not eng.runner.cache.requests
