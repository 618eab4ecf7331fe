"""Replay on the GPU against the plain implementation: each request alone and whole; most of it
in one step and the last 32 tokens one by one; in portions of changing size down to two tokens;
and mixed, up to four live requests with so few pages that they are used again — in 32-bit and in
bfloat16, in process and through bin/trace_run."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_cases as rc
from helpers import make_model_dir, plain_model
from plain import model as pm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAMILIES = {"whole": rc.whole, "tail": rc.tail_decode, "portions": rc.portions, "mixed": rc.mixed}
# 32-bit: sums in another order than the plain implementation's, nothing else.
# bfloat16: activations are rounded to 8 bits of mantissa between kernels.
# ``rel_fro`` (the error's norm over the logits' norm) is the bound that a wrong key, page or position breaks;
# ``max_abs`` is taken against the largest logit of the request (about 0.2 for the tiny models) and is there for a
# single wild element, which a norm over tens of thousands of logits would hide.
TOL = {"float32": dict(max_abs=6e-5, rel_fro=2e-5), "bfloat16": dict(max_abs=6e-2, rel_fro=2.5e-2)}


def check(got, want, dtype, what):
    err = (got.double() - want.double())
    max_abs = err.abs().max().item()
    rel = (err.norm() / want.double().norm()).item()
    t = TOL[dtype]
    assert max_abs < t["max_abs"] * want.abs().max().item() and rel < t["rel_fro"], \
        f"{what}: max abs {max_abs:.3e} (largest logit {want.abs().max().item():.3e}), relative {rel:.3e}"


def requests_for(vocab, lens=(5, 17, 33, 70, 100, 41), seed=3):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lens)}


def runner_for(model_dir, dtype, max_tokens, page_size=16, poison=True):
    from omniserver_b200 import EngineConfig, build_runner
    ec = EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=8)
    r = build_runner(model_dir=model_dir, engine_config=ec)
    r.cache.poison_freed = poison   # a read of a page that was given back shows up as NaN
    return r


def replay_in_process(runner, steps):
    from omniserver_b200.replay import TraceReplayer
    rp, outs = TraceReplayer(runner), {}
    with torch.inference_mode():
        for st in steps:
            lg = rp.run_step(st)
            if lg is not None:
                outs[st["step"]] = lg.float().cpu()
            runner.cache.check_invariants()
    assert not runner.cache.requests and all(p == 0 for p in runner.cache.pages_in_use())
    return outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("family", list(FAMILIES))
def test_replay_matches_plain(dtype, name, family, tmp_path):
    store = "float32" if dtype == "float32" else "bfloat16"
    d = make_model_dir(tmp_path, name, store)
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V)
    steps = FAMILIES[family](reqs)
    runner = runner_for(d, dtype, rc.max_live_tokens(steps))
    got = rc.collect(steps, replay_in_process(runner, steps))
    for rid, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        assert torch.isfinite(got[rid]).all(), f"{family}/{rid}: non-finite logits (a stale page was read?)"
        check(got[rid], want, dtype, f"{name}/{family}/{rid}")


@pytest.mark.parametrize("family", list(FAMILIES))
def test_replay_through_the_serving_kernels_of_decode_steps(family, tmp_path):
    """The tiny configuration whose sizes the weight-streaming kernels and the streaming decode attention take: the
    replay families in bfloat16 run decode steps (and mixed steps of up to 16 rows) through those kernels inside
    the engine, with pages that are used again; the kernels' use is checked by their launch counts."""
    from omniserver_b200 import ops
    d = make_model_dir(tmp_path, "tiny_d", "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V)
    steps = FAMILIES[family](reqs)
    runner = runner_for(d, "bfloat16", rc.max_live_tokens(steps))
    counts = ops.kernels().counts
    before = dict(counts)
    got = rc.collect(steps, replay_in_process(runner, steps))
    if family in ("tail", "mixed"):
        for what in ("stream_ffn", "stream_linear", "attn_decode_stream"):
            assert counts.get(what, 0) > before.get(what, 0), f"{what} did not run in the {family} family"
    if family == "portions":
        # portions of 17 to 63 tokens: the gate/up product of the few-rows tcgen05 kernel
        assert counts.get("gemm_fewrows_tc", 0) > before.get("gemm_fewrows_tc", 0)
    for rid, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        assert torch.isfinite(got[rid]).all()
        check(got[rid], want, "bfloat16", f"tiny_d/{family}/{rid}")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_c"])
def test_fp32_logits_do_not_depend_on_the_cut(name, tmp_path):
    """In 32-bit every kernel sums in an order fixed by the element, so whole, token by token,
    portions and mixed batches give bitwise the same logits."""
    d = make_model_dir(tmp_path, name, "float32")
    cfg, _ = plain_model(d)
    reqs = requests_for(cfg.V)
    base = None
    for family, make in FAMILIES.items():
        steps = make(reqs)
        got = rc.collect(steps, replay_in_process(runner_for(d, "float32", rc.max_live_tokens(steps)), steps))
        if base is None:
            base = got
        else:
            for rid in reqs:
                assert torch.equal(got[rid], base[rid]), f"{family}/{rid} differs from whole"


@pytest.mark.parametrize("page_size", [16, 64])
def test_long_decoding_and_first_tokens(page_size, tmp_path):
    """A request decoded one token at a time from its first token on, over many pages."""
    d = make_model_dir(tmp_path, "tiny_c", "float32")
    cfg, w = plain_model(d)
    toks = requests_for(cfg.V, (300,), seed=9)["r0"]
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == len(toks) - 1 else []}
             for i, t in enumerate(toks)]
    got = rc.collect(steps, replay_in_process(runner_for(d, "float32", 320, page_size), steps))
    check(got["x"], pm.forward(cfg, w, torch.tensor(toks)), "float32", "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_across_buckets_and_batch_sizes(dtype, tmp_path):
    """Pure decode steps replay CUDA graphs, one per (batch size, block-table width rounded up to 32 pages).
    A request decoded from 500 to 530 tokens crosses 512 = 32 pages of 16, where the next graph is built by a
    warm-up forward that writes the step's keys a second time; beside it the batch shrinks when a request
    ends and grows when one joins. Every decoded place against the plain model; more than one graph is used."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_a", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (530, 60, 45, 38), seed=12)
    runner = runner_for(d, dtype, 1024)
    assert runner.use_graphs
    runner.graph_min_uses = 1              # every shape gets its graph at once
    pos = {"r0": 500, "r1": 40, "r2": 0, "r3": 0}
    got = {r: {} for r in reqs}
    live = []

    def prefill(r, n):
        runner.start_request(r)
        lg = runner.step([StepEntry(r, reqs[r][:n], want=[n - 1])]).float().cpu()
        got[r][n - 1] = lg[0]
        pos[r] = n
        live.append(r)

    with torch.inference_mode():
        prefill("r0", 500)
        prefill("r1", 40)
        for step in range(30):
            if step == 8:
                prefill("r2", 30)          # the batch grows
            if step == 12:
                prefill("r3", 21)
            entries = [StepEntry(r, [reqs[r][pos[r]]], want=[0]) for r in live]
            lg = runner.step(entries).float().cpu()
            for i, r in enumerate(list(live)):
                got[r][pos[r]] = lg[i]
                pos[r] += 1
                if pos[r] == len(reqs[r]):     # the batch shrinks
                    runner.end_request(r)
                    live.remove(r)
            runner.cache.check_invariants()
        assert pos["r0"] == 530
        for r in list(live):
            runner.end_request(r)
    keys = set(runner._graphs)
    assert len({k[0] for k in keys}) >= 3, keys            # several batch sizes
    assert len({k[1] for k in keys}) >= 2, keys            # and two block-table widths
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        assert len(rows) >= 16
        check(torch.stack([got[r][p] for p in rows]), want[rows], dtype, f"graphs/{r}")


def test_a_decode_graph_may_wait_until_its_shape_comes_back(tmp_path):
    """With ``graph_min_uses`` = 3 a shape of decode step (batch size, table width) is launched kernel by kernel the
    first two times and replayed from a graph from the third on; shapes that come by once or twice never get one.
    The logits are the plain model's either way."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_b", "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (40, 33, 29, 31), seed=31)
    runner = runner_for(d, "bfloat16", 512)
    assert runner.use_graphs and runner.graph_min_uses == 1
    runner.graph_min_uses = 3
    runner.graph_min_uses_prompt = 0       # (no graphs for the prompts' steps: only decode shapes are counted below)
    got = {r: {} for r in reqs}
    n_graphs = []
    with torch.inference_mode():
        for r, toks in reqs.items():
            runner.start_request(r)
            runner.step([StepEntry(r, toks[:20], want=[])])
        pos = {r: 20 for r in reqs}
        names = list(reqs)
        for live in ([names[:4]] * 5 + [names[:2]] * 2 + [names[:1]] * 4):
            lg = runner.step([StepEntry(r, [reqs[r][pos[r]]], want=[0]) for r in live]).float().cpu()
            for i, r in enumerate(live):
                got[r][pos[r]] = lg[i]
                pos[r] += 1
            n_graphs.append(len(runner._graphs))
        for r in reqs:
            runner.end_request(r)
    assert n_graphs == [0, 0, 1, 1, 1, 1, 1, 1, 1, 2, 2], n_graphs     # batch 4 at its third step, batch 2 never, batch 1 at its third
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        check(torch.stack([got[r][p] for p in rows]), want[rows], "bfloat16", f"late graphs/{r}")


def test_only_uses_that_follow_one_another_count_towards_a_graph(tmp_path):
    """Two shapes of decode step in turn, each coming back every second step: with ``graph_use_window`` = 1 their
    uses never add up and no graph is built (a workload that brings many shapes back now and then must not build
    them all, more than are kept, again and again); with a window of 2 both get their graph on their next use."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_b", "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (40, 33), seed=37)
    runner = runner_for(d, "bfloat16", 512)
    runner.graph_min_uses, runner.graph_min_uses_prompt, runner.graph_use_window = 2, 0, 1
    names = list(reqs)
    got = {r: {} for r in reqs}
    n_graphs = []
    with torch.inference_mode():
        for r, toks in reqs.items():
            runner.start_request(r)
            runner.step([StepEntry(r, toks[:20], want=[])])
        pos = {r: 20 for r in reqs}
        for i, live in enumerate([names, names[:1]] * 5):
            if i == 6:
                runner.graph_use_window = 2
            lg = runner.step([StepEntry(r, [reqs[r][pos[r]]], want=[0]) for r in live]).float().cpu()
            for j, r in enumerate(live):
                got[r][pos[r]] = lg[j]
                pos[r] += 1
            n_graphs.append(len(runner._graphs))
        for r in reqs:
            runner.end_request(r)
    assert n_graphs == [0, 0, 0, 0, 0, 0, 1, 2, 2, 2], n_graphs     # (the use two steps back counts once the window is 2)
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        check(torch.stack([got[r][p] for p in rows]), want[rows], "bfloat16", f"graph window/{r}")


def test_decode_steps_are_padded_to_the_batch_sizes_of_graphs(tmp_path):
    """Eleven, nine, five and then four decoding requests: the steps of eleven and of nine replay the graph of sixteen
    rows, that of five the graph of eight, padded with rows that are no requests (spare state slots, a page that
    goes back after every step); four need none. Every request's logits are the plain model's, the fillers hold
    nothing between steps and take no request's slot."""
    from omniserver_b200 import EngineConfig, build_runner
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_b", "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, tuple(30 + (i % 4) for i in range(11)), seed=41)
    runner = build_runner(model_dir=d, engine_config=EngineConfig(dtype="bfloat16", page_size=16, max_cache_tokens=1024,
                                                               max_requests=12))
    runner.cache.poison_freed = True
    runner.graph_min_uses = 1
    runner.graph_min_uses_prompt = 0
    got = {r: {} for r in reqs}
    names = list(reqs)
    with torch.inference_mode():
        for r, toks in reqs.items():
            runner.start_request(r)
            runner.step([StepEntry(r, toks[:12], want=[])])
        pos = {r: 12 for r in reqs}
        free_slots = runner.cache.state.num_free
        for live in ([names] * 4 + [names[:9]] * 4 + [names[:5]] * 3 + [names[:4]] * 2):
            lg = runner.step([StepEntry(r, [reqs[r][pos[r]]], want=[0]) for r in live]).float().cpu()
            assert lg.shape[0] == len(live) and runner.logit_slots.shape[0] == len(live)
            for i, r in enumerate(live):
                got[r][pos[r]] = lg[i]
                pos[r] += 1
            runner.cache.check_invariants()
            assert runner.cache.state.num_free == free_slots
            for f in runner._filler_ids:
                rc = runner.cache.requests[f]
                assert rc.cursor == 0 and rc.reserved == 0 and all(len(t) == 0 for t in rc.tables)
        assert {k[0] for k in runner._graphs} == {16, 8, 4} and len(runner._filler_ids) == 7
        for r in reqs:
            runner.end_request(r)
    assert all(p == 0 for p in runner.cache.pages_in_use())
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        check(torch.stack([got[r][p] for p in rows]), want[rows], "bfloat16", f"padded/{r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_with_prompt_portions_replay_graphs_of_their_shape(dtype, tmp_path):
    """A long prompt in portions of 16 tokens beside two decoding requests: the shape (1, 1, 16 tokens) comes by
    again and again and is replayed from a graph from its third time on, with other tokens, positions in the cache,
    pages and wanted rows every time; so is a lone portion of 24 tokens of several requests. Logits against the plain
    model at every wanted place."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_b", dtype)
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (140, 60, 50, 72, 72, 72, 72), seed=51)
    runner = runner_for(d, dtype, 1024)
    assert runner.use_graphs and runner.graph_min_uses_prompt == 3
    got = {r: {} for r in reqs}
    names = list(reqs)
    long, d1, d2 = names[:3]
    with torch.inference_mode():
        for r in (d1, d2):
            runner.start_request(r)
            runner.step([StepEntry(r, reqs[r][:30], want=[])])
        pos = {d1: 30, d2: 30, long: 0}
        runner.start_request(long)
        shape_graphs = []
        for step in range(8):           # 8 x 16 = 128 tokens of the long prompt, each beside two decoded tokens
            entries = [StepEntry(d1, [reqs[d1][pos[d1]]], want=[0]), StepEntry(d2, [reqs[d2][pos[d2]]], want=[0]),
                       StepEntry(long, reqs[long][pos[long]:pos[long] + 16], want=[step % 15, 15])]   # two rows, other places
            lg = runner.step(entries).float().cpu()
            got[d1][pos[d1]], got[d2][pos[d2]] = lg[0], lg[1]
            for j, wrow in enumerate(entries[2].want):
                got[long][pos[long] + wrow] = lg[2 + j]
            pos[d1] += 1; pos[d2] += 1; pos[long] += 16
            shape_graphs.append(sum(1 for k in runner._graphs if k[0] == "shape"))
            runner.cache.check_invariants()
        assert shape_graphs == [0, 0, 1, 1, 1, 1, 1, 1], shape_graphs
        for r in (long, d1, d2):
            runner.end_request(r)
        # lone portions of 24 tokens of four other requests, three portions each
        for r in names[3:]:
            runner.start_request(r)
            for o in range(0, 72, 24):
                lg = runner.step([StepEntry(r, reqs[r][o:o + 24], want=[23])]).float().cpu()
                got[r][o + 23] = lg[0]
            runner.end_request(r)
        assert sum(1 for k in runner._graphs if k[0] == "shape") >= 2
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        assert rows
        check(torch.stack([got[r][p] for p in rows]), want[rows], dtype, f"shape graphs/{r}")


def test_the_number_of_decode_graphs_is_bounded(tmp_path):
    """With room for two graphs, a batch that keeps changing its size makes the runner drop the graph used longest
    ago and build it again later; the logits stay those of the plain model."""
    from omniserver_b200.engine.step import StepEntry
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (30, 30, 30, 30), seed=14)
    runner = runner_for(d, "float32", 512)
    runner.graph_max_count = 2
    runner.graph_min_uses = 1
    got = {r: {} for r in reqs}
    with torch.inference_mode():
        for r, toks in reqs.items():
            runner.start_request(r)
            runner.step([StepEntry(r, toks[:10], want=[])])
        pos = {r: 10 for r in reqs}
        names = list(reqs)
        for step in range(20):
            live = names[:1 + step % 4]              # batch sizes 1, 2, 3, 4, 1, ...
            lg = runner.step([StepEntry(r, [reqs[r][pos[r]]], want=[0]) for r in live]).float().cpu()
            for i, r in enumerate(live):
                got[r][pos[r]] = lg[i]
                pos[r] += 1
            assert len(runner._graphs) <= 2
        for r in reqs:
            runner.end_request(r)
    for r, toks in reqs.items():
        want = pm.forward(cfg, w, torch.tensor(toks))
        rows = sorted(got[r])
        check(torch.stack([got[r][p] for p in rows]), want[rows], "float32", f"bounded graphs/{r}")


def test_positions_and_embeddings_given_with_the_prompt(tmp_path):
    """A prompt with a 24-token span whose embeddings are given and whose positions run over a
    4 x 6 grid; text after it resumes at max + 1. Cut into portions of 16 that split the span."""
    d = make_model_dir(tmp_path, "tiny_b", "float32")
    cfg, w = plain_model(d)
    L, start = 100, 10
    toks = requests_for(cfg.V, (L,), seed=5)["r0"]
    pos, delta = pm.image_span_positions(L, start, 1, 4, 6)
    rows = torch.arange(start, start + 24)
    vals = torch.randn(24, cfg.H, generator=torch.Generator().manual_seed(2))
    want = pm.forward(cfg, w, torch.tensor(toks), pos, rows, vals)
    steps = []
    for i, a in enumerate(range(0, L, 16)):
        b = min(a + 16, L)
        pick = [r for r in range(a, b) if start <= r < start + 24]
        e = {"id": "img", "tokens": toks[a:b], "want": list(range(b - a)), "positions": pos[:, a:b].tolist()}
        if pick:
            e["embeds"] = {"rows": [r - a for r in pick], "values": vals[[r - start for r in pick]].tolist()}
        steps.append({"step": i, "entries": [e], "end": []})
    # then decoded tokens continue at cursor + delta on all axes: the encoding derives that from the prompt's positions
    extra = requests_for(cfg.V, (6,), seed=6)["r0"]
    runner = runner_for(d, "float32", 128)
    from omniserver_b200.engine.step import StepEntry
    with torch.inference_mode():
        runner.start_request("img", pos.numpy(), L)
        outs = []
        for st in steps:
            e = st["entries"][0]
            emb = e.get("embeds")
            outs.append(runner.step([StepEntry("img", e["tokens"], e["want"], np.asarray(e["positions"]),
                                               emb["rows"] if emb else None,
                                               torch.tensor(emb["values"]) if emb else None)]).cpu())
        for t in extra:
            outs.append(runner.step([StepEntry("img", [t], [0])]).cpu())
        runner.end_request("img")
    got = torch.cat(outs)
    full = toks + extra
    pos_full = pm.extend_positions(pos, delta, len(full))
    want_full = pm.forward(cfg, w, torch.tensor(full), pos_full, rows, vals)
    check(got, want_full, "float32", "image span")
    assert delta == -18


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """The program itself: JSON lines in, <step>.f32 files and 'done <step>' lines out."""
    d = make_model_dir(tmp_path, "tiny_b", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = plain_model(d)
    reqs = requests_for(cfg.V, (40, 9, 64, 100, 23), seed=8)
    steps = rc.mixed(reqs, seed=4)
    steps.append({"step": len(steps), "entries": [{"id": "nolog", "tokens": [1, 2, 3], "want": []}], "end": ["nolog"]})
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(rc.max_live_tokens(steps))],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    assert not (out / f"{len(steps) - 1}.f32").exists()
    outputs = {}
    for st in steps[:-1]:
        n = sum(len(e["want"]) for e in st["entries"])
        arr = np.fromfile(out / f"{st['step']}.f32", dtype="<f4")
        assert arr.size == n * cfg.V
        outputs[st["step"]] = torch.from_numpy(arr.reshape(n, cfg.V).copy())
    got = rc.collect(steps[:-1], outputs)
    for rid, toks in reqs.items():
        check(got[rid], pm.forward(cfg, w, torch.tensor(toks)), dtype, f"trace_run/{rid}")
