"""The engine at the layer sizes of Qwen2-VL-2B (hidden 1536, 12 heads in 2 groups, head size 128,
intermediate 8960, vocabulary 151936, tied head) with two layers and random weights: logits of
whole prompts, of portions and of mixed batches against the plain implementation, in 32-bit (where
they must also be bitwise independent of the cut) and in bfloat16 (tensor-core kernels at their
real shapes: tcgen05 GEMM, paged prefill attention, split-key decode attention, skinny GEMM)."""

import pytest
import torch

import replay_cases as rc
from plain import model as pm

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["Qwen2VLForConditionalGeneration"], "hidden_size": 1536, "num_hidden_layers": 2,
    "num_attention_heads": 12, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960,
    "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]}, "tie_word_embeddings": True,
}


def build(dtype, max_tokens):
    from omniserver_b200 import EngineConfig, build_runner
    ec = EngineConfig(dtype=dtype, max_cache_tokens=max_tokens, max_requests=8)
    r = build_runner(config=CONFIG, seed=2, engine_config=ec, init_std=0.03, norm_noise=0.1)
    r.cache.poison_freed = True
    return r


def plain_weights(model):
    f = lambda t: t.detach().float().cpu()
    w = {"embed_tokens.weight": f(model.embed.weight), "norm.weight": f(model.final_norm.weight)}
    nq, nkv = 12 * 128, 2 * 128
    for i, blk in enumerate(model.blocks):
        p = f"layers.{i}."
        qkv_w, qkv_b = f(blk.mixer.qkv.weight), f(blk.mixer.qkv.bias)
        w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"] = \
            qkv_w[:nq], qkv_w[nq:nq + nkv], qkv_w[nq + nkv:]
        w[p + "self_attn.q_proj.bias"], w[p + "self_attn.k_proj.bias"], w[p + "self_attn.v_proj.bias"] = \
            qkv_b[:nq], qkv_b[nq:nq + nkv], qkv_b[nq + nkv:]
        w[p + "self_attn.o_proj.weight"] = f(blk.mixer.out.weight)
        gu = f(blk.ffn.gate_up.weight)
        w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"] = gu[:8960], gu[8960:]
        w[p + "mlp.down_proj.weight"] = f(blk.ffn.down.weight)
        w[p + "input_layernorm.weight"] = f(blk.mixer_norm.weight)
        w[p + "post_attention_layernorm.weight"] = f(blk.ffn_norm.weight)
    return w


def replay(runner, steps):
    from omniserver_b200.replay import TraceReplayer
    rp, outs = TraceReplayer(runner), {}
    with torch.inference_mode():
        for st in steps:
            lg = rp.run_step(st)
            if lg is not None:
                outs[st["step"]] = lg.float().cpu()
    return outs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_logits_match_plain_for_every_cut(dtype):
    g = torch.Generator().manual_seed(4)
    reqs = {f"r{i}": torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate((1100, 40, 97))}
    # logits only at a few places per request: [wanted, 151936] rows are large
    def thin(steps):
        for st in steps:
            for e in st["entries"]:
                e["want"] = [w for w in e["want"] if w == len(e["tokens"]) - 1]
        return steps
    runner = build(dtype, 1536)
    cfg = pm.PlainConfig(CONFIG)
    w = plain_weights(runner.model)
    # plain logits only at the rows some cut asks for (the [T, 151936] matrix of the long prompt
    # would take minutes on the CPU): computed lazily per (request, row) from the final hidden states
    hidden = {}
    for r, t in reqs.items():
        hidden[r] = pm.forward(cfg, w, torch.tensor(t), return_hidden=True, rows=[len(t) - 1])[1]

    class Want(dict):
        def __missing__(self, rid):
            self[rid] = Rows(rid)
            return self[rid]

    class Rows(dict):
        def __init__(self, rid):
            self.rid = rid

        def __missing__(self, p):
            self[p] = pm.lm_head(hidden[self.rid][p:p + 1], w["embed_tokens.weight"])[0]
            return self[p]
    want = Want()
    base = None
    for family in (rc.whole, rc.portions, rc.mixed, rc.tail_decode):
        steps = thin(family(reqs))
        outs = replay(runner, steps)
        got = {}
        for st in steps:
            o = 0
            pos = got.setdefault("_pos", {})
            for e in st["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
                if e["want"]:
                    got.setdefault(e["id"], {})[pos[e["id"]] - 1] = outs[st["step"]][o]
                    o += 1
            for rid in st["end"]:
                pos.pop(rid, None)
        got.pop("_pos")
        for rid, rows in got.items():
            for p, lg in rows.items():
                ref = want[rid][p]
                err = (lg - ref).abs().max().item()
                scale = ref.abs().max().item()
                if dtype == "float32":
                    assert err < 2e-4 * max(1.0, scale), f"{family.__name__}/{rid}@{p}: {err}"
                else:
                    assert err < 5e-2 * max(1.0, scale), f"{family.__name__}/{rid}@{p}: {err}"
                    assert ((lg - ref).norm() / ref.norm()).item() < 3e-2
        if dtype == "float32":
            if base is None:
                base = got
            else:
                for rid, rows in got.items():
                    for p, lg in rows.items():
                        if p in base.get(rid, {}):
                            assert torch.equal(lg, base[rid][p]), f"{family.__name__}/{rid}@{p} differs bitwise from whole"


def test_full_width_many_live_requests_bfloat16():
    """24 live requests at the real layer sizes: their prompts packed into two steps, then four steps that
    decode all of them at once. That is the regime of the few-rows tcgen05 kernel (gate/up with its activation and
    the down projection at 17 to 64 rows) and of the library GEMM (qkv, o), of the streaming decode
    attention with several splits merged through scratch memory, and of CUDA-graph replay at a batch size
    the other tests do not reach. Logits of every request at every decoded place against the plain model."""
    from omniserver_b200 import EngineConfig, build_runner
    from omniserver_b200.engine.step import StepEntry
    n_req, n_dec = 24, 4
    g = torch.Generator().manual_seed(9)
    lens = [int(x) for x in torch.randint(3, 90, (n_req,), generator=g)]
    lens[0], lens[1] = 200, 1                       # several key blocks; a prompt of one token
    toks = [torch.randint(0, CONFIG["vocab_size"], (n + n_dec,), generator=g).tolist() for n in lens]
    ec = EngineConfig(dtype="bfloat16", max_cache_tokens=4096, max_requests=n_req + 2)
    runner = build_runner(config=CONFIG, seed=2, engine_config=ec, init_std=0.03, norm_noise=0.1)
    cfg = pm.PlainConfig(CONFIG)
    w = plain_weights(runner.model)
    got = {i: [] for i in range(n_req)}
    with torch.inference_mode():
        for i in range(n_req):
            runner.start_request(f"m{i}")
        for part in (range(0, 12), range(12, n_req)):
            lg = runner.step([StepEntry(f"m{i}", toks[i][:lens[i]], want=[lens[i] - 1]) for i in part]).float().cpu()
            for j, i in enumerate(part):
                got[i].append(lg[j])
        for d in range(n_dec):
            lg = runner.step([StepEntry(f"m{i}", [toks[i][lens[i] + d]], want=[0]) for i in range(n_req)]).float().cpu()
            for i in range(n_req):
                got[i].append(lg[i])
        for i in range(n_req):
            runner.end_request(f"m{i}")
    assert all(p == 0 for p in runner.cache.pages_in_use())
    for i in range(n_req):
        rows = list(range(lens[i] - 1, lens[i] + n_dec))
        hid = pm.forward(cfg, w, torch.tensor(toks[i]), return_hidden=True, rows=[rows[-1]])[1]
        for k, p in enumerate(rows):
            ref = pm.lm_head(hid[p:p + 1], w["embed_tokens.weight"])[0]
            lg = got[i][k]
            err = (lg - ref).abs().max().item()
            assert err < 5e-2 * max(1.0, ref.abs().max().item()), f"request {i} place {p}: {err}"
            assert ((lg - ref).norm() / ref.norm()).item() < 3e-2, f"request {i} place {p}"


_PLAIN_ROWS = {}


def _plain_rows(cfg, w, key, toks, rows):
    """Plain logits of one request at the given rows, kept for the tests that share requests."""
    if key not in _PLAIN_ROWS:
        hid = pm.forward(cfg, w, torch.tensor(toks), return_hidden=True, rows=[rows[-1]])[1]
        _PLAIN_ROWS[key] = {p: pm.lm_head(hid[p:p + 1], w["embed_tokens.weight"])[0] for p in rows}
    return _PLAIN_ROWS[key]


@pytest.mark.parametrize("n_req", [8, 16])
def test_benchmarked_decode_steps_match_plain(n_req):
    """The configuration that the benchmark times, with two layers: 8 and 16 requests with contexts of about
    2,040 tokens decode together for 12 steps, so that every context crosses 2,048 tokens and a page's edge at
    a step of its own. Default switches: CUDA graphs, the weight-streaming kernels for up to 8 rows and their
    forms with two column tiles for 9 to 16 rows, the streaming decode attention with its splits merged in a
    cluster or through scratch memory. Logits of every request at every decoded place against the plain model."""
    from omniserver_b200 import EngineConfig, build_runner
    from omniserver_b200.engine.step import StepEntry
    n_dec = 12
    g = torch.Generator().manual_seed(21)
    lens = [2040 - 3 * i for i in range(16)][:n_req]       # 2040, 2037, ...: they cross 2,048 at different steps
    toks = [torch.randint(0, CONFIG["vocab_size"], (n + n_dec,), generator=g).tolist() for n in [2040 - 3 * i for i in range(16)]][:n_req]
    ec = EngineConfig(dtype="bfloat16", max_cache_tokens=n_req * 2112, max_requests=n_req + 2)
    runner = build_runner(config=CONFIG, seed=2, engine_config=ec, init_std=0.03, norm_noise=0.1)
    assert runner.use_graphs
    cfg = pm.PlainConfig(CONFIG)
    w = plain_weights(runner.model)
    got = {i: [] for i in range(n_req)}
    with torch.inference_mode():
        for i in range(n_req):
            runner.start_request(f"b{i}")
            got[i].append(runner.step([StepEntry(f"b{i}", toks[i][:lens[i]], want=[lens[i] - 1])]).float().cpu()[0])
        for d in range(n_dec):
            lg = runner.step([StepEntry(f"b{i}", [toks[i][lens[i] + d]], want=[0]) for i in range(n_req)]).float().cpu()
            for i in range(n_req):
                got[i].append(lg[i])
        from omniserver_b200 import ops
        ops.kernels().check_device_errors()
        for i in range(n_req):
            runner.end_request(f"b{i}")
    assert len(runner._graphs) >= 1 and all(p == 0 for p in runner.cache.pages_in_use())
    for i in range(n_req):
        rows = list(range(lens[i] - 1, lens[i] + n_dec))
        want = _plain_rows(cfg, w, ("bench", i), toks[i], rows)
        for k, p in enumerate(rows):
            ref, lg = want[p], got[i][k]
            err = (lg - ref).abs().max().item()
            assert err < 5e-2 * max(1.0, ref.abs().max().item()), f"request {i} place {p}: {err}"
            assert ((lg - ref).norm() / ref.norm()).item() < 3e-2, f"request {i} place {p}"
