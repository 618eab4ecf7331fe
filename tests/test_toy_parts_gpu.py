"""Generality of the layer machinery, shown with toy parts that are defined here and registered
without a change to the framework's files: a mixer with per-request state of its own (no pages), a
feed-forward with routing, and a position encoding without rotation; and a layer schedule that
runs a layer twice and lets one run read another run's cache.  The toy model is stepped through
the product's step function in several cuts and compared with a plain whole-sequence evaluation
written here.  The toy parts use torch ops on the GPU; they are test code, not a model of anyone's.
"""

import math

import pytest
import torch

from plain import model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
H, NH, NKV, HD, I, V = 64, 4, 2, 16, 96, 300
DECAY = 0.8


def _register():
    from omniserver_b200.parts import base as pb
    from omniserver_b200.parts.base import FeedForward, Mixer, ParamSpec, PositionEncoding, StateNeed

    class DecayMixer(Mixer):
        """y_t = W s_t with s_t = decay * s_{t-1} + x_t: a running state per request, carried
        across steps in the request's state slot."""

        def __init__(self, hidden_size, decay, prefix, position=None):
            self.h, self.decay, self.prefix = hidden_size, decay, prefix
            self.w_weight = None

        def param_specs(self):
            return [ParamSpec("w_weight", ("w.weight",), ((self.h, self.h),))]

        def cache_needs(self):
            return [StateNeed("acc", (self.h,), torch.float32)]

        def forward(self, ctx, x, binding):
            state = binding.state["acc"]
            y = torch.empty_like(x)
            slots = ctx.state_slot.tolist()
            cu = ctx.cu_q.tolist()
            for s, slot in enumerate(slots):
                acc = state[slot]
                for t in range(cu[s], cu[s + 1]):
                    acc = self.decay * acc + x[t].float()
                    y[t] = (self.w_weight.float() @ acc).to(x.dtype)
                state[slot] = acc
            return y

    class RoutedFFN(FeedForward):
        """Two experts, the router picks one per token (argmax of the router logits in fp32)."""

        def __init__(self, hidden_size, prefix):
            self.h, self.prefix = hidden_size, prefix

        def param_specs(self):
            return [ParamSpec("router", ("router.weight",), ((2, self.h),)),
                    ParamSpec("e0", ("experts.0.weight",), ((self.h, self.h),)),
                    ParamSpec("e1", ("experts.1.weight",), ((self.h, self.h),))]

        def forward(self, ctx, x):
            pick = (x.float() @ self.router.float().T).argmax(-1)
            y0, y1 = x.float() @ self.e0.float().T, x.float() @ self.e1.float().T
            return torch.where(pick[:, None] == 0, y0, y1).to(x.dtype)

    class NoRotation(PositionEncoding):
        """A position encoding that leaves queries and keys alone: it has no tables and is no rotation."""

        def __init__(self):
            pass

        def prepare(self, ctx, state):
            return None

    class ShiftedIndexScale(PositionEncoding):
        """Another encoding, nothing like a rotation: every query and key is scaled by 1 + slope * p, where p
        is the token's position: one column given with the prompt, and index + shift for the tokens after it,
        with the shift kept in a state field of the encoding's own."""

        position_columns = 1

        def __init__(self, slope):
            self.slope = float(slope)

        def state_needs(self):
            return [StateNeed("toy_shift", (1,), torch.int32, shared=True)]

        def request_state(self, given, num_prompt_tokens):
            shift = 0 if given is None else int(given.max()) + 1 - num_prompt_tokens
            return {"toy_shift": [shift]}

        def prepare(self, ctx, state):
            # tokens with given positions read their column; the others sit at their index in the request + shift
            q_len = ctx.cu_q[1:] - ctx.cu_q[:-1]
            first = (ctx.seq_lens - q_len)[ctx.tok_seq.long()]
            offset = torch.arange(ctx.T, device=ctx.device, dtype=torch.int32) - ctx.cu_q[ctx.tok_seq.long()]
            derived = first + offset + state["toy_shift"][ctx.state_slot.long(), 0][ctx.tok_seq.long()]
            given = ctx.pos_mode[ctx.tok_seq.long()] == 0
            return torch.where(given, ctx.positions[0], derived)

        def apply(self, ctx, tables, qkv, num_heads, num_kv_heads, head_dim):
            n = (num_heads + num_kv_heads) * head_dim
            qkv[:, :n] = (qkv[:, :n].float() * (1.0 + self.slope * tables.float())[:, None]).to(qkv.dtype)

    if "toy_decay" not in pb.MIXERS:
        pb.register_mixer("toy_decay", DecayMixer)
        pb.register_feed_forward("toy_routed", RoutedFFN)
        pb.register_position_encoding("toy_none", NoRotation)
        pb.register_position_encoding("toy_scale", ShiftedIndexScale)


def _spec():
    from omniserver_b200.models import LayerSpec, ModelSpec, ScheduleEntry
    from omniserver_b200.parts.base import PartSpec
    norm = PartSpec("rmsnorm", {"dim": H, "eps": 1e-5})
    rope = PartSpec("mrope", {"head_dim": HD, "theta": 1e4, "sections": (2, 3, 3)})
    none = PartSpec("toy_none", {})
    attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD})
    swiglu = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I})
    layers = [
        LayerSpec("layers.0.", PartSpec("toy_decay", {"hidden_size": H, "decay": DECAY}), swiglu, norm, norm),
        LayerSpec("layers.1.", attn, PartSpec("toy_routed", {"hidden_size": H}), norm, norm, position=rope),
        LayerSpec("layers.2.", attn, swiglu, norm, norm, position=none),
    ]
    # layer 1 runs twice (two caches of its own); the run of layer 2 reads the first run's cache
    schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=1), ScheduleEntry(1)]
    return ModelSpec("ToyForTests", V, H, layers, schedule, norm, tie_word_embeddings=True)


def _build(dtype):
    from omniserver_b200.cache import CacheManager
    from omniserver_b200.engine.step import ModelRunner
    from omniserver_b200.models import DecoderModel
    from omniserver_b200.weights import fill_random
    _register()
    model = DecoderModel(_spec())
    fill_random(model, 7, dtype, DEV, std=0.08, norm_noise=0.1, store_dtype=torch.float32 if dtype == torch.float32 else torch.bfloat16)
    cache = CacheManager(model.entry_needs(), model.shared_state_needs(), 16, 32, 4, dtype, DEV)
    return model, ModelRunner(model, cache, dtype, DEV)


def _plain(model, toks):
    """Whole sequence, no cache, float32 on the CPU, from the same tensors."""
    T = len(toks)
    f = lambda t: t.detach().float().cpu()
    x = f(model.embed.weight)[torch.tensor(toks)]
    res = None
    pos = pm.text_positions(T)
    cos, sin = pm.mrope_cos_sin(pos, 1e4, HD, (2, 3, 3))
    kv_of_entry = {}
    for ei, e in enumerate(model.spec.schedule):
        blk = model.blocks[e.layer]
        res = pm.add_residual(res, x)
        y = pm.rms_norm(res, f(blk.mixer_norm.weight), 1e-5)
        mx = blk.mixer
        if e.layer == 0:
            acc = torch.zeros(H)
            out = []
            for t in range(T):
                acc = DECAY * acc + y[t]
                out.append(f(mx.w_weight) @ acc)
            x = torch.stack(out)
        else:
            w, b = f(mx.qkv.weight), f(mx.qkv.bias)
            qkv = y @ w.T + b
            q = qkv[:, :NH * HD].view(T, NH, HD)
            k = qkv[:, NH * HD:(NH + NKV) * HD].view(T, NKV, HD)
            v = qkv[:, (NH + NKV) * HD:].view(T, NKV, HD)
            if e.layer == 1:
                q, k = pm.apply_rotary(q, cos, sin), pm.apply_rotary(k, cos, sin)
            if e.cache_of is None:
                kv_of_entry[ei] = (k, v)
            else:
                k, v = kv_of_entry[e.cache_of]
            x = pm.o_proj(pm.attention(q, k, v), f(mx.out.weight))
        res = pm.add_residual(res, x)
        y = pm.rms_norm(res, f(blk.ffn_norm.weight), 1e-5)
        ff = blk.ffn
        if e.layer == 1:
            pick = (y @ f(ff.router).T).argmax(-1)
            x = torch.where(pick[:, None] == 0, y @ f(ff.e0).T, y @ f(ff.e1).T)
        else:
            gu = f(ff.gate_up.weight)
            x = pm.swiglu(y, gu[:I], gu[I:], f(ff.down.weight))
    res = pm.add_residual(res, x)
    return pm.lm_head(pm.rms_norm(res, f(model.final_norm.weight), 1e-5), f(model.embed.weight))


def test_toy_parts_register_build_and_step():
    from omniserver_b200.engine.step import StepEntry
    model, runner = _build(torch.float32)
    needs = model.entry_needs()
    assert [n.kv is None for n in needs] == [True, False, False, False]
    assert needs[0].states[0].name == "acc" and needs[2].cache_of == 1
    assert len(runner.cache.groups) == 1 and runner.cache.groups[0].entries == [1, 3]   # the borrower owns no pages
    g = torch.Generator().manual_seed(1)
    seqs = {r: torch.randint(0, V, (n,), generator=g).tolist() for r, n in (("a", 37), ("b", 20), ("c", 9))}
    want = {r: _plain(model, t) for r, t in seqs.items()}
    # a: whole; then the same requests in portions, mixed in one batch, with decode steps at the end
    with torch.inference_mode():
        runner.start_request("a")
        got = runner.step([StepEntry("a", seqs["a"], list(range(37)))]).cpu()
        runner.end_request("a")
        assert (got - want["a"]).abs().max() < 1e-4
        cuts = {"a": [5, 2, 17, 1, 1, 11], "b": [3, 16, 1], "c": [2, 2, 5]}
        pos = {r: 0 for r in seqs}
        out = {r: [] for r in seqs}
        for r in seqs:
            runner.start_request(r)
        step = 0
        while any(pos[r] < len(seqs[r]) for r in seqs):
            entries = []
            for r in seqs:
                if pos[r] < len(seqs[r]) and step < len(cuts[r]) + 8:
                    n = cuts[r][step] if step < len(cuts[r]) else 1
                    n = min(n, len(seqs[r]) - pos[r])
                    entries.append(StepEntry(r, seqs[r][pos[r]:pos[r] + n], list(range(n))))
            lg = runner.step(entries).cpu()
            o = 0
            for e in entries:
                n = len(e.tokens)
                out[e.request_id].append(lg[o:o + n])
                o += n
                pos[e.request_id] += n
            step += 1
        for r in seqs:
            runner.end_request(r)
            assert (torch.cat(out[r]) - want[r]).abs().max() < 1e-4, r
    # the state slot of a finished request is zeroed for its next user
    assert runner.cache.state.num_free == 4


def test_toy_model_in_bfloat16_runs_on_the_fast_kernels():
    from omniserver_b200.engine.step import StepEntry
    model, runner = _build(torch.bfloat16)
    toks = torch.randint(0, V, (50,), generator=torch.Generator().manual_seed(2)).tolist()
    want = _plain(model, toks)
    with torch.inference_mode():
        runner.start_request("x")
        a = runner.step([StepEntry("x", toks[:33], list(range(33)))]).cpu()
        b = torch.cat([runner.step([StepEntry("x", [t], [0])]).cpu() for t in toks[33:]])
        runner.end_request("x")
    got = torch.cat([a, b])
    rel = ((got - want).norm() / want.norm()).item()
    assert rel < 3e-2, rel


def test_a_position_encoding_with_one_column_and_state_of_its_own():
    """An encoding defined in the test: one position column per token, a state field of its own that its
    ``request_state`` fills from the prompt's positions, and a change of q and k that is no rotation. The
    engine's files know none of this; it carries the column, writes the state row and asks the encoding
    which columns to send with a span."""
    import numpy as np
    from omniserver_b200.cache import CacheManager
    from omniserver_b200.engine.step import ModelRunner, StepEntry
    from omniserver_b200.models import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry
    from omniserver_b200.parts.base import PartSpec
    from omniserver_b200.weights import fill_random
    _register()
    slope = 0.01
    norm = PartSpec("rmsnorm", {"dim": H, "eps": 1e-5})
    scale = PartSpec("toy_scale", {"slope": slope})
    attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": NH, "num_kv_heads": NKV, "head_dim": HD})
    swiglu = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I})
    layers = [LayerSpec(f"layers.{i}.", attn, swiglu, norm, norm, position=scale) for i in range(2)]
    spec = ModelSpec("ToyScaleForTests", V, H, layers, [ScheduleEntry(0), ScheduleEntry(1)], norm, tie_word_embeddings=True)
    model = DecoderModel(spec)
    assert model.position_columns == 1
    fill_random(model, 11, torch.float32, DEV, std=0.08, norm_noise=0.1, store_dtype=torch.float32)
    cache = CacheManager(model.entry_needs(), model.shared_state_needs(), 16, 16, 2, torch.float32, DEV)
    assert "toy_shift" in cache.state.fields
    runner = ModelRunner(model, cache, torch.float32, DEV)

    n_prompt, n_more = 21, 5
    toks = torch.randint(0, V, (n_prompt + n_more,), generator=torch.Generator().manual_seed(3)).tolist()
    given = np.concatenate([np.arange(8), 8 + 3 * np.arange(n_prompt - 8)])[None, :]    # the prompt's own positions
    shift = int(given.max()) + 1 - n_prompt
    pos_all = torch.tensor(np.concatenate([given[0], np.arange(n_prompt, n_prompt + n_more) + shift]), dtype=torch.float32)

    def plain():
        f = lambda t: t.detach().float().cpu()
        T = len(toks)
        x = f(model.embed.weight)[torch.tensor(toks)]
        res = None
        for blk in model.blocks:
            res = pm.add_residual(res, x)
            y = pm.rms_norm(res, f(blk.mixer_norm.weight), 1e-5)
            qkv = y @ f(blk.mixer.qkv.weight).T + f(blk.mixer.qkv.bias)
            s = (1.0 + slope * pos_all)[:, None, None]
            q = qkv[:, :NH * HD].view(T, NH, HD) * s
            k = qkv[:, NH * HD:(NH + NKV) * HD].view(T, NKV, HD) * s
            v = qkv[:, (NH + NKV) * HD:].view(T, NKV, HD)
            x = pm.o_proj(pm.attention(q, k, v), f(blk.mixer.out.weight))
            res = pm.add_residual(res, x)
            y = pm.rms_norm(res, f(blk.ffn_norm.weight), 1e-5)
            gu = f(blk.ffn.gate_up.weight)
            x = pm.swiglu(y, gu[:I], gu[I:], f(blk.ffn.down.weight))
        res = pm.add_residual(res, x)
        return pm.lm_head(pm.rms_norm(res, f(model.final_norm.weight), 1e-5), f(model.embed.weight))

    want = plain()
    with torch.inference_mode():
        runner.start_request("r", given, n_prompt)
        assert int(cache.state.tensors["toy_shift"][cache.requests["r"].slot, 0]) == shift
        outs, a = [], 0
        for n in (7, 2, 9, 6):      # the last portion reaches 3 tokens past the prompt
            b = a + n
            outs.append(runner.step([StepEntry("r", toks[a:b], list(range(n)),
                                               positions=runner.positions_for(given, n_prompt, a, b)
                                               if b <= n_prompt else None if a >= n_prompt else
                                               np.concatenate([given[:, a:], (np.arange(n_prompt, b) + shift)[None, :]], axis=1))]).cpu())
            a = b
        for t in toks[a:]:
            outs.append(runner.step([StepEntry("r", [t], [0])]).cpu())
        runner.end_request("r")
    assert (torch.cat(outs) - want).abs().max() < 1e-4
    with pytest.raises(ValueError):
        runner.start_request("bad", np.zeros((3, 4), dtype=np.int64), 4)    # three columns where the model takes one
