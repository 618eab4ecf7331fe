"""Which schedule entries the model hands to a multi-layer kernel as one run: found by asking the blocks to
describe themselves, never by the architecture's name. Blocks here are stand-ins defined in the test."""

import torch

from omniserver_b200.models.layer_run import FusedLayerRun, find_runs
from omniserver_b200.models.spec import ScheduleEntry
from omniserver_b200.parts.base import CacheBinding


class Position:
    pass


POS = Position()


def desc(nh=4, nkv=2, hd=64, H=256, I=512, bias=True, position=POS, window=None):
    t = lambda *shape: torch.zeros(*shape, dtype=torch.bfloat16)
    return {"block": "prenorm_rms", "norm_attn": t(H), "eps_attn": 1e-6, "norm_ffn": t(H), "eps_ffn": 1e-5,
            "mixer": {"kind": "gqa_rope", "w_qkv": t((nh + 2 * nkv) * hd, H), "b_qkv": t((nh + 2 * nkv) * hd) if bias else None,
                      "w_o": t(H, nh * hd), "nh": nh, "nkv": nkv, "hd": hd, "scale": hd ** -0.5, "window": window,
                      "position": position},
            "ffn": {"kind": "swiglu", "w_gate_up": t(2 * I, H), "w_down": t(H, I), "intermediate_size": I}}


class Block:
    def __init__(self, d):
        self.d = d

    def decode_descriptor(self):
        return self.d


def binding(group=0, nkv=2, hd=64, writes=True):
    c = torch.zeros(3, nkv, 8, hd, dtype=torch.bfloat16)
    return CacheBinding(group=group, k_cache=c, v_cache=c.clone(), writes=writes)


def runs_of(blocks, schedule, bindings):
    return {i: (r.start, r.end) for i, r in find_runs(blocks, schedule, bindings).items()}


def test_alike_layers_form_one_run():
    blocks = [Block(desc()) for _ in range(5)]
    sched = [ScheduleEntry(i) for i in range(5)]
    assert runs_of(blocks, sched, [binding() for _ in range(5)]) == {0: (0, 5)}


def test_a_part_without_a_descriptor_splits_the_run_and_runs_alone():
    blocks = [Block(desc()), Block(desc()), Block(None), Block(desc()), Block(desc()), Block(desc())]
    sched = [ScheduleEntry(i) for i in range(6)]
    assert runs_of(blocks, sched, [binding() for _ in range(6)]) == {0: (0, 2), 3: (3, 6)}
    # another kind of mixer or feed-forward is no part of a run either
    d = desc()
    d["mixer"]["kind"] = "decayed_sum"
    blocks[1] = Block(d)
    assert runs_of(blocks, sched, [binding() for _ in range(6)]) == {3: (3, 6)}


def test_sizes_groups_and_positions_must_agree():
    sched = [ScheduleEntry(i) for i in range(4)]
    blocks = [Block(desc()), Block(desc()), Block(desc(I=1024)), Block(desc(I=1024))]
    assert runs_of(blocks, sched, [binding() for _ in range(4)]) == {0: (0, 2), 2: (2, 4)}
    blocks = [Block(desc()) for _ in range(4)]
    assert runs_of(blocks, sched, [binding(0), binding(0), binding(1), binding(1)]) == {0: (0, 2), 2: (2, 4)}
    blocks = [Block(desc()), Block(desc()), Block(desc(position=Position())), Block(desc())]
    assert runs_of(blocks, sched, [binding() for _ in range(4)]) == {0: (0, 2)}
    # a window is a constant of the layer, not of the run
    blocks = [Block(desc(window=64)), Block(desc()), Block(desc(window=8))]
    assert runs_of(blocks, sched[:3], [binding() for _ in range(3)]) == {0: (0, 3)}


def test_repeated_layers_and_borrowed_caches_stay_out():
    blocks = [Block(desc()) for _ in range(4)]
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(3)]
    assert runs_of(blocks, sched, [binding() for _ in range(5)]) == {3: (3, 5)}
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=0), ScheduleEntry(3)]
    bs = [binding(), binding(), binding(writes=False), binding()]
    assert runs_of(blocks, sched, bs) == {0: (0, 2)}


def test_run_collects_what_the_kernel_needs():
    blocks = [Block(desc(window=None)), Block(desc(window=32))]
    bs = [binding(), binding()]
    run = find_runs(blocks, [ScheduleEntry(0), ScheduleEntry(1)], bs)[0]
    assert isinstance(run, FusedLayerRun) and (run.nh, run.nkv, run.hd, run.I, run.H, run.group) == (4, 2, 64, 512, 256, 0)
    assert [l["window"] for l in run._layers] == [None, 32]
    assert run._layers[1]["k_cache"] is bs[1].k_cache and run._layers[0]["eps_ffn"] == 1e-5
