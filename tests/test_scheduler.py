"""The scheduler's decisions without a GPU: admission, portions under the token budget, decodes
first, retirement, and what happens when pages run out (cut, wait, preempt, abort)."""

import pytest
import torch

from omniserver_b200.cache import CacheManager
from omniserver_b200.engine import Request, SamplingParams, Scheduler, SchedulerConfig, Sequence, Status
from omniserver_b200.models.decoder import EntryNeeds
from omniserver_b200.parts.base import KVCacheNeed


def cache(num_pages=64, page_size=4, max_requests=8, window=None):
    needs = [EntryNeeds(KVCacheNeed(1, 8, window), [], None)]
    return CacheManager(needs, [], page_size, num_pages, max_requests, torch.float32, "cpu", allocate=False)


def seq(n_prompt, max_new=4, rid=None):
    r = Request(prompt=list(range(1, n_prompt + 1)), sampling=SamplingParams(max_new_tokens=max_new))
    if rid:
        r.request_id = rid
    return Sequence(request=r)


def run_step(sched, cm, token=7):
    """What the engine does around schedule(): run the entries, append tokens, retire."""
    out = sched.schedule()
    for e in out.entries:
        cm.reserve(e.seq.request_id, e.count)
    for e in out.entries:
        cm.commit(e.seq.request_id, e.count)
        e.seq.num_computed += e.count
        if e.wants_logits:
            e.seq.append_token(token)
            e.seq.maybe_finish()
    cm.check_invariants()
    sched.free_finished()
    return out


def test_whole_prompts_are_packed_then_decoded_together():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_running=8, max_prefill_per_step=8, max_prefill_tokens=100), cm)
    a, b, c = seq(5), seq(17), seq(33)
    for x in (a, b, c):
        s.add(x)
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count, e.wants_logits) for e in out.entries] == [(a, 0, 5, True), (b, 0, 17, True), (c, 0, 33, True)]
    out = run_step(s, cm)
    assert [e.is_decode for e in out.entries] == [True] * 3 and out.decode == [a, b, c]
    assert [e.start for e in out.entries] == [5, 17, 33]


def test_budget_cuts_prompts_into_portions_beside_decodes():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_running=4, max_prefill_per_step=1, max_prefill_tokens=16), cm)
    a, b = seq(5, max_new=50), seq(40)
    s.add(a)
    s.add(b)
    out = run_step(s, cm)
    assert [(e.seq, e.count) for e in out.entries] == [(a, 5)]          # one admission per step
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count, e.wants_logits) for e in out.entries] == [(a, 5, 1, True), (b, 0, 16, False)]
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count) for e in out.entries] == [(a, 6, 1), (b, 16, 16)]
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count, e.wants_logits) for e in out.entries] == [(a, 7, 1, True), (b, 32, 8, True)]
    out = run_step(s, cm)
    assert out.decode == [a, b] and out.num_tokens == 2


def test_budget_is_shared_by_prompts_in_flight_oldest_first():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_running=4, max_prefill_per_step=2, max_prefill_tokens=10), cm)
    a, b = seq(14), seq(9)
    s.add(a)
    s.add(b)
    out = run_step(s, cm)
    assert [(e.seq, e.count) for e in out.entries] == [(a, 10)]          # budget used up by the first
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count) for e in out.entries] == [(a, 10, 4), (b, 0, 6)]
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count) for e in out.entries] == [(a, 14, 1), (b, 6, 3)]


def test_max_running_and_retirement_free_everything():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_running=2, max_prefill_per_step=4, max_prefill_tokens=64), cm)
    seqs = [seq(6, max_new=2) for _ in range(5)]
    for x in seqs:
        s.add(x)
    steps = 0
    while s.has_work():
        out = run_step(s, cm)
        assert len(s.running) <= 2
        steps += 1
        assert steps < 50
    assert all(x.status == Status.FINISHED and x.num_output_tokens == 2 for x in seqs)
    assert cm.pages_in_use() == [0] and cm.state.num_free == 8 and not cm.requests


def test_stop_token_finishes_and_max_seq_len_is_enforced():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_seq_len=20), cm)
    with pytest.raises(ValueError, match="max_seq_len"):
        s.add(seq(18, max_new=4))
    a = seq(3, max_new=10)
    a.request.sampling.stop_token_ids.append(7)
    s.add(a)
    run_step(s, cm, token=7)
    assert a.status == Status.FINISHED and a.output_token_ids == [7] and not s.has_work()


def test_abort_waiting_and_running():
    cm = cache()
    s = Scheduler(SchedulerConfig(max_running=1), cm)
    a, b = seq(4, rid="a"), seq(4, rid="b")
    s.add(a)
    s.add(b)
    run_step(s, cm)
    s.abort("b")
    s.abort("a")
    assert b.status == Status.ABORTED and not s.waiting
    out = s.schedule()
    assert not out.entries and not s.running and cm.pages_in_use() == [0]


def test_a_portion_is_cut_to_the_free_pages_or_waits():
    cm = cache(num_pages=6, page_size=4)                      # 24 tokens
    s = Scheduler(SchedulerConfig(max_running=4, max_prefill_per_step=2, max_prefill_tokens=64), cm)
    a, b = seq(14, max_new=2), seq(20, max_new=2)
    s.add(a)
    s.add(b)
    out = run_step(s, cm)
    # a takes 4 pages (14 tokens); b is cut to the 2 pages left
    assert [(e.seq, e.count, e.wants_logits) for e in out.entries] == [(a, 14, True), (b, 8, False)]
    out = run_step(s, cm)
    # a decodes inside its last page; b cannot grow and waits without being preempted
    assert [(e.seq, e.count) for e in out.entries] == [(a, 1)] and not out.preempted
    assert a.status == Status.FINISHED
    out = run_step(s, cm)
    assert [(e.seq, e.start, e.count) for e in out.entries] == [(b, 8, 12)]


def test_a_decode_without_a_page_preempts_the_request_admitted_last():
    cm = cache(num_pages=4, page_size=4)                      # 16 tokens
    s = Scheduler(SchedulerConfig(max_running=4, max_prefill_per_step=2, max_prefill_tokens=64), cm)
    a, b = seq(8, max_new=6, rid="a"), seq(7, max_new=6, rid="b")
    s.add(a)
    s.add(b)
    run_step(s, cm)                                           # both prompts in, 4 pages held
    out = run_step(s, cm)                                     # a needs a 3rd page: b (admitted last) gives way
    assert out.preempted == [b] and [(e.seq, e.count) for e in out.entries] == [(a, 1)]
    assert b.status == Status.WAITING and b.num_computed == 0 and b.num_output_tokens == 1
    assert s.waiting[0] is b and "b" not in cm.requests
    while a.status == Status.RUNNING:
        out = run_step(s, cm)
    # b comes back: prompt and its first token are recomputed as one prompt
    while b.status != Status.FINISHED:
        out = run_step(s, cm)
        if out.entries and out.entries[0].seq is b and out.entries[0].start == 0:
            assert out.entries[0].count == 8 and out.entries[0].wants_logits
    assert b.num_output_tokens == 6 and b.num_preemptions >= 1 and s.num_preemptions >= 1
    assert cm.pages_in_use() == [0]


def test_the_decoding_request_itself_may_be_the_one_preempted():
    cm = cache(num_pages=4, page_size=4)
    s = Scheduler(SchedulerConfig(max_running=4, max_prefill_per_step=1, max_prefill_tokens=64), cm)
    a, b = seq(8, max_new=2, rid="a"), seq(8, max_new=8, rid="b")
    s.add(a)
    s.add(b)
    run_step(s, cm)
    run_step(s, cm)            # a decodes (needs page 3), b's prompt enters: 2+... pages
    # now both decode; whoever was admitted last (b) gives way when pages run out
    out = run_step(s, cm)
    while s.has_work():
        out = run_step(s, cm)
    assert a.status == b.status == Status.FINISHED and cm.pages_in_use() == [0]


def test_a_request_that_can_never_fit_is_aborted():
    cm = cache(num_pages=3, page_size=4)                      # 12 tokens
    s = Scheduler(SchedulerConfig(max_running=2, max_prefill_tokens=64), cm)
    a = seq(10, max_new=8)
    s.add(a)
    steps = 0
    aborted = []
    while s.has_work():
        aborted += run_step(s, cm).aborted
        steps += 1
        assert steps < 20
    assert aborted == [a] and a.status == Status.ABORTED and a.num_output_tokens == 3
    assert cm.pages_in_use() == [0] and not cm.requests
    b = seq(30, max_new=1)
    s.add(b)
    while s.has_work():
        aborted += run_step(s, cm).aborted
        steps += 1
        assert steps < 40
    assert b in aborted and cm.pages_in_use() == [0]


def test_windowed_group_lets_a_long_request_run_in_few_pages():
    cm = cache(num_pages=5, page_size=4, window=6)            # 20 tokens of pages, window 6
    s = Scheduler(SchedulerConfig(max_running=1, max_prefill_tokens=8, max_seq_len=200), cm)
    a = seq(30, max_new=40)
    s.add(a)
    while s.has_work():
        out = run_step(s, cm)
        assert not out.preempted and not out.aborted
        assert cm.pages_in_use()[0] <= 5
    assert a.status == Status.FINISHED and a.num_output_tokens == 40
