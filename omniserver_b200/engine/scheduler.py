"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, retires, and decides what happens when pages run out.

It follows omniserve/scheduler.py:36-121 in names and in the shape of a step (retire, continue
prompts in flight, admit, decode everything that is ready), with these differences:

* a prompt is just portions: several prompts may be in flight and a portion may be cut anywhere
  (the reference allows one chunked prompt at a time and admits nothing beside it, scheduler.py:63-94);
* ``max_prefill_tokens`` is the step's budget of prompt tokens, as in the reference (decoded
  tokens are not counted, scheduler.py:58,96), and also the largest portion;
* pages are finite.  Before a step every entry must get its pages.  Decodes come first, oldest
  request first.  A prompt portion that does not fit is cut to the free pages or left for a later
  step.  A decode that does not fit preempts the request admitted last (possibly itself): its
  pages are given back, it returns to the front of the waiting queue and is later recomputed
  from its prompt plus the tokens it already produced.  A lone request that cannot fit at all
  is aborted, since waiting would not help.
* ``max_seq_len`` is enforced when a request is added (the reference declares it and never
  checks it, scheduler.py:25).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, List, Optional, Tuple

from .request import Sequence, Status


@dataclass
class SchedulerConfig:
    max_running: int = 8             # most requests in the batch at once
    max_prefill_per_step: int = 1    # most new requests admitted in one step
    max_prefill_tokens: int = 8192   # prompt tokens per step, over all prompts in flight
    max_seq_len: int = 4096          # hard limit of prompt + generated tokens


@dataclass
class ScheduledEntry:
    seq: Sequence
    start: int        # first token (index into prompt + outputs) this step computes
    count: int        # how many tokens
    wants_logits: bool  # the portion ends at the request's last token

    @property
    def is_decode(self) -> bool:
        return self.count == 1 and self.seq.num_output_tokens > 0 and self.wants_logits


@dataclass
class SchedulerOutput:
    entries: List[ScheduledEntry] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    aborted: List[Sequence] = field(default_factory=list)

    @property
    def decode(self) -> List[Sequence]:
        return [e.seq for e in self.entries if e.is_decode]

    @property
    def prefill(self) -> List[Sequence]:
        return [e.seq for e in self.entries if not e.is_decode]

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    """``cache`` is the cache manager (only its host-side accounting is used here)."""

    def __init__(self, config: SchedulerConfig, cache, on_admit: Optional[Callable[[Sequence], None]] = None,
                 on_release: Optional[Callable[[Sequence], None]] = None):
        self.config = config
        self.cache = cache
        # hooks by which the engine starts and ends a request's cache (state slot, pages)
        self.on_admit = on_admit or (lambda seq: cache.begin(seq.request_id))
        self.on_release = on_release or (lambda seq: cache.finish(seq.request_id))
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self._admitted = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def add(self, seq: Sequence) -> None:
        limit = self.config.max_seq_len
        need = seq.num_prompt_tokens + seq.request.sampling.max_new_tokens
        if need > limit:
            raise ValueError(f"request {seq.request_id}: prompt ({seq.num_prompt_tokens}) + max_new_tokens "
                             f"({seq.request.sampling.max_new_tokens}) exceeds max_seq_len ({limit})")
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, request_id: str) -> None:
        for q in (self.waiting, self.running):
            for seq in list(q):
                if seq.request_id == request_id:
                    seq.status = Status.ABORTED
                    if seq in self.waiting:
                        self.waiting.remove(seq)

    # ------------------------------------------------------------------ one step's decision
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        cfg = self.config
        cache = self.cache
        self.free_finished()  # requests aborted between steps leave here
        granted: List[Tuple[Sequence, int]] = []
        free = list(cache.free_pages())

        def needed(seq: Sequence, n: int) -> List[int]:
            return cache.pages_needed(seq.request_id, n)

        def fits(seq: Sequence, n: int) -> bool:
            return all(k <= f for k, f in zip(needed(seq, n), free))

        def grant(seq: Sequence, n: int) -> None:
            for gi, k in enumerate(needed(seq, n)):
                free[gi] -= k
            granted.append((seq, n))

        def refresh_free() -> None:
            free[:] = cache.free_pages()
            for s, n in granted:
                for gi, k in enumerate(needed(s, n)):
                    free[gi] -= k

        def largest_fit(seq: Sequence, n: int) -> int:
            lo, hi = 0, n
            while lo < hi:
                mid = (lo + hi + 1) // 2
                if fits(seq, mid):
                    lo = mid
                else:
                    hi = mid - 1
            return lo

        # 1) decodes first, oldest request first; a decode without a page preempts the request
        #    admitted last (which may be itself)
        for seq in sorted([s for s in self.running if s.is_decoding], key=lambda s: s.admit_order):
            if seq.status != Status.RUNNING:
                continue  # preempted by an older decode (a request that left ``running`` is no longer RUNNING)
            while not fits(seq, 1):
                victim = max(self.running, key=lambda s: s.admit_order)
                if victim is seq and len(self.running) == 1:
                    self._abort_running(seq)
                    out.aborted.append(seq)
                    break
                self._preempt(victim)
                out.preempted.append(victim)
                refresh_free()
                if victim is seq:
                    break
            if seq.status == Status.RUNNING:
                grant(seq, 1)

        # 2) prompts in flight, oldest first: as much as the budget and the free pages allow
        budget = cfg.max_prefill_tokens
        for seq in sorted([s for s in self.running if not s.is_decoding], key=lambda s: s.admit_order):
            n = largest_fit(seq, min(seq.remaining, budget))
            if n > 0:
                grant(seq, n)
                budget -= n

        # 3) admit new requests while there is room for them to start (never in a step that had to
        #    preempt: the pages just won back are for the requests that are running)
        admitted = 0
        while (not out.preempted and self.waiting and len(self.running) < cfg.max_running and admitted < cfg.max_prefill_per_step
               and budget > 0 and cache.state.num_free > 0 and all(f > 0 for f in free)):
            seq = self.waiting.popleft()
            if seq.status == Status.ABORTED:
                continue
            seq.status = Status.RUNNING
            seq.admit_order = self._admitted
            self._admitted += 1
            self.running.append(seq)
            self.on_admit(seq)
            n = largest_fit(seq, min(seq.remaining, budget))
            if n > 0:
                grant(seq, n)
                budget -= n
            admitted += 1

        # 4) nothing can move: every page is held by prompts that cannot grow. The request admitted
        #    last gives way; alone, it can never fit and is aborted.
        if not granted and self.running:
            victim = max(self.running, key=lambda s: s.admit_order)
            if len(self.running) == 1:
                self._abort_running(victim)
                out.aborted.append(victim)
            else:
                self._preempt(victim)
                out.preempted.append(victim)

        for seq, n in granted:
            seq.scheduled = n
            out.entries.append(ScheduledEntry(seq, seq.num_computed, n, seq.num_computed + n == seq.total_len))
        # decodes first keeps the rows of running requests stable (omniserve/runners/multimodal.py:255-263)
        out.entries.sort(key=lambda e: (0 if e.is_decode else 1, e.seq.admit_order))
        return out

    def _preempt(self, victim: Sequence) -> None:
        """The victim's cache is given back; it returns to the front of the queue and will be
        recomputed from its prompt plus the tokens it has produced."""
        self.running.remove(victim)
        self.on_release(victim)
        victim.num_computed = 0
        victim.scheduled = 0
        victim.num_preemptions += 1
        victim.status = Status.WAITING
        self.num_preemptions += 1
        self.waiting.appendleft(victim)

    def _abort_running(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.on_release(seq)
        seq.status = Status.ABORTED

    # ------------------------------------------------------------------ after the step
    def free_finished(self) -> List[Sequence]:
        """Retires the requests that ended (finished or aborted): their pages and slot are given
        back. Returns them so that the engine can tell its clients."""
        done = [s for s in self.running if s.status != Status.RUNNING]
        self.running = [s for s in self.running if s.status == Status.RUNNING]
        for s in done:
            self.on_release(s)
        return done
