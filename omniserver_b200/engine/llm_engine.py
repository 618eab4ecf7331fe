"""LLMEngine: the Python entry point. Names and meanings follow omniserve/engine.py:27-92
(add_request, step, has_unfinished, abort, sequences, run_until_complete, StepDelta).

A step is: schedule -> one forward of the whole mixed batch -> sample -> retire.  The reference
runs up to two forwards per step (packed prefill, then decode or chunk+decode, engine.py:57-65);
here the scheduler's entries always run as one batch.
"""

from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import torch

from .. import ops
from ..config import EngineConfig, resolve, resolve_dir
from ..config.model_config import read_config_dict
from ..sampling import SampleHandle, Sampler
from .request import PENDING_TOKEN, Request, SamplingParams, Sequence, Status
from .scheduler import Scheduler, SchedulerConfig, SchedulerOutput
from .step import ModelRunner, StepEntry



@dataclass
class _InFlight:
    """A launched step whose tokens have not been read yet."""

    handle: SampleHandle
    wanting: List[Sequence]      # row i of the sampled tokens belongs to wanting[i] ...
    fill_at: List[int]           # ... and goes to this place of its output_token_ids
    seqs: List[Sequence]         # every sequence that took part


@dataclass
class StepDelta:
    """What one request produced in one step. ``text`` is filled when a tokenizer is attached."""

    request_id: str
    new_token_ids: List[int]
    finished: bool
    text: str = ""


@torch.inference_mode(False)   # weights, caches and state outlive any inference-mode block of the caller
def build_runner(model_dir: Optional[str] = None, engine_config: Optional[EngineConfig] = None,
                 config: Optional[dict] = None, seed: int = 0, init_std: float = 0.02, norm_noise: float = 0.0,
                 random_on_device: bool = False, allocate: bool = True) -> ModelRunner:
    """Model + weights + cache + step function from a model folder, or from a configuration
    dictionary and a seed (random weights)."""
    from ..cache import CacheManager
    from ..models import DecoderModel
    from ..weights import fill_random, load_weights

    ec = engine_config or EngineConfig()
    dtype = ec.torch_dtype
    device = torch.device(ec.device)
    if model_dir is not None:
        cfg, spec = resolve_dir(model_dir)
    elif config is not None:
        cfg, spec = resolve(config)
    else:
        raise ValueError("give a model folder or a configuration")
    model = DecoderModel(spec)
    if model_dir is not None:
        load_weights(model, model_dir, dtype, device)
    else:
        fill_random(model, seed, dtype, device, std=init_std, norm_noise=norm_noise, on_device=random_on_device)
    num_pages = (ec.max_cache_tokens + ec.page_size - 1) // ec.page_size
    spare = ModelRunner.GRAPH_FILLERS if (ec.cuda_graphs and device.type == "cuda") else 0
    cache = CacheManager(model.entry_needs(), model.shared_state_needs(), ec.page_size, num_pages, ec.max_requests,
                         dtype, device, allocate=allocate, spare_slots=spare)
    runner = ModelRunner(model, cache, dtype, device, check_device_errors=ec.check_device_errors,
                         use_graphs=ec.cuda_graphs)
    runner.model_config = cfg
    return runner


class LLMEngine:
    def __init__(self, runner: ModelRunner, sched_config: Optional[SchedulerConfig] = None, seed: int = 0,
                 eos_token_id: Optional[int] = None, detokenize=None, overlap: Optional[bool] = None):
        self.runner = runner
        self.scheduler = Scheduler(sched_config or SchedulerConfig(), runner.cache,
                                   on_admit=lambda s: runner.start_request(s.request_id, s.prompt_positions, s.num_prompt_tokens),
                                   on_release=lambda s: runner.end_request(s.request_id))
        self.sampler = Sampler(seed)
        cfg = getattr(runner, "model_config", None)
        self.eos_token_id = eos_token_id if eos_token_id is not None else getattr(cfg, "eos_token_id", None)
        self._detokenize = detokenize
        self._seqs: Dict[str, Sequence] = {}
        self._history: Dict[str, Sequence] = {}
        #: launch step t+1 before reading the tokens of step t (see ``step``); on by default on a GPU
        self.overlap = (runner.device.type == "cuda") if overlap is None else bool(overlap)
        self._pending: Optional[_InFlight] = None
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0, "overlapped_steps": 0}

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_model_dir(cls, model_dir: str, engine_config: Optional[EngineConfig] = None,
                       sched_config: Optional[SchedulerConfig] = None, seed: int = 0) -> "LLMEngine":
        return cls(build_runner(model_dir=model_dir, engine_config=engine_config), sched_config, seed)

    @classmethod
    def from_random(cls, config: dict, seed: int = 0, engine_config: Optional[EngineConfig] = None,
                    sched_config: Optional[SchedulerConfig] = None, **init) -> "LLMEngine":
        return cls(build_runner(config=config, seed=seed, engine_config=engine_config, **init), sched_config, seed)

    # ------------------------------------------------------------------ requests (omniserve/engine.py:35-51)
    def add_request(self, request: Request) -> str:
        seq = Sequence(request=request)
        if request.request_id in self._seqs:
            raise ValueError(f"request id {request.request_id!r} is already in use")
        V = self.runner.vocab_size
        if min(seq.prompt_token_ids) < 0 or max(seq.prompt_token_ids) >= V:
            raise ValueError(f"request {request.request_id!r}: token id outside [0, {V})")
        if seq.prompt_positions is not None:
            self.runner.check_positions(seq.prompt_positions, seq.num_prompt_tokens)
        if request.embed_rows is not None and len(request.embed_rows):
            rows = [int(r) for r in request.embed_rows]
            if min(rows) < 0 or max(rows) >= seq.num_prompt_tokens:
                raise ValueError(f"request {request.request_id!r}: embedding row outside its prompt")
            if request.embed_values is None or tuple(request.embed_values.shape) != (len(rows), self.runner.hidden_size):
                raise ValueError(f"request {request.request_id!r}: embed_values must be "
                                 f"[{len(rows)}, {self.runner.hidden_size}]")
        sp = request.sampling
        if self.eos_token_id is not None and not sp.ignore_eos and self.eos_token_id not in sp.stop_token_ids:
            sp.stop_token_ids.append(self.eos_token_id)   # omniserve/runners/multimodal.py:53-56
        self.scheduler.add(seq)
        self._seqs[seq.request_id] = seq
        self._history[seq.request_id] = seq
        return seq.request_id

    def sequences(self) -> List[Sequence]:
        return list(self._history.values())

    def abort(self, request_id: str) -> None:
        self.scheduler.abort(request_id)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work() or self._pending is not None

    # ------------------------------------------------------------------ the step (omniserve/engine.py:53-84)
    def step(self) -> List[StepDelta]:
        """Schedules and launches one step and returns what has become known since the last call.

        With ``overlap`` the host does not wait for the step it has just launched: sampled tokens stay
        on the device for the next step's embedding lookup (``StepEntry.from_device``) and are read one
        call later, so that scheduling and launching step t+1 overlaps the device's work on step t.
        That is done whenever no preemption can happen in the next step (pages to spare for all it may
        take); otherwise the step in flight is read before the next is scheduled.
        A request that ends on a stop token is found out one step late; the token computed for it
        meanwhile is dropped."""
        deltas: List[StepDelta] = []
        pend = self._pending
        if pend is not None and not (self.overlap and self._steady_decode()):
            deltas += self._finalize(pend)
            pend = self._pending = None
        out = self.scheduler.schedule()
        self.counters["preemptions"] += len(out.preempted)
        for seq in out.aborted:
            self._seqs.pop(seq.request_id, None)
            deltas.append(StepDelta(seq.request_id, [], True))
        new = self._launch(out) if out.entries else None
        if pend is not None:
            self.counters["overlapped_steps"] += 1 if new is not None else 0
            deltas += self._finalize(pend)
        self._pending = new
        if new is not None and not self.overlap:
            deltas += self._finalize(new)
            self._pending = None
        self.counters["steps"] += 1
        for seq in self.scheduler.free_finished():
            self._seqs.pop(seq.request_id, None)
        return deltas

    def _steady_decode(self) -> bool:
        """Whether the next step can be scheduled before the tokens of the step in flight are known: whenever no
        request can be preempted in it (a preempted request is computed again from its tokens, and its newest one
        is still on the device). The step then takes the tokens it lacks from the device (``from_device``), be it a
        decode step or one that also brings portions of prompts and admits requests."""
        sch = self.scheduler
        cfg = sch.config
        live = [s for s in sch.running if s.status == Status.RUNNING]
        ps = self.runner.cache.page_size
        # the most pages the next step can take: one per decoding request; for the prompts in flight and those that
        # may be admitted, the tokens the budget lets through and a page more each (a portion may start inside a page)
        admit = min(len(sch.waiting), cfg.max_prefill_per_step, max(0, cfg.max_running - len(live)))
        prompts = [s for s in live if not s.is_decoding] + list(itertools.islice(sch.waiting, admit))
        tokens = min(cfg.max_prefill_tokens, sum(s.remaining for s in prompts))
        need = (len(live) + admit - len(prompts)) + -(-tokens // ps) + len(prompts)
        free = self.runner.cache.free_pages()
        if free and min(free) < need:
            return False
        return admit == 0 or self.runner.cache.state.num_free >= admit

    def _launch(self, out: SchedulerOutput) -> "_InFlight":
        entries = []
        wanting: List[Sequence] = []
        for e in out.entries:
            seq = e.seq
            stop = e.start + e.count
            rows = vals = None
            req = seq.request
            if req.embed_rows is not None and e.start < seq.num_prompt_tokens:
                pick = [i for i, r in enumerate(req.embed_rows) if e.start <= r < stop]
                if pick:
                    rows = [req.embed_rows[i] - e.start for i in pick]
                    vals = req.embed_values[pick]
            toks = seq.tokens(e.start, stop)
            from_device = e.count == 1 and toks[0] == PENDING_TOKEN
            if from_device:
                toks = [0]
            elif PENDING_TOKEN in toks:
                raise RuntimeError(f"request {seq.request_id!r}: a token still on the device is needed on the host")
            entries.append(StepEntry(seq.request_id, toks, want=[e.count - 1] if e.wants_logits else [],
                                     positions=self.runner.positions_for(seq.prompt_positions, seq.num_prompt_tokens, e.start, stop),
                                     embed_rows=rows, embed_values=vals,
                                     from_device=from_device))
            if e.wants_logits:
                wanting.append(seq)
            self.counters["decode_tokens" if e.is_decode else "prefill_tokens"] += e.count
        logits = self.runner.step(entries, copy_logits=False)
        handle = self.sampler.sample_async(logits, wanting, self.runner.last_token,
                                           self.runner.logit_slots if self.runner.last_token is not None else None)
        for e in out.entries:
            e.seq.num_computed += e.count
            e.seq.scheduled = 0
        fill_at = []
        for seq in wanting:
            fill_at.append(seq.num_output_tokens)
            seq.append_token(PENDING_TOKEN)
            seq.maybe_finish()          # by count; a stop token shows when the value is read
        return _InFlight(handle, wanting, fill_at, [e.seq for e in out.entries])

    def _finalize(self, fl: "_InFlight") -> List[StepDelta]:
        """Reads the tokens of a launched step (waits for the device) and retires what ended."""
        for seq, idx, tok in zip(fl.wanting, fl.fill_at, fl.handle.result()):
            if idx >= seq.num_output_tokens:
                continue                # the request ended on an earlier token; this one is dropped
            seq.output_token_ids[idx] = int(tok)
            if int(tok) in seq.request.sampling.stop_token_ids:
                del seq.output_token_ids[idx + 1:]
                if seq.status == Status.RUNNING:
                    seq.maybe_finish()
        deltas: List[StepDelta] = []
        seen = set()
        for seq in fl.seqs:
            if id(seq) in seen:
                continue
            seen.add(id(seq))
            outs = seq.output_token_ids
            known = seq.num_streamed
            while known < len(outs) and outs[known] != PENDING_TOKEN:
                known += 1
            if known > seq.num_streamed:
                new_ids = outs[seq.num_streamed:known]
                seq.num_streamed = known
                text = self._detokenize(new_ids) if self._detokenize else ""
                done = seq.status != Status.RUNNING and known == len(outs)
                deltas.append(StepDelta(seq.request_id, list(new_ids), done, text))
        return deltas

    def run_until_complete(self) -> Dict[str, List[int]]:
        """Runs until every request has ended; returns the generated token ids per request."""
        outs: Dict[str, List[int]] = {rid: [] for rid in self._seqs}
        while self.has_unfinished():
            for d in self.step():
                outs.setdefault(d.request_id, []).extend(d.new_token_ids)
        if self.runner.check_device_errors:
            ops.kernels().check_device_errors()     # the steps only looked at what had already come back
        return outs

    def generate(self, prompts: Seq[Seq[int]], sampling: Optional[SamplingParams] = None) -> List[List[int]]:
        """Convenience: token-id prompts in, generated token ids out, in the prompts' order."""
        ids = []
        for p in prompts:
            sp = SamplingParams(**{**sampling.__dict__, "stop_token_ids": list(sampling.stop_token_ids)}) \
                if sampling else SamplingParams()
            ids.append(self.add_request(Request(prompt=list(p), sampling=sp)))
        outs = self.run_until_complete()
        return [outs.get(i, []) for i in ids]

    def stats(self) -> Dict[str, object]:
        c = dict(self.counters)
        c["pages_in_use"] = sum(self.runner.cache.pages_in_use())
        c["running"] = len(self.scheduler.running)
        c["waiting"] = len(self.scheduler.waiting)
        if self.runner.device.type == "cuda":
            # launches by kernel entry point since the process began: which kernels the steps have been taking
            c["kernel_launches"] = dict(ops.kernels().counts)
        return c
