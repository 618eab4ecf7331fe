"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference has four entry points for what is one computation — packed whole prompts, one
chunk, decode tokens plus one chunk, decode only (omniserve/runners/base.py:31-49,
omniserve/runners/multimodal.py:79-304); each appends ``new_len`` tokens per request at its cache
length and attends causally over that request's cache (omniserve/cache/kv_prealloc.py:110-146).
Here there is one: any number of requests, each bringing one or more tokens (a decoded token, a
portion of a prompt cut anywhere, a whole prompt), flattened into one varlen batch.  It runs only
the tokens it is given and returns fp32 logits at the wanted places.
"""

from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..models.decoder import DecoderModel


@dataclass
class StepEntry:
    """A request's next tokens in one step.

    ``want``: places among ``tokens`` whose logits are wanted (may be empty).
    ``positions``: int array [columns, n] of given positions, as many columns as the model's position
    encoding takes (``ModelRunner.position_columns``); None means the tokens continue the request and the
    encoding finds their positions from the request's state.
    ``embed_rows``/``embed_values``: places among ``tokens`` whose looked-up embedding is replaced
    by the given rows [len(embed_rows), hidden] (the hook the vision tower's output uses).
    ``from_device``: the entry brings one token, the one the sampler last kept for this request on
    the device (``ModelRunner.last_token``); ``tokens[0]`` is only a placeholder. This lets the next
    step be launched before the host has read the token.
    """

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()
    positions: Optional[np.ndarray] = None
    embed_rows: Optional[Sequence[int]] = None
    embed_values: Optional[torch.Tensor] = None
    from_device: bool = False


class StepContext:
    """Device-side description of one step, shared by all layers."""

    def __init__(self) -> None:
        self.device: torch.device = None
        self.act_dtype: torch.dtype = None
        self.T = self.S = self.num_logit_rows = 0
        self.token_ids = self.cu_q = self.seq_lens = self.tok_seq = self.state_slot = None
        self.token_src: Optional[torch.Tensor] = None      # [T]: slot of last_token to take the id from, or -1
        self.last_token: Optional[torch.Tensor] = None     # [slots]: the token last sampled for each request
        self.positions = self.pos_mode = self.logit_rows = None
        self.block_tables: List[torch.Tensor] = []
        self.slot_maps: List[torch.Tensor] = []
        self.override_rows: Optional[torch.Tensor] = None
        self.override_vals: Optional[torch.Tensor] = None
        self.max_q_len = self.max_kv_len = 0
        self.q_lens: List[int] = []
        self.kv_lens: List[int] = []
        self.page_size = 0
        self.logit_slots: Optional[torch.Tensor] = None    # [wanted rows]: the request slot of each logits row
        self.decode_index: Optional[torch.Tensor] = None   # [S]: index among requests bringing one token, else -1
        self.attn_order: Optional[torch.Tensor] = None     # [S]: the requests by falling length (attention starts long ones first)
        self.kv_uneven = False                             # the single-token requests' lengths differ much
        self.prefill_units: Optional[torch.Tensor] = None  # [n, 2]: (request, 128-row tile) with work, most keys first
        self.n_decode = self.n_multi = 0
        self.scratch: Dict[str, torch.Tensor] = {}         # per-step scratch buffers shared by the layers
        self.advance_state = True                          # False: a dry run that must not move cursors
        self._model: Optional[DecoderModel] = None
        self._tables: Dict[int, Any] = {}

    def bind_model(self, model: DecoderModel) -> None:
        self._model = model
        self._tables = {}

    def position_tables(self, position: Any) -> Any:
        """Per-step tables of a position encoding, computed once and shared by the layers using it."""
        k = id(position)
        if k not in self._tables:
            self._tables[k] = position.prepare(self, self._model.shared_state)
        return self._tables[k]


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    """Owns the model, its cache and the step function."""

    def __init__(self, model: DecoderModel, cache: CacheManager, act_dtype: torch.dtype, device,
                 check_device_errors: bool = True, use_graphs: bool = False):
        self.model = model
        self.cache = cache
        self.act_dtype = act_dtype
        self.device = torch.device(device)
        self.check_device_errors = check_device_errors
        self.vocab_size = model.spec.vocab_size
        self.hidden_size = model.spec.hidden_size
        self.steps = 0
        self._scratch: Dict[str, torch.Tensor] = {}
        #: replay pure decode steps from CUDA graphs (one per batch size and block-table width)
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda"
        self.graph_max_batch = 256
        self.graph_bt_round = 32          # block-table width is rounded up to this many pages times a power of two
        #: most graphs kept; the one used longest ago goes when another is needed. All graphs allocate from one
        #: memory pool (they replay one after the other on one stream), so their activations share memory.
        self.graph_max_count = 32
        #: a graph is built when its shape comes by for this many-th time; before that the step is launched kernel
        #: by kernel (1: build at once)
        self.graph_min_uses = 1
        #: the same for steps that bring portions of prompts (0: never a graph for them). Their shapes (tokens per
        #: request) are many, and most come by once
        self.graph_min_uses_prompt = 3
        self.graph_min_free_bytes = 8 << 30     # no new graph for such a step with less free device memory than this
        self.graph_use_window = 64              # steps within which a shape has to come back for its uses to add up
        self._graph_seen: Dict[Any, Tuple[int, int]] = {}    # shape -> (uses that followed one another, step of the last)
        #: rows that pad a decode step to the next batch size for which graphs are kept (``_graph_bucket``): requests
        #: of one token at position 0 on spare state slots, whose page goes back after every step
        self._filler_ids: List[str] = []
        self._graphs: "collections.OrderedDict[Any, Dict[str, Any]]" = collections.OrderedDict()
        self._graph_pool = None
        model.attach_cache(cache.bindings(), cache.shared_state())
        #: rows of the positions a request may give per token (what the model's position encoding takes)
        self.position_columns = model.position_columns
        #: per request slot, the token the sampler last kept on the device (see StepEntry.from_device)
        self.last_token: Optional[torch.Tensor] = None
        #: after a step: the request slot of each returned logits row, on the device (for Sampler.sample_async)
        self.logit_slots: Optional[torch.Tensor] = None
        self.last_h2d_bytes = 0           # size of the last step's metadata copy
        #: set when a kernel reported an error: the text of it; the runner then refuses further steps
        self.failed: Optional[str] = None
        if cache.state.tensors or self.device.type == "cuda":
            with torch.inference_mode(False):
                self.last_token = torch.zeros(max(cache.state.num_slots, 1), dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ request life
    def start_request(self, request_id: str, prompt_positions: Optional[np.ndarray] = None,
                      num_prompt_tokens: int = 0) -> None:
        """The request takes a state slot. ``prompt_positions`` ([position_columns, num_prompt_tokens]) are
        the positions that came with its prompt, if any: the model's position encodings turn them into
        their rows of the request's state."""
        if prompt_positions is not None:
            self.check_positions(prompt_positions, num_prompt_tokens)
        rc = self.cache.begin(request_id)
        self._write_request_state(rc.slot, prompt_positions, num_prompt_tokens)

    def end_request(self, request_id: str) -> None:
        self.cache.finish(request_id)
        if self._filler_ids and len(self.cache.requests) == len(self._filler_ids):
            for rid in self._filler_ids:       # the last request has gone: so do the rows that padded its steps
                self.cache.finish(rid)
            self._filler_ids = []

    def reset_request(self, request_id: str, prompt_positions: Optional[np.ndarray] = None,
                      num_prompt_tokens: int = 0) -> None:
        if prompt_positions is not None:
            self.check_positions(prompt_positions, num_prompt_tokens)
        self.cache.reset(request_id)
        self._write_request_state(self.cache.requests[request_id].slot, prompt_positions, num_prompt_tokens)

    def _write_request_state(self, slot: int, prompt_positions: Optional[np.ndarray], num_prompt_tokens: int) -> None:
        if not self.cache.state.tensors:
            return
        for name, row in self.model.request_state(prompt_positions, num_prompt_tokens).items():
            if name in self.cache.state.tensors:
                self.cache.state.write(name, slot, row)

    def check_positions(self, positions: np.ndarray, n: int) -> None:
        p = np.asarray(positions)
        if p.shape != (self.position_columns, n):
            raise ValueError(f"positions must be [{self.position_columns}, {n}], got {tuple(p.shape)}")

    def positions_for(self, prompt_positions: Optional[np.ndarray], num_prompt_tokens: int, start: int, stop: int
                      ) -> Optional[np.ndarray]:
        """The ``StepEntry.positions`` of tokens [start, stop) of a request whose prompt came with positions."""
        return self.model.positions_for(prompt_positions, num_prompt_tokens, start, stop)

    # ------------------------------------------------------------------ the step
    def _plan(self, entries: Sequence[StepEntry], bt_round: int = 1) -> Dict[str, Any]:
        """Validates the entries, takes their pages and lays out the step's host-side metadata."""
        cache = self.cache
        S = len(entries)
        if S == 0:
            raise ValueError("a step needs at least one entry")
        rids = [e.request_id for e in entries]
        if len(set(rids)) != S:
            raise ValueError("a request may appear once in a step")
        q_lens = [len(e.tokens) for e in entries]
        if min(q_lens) <= 0:
            raise ValueError("every entry of a step brings at least one token")
        T = int(sum(q_lens))
        for e in entries:
            if not cache.has(e.request_id):
                raise KeyError(f"request {e.request_id!r} was not started")

        # every entry is checked before a page is taken: a bad entry leaves the cache as it was
        cu_q = np.zeros(S + 1, dtype=np.int32)
        cu_q[1:] = np.cumsum(q_lens)
        token_ids = np.empty(T, dtype=np.int32)
        tok_src = np.full(T, -1, dtype=np.int32)
        tok_seq = np.empty(T, dtype=np.int32)
        C = self.position_columns
        positions = np.zeros((C, T), dtype=np.int32)
        pos_mode = np.ones(S, dtype=np.int32)
        logit_rows: List[int] = []
        logit_slots: List[int] = []
        ov_rows: List[int] = []
        ov_vals: List[torch.Tensor] = []
        V = self.vocab_size
        for i, e in enumerate(entries):
            a, b = int(cu_q[i]), int(cu_q[i + 1])
            toks = np.asarray(e.tokens, dtype=np.int64)
            if e.from_device:
                if b - a != 1:
                    raise ValueError(f"request {e.request_id!r}: a token taken from the device comes alone")
                toks = np.zeros(1, dtype=np.int64)
                tok_src[a] = cache.requests[e.request_id].slot
            if toks.min() < 0 or toks.max() >= V:
                raise ValueError(f"request {e.request_id!r}: token id outside [0, {V})")
            token_ids[a:b] = toks
            tok_seq[a:b] = i
            if e.positions is not None:
                p = np.asarray(e.positions)
                if p.shape != (C, b - a):
                    raise ValueError(f"request {e.request_id!r}: positions must be [{C}, {b - a}], got {p.shape}")
                positions[:, a:b] = p
                pos_mode[i] = 0
            for w in e.want:
                if not (0 <= w < b - a):
                    raise ValueError(f"request {e.request_id!r}: wanted place {w} outside its {b - a} tokens")
                logit_rows.append(a + int(w))
                logit_slots.append(cache.requests[e.request_id].slot)
            if e.embed_rows is not None and len(e.embed_rows):
                rows = [int(r) for r in e.embed_rows]
                if min(rows) < 0 or max(rows) >= b - a:
                    raise ValueError(f"request {e.request_id!r}: embedding row outside its tokens")
                if e.embed_values is None or tuple(e.embed_values.shape) != (len(rows), self.hidden_size):
                    raise ValueError(f"request {e.request_id!r}: embed_values must be [{len(rows)}, {self.hidden_size}]")
                ov_rows += [a + r for r in rows]
                ov_vals.append(e.embed_values)

        if not cache.can_reserve(list(zip(rids, q_lens))):
            from ..cache.page_pool import OutOfPages
            raise OutOfPages(f"the step needs more pages than are free ({cache.free_pages()} free)")
        cursors = [cache.requests[r].cursor for r in rids]
        kv_lens = [c + n for c, n in zip(cursors, q_lens)]
        for r, n in zip(rids, q_lens):
            cache.reserve(r, n)
        slots = np.asarray([cache.requests[r].slot for r in rids], dtype=np.int32)
        G = len(cache.groups)
        bts = [cache.block_table(g, rids, bt_round, pow2=bt_round > 1) for g in range(G)]
        sms = [cache.slot_map(g, rids, q_lens) for g in range(G)]
        ql = np.asarray(q_lens)
        single = ql == 1
        decode_index = np.where(single, np.cumsum(single) - 1, -1).astype(np.int32)
        segs: List[Tuple[str, np.ndarray]] = [
            ("token_ids", token_ids), ("cu_q", cu_q), ("seq_lens", np.asarray(kv_lens, dtype=np.int32)),
            ("tok_seq", tok_seq), ("state_slot", slots), ("positions", positions.reshape(-1)),
            ("pos_mode", pos_mode), ("logit_rows", np.asarray(logit_rows, dtype=np.int32)),
            ("override_rows", np.asarray(ov_rows, dtype=np.int32)), ("decode_index", decode_index),
            ("token_src", tok_src), ("logit_slots", np.asarray(logit_slots, dtype=np.int32)),
            ("attn_order", np.argsort(-np.asarray(kv_lens), kind="stable").astype(np.int32)),
            ("prefill_units", ops.CudaKernels.prefill_units(q_lens, kv_lens).reshape(-1)),
        ]
        for g in range(G):
            segs.append((f"bt{g}", bts[g].reshape(-1)))
            segs.append((f"sm{g}", sms[g]))
        return dict(S=S, T=T, segs=segs, q_lens=q_lens, kv_lens=kv_lens, bt_widths=[b.shape[1] for b in bts],
                    n_logit_rows=len(logit_rows), ov_vals=ov_vals, n_decode=int(single.sum()),
                    explicit_positions=bool((pos_mode == 0).any()),
                    uneven=self._uneven(np.asarray(kv_lens)[single]))

    def _plan_decode(self, entries: Sequence[StepEntry], bt_round: int, n_real: Optional[int] = None) -> Dict[str, Any]:
        """``_plan`` for a step in which every request brings one token and wants its logits: the same
        result, built with array operations instead of a loop over entries."""
        cache = self.cache
        ps = cache.page_size
        S = len(entries)
        rids = [e.request_id for e in entries]
        if len(set(rids)) != S:
            raise ValueError("a request may appear once in a step")
        try:
            rcs = [cache.requests[r] for r in rids]
        except KeyError as k:
            raise KeyError(f"request {k.args[0]!r} was not started") from None
        from_dev = np.fromiter((e.from_device for e in entries), dtype=bool, count=S)
        token_ids = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=S)
        token_ids[from_dev] = 0
        if token_ids.min() < 0 or token_ids.max() >= self.vocab_size:
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        boundary = [rc for rc in rcs if (rc.cursor + rc.reserved) % ps == 0]
        if boundary and len(boundary) > min(cache.free_pages(), default=len(boundary)):
            from ..cache.page_pool import OutOfPages
            raise OutOfPages(f"the step needs more pages than are free ({cache.free_pages()} free)")
        for rc in rcs:
            if (rc.cursor + rc.reserved) % ps == 0:
                cache.reserve(rc.request_id, 1)
            else:
                rc.reserved += 1
        cursors = np.fromiter((rc.cursor for rc in rcs), dtype=np.int32, count=S)
        ar = np.arange(S + 1, dtype=np.int32)
        G = len(cache.groups)
        bts = [cache.block_table(g, rids, bt_round, pow2=bt_round > 1) for g in range(G)]
        sms = []
        for g in range(G):
            pages = np.fromiter((rc.tables[g][rc.cursor // ps] for rc in rcs), dtype=np.int32, count=S)
            if (pages < 0).any():
                raise RuntimeError("a token of this step maps to a page that was given back")
            sms.append(pages * ps + cursors % ps)
        slots = np.fromiter((rc.slot for rc in rcs), dtype=np.int32, count=S)
        segs: List[Tuple[str, np.ndarray]] = [
            ("token_ids", token_ids.astype(np.int32)), ("cu_q", ar), ("seq_lens", cursors + 1), ("tok_seq", ar[:S]),
            ("state_slot", slots),
            ("positions", np.zeros(self.position_columns * S, dtype=np.int32)), ("pos_mode", np.ones(S, dtype=np.int32)),
            ("logit_rows", ar[:S]), ("override_rows", np.zeros(0, dtype=np.int32)), ("decode_index", ar[:S]),
            ("token_src", np.where(from_dev, slots, -1).astype(np.int32)), ("logit_slots", slots),
            ("attn_order", np.argsort(-cursors, kind="stable").astype(np.int32)),
            ("prefill_units", np.zeros(0, dtype=np.int32)),
        ]
        for g in range(G):
            segs.append((f"bt{g}", bts[g].reshape(-1)))
            segs.append((f"sm{g}", sms[g].astype(np.int32)))
        kv_lens = (cursors + 1).tolist()
        return dict(S=S, T=S, segs=segs, q_lens=[1] * S, kv_lens=kv_lens, bt_widths=[b.shape[1] for b in bts],
                    n_logit_rows=S, ov_vals=[], n_decode=S, explicit_positions=False,
                    uneven=self._uneven((cursors + 1)[:n_real]))      # (rows behind n_real only pad the step)

    @staticmethod
    def _uneven(lens: np.ndarray) -> bool:
        """Whether the lengths of the requests that bring one token differ much: the longest 1.5 times the mean or
        more (the attention kernel may then cut the keys into more parts)."""
        return bool(lens.size >= 2 and lens.max() >= 1.5 * lens.mean())

    @staticmethod
    def _layout(segs: List[Tuple[str, np.ndarray]]) -> Tuple[Dict[str, Tuple[int, int]], int]:
        offs, total = {}, 0
        for name, arr in segs:
            offs[name] = (total, arr.size)
            total += _align4(arr.size)
        return offs, max(total, 4)

    def _context(self, plan: Dict[str, Any], dev: torch.Tensor, offs: Dict[str, Tuple[int, int]]) -> StepContext:
        S, T = plan["S"], plan["T"]
        G = len(self.cache.groups)

        def seg(name: str) -> torch.Tensor:
            o, n = offs[name]
            return dev[o:o + n]

        ctx = StepContext()
        ctx.device, ctx.act_dtype = self.device, self.act_dtype
        ctx.T, ctx.S, ctx.num_logit_rows = T, S, plan["n_logit_rows"]
        ctx.token_ids, ctx.cu_q, ctx.seq_lens = seg("token_ids"), seg("cu_q"), seg("seq_lens")
        ctx.tok_seq, ctx.state_slot = seg("tok_seq"), seg("state_slot")
        ctx.positions = seg("positions").view(self.position_columns, T)
        ctx.pos_mode, ctx.logit_rows = seg("pos_mode"), seg("logit_rows")
        ctx.block_tables = [seg(f"bt{g}").view(S, plan["bt_widths"][g]) for g in range(G)]
        ctx.slot_maps = [seg(f"sm{g}") for g in range(G)]
        if plan["ov_vals"]:
            ctx.override_rows = seg("override_rows")
            ctx.override_vals = torch.cat([v.to(self.device) for v in plan["ov_vals"]], dim=0).contiguous()
        ctx.q_lens, ctx.kv_lens = plan["q_lens"], plan["kv_lens"]
        ctx.max_q_len, ctx.max_kv_len = max(plan["q_lens"]), max(plan["kv_lens"])
        ctx.page_size = self.cache.page_size
        ctx.decode_index = seg("decode_index")
        ctx.attn_order = seg("attn_order")      # the requests by falling length: long ones start first
        ctx.kv_uneven = plan["uneven"]
        ctx.prefill_units = seg("prefill_units").view(-1, 2)   # (request, row tile) of the requests bringing several tokens
        if self.last_token is not None:
            ctx.token_src, ctx.last_token = seg("token_src"), self.last_token
        ctx.logit_slots = seg("logit_slots")
        ctx.n_decode = plan["n_decode"]
        ctx.n_multi = S - ctx.n_decode
        ctx.scratch = self._scratch
        return ctx

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        return self._context_of_plan(self._plan(entries))

    def _context_of_plan(self, plan: Dict[str, Any]) -> StepContext:
        offs, total = self._layout(plan["segs"])
        # one staging buffer, one host-to-device copy
        host = torch.empty(total, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        hv = host.numpy()
        for name, arr in plan["segs"]:
            o, n = offs[name]
            hv[o:o + n] = arr
        dev = host.to(self.device, non_blocking=True)
        ctx = self._context(plan, dev, offs)
        ctx.h2d_bytes = self.last_h2d_bytes = total * 4
        return ctx

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], copy_logits: bool = True) -> torch.Tensor:
        """Runs the entries as one batch; returns fp32 logits [wanted, vocab] in the order of the
        entries and of their ``want``. The requests' tokens are in the cache afterwards.

        Nothing here waits for the device. ``copy_logits=False`` may return a buffer that the next
        step overwrites: for callers that consume the logits (sample from them) on the same stream
        before they step again."""
        if self.use_graphs and self._graphable(entries):
            return self._graph_step(entries, copy_logits)
        if self.use_graphs and self._shape_graphable(entries):
            return self._shape_graph_step(entries, copy_logits)
        self._before_step()
        try:
            ctx = self.build_context(entries)
            self.logit_slots = ctx.logit_slots
            ops.profile_mark("plan")     # what came before is the host laying out the step
            with ops.kernels().pinned_stream():
                logits = self.model.forward(ctx)
        except Exception:
            self._rollback(entries)
            raise
        self._after_step(entries)
        return logits

    def _planned_step(self, entries: Sequence[StepEntry], plan: Dict[str, Any], fill: Sequence[StepEntry] = ()
                      ) -> torch.Tensor:
        """Runs a step whose plan exists (its pages are taken) kernel by kernel. ``fill``: the rows behind those of
        ``entries`` that only pad the step."""
        n_real = len(entries)
        try:
            ctx = self._context_of_plan(plan)
            self.logit_slots = ctx.logit_slots[:n_real]
            ops.profile_mark("plan")
            with ops.kernels().pinned_stream():
                logits = self.model.forward(ctx)
        except Exception:
            self._rollback(list(entries) + list(fill))
            raise
        self._after_step(entries)
        for e in fill:
            self.cache.rollback(e.request_id)
        return logits[:n_real] if fill else logits

    def _rollback(self, entries: Sequence[StepEntry]) -> None:
        """A step that failed gives back what it reserved: its requests hold the pages of their cursors again."""
        for e in entries:
            if self.cache.has(e.request_id):
                self.cache.rollback(e.request_id)

    def _before_step(self) -> None:
        """What a kernel of an earlier step reported is raised here, before this step takes a page or moves a
        cursor, and the runner refuses further steps: cursors on the device and on the host may disagree."""
        if self.failed is not None:
            raise RuntimeError(f"this runner stopped after a kernel error ({self.failed}); build a new one")
        if self.check_device_errors and self.device.type == "cuda":
            try:
                ops.kernels().check_device_errors_async()
            except Exception as e:
                self.failed = str(e)
                raise

    def _after_step(self, entries: Sequence[StepEntry]) -> None:
        # no wait for the device here: what a kernel of this step reports is raised at the start of a later
        # step (``_before_step``) or by the caller's own ``ops.kernels().check_device_errors()``, which waits
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps += 1

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        """Pure decode steps (one token and one wanted row per request, positions from the state
        slot, no given embeddings) have a fixed launch sequence for a given batch size."""
        if self.device.type != "cuda" or len(entries) > self.graph_max_batch:
            return False
        for e in entries:
            if len(e.tokens) != 1 or e.positions is not None or e.embed_rows is not None or list(e.want) != [0]:
                return False
        return True

    #: spare state slots for the rows that pad a decode step (the largest gap between two graph batch sizes)
    GRAPH_FILLERS = 127

    @staticmethod
    def _graph_bucket(n: int) -> int:
        """The batch size of the graph that a decode step of ``n`` requests replays: the next power of two. While
        the requests of a run end one after the other every batch size comes by once or twice, and building a graph
        costs as much as five to ten steps; padded, 33 to 63 requests replay the graph of 64 (a decode step of up to
        64 rows is bound by the weights it streams: the rows that pad it cost next to nothing, their attention is
        one key long)."""
        b = 1
        while b < n:
            b *= 2
        return b

    def _fillers(self, entries: Sequence[StepEntry]) -> List[StepEntry]:
        """Entries that pad ``entries`` to the batch size of a graph, or none (no spare slots, or no page left)."""
        n = min(self._graph_bucket(len(entries)), self.graph_max_batch) - len(entries)
        if n <= 0:
            return []
        from ..cache.state_slots import OutOfSlots
        while len(self._filler_ids) < n:
            rid = "\x00filler%d" % len(self._filler_ids)
            try:
                self.cache.begin(rid, spare=True)
            except OutOfSlots:
                return []
            self._filler_ids.append(rid)
        fill = [StepEntry(r, [0], want=[0]) for r in self._filler_ids[:n]]
        if not self.cache.can_reserve([(e.request_id, 1) for e in list(entries) + fill]):
            return []
        return fill

    def _graph_step(self, entries: Sequence[StepEntry], copy_logits: bool = True) -> torch.Tensor:
        """A decode step replayed from a CUDA graph: the launch-bound inner loop of generation.

        One graph per (batch size, block-table width bucket, lengths uneven or not). The step's metadata goes into a
        buffer at a fixed address (one host-to-device copy); everything the kernels need that
        changes from step to step is read from that buffer or from the state slots.
        """
        round_to = self.graph_bt_round
        self._before_step()
        n_real = len(entries)
        fill = self._fillers(entries)
        real, entries = entries, list(entries) + fill      # ``entries``: what runs; ``real``: what the caller sees
        try:
            plan = self._plan_decode(entries, bt_round=round_to, n_real=n_real)
        except Exception:
            self._rollback(entries)
            raise
        key = (plan["S"], tuple(plan["bt_widths"]), plan["uneven"])   # (the attention's splits depend on the last)
        return self._replay(key, plan, real, fill, copy_logits, self.graph_min_uses)

    def _shape_graphable(self, entries: Sequence[StepEntry]) -> bool:
        """Steps that bring portions of prompts have a fixed launch sequence too, for given token counts per
        request: all that changes from one such step to the next (tokens, positions, tables, wanted rows) is data in
        the step's buffer. Not with given embedding rows (a tensor of the step's own)."""
        if self.device.type != "cuda" or len(entries) > self.graph_max_batch or self.graph_min_uses_prompt <= 0:
            return False
        return all(e.embed_rows is None for e in entries)

    def _shape_graph_step(self, entries: Sequence[StepEntry], copy_logits: bool = True) -> torch.Tensor:
        """A step of any shape replayed from a CUDA graph once its shape (tokens and wanted rows per request,
        block-table width bucket) has come by ``graph_min_uses_prompt`` times: a 2,048-token portion is 232 launches,
        which the host issues in 3.4 ms while the device needs 5.1 ms for them and waits now and then (5.8 ms from
        the call to the logits launched kernel by kernel, 5.1 ms replayed)."""
        self._before_step()
        try:
            plan = self._plan(entries, bt_round=self.graph_bt_round)
        except Exception:
            self._rollback(entries)
            raise
        key = ("shape", tuple(plan["q_lens"]), tuple(len(e.want) for e in entries), tuple(plan["bt_widths"]),
               plan["uneven"], plan["explicit_positions"])
        if key not in self._graphs and torch.cuda.mem_get_info(self.device)[0] < self.graph_min_free_bytes:
            return self._planned_step(entries, plan)     # a graph keeps the step's activations: not with memory this short
        return self._replay(key, plan, entries, [], copy_logits, self.graph_min_uses_prompt)

    def _replay(self, key, plan: Dict[str, Any], real: Sequence[StepEntry], fill: Sequence[StepEntry],
                copy_logits: bool, min_uses: int) -> torch.Tensor:
        """Runs a planned step from the graph of its shape (built now if the shape has come by often enough, else
        the step is launched kernel by kernel)."""
        k = ops.kernels()
        entries = list(real) + list(fill)
        n_real = len(real)
        slot = self._graphs.get(key)
        if slot is None and min_uses > 1:
            # Building a graph costs about as much as ten steps (a warm-up forward, a wait for the device, the
            # capture): a shape that comes by once or twice is launched kernel by kernel instead.
            # And only uses that follow one another within ``graph_use_window`` steps count: shapes that a workload
            # brings back now and then (the same requests served again a few hundred steps later) would otherwise
            # all be built on their third visit, more of them than are kept, each built again on its next.
            if len(self._graph_seen) > 4096:
                self._graph_seen.clear()
            seen, last = self._graph_seen.get(key, (0, self.steps))
            seen = seen + 1 if self.steps - last <= self.graph_use_window else 1
            self._graph_seen[key] = (seen, self.steps)
            if seen < min_uses:
                return self._planned_step(real, plan, fill)
        if slot is not None:
            self._graphs.move_to_end(key)
        else:
            if len(self._graphs) >= max(1, self.graph_max_count):
                torch.cuda.synchronize()             # the graph that goes may still be running
                self._graphs.popitem(last=False)
            offs, total = self._layout(plan["segs"])
            with torch.inference_mode(False):
                # two staging buffers in turn: the host may fill one while the copy out of the other waits
                # behind the step before on the stream
                hosts = [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
                dev = torch.zeros(total, dtype=torch.int32, device=self.device)
            slot = {"offs": offs, "hosts": hosts, "dev": dev, "graph": None, "logits": None, "launches": 0,
                    "copied": [torch.cuda.Event(), torch.cuda.Event()], "turn": 0, "used": [False, False]}
            self._graphs[key] = slot
        turn = slot["turn"]
        slot["turn"] = turn ^ 1
        if slot["used"][turn]:
            slot["copied"][turn].synchronize()      # the last copy out of this pinned buffer has finished
        host = slot["hosts"][turn]
        hv = host.numpy()
        for name, arr in plan["segs"]:
            o, n = slot["offs"][name]
            hv[o:o + n] = arr
        slot["dev"].copy_(host, non_blocking=True)
        self.last_h2d_bytes = host.numel() * 4
        slot["copied"][turn].record()
        slot["used"][turn] = True
        try:
            if slot["graph"] is None:
                ctx = self._context(plan, slot["dev"], slot["offs"])
                # the kernels' grids must not depend on this step's lengths: size them for the bucket
                ctx.max_kv_len = max(plan["bt_widths"]) * self.cache.page_size
                ctx.advance_state = False
                self.model.forward(ctx)                      # warm-up; same cache writes as the real run
                torch.cuda.synchronize()
                ctx.advance_state = True
                g = torch.cuda.CUDAGraph()
                l0 = k.launches
                if self._graph_pool is None:
                    self._graph_pool = torch.cuda.graph_pool_handle()
                with torch.cuda.graph(g, pool=self._graph_pool):
                    slot["logits"] = self.model.forward(ctx)
                slot["launches"] = k.launches - l0
                slot["graph"] = g
                k.launches = l0
            slot["graph"].replay()
            k.launches += slot["launches"]
        except Exception:
            self._rollback(entries)
            raise
        self._after_step(real)
        for e in fill:
            self.cache.rollback(e.request_id)       # the filler's page goes back; it stays at position 0
        o, n = slot["offs"]["logit_slots"]
        self.logit_slots = slot["dev"][o:o + n] if not fill else slot["dev"][o:o + n_real]
        logits = slot["logits"] if not fill else slot["logits"][:n_real]
        return logits.clone() if copy_logits else logits
