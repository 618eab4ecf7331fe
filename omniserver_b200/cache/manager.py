"""The cache manager: keys and values in pages with a block table per request, page groups for
layers with different needs, and slots of fixed-size per-request state.

The reference's pool gives every request one slot of ``max_len`` tokens per layer and compacts by
copying on every finish (omniserve/cache/kv_prealloc.py:20-57, omniserve/runners/multimodal.py:359-369).
Here a request holds only the pages its tokens need:

* Layer runs whose mixers ask for the same kind of cache (kv heads, head size, window) form a
  *group*; a group has its own pool and every request has one block table per group, shared by
  all layers of the group (page p of a request is page p in each of the group's layers).
* Pages are taken when a step brings tokens (``reserve``), given back when a request ends, and,
  in a group with a window, as soon as every position of the page is older than any future query
  can see (``commit``).  A freed page is the next one handed out.
* Storage per group: ``[layers, 2, pages, kv_heads, page_size, head_dim]`` (keys, values).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheBinding, KVCacheNeed, StateNeed
from .page_pool import OutOfPages, PagePool
from .state_slots import OutOfSlots, StateSlots


@dataclass
class PageGroup:
    need: KVCacheNeed
    entries: List[int]                      # schedule entries that own a cache in this group
    pool: PagePool
    storage: Optional[torch.Tensor] = None  # [layers, 2, pages, nkv, page_size, hd]

    @property
    def window(self) -> Optional[int]:
        return self.need.window


class PageTable:
    """A request's page ids in one group (-1 = given back), kept as a growing int32 array so that a
    step's block table is a row copy instead of a walk over Python lists."""

    __slots__ = ("_a", "_n")

    def __init__(self) -> None:
        self._a = np.full(16, -1, dtype=np.int32)
        self._n = 0

    def __len__(self) -> int:
        return self._n

    def append(self, page: int) -> None:
        if self._n == self._a.shape[0]:
            grown = np.full(2 * self._n, -1, dtype=np.int32)
            grown[:self._n] = self._a
            self._a = grown
        self._a[self._n] = page
        self._n += 1

    def __getitem__(self, i):
        if isinstance(i, slice):
            return self._a[:self._n][i].tolist()
        if i < 0:
            i += self._n
        if not (0 <= i < self._n):
            raise IndexError(i)
        return int(self._a[i])

    def __setitem__(self, i: int, v: int) -> None:
        if not (0 <= i < self._n):
            raise IndexError(i)
        self._a[i] = v

    def __iter__(self):
        return iter(self._a[:self._n].tolist())

    def __eq__(self, other) -> bool:
        return list(self) == list(other)

    def array(self) -> np.ndarray:
        return self._a[:self._n]

    def truncate(self, n: int) -> None:
        """Forget the entries from index ``n`` on."""
        if 0 <= n < self._n:
            self._a[n:self._n] = -1
            self._n = n


@dataclass
class RequestCache:
    request_id: str
    slot: int
    cursor: int = 0                          # tokens of the request in the cache
    reserved: int = 0                        # tokens reserved for the running step
    tables: List[PageTable] = field(default_factory=list)   # per group: page id per page index, -1 = given back
    first_live: List[int] = field(default_factory=list)     # per group: first page index still held


class CacheManager:
    def __init__(self, entry_needs, shared_state_needs: Sequence[StateNeed], page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype, device, allocate: bool = True, poison_freed: bool = False,
                 spare_slots: int = 0):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.dtype = dtype
        self.device = device
        self.poison_freed = poison_freed and allocate
        self.groups: List[PageGroup] = []
        self._entry_group: List[Optional[Tuple[int, int]]] = []   # entry -> (group, layer within group)
        self._entry_needs = list(entry_needs)
        key_to_group: Dict[KVCacheNeed, int] = {}
        for i, n in enumerate(self._entry_needs):
            if n.kv is None or n.cache_of is not None:
                self._entry_group.append(None)
                continue
            if n.kv not in key_to_group:
                key_to_group[n.kv] = len(self.groups)
                self.groups.append(PageGroup(n.kv, [], PagePool(self.num_pages)))
            g = key_to_group[n.kv]
            self._entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(i)
        for i, n in enumerate(self._entry_needs):
            if n.cache_of is not None and n.kv is not None:
                src = self._entry_needs[n.cache_of]
                if src.kv != n.kv:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {n.cache_of}: "
                                     f"it needs {n.kv}, the cache is {src.kv}")
        fields: Dict[str, Tuple[Tuple[int, ...], torch.dtype]] = {}
        for s in shared_state_needs:
            fields[s.name] = (tuple(s.shape), s.dtype)
        self._entry_state_names: List[Dict[str, str]] = []
        for i, n in enumerate(self._entry_needs):
            names = {}
            for s in n.states:
                full = s.name if s.shared else f"entry{i}.{s.name}"
                fields[full] = (tuple(s.shape), s.dtype)
                names[s.name] = full
            self._entry_state_names.append(names)
        self._shared_names = [s.name for s in shared_state_needs]
        self.state = StateSlots(max_requests, fields, device, allocate=allocate, spare=spare_slots)
        if allocate:
            for g in self.groups:
                g.storage = torch.zeros((len(g.entries), 2, self.num_pages, g.need.num_kv_heads, self.page_size,
                                         g.need.head_dim), dtype=dtype, device=device)
        self.requests: Dict[str, RequestCache] = {}
        self._no_pages = [0] * len(self.groups)

    # ------------------------------------------------------------------ wiring
    def bindings(self) -> List[CacheBinding]:
        out: List[CacheBinding] = []
        for i, n in enumerate(self._entry_needs):
            b = CacheBinding()
            src = i if n.cache_of is None else n.cache_of
            eg = self._entry_group[src]
            if eg is not None:
                g, layer = eg
                b.group = g
                st = self.groups[g].storage
                if st is not None:
                    b.k_cache, b.v_cache = st[layer, 0], st[layer, 1]
                b.writes = n.cache_of is None
            b.state = {short: self.state.tensors.get(full) for short, full in self._entry_state_names[i].items()}
            out.append(b)
        return out

    def shared_state(self) -> Dict[str, torch.Tensor]:
        return {n: self.state.tensors[n] for n in self._shared_names if n in self.state.tensors}

    # ------------------------------------------------------------------ request life
    def begin(self, request_id: str, spare: bool = False) -> RequestCache:
        """``spare``: the slot comes out of the spare ones (a row that is no request)."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.state.alloc(spare=spare)
        rc = RequestCache(request_id, slot, tables=[PageTable() for _ in self.groups],
                          first_live=[0 for _ in self.groups])
        self.requests[request_id] = rc
        return rc

    def has(self, request_id: str) -> bool:
        return request_id in self.requests

    def _first_needed_page(self, g: PageGroup, next_pos: int) -> int:
        """Index of the first page a query at position >= next_pos can still see."""
        if g.window is None:
            return 0
        lo = next_pos - g.window + 1
        return max(0, lo) // self.page_size

    def pages_needed(self, request_id: str, n_new: int) -> List[int]:
        """New pages per group that ``n_new`` more tokens of this request need."""
        rc = self.requests[request_id]
        end = rc.cursor + rc.reserved + n_new
        if n_new == 1 and (end - 1) % self.page_size != 0 and all(len(t) * self.page_size >= end for t in rc.tables):
            return self._no_pages       # a decoded token inside a page the request already holds
        need = []
        for gi, g in enumerate(self.groups):
            have = len(rc.tables[gi])
            total = (end + self.page_size - 1) // self.page_size
            # pages that the window has passed before they were ever needed are not taken
            first = min(self._first_needed_page(g, rc.cursor + rc.reserved), total)
            need.append(max(0, total - max(have, first)))
        return need

    def can_reserve(self, items: Sequence[Tuple[str, int]]) -> bool:
        tot = [0] * len(self.groups)
        for rid, n in items:
            for gi, k in enumerate(self.pages_needed(rid, n)):
                tot[gi] += k
        return all(t <= g.pool.num_free for t, g in zip(tot, self.groups))

    def reserve(self, request_id: str, n_new: int) -> None:
        """Takes the pages for ``n_new`` tokens at the request's cursor. All or nothing."""
        rc = self.requests[request_id]
        need = self.pages_needed(request_id, n_new)
        for k, g in zip(need, self.groups):
            if k > g.pool.num_free:
                raise OutOfPages(f"request {request_id!r} needs {k} pages, {g.pool.num_free} are free")
        end = rc.cursor + rc.reserved + n_new
        total = (end + self.page_size - 1) // self.page_size
        for gi, g in enumerate(self.groups):
            first = min(self._first_needed_page(g, rc.cursor + rc.reserved), total)
            tbl = rc.tables[gi]
            while len(tbl) < total:
                if len(tbl) < first:
                    tbl.append(-1)
                    rc.first_live[gi] = max(rc.first_live[gi], len(tbl))
                else:
                    tbl.append(g.pool.alloc())
        rc.reserved += n_new

    def commit(self, request_id: str, n_new: int) -> None:
        """The step ran: the tokens are in the cache. Gives back pages a window has passed."""
        rc = self.requests[request_id]
        if n_new > rc.reserved:
            raise ValueError("commit of more tokens than were reserved")
        rc.cursor += n_new
        rc.reserved -= n_new
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            first = min(self._first_needed_page(g, rc.cursor), len(rc.tables[gi]))
            for pi in range(rc.first_live[gi], first):
                self._release(g, rc.tables[gi][pi])
                rc.tables[gi][pi] = -1
            rc.first_live[gi] = max(rc.first_live[gi], first)

    def rollback(self, request_id: str) -> None:
        """Undoes the reservations of a step that did not run: the pages taken beyond the request's cursor go
        back to the pool and nothing stays reserved."""
        rc = self.requests[request_id]
        keep = (rc.cursor + self.page_size - 1) // self.page_size
        for gi, g in enumerate(self.groups):
            tbl = rc.tables[gi]
            for pi in range(keep, len(tbl)):
                self._release(g, tbl[pi])
            tbl.truncate(keep)
            rc.first_live[gi] = min(rc.first_live[gi], keep)
        rc.reserved = 0

    def _release(self, g: PageGroup, page: int) -> None:
        if page < 0:
            return
        if self.poison_freed and g.storage is not None:
            g.storage[:, :, page] = float("nan")
        g.pool.free(page)

    def finish(self, request_id: str) -> None:
        """Gives back everything the request holds."""
        rc = self.requests.pop(request_id)
        for gi, g in enumerate(self.groups):
            for p in rc.tables[gi]:
                self._release(g, p)
        self.state.free(rc.slot)

    def reset(self, request_id: str) -> None:
        """Drops the request's pages and rewinds its cursor; it keeps its slot (used on preemption)."""
        rc = self.requests[request_id]
        for gi, g in enumerate(self.groups):
            for p in rc.tables[gi]:
                self._release(g, p)
            rc.tables[gi] = PageTable()
            rc.first_live[gi] = 0
        rc.cursor = 0
        rc.reserved = 0
        for t in self.state.tensors.values():
            t[rc.slot].zero_()

    # ------------------------------------------------------------------ per-step tables
    def block_table(self, group: int, request_ids: Sequence[str], round_to: int = 1, pow2: bool = False) -> np.ndarray:
        """[requests, width] page ids, -1 where a request has none. The width is that of the longest table, rounded up
        to a multiple of ``round_to``, or (``pow2``) to ``round_to`` times a power of two."""
        width = max(1, max((len(self.requests[r].tables[group]) for r in request_ids), default=1))
        width = -(-width // round_to) * round_to
        if pow2:
            w = round_to
            while w < width:
                w *= 2
            width = w
        bt = np.full((len(request_ids), width), -1, dtype=np.int32)
        for i, r in enumerate(request_ids):
            t = self.requests[r].tables[group].array()
            bt[i, :t.shape[0]] = t
        return bt

    def slot_map(self, group: int, request_ids: Sequence[str], q_lens: Sequence[int]) -> np.ndarray:
        """Flat cache slot (page * page_size + offset) of every token of the step, in batch order."""
        out = np.empty(int(sum(q_lens)), dtype=np.int32)
        o = 0
        ps = self.page_size
        for r, n in zip(request_ids, q_lens):
            rc = self.requests[r]
            if n == 1:
                page = rc.tables[group][rc.cursor // ps]
                if page < 0:
                    raise RuntimeError(f"request {r!r}: a token of this step maps to a page that was given back")
                out[o] = page * ps + rc.cursor % ps
                o += 1
                continue
            pos = np.arange(rc.cursor, rc.cursor + n)
            pages = rc.tables[group].array().astype(np.int64)[pos // ps]
            if (pages < 0).any():
                raise RuntimeError(f"request {r!r}: a token of this step maps to a page that was given back")
            out[o:o + n] = pages * ps + pos % ps
            o += n
        return out

    # ------------------------------------------------------------------ accounting
    def pages_in_use(self) -> List[int]:
        return [g.pool.num_held for g in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check_invariants(self) -> None:
        """No page lost, none held twice: every held page is in exactly one live table."""
        for gi, g in enumerate(self.groups):
            seen = set()
            for rc in self.requests.values():
                for p in rc.tables[gi]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise AssertionError(f"group {gi}: page {p} is in two block tables")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"group {gi}: page {p} is in a block table but free")
                    seen.add(p)
            if len(seen) != g.pool.num_held:
                raise AssertionError(f"group {gi}: {g.pool.num_held} pages held, {len(seen)} in block tables")
