"""The cache manager: paged keys and values per layer group, block tables per request,
and slots for per-request state of fixed size.

tamnd/fastmlx keeps, per request and layer, two tensors that grow by concatenation
(compute/models/cache.go:51-69) and plans a contiguous buffer in 256-token steps
(compute/kvcache.go:21,78-106); its blocks exist only as hash units (cache/blockhash.go:23).
Pages, block tables and what happens when pages run out are this engine's own.

Schedule entries whose mixers ask for the same (kv heads, head size, window) form a
group with one pool, one page geometry and one block table per request; a group with a
window gives a page back as soon as every position on it is out of every later query's
reach.  Memory of a layer: [num_pages, 2 (k|v), kv_heads, page_size, head_dim].
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import PagedKVSpec, StateSpec
from .pages import BlockTable, OutOfPages, PagePool


@dataclass
class CacheGroup:
    spec: PagedKVSpec
    entries: list[int]                  # schedule positions that own a cache in this group
    pool: PagePool
    kv: torch.Tensor | None = None      # [len(entries), num_pages, 2, nkv, page_size, hd]

    def page_bytes(self, elem: int) -> int:
        return 2 * self.spec.num_kv_heads * self.pool.page_size * self.spec.head_dim * elem * len(self.entries)


@dataclass
class RequestCache:
    """What one live request holds: a state slot, a block table per group, its length."""
    request_id: object
    slot: int
    tables: list[BlockTable]
    length: int = 0                     # tokens whose keys are in the cache
    reserved: int = 0                   # tokens of the running step, pages taken, not yet committed
    _new_pages: list[list[int]] = field(default_factory=list)


@dataclass
class EntryCache:
    """What a schedule entry's mixer sees: its layer of a group's pages, whether it writes
    them, and its state tensor [max_requests, *shape]."""
    kv: torch.Tensor | None
    group: int
    writable: bool
    state: torch.Tensor | None


class CacheManager:
    def __init__(self, cache_needs, *, page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.bfloat16, device="cpu", allocate: bool = True):
        """`cache_needs`: per schedule entry (PagedKVSpec | None, StateSpec | None,
        cache_from | None), as Model.cache_needs() returns it.  `num_pages` is per group: one
        number for all, or one per group in the order in which the schedule first names them
        (a group with a window needs far fewer than one that keeps every key)."""
        self.page_size, self.max_requests = int(page_size), int(max_requests)
        self.dtype, self.device = dtype, device
        self.groups: list[CacheGroup] = []
        by_spec: dict[PagedKVSpec, int] = {}
        entry_group: list[tuple[int, int] | None] = []
        for pos, (kv, _state, src) in enumerate(cache_needs):
            if kv is None:
                entry_group.append(None)
                continue
            if kv not in by_spec:
                by_spec[kv] = len(self.groups)
                n = num_pages if isinstance(num_pages, int) else list(num_pages)[len(self.groups)]
                self.groups.append(CacheGroup(kv, [], PagePool(int(n), page_size)))
            g = by_spec[kv]
            entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(pos)
        if allocate:
            for g in self.groups:
                g.kv = torch.empty((len(g.entries), g.pool.num_pages, 2, g.spec.num_kv_heads,
                                    page_size, g.spec.head_dim), dtype=dtype, device=device)
        self.entries: list[EntryCache] = []
        for pos, (kv, state, src) in enumerate(cache_needs):
            st = None
            if state is not None and allocate:
                st = torch.zeros((max_requests, *state.shape), dtype=state.dtype, device=device)
            if src is not None:
                if entry_group[src] is None:
                    raise ValueError(f"schedule[{pos}] reads the cache of entry {src}, which has none")
                g, i = entry_group[src]
                self.entries.append(EntryCache(self.groups[g].kv[i] if allocate else None, g, False, st))
            elif entry_group[pos] is not None:
                g, i = entry_group[pos]
                self.entries.append(EntryCache(self.groups[g].kv[i] if allocate else None, g, True, st))
            else:
                self.entries.append(EntryCache(None, -1, False, st))
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self.requests: dict[object, RequestCache] = {}
        # block tables by slot, as the step's batch builder wants them: one array per group,
        # -1 where there is no page; widened on demand
        self.table_mirror = [np.full((self.max_requests, 16), -1, dtype=np.int32) for _ in self.groups]

    # ------------------------------------------------------------------ sizes
    def bytes_per_token(self) -> int:
        e = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.page_bytes(e) // self.page_size for g in self.groups)

    def kv_bytes_read(self, req: RequestCache) -> int:
        """Bytes of keys and values a decode step of this request reads."""
        e = torch.empty((), dtype=self.dtype).element_size()
        total = 0
        for g in self.groups:
            n = req.length if g.spec.window <= 0 else min(req.length, g.spec.window)
            total += 2 * g.spec.num_kv_heads * g.spec.head_dim * e * len(g.entries) * n
        return total

    @property
    def free_pages(self) -> int:
        return min((g.pool.free_pages for g in self.groups), default=0)

    def pages_needed(self, req: RequestCache | None, n_new: int, length: int = 0) -> int:
        """Most pages any group must take so that `n_new` more tokens fit.  (A block table has
        an entry for every page of positions, given back or not, so a group with a window asks
        for as many new pages as one without.)"""
        cur = length if req is None else req.length + req.reserved
        total = -(-(cur + n_new) // self.page_size)
        if req is None or not req.tables:
            return max(0, total)
        return max(max(0, total - len(bt.pages)) for bt in req.tables)

    def holds_alone(self, n_tokens: int, portion: int) -> int:
        """0 if a request of `n_tokens` fed in portions of at most `portion` tokens fits the
        pools when it runs alone; else the number of tokens the tightest group can hold.  A
        group with a window holds the window and the running portion, not the whole request."""
        for g in self.groups:
            room = g.pool.num_pages * self.page_size
            w = g.spec.window
            need = n_tokens if w <= 0 else min(n_tokens, w + min(portion, n_tokens) + self.page_size)
            if need > room:
                return room
        return 0

    # ------------------------------------------------------------------ per-request state
    @property
    def has_state(self) -> bool:
        return any(e.state is not None for e in self.entries)

    def snapshot_state(self, slots=None):
        """Copies of the state slots (all, or the given ones): what `restore_state` puts back
        after a step that must not count (a failed one, or the warm-up run before a capture)."""
        idx = None if slots is None else torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        return idx, [None if e.state is None else (e.state.clone() if idx is None else e.state[idx].clone())
                     for e in self.entries]

    def restore_state(self, snapshot) -> None:
        idx, saved = snapshot
        for e, s in zip(self.entries, saved):
            if s is not None:
                if idx is None:
                    e.state.copy_(s)
                else:
                    e.state[idx] = s

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        for e in self.entries:
            if e.state is not None:
                e.state[slot].zero_()
        rc = RequestCache(request_id, slot, [BlockTable() for _ in self.groups])
        self.requests[request_id] = rc
        return rc

    def reserve(self, req: RequestCache, n_new: int) -> None:
        """Take the pages that positions [length, length + n_new) need, in every group, or
        none at all."""
        if req.reserved:
            raise RuntimeError("a request can take part in a step only once")
        taken: list[list[int]] = []
        try:
            for g, bt in zip(self.groups, req.tables):
                need = -(-(req.length + n_new) // self.page_size) - len(bt.pages)
                taken.append(g.pool.take(max(0, need)))
        except OutOfPages:
            for g, pages in zip(self.groups, taken):
                g.pool.give(pages)
            raise
        for gi, (bt, pages) in enumerate(zip(req.tables, taken)):
            if pages:
                at = len(bt.pages)
                bt.pages.extend(pages)
                self._mirror_set(gi, req.slot, at, pages)
        req.reserved, req._new_pages = n_new, taken

    def rollback(self, req: RequestCache) -> None:
        """Undo `reserve` after a step that failed: no state has advanced."""
        for gi, (g, bt, pages) in enumerate(zip(self.groups, req.tables, req._new_pages)):
            if pages:
                del bt.pages[len(bt.pages) - len(pages):]
                self.table_mirror[gi][req.slot, len(bt.pages): len(bt.pages) + len(pages)] = -1
                g.pool.give(pages)
        req.reserved, req._new_pages = 0, []

    def commit(self, req: RequestCache) -> None:
        """The step ran: the reserved tokens are in the cache.  Pages that a window has
        passed go back to the pool."""
        req.length += req.reserved
        req.reserved, req._new_pages = 0, []
        for gi, (g, bt) in enumerate(zip(self.groups, req.tables)):
            w = g.spec.window
            if w <= 0:
                continue
            # the next query sits at position >= length and sees keys > position - w
            first_needed = req.length - w + 1
            while bt.first_live < len(bt.pages) and (bt.first_live + 1) * self.page_size <= first_needed:
                g.pool.give([bt.pages[bt.first_live]])
                bt.pages[bt.first_live] = -1
                self.table_mirror[gi][req.slot, bt.first_live] = -1
                bt.first_live += 1

    def free(self, request_id) -> None:
        """Give back everything the request holds (finished, aborted or preempted)."""
        req = self.requests.pop(request_id)
        for gi, (g, bt) in enumerate(zip(self.groups, req.tables)):
            g.pool.give(bt.live())
            bt.pages, bt.first_live = [], 0
            self.table_mirror[gi][req.slot, :] = -1
        self._free_slots.append(req.slot)

    def _mirror_set(self, gi: int, slot: int, at: int, pages) -> None:
        m = self.table_mirror[gi]
        if at + len(pages) > m.shape[1]:
            wider = np.full((m.shape[0], max(2 * m.shape[1], at + len(pages))), -1, dtype=np.int32)
            wider[:, :m.shape[1]] = m
            self.table_mirror[gi] = m = wider
        m[slot, at: at + len(pages)] = pages

    def free_all(self) -> None:
        for rid in list(self.requests):
            self.free(rid)

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = []
            for r in self.requests.values():
                bt = r.tables[gi]
                assert all(p == -1 for p in bt.pages[:bt.first_live])
                held.extend(bt.live())
            assert len(held) == len(set(held)), "a page is in two block tables"
            assert all(0 <= p < g.pool.num_pages for p in held)
            assert len(held) == g.pool.used_pages, "pages held by no request"
            m = self.table_mirror[gi]
            for r in self.requests.values():
                n = len(r.tables[gi].pages)
                assert m[r.slot, :n].tolist() == r.tables[gi].pages and (m[r.slot, n:] == -1).all(), "mirror out of step"
            free = [s for s in self._free_slots]
            assert (m[free] == -1).all(), "a free slot still has pages in the mirror"
        slots = [r.slot for r in self.requests.values()]
        assert len(set(slots)) == len(slots)
        assert sorted(slots + self._free_slots) == list(range(self.max_requests)), "a slot is lost"
