"""The cache manager: pages of keys and values with a block table per request, and slots
for per-request state of fixed size.

AIR's CUDA cache allocates a device page per request on demand, all layers in one page,
and keeps a table of page pointers per sequence (src/cuda/cuda_backend.cu:1186-1433).  Here
the memory is one slab per layer made at start, pages are numbers, and:

* What a run keeps is described by its mixer's needs (air_b200.parts.base.CacheNeed).  The
  manager knows no kinds of need: a paged need states the shape of one page of it and whether
  old pages may go back (a window), a need that is not paged states the shape of its per-request
  state; the mixer receives what the need's `view` makes of the memory.
* Runs with paged needs of the same group key (for keys and values: kv heads, head size, window)
  form a *group*.  A group has its own pool of pages and its own block table per request; page n
  of a group is row n of every run's slab in that group.
* A page belongs to one request from `reserve` until the request is closed, or, in a group
  with a window, until every key in it is older than the window of any future query.
  Freed pages go back on the pool's stack and are handed out again at once.
* `reserve` for a batch either gets every page the batch needs or changes nothing.
* A request's length advances only at `commit`, after the step has succeeded
  (AIR: begin_transaction / commit_kv / rollback, src/cuda/cuda_backend.cu:1397-1432, 2291-2298).
* A request also holds one slot index; every run that keeps a fixed-size state has a tensor
  [slots, *shape] that is zeroed at the slot's row when the request opens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, PagedKV, PagedKVView, SlotState, SlotStateView  # noqa: F401 (views: old import path)


class OutOfPages(RuntimeError):
    """The pool of a group cannot hold what a step needs.  Nothing was changed."""


class CacheError(RuntimeError):
    pass


class PagePool:
    """Page numbers 0..n-1 with an owner each.  LIFO: the page freed last is reused first."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._owner: List[Optional[Hashable]] = [None] * num_pages
        self.peak_used = 0
        self.takes = 0      # pages handed out so far; more than num_pages means pages were used again

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, owner: Hashable) -> int:
        if owner is None:
            raise CacheError("a page needs an owner")
        if not self._free:
            raise OutOfPages("out of KV pages")
        page = self._free.pop()
        if self._owner[page] is not None:
            raise CacheError(f"page {page} was on the free stack while owned by {self._owner[page]!r}")
        self._owner[page] = owner
        self.takes += 1
        self.peak_used = max(self.peak_used, self.used_pages)
        return page

    def give(self, page: int, owner: Hashable) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} does not exist")
        if self._owner[page] is None:
            raise CacheError(f"page {page} is freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} belongs to {self._owner[page]!r}, not to {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """No page lost, none held twice: free and owned pages partition the pool."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free stack twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise CacheError(f"page {p} is {'both free and owned' if p in free else 'neither free nor owned'}")


@dataclass
class Group:
    key: Hashable                 # the needs' group key
    window: Optional[int]         # None: every page is kept until the request ends
    pool: PagePool
    runs: List[int] = field(default_factory=list)


@dataclass
class Sequence_:
    request: Hashable
    slot: int
    length: int = 0                      # committed tokens
    pages: List[List[int]] = field(default_factory=list)  # per group: page of block b, or -1 once given back


class CacheManager:
    """needs_per_run[i]: the needs of the i-th run of the order list (empty for a run that
    reads another run's cache).  allocate=False builds the bookkeeping without device memory
    (for tests of the bookkeeping)."""

    def __init__(self, needs_per_run: Sequence[Sequence[object]], page_tokens: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype = torch.float32, device="cpu", allocate: bool = True,
                 max_blocks: Optional[int] = None):
        if page_tokens <= 0 or page_tokens % 16:
            raise CacheError(f"page size {page_tokens} must be a positive multiple of 16")
        if num_pages <= 0:
            raise CacheError("the pool needs at least one page")
        self.page_tokens, self.num_pages, self.max_requests = page_tokens, num_pages, max_requests
        self.dtype, self.device = dtype, device
        self.groups: List[Group] = []
        self._views: List[Tuple[object, ...]] = []
        self._state_tensors: List[torch.Tensor] = []
        for run, needs in enumerate(needs_per_run):
            views = []
            for need in needs:
                if not isinstance(need, CacheNeed):
                    raise CacheError(f"run {run}: {need!r} is not a cache need")
                memory, g = None, None
                if need.paged:
                    g = self._group_of(need)
                    if run not in self.groups[g].runs:
                        self.groups[g].runs.append(run)
                    if allocate:
                        memory = torch.zeros((num_pages,) + tuple(need.page_shape(page_tokens)),
                                             dtype=need.element_dtype(dtype), device=device)
                elif allocate:
                    memory = torch.zeros((max_requests,) + tuple(need.slot_shape()),
                                         dtype=need.element_dtype(dtype), device=device)
                    self._state_tensors.append(memory)
                views.append(need.view(memory, g))
            self._views.append(tuple(views))
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.sequences: Dict[Hashable, Sequence_] = {}
        # Block tables on the device, one per group: row = the request's slot, column = block of
        # page_tokens positions, value = page (or -1).  They are kept up to date by small updates
        # (slot, block, page) that `flush_tables` sends before a step, so a step copies no tables.
        # max_blocks bounds a request's length (in a group with a window a request may be longer
        # than the whole pool, since it gives old pages back).
        self.max_blocks = max_blocks if max_blocks is not None else (num_pages if allocate else 1 << 30)
        self.tables: List[Optional[torch.Tensor]] = []
        self._updates: List[Dict[Tuple[int, int], int]] = []   # (slot, block) -> page: the last write wins
        for _ in self.groups:
            self.tables.append(torch.full((max_requests, self.max_blocks), -1, dtype=torch.int32, device=device)
                               if allocate else None)
            self._updates.append({})

    def _group_of(self, need: CacheNeed) -> int:
        key = need.group_key()
        for i, g in enumerate(self.groups):
            if g.key == key:
                return i
        self.groups.append(Group(key, need.window, PagePool(self.num_pages)))
        return len(self.groups) - 1

    @staticmethod
    def bytes_per_page(needs_per_run: Sequence[Sequence[object]], page_tokens: int, dtype: torch.dtype) -> int:
        """Device bytes that one page number costs over all runs (every run has a slab of its own)."""
        return sum(need.bytes_per_page(page_tokens, dtype) for needs in needs_per_run for need in needs
                   if getattr(need, "paged", False))

    # ------------------------------------------------------------------ what mixers see
    def views(self, run: int):
        return self._views[run]

    # ------------------------------------------------------------------ requests
    def open(self, request: Hashable) -> Sequence_:
        if request in self.sequences:
            raise CacheError(f"request {request!r} is already open")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        for st in self._state_tensors:
            st[slot].zero_()
        seq = Sequence_(request, slot, 0, [[] for _ in self.groups])
        self.sequences[request] = seq
        return seq

    def close(self, request: Hashable) -> None:
        seq = self.sequences.pop(request, None)
        if seq is None:
            raise CacheError(f"request {request!r} is not open")
        for g, pages in zip(self.groups, seq.pages):
            for p in pages:
                if p >= 0:
                    g.pool.give(p, request)
        self._free_slots.append(seq.slot)

    def pages_needed(self, tokens: int) -> int:
        return -(-tokens // self.page_tokens)

    def _first_live_block(self, window: Optional[int], length: int) -> int:
        """Blocks below this hold only tokens that no query at position >= length can see."""
        if window is None:
            return 0
        return max(0, length - window + 1) // self.page_tokens

    def reserve(self, batch: Sequence[Tuple[Hashable, int]]) -> None:
        """Makes room for `n` more tokens of each request in the batch: all of it or none."""
        taken: List[Tuple[int, Hashable, int]] = []  # (group, request, blocks appended)
        for request, n in batch:
            want = self.pages_needed(self.sequences[request].length + n)
            if want > self.max_blocks:
                raise CacheError(f"request {request!r} would need {want} blocks, tables have {self.max_blocks}")
        try:
            for request, n in batch:
                seq = self.sequences[request]
                want = self.pages_needed(seq.length + n)
                for gi, g in enumerate(self.groups):
                    pages = seq.pages[gi]
                    while len(pages) < want:
                        pages.append(g.pool.take(request))
                        taken.append((gi, request, 1))
                        self._updates[gi][(seq.slot, len(pages) - 1)] = pages[-1]
        except OutOfPages:
            for gi, request, _ in reversed(taken):
                page = self.sequences[request].pages[gi].pop()
                self.groups[gi].pool.give(page, request)
                seq = self.sequences[request]
                self._updates[gi].pop((seq.slot, len(seq.pages[gi])), None)
            raise

    def commit(self, request: Hashable, n: int) -> None:
        """The step that wrote `n` more tokens of the request has succeeded."""
        seq = self.sequences[request]
        seq.length += n
        if self.groups and seq.length > len(seq.pages[0]) * self.page_tokens:
            raise CacheError(f"request {request!r} holds fewer pages than its length needs")
        for gi, g in enumerate(self.groups):
            first = self._first_live_block(g.window, seq.length)
            pages = seq.pages[gi]
            for b in range(min(first, len(pages))):
                if pages[b] >= 0:
                    g.pool.give(pages[b], request)
                    pages[b] = -1
                    self._updates[gi][(seq.slot, b)] = -1

    def flush_tables(self) -> None:
        """Sends the pending updates of the block tables to the device."""
        for gi, upd in enumerate(self._updates):
            if upd and self.tables[gi] is not None:
                from ..csrc import ops
                host = torch.tensor([x for (slot, block), page in upd.items() for x in (slot, block, page)],
                                    dtype=torch.int32)
                if self.tables[gi].is_cuda:
                    ops.table_update(self.tables[gi], host.pin_memory().to(self.tables[gi].device, non_blocking=True))
                else:
                    u = host.view(-1, 3).long()
                    self.tables[gi][u[:, 0], u[:, 1]] = u[:, 2].int()
            upd.clear()

    def trim(self, request: Hashable) -> None:
        """Gives back pages beyond the committed length (after a step that failed)."""
        seq = self.sequences[request]
        keep = self.pages_needed(seq.length)
        for gi, g in enumerate(self.groups):
            pages = seq.pages[gi]
            while len(pages) > keep:
                p = pages.pop()
                if p >= 0:
                    g.pool.give(p, request)

    # ------------------------------------------------------------------ figures
    def length(self, request: Hashable) -> int:
        return self.sequences[request].length

    def free_pages(self) -> int:
        return min((g.pool.free_pages for g in self.groups), default=self.num_pages)

    def used_pages(self, request: Optional[Hashable] = None) -> int:
        if request is None:
            return max((g.pool.used_pages for g in self.groups), default=0)
        seq = self.sequences[request]
        return max((sum(1 for p in pages if p >= 0) for pages in seq.pages), default=0)

    def check(self) -> None:
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = {}
            for seq in self.sequences.values():
                for p in seq.pages[gi]:
                    if p < 0:
                        continue
                    if p in held:
                        raise CacheError(f"page {p} of group {gi} is held by {held[p]!r} and {seq.request!r}")
                    held[p] = seq.request
                    if g.pool.owner(p) != seq.request:
                        raise CacheError(f"page {p} of group {gi}: table and pool disagree on the owner")
            if len(held) != g.pool.used_pages:
                raise CacheError(f"group {gi}: {g.pool.used_pages - len(held)} pages are owned but in no table")
        slots = [s.slot for s in self.sequences.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")
