"""Cache manager: keys and values in pages, one block table per request and
layer group, and slots for per-request state of fixed size.

Layers with the same needs form a group (same window rule, same number of kv
heads and head size).  A group owns its pages: a page id addresses the same
page in every cache of the group, so one block table per (request, group)
serves all of the group's layers.  A block table is indexed by the logical page
`position // page_size`; an entry is -1 once the group's window has passed the
page, and that page is back in the pool.

Pages are given back
  * when the request ends (`release`), and
  * after a step (`commit`), for every page that lies wholly before the first
    position the group's window still lets a later token read.  Within a step the
    old pages are still held, because a portion that crosses a window boundary
    reads the old window with its first tokens and writes the new one with its last.

This module is host-side bookkeeping only (no tensors); `storage.py` owns the
device memory the page ids address.

Counterpart in giveen/spite: `BlockPool` / `PagedSeqCache` / `RingCache`
(crates/spite-kvcache/src/paged.rs:51-171, crates/spite-kvcache/src/lib.rs:266-326),
which no forward pass uses there; errors follow `CacheError` (lib.rs:233-241).
"""
from __future__ import annotations

from dataclasses import dataclass


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """A group's pool cannot supply the pages a step needs.  Nothing was changed."""


class OutOfSlots(CacheError):
    """Every per-request state slot is taken."""


@dataclass(frozen=True)
class Window:
    """Which earlier positions a layer may read: all ("full"), those of the
    reader's own chunk ("chunk", size C), or the last W ("sliding", size W)."""
    kind: str
    size: int = 0

    def __post_init__(self):
        if self.kind not in ("full", "chunk", "sliding"):
            raise ValueError(f"unknown window kind {self.kind!r}")
        if self.kind != "full" and self.size < 1:
            raise ValueError("a chunk or sliding window needs a positive size")

    def first_needed(self, next_pos: int) -> int:
        """Lowest position that a token at `next_pos` or later can still read."""
        if self.kind == "full":
            return 0
        if self.kind == "chunk":
            return (next_pos // self.size) * self.size
        return max(0, next_pos - self.size + 1)

    def lowest_visible(self, pos: int) -> int:
        """Lowest position visible to the token at `pos` (the kernels use the same rule)."""
        return self.first_needed(pos)


@dataclass(frozen=True)
class GroupKey:
    window: Window
    num_kv_heads: int
    head_dim: int


class PagePool:
    """Free pages of one group.  Last freed, first reused."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool exhausted")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int):
        if not 0 <= page < self.n_pages or not self._held[page]:
            raise CacheError(f"page {page} freed but not held")
        self._held[page] = False
        self._free.append(page)


class SlotPool:
    """Slots for per-request state of fixed size (also the request's row in
    per-request device tables).  Lowest free slot first."""

    def __init__(self, n_slots: int):
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = [False] * n_slots

    @property
    def n_free(self):
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.n_slots} request slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, slot: int):
        if not 0 <= slot < self.n_slots or not self._held[slot]:
            raise CacheError(f"slot {slot} freed but not held")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


class RequestCache:
    """What one live request holds."""

    def __init__(self, slot: int, n_groups: int):
        self.slot = slot
        self.n_tokens = 0                      # positions whose keys and values are cached
        self.tables = [[] for _ in range(n_groups)]   # logical page -> physical page or -1
        self.pending = [[] for _ in range(n_groups)]  # logical pages allocated by an uncommitted reserve
        self.len_before = [0] * n_groups       # block-table lengths before the uncommitted reserve
        self.reserved = 0                      # tokens covered by the uncommitted reserve
        self.fresh = True                      # no step has run yet: fixed-size state must be cleared


class CacheManager:
    def __init__(self, groups: list[GroupKey], page_size: int, pages_per_group, n_slots: int):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(self.groups)
        self.pools = [PagePool(n) for n in pages_per_group]
        self.slots = SlotPool(n_slots)
        self.requests: dict[object, RequestCache] = {}

    # ---------------------------------------------------------------- requests
    def admit(self, req_id) -> RequestCache:
        if req_id in self.requests:
            raise CacheError(f"request {req_id!r} is already live")
        rc = RequestCache(self.slots.alloc(), len(self.groups))
        self.requests[req_id] = rc
        return rc

    def get(self, req_id) -> RequestCache:
        try:
            return self.requests[req_id]
        except KeyError:
            raise CacheError(f"request {req_id!r} is not live") from None

    def release(self, req_id):
        """The request ends: everything it holds goes back."""
        rc = self.get(req_id)
        for g, table in enumerate(rc.tables):
            for page in table:
                if page >= 0:
                    self.pools[g].free(page)
        self.slots.free(rc.slot)
        del self.requests[req_id]

    # ---------------------------------------------------------------- pages
    def pages_needed(self, req_id, n_new: int) -> list[int]:
        """Pages each group must newly supply to cache `n_new` more tokens."""
        rc = self.requests.get(req_id)
        have = [len(t) for t in rc.tables] if rc else [0] * len(self.groups)
        start = rc.n_tokens if rc else 0
        end = start + n_new
        need_total = -(-end // self.page_size)
        out = []
        for g, key in enumerate(self.groups):
            # pages before the window of the portion's first token are never touched
            first = key.window.first_needed(start) // self.page_size
            out.append(max(0, need_total - max(have[g], first)))
        return out

    def can_reserve(self, wants: dict) -> bool:
        """True if the pools can supply every (request -> n_new) of `wants` together."""
        total = [0] * len(self.groups)
        for req_id, n in wants.items():
            for g, k in enumerate(self.pages_needed(req_id, n)):
                total[g] += k
        return all(t <= p.n_free for t, p in zip(total, self.pools))

    def reserve(self, req_id, n_new: int):
        """Make every group's block table cover positions [n_tokens, n_tokens + n_new).
        All or nothing: on `OutOfPages` the request holds what it held before."""
        rc = self.get(req_id)
        if rc.reserved:
            raise CacheError(f"request {req_id!r} already has an uncommitted reserve")
        if n_new < 1:
            raise CacheError("reserve needs at least one token")
        need = self.pages_needed(req_id, n_new)
        for g, k in enumerate(need):
            if k > self.pools[g].n_free:
                raise OutOfPages(
                    f"group {g} ({self.groups[g].window.kind}) needs {k} pages for request {req_id!r}, "
                    f"{self.pools[g].n_free} of {self.pools[g].n_pages} are free")
        end_pages = -(-(rc.n_tokens + n_new) // self.page_size)
        rc.len_before = [len(t) for t in rc.tables]
        for g, key in enumerate(self.groups):
            table = rc.tables[g]
            first = key.window.first_needed(rc.n_tokens) // self.page_size
            while len(table) < end_pages:
                lp = len(table)
                if lp < first:
                    table.append(-1)
                else:
                    table.append(self.pools[g].alloc())
                    rc.pending[g].append(lp)
        rc.reserved = n_new

    def rollback(self, req_id):
        """Undo an uncommitted reserve (the step did not run)."""
        rc = self.get(req_id)
        if not rc.reserved:
            raise CacheError(f"request {req_id!r} has nothing reserved")
        for g, lps in enumerate(rc.pending):
            for lp in lps:
                self.pools[g].free(rc.tables[g][lp])
            del rc.tables[g][rc.len_before[g]:]
            rc.pending[g] = []
        rc.reserved = 0

    def commit(self, req_id) -> list[list[int]]:
        """The step ran: the reserved tokens are cached.  Pages that every later
        token's window has passed are freed; returns them per group."""
        rc = self.get(req_id)
        if not rc.reserved:
            raise CacheError(f"request {req_id!r} has nothing reserved")
        rc.n_tokens += rc.reserved
        rc.reserved = 0
        rc.fresh = False
        freed = []
        for g, key in enumerate(self.groups):
            rc.pending[g] = []
            rc.len_before[g] = len(rc.tables[g])
            first_live = key.window.first_needed(rc.n_tokens) // self.page_size
            out = []
            table = rc.tables[g]
            for lp in range(min(first_live, len(table))):
                if table[lp] >= 0:
                    self.pools[g].free(table[lp])
                    out.append(table[lp])
                    table[lp] = -1
            freed.append(out)
        return freed

    def pending_pages(self, req_id) -> list[list[int]]:
        """Per group, the pages that the request's uncommitted reserve took from the pool."""
        rc = self.get(req_id)
        return [[rc.tables[g][lp] for lp in lps] for g, lps in enumerate(rc.pending)]

    # ---------------------------------------------------------------- views
    def block_table(self, req_id, group: int) -> list[int]:
        return self.get(req_id).tables[group]

    def free_pages(self) -> list[int]:
        return [p.n_free for p in self.pools]

    def check_invariants(self):
        """No page lost, none held twice.  For tests and debugging."""
        for g, pool in enumerate(self.pools):
            held = []
            for rc in self.requests.values():
                held += [p for p in rc.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            if set(held) & set(pool._free):
                raise CacheError(f"group {g}: a held page is on the free list")
            if len(set(pool._free)) != len(pool._free):
                raise CacheError(f"group {g}: a page is on the free list twice")
            if len(held) + pool.n_free != pool.n_pages:
                raise CacheError(f"group {g}: {pool.n_pages - len(held) - pool.n_free} pages lost")
            for p in range(pool.n_pages):
                if pool._held[p] != (p in held):
                    raise CacheError(f"group {g}: held flag of page {p} is wrong")
        slots = [rc.slot for rc in self.requests.values()]
        if len(slots) != len(set(slots)):
            raise CacheError("a state slot is held twice")
        if len(slots) + self.slots.n_free != self.slots.n_slots:
            raise CacheError("a state slot was lost")
