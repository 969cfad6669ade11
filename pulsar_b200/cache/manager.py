"""Cache manager: paged keys and values with a block table per request, page pools per
group of layers, and slots for fixed-size per-request state.

What the reference's ``ActiveBuffer`` does for the one kind of layer it knows
(pulsar-core/src/runtime/kv/active_buffer.cpp:32-82 pools and LIFO free list, :152-228
claim/allocate/append/free, :255-279 slot mapping) is done here for several groups:
cache entries (one per entry of the model's run order) whose needs are equal (heads,
head size, window) share one pool, one free list and one block table per request.  A
group with a window gives pages back as soon as every future query has passed them.
Beside the pages every request holds one slot index into the fixed-state arenas of
the entries that declare such state (none do for Qwen3 dense, the slot exists anyway).

The accounting (``PageAllocator``, ``CacheManager`` with ``device=None``) is pure host
code and is tested without a GPU.

Physical layout of a group's pool: ``[entries, 2 (k, v), pages, kv_heads, page_size,
head_dim]``, so that one (page, kv head) tile of keys is contiguous
(``page_size * head_dim`` elements) for bulk copies.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch


class OutOfPages(RuntimeError):
    """No free page (or state slot) is left for what was asked."""


class CacheError(RuntimeError):
    """The manager was used wrongly (unknown request, double free, ...)."""


@dataclass(frozen=True)
class CacheNeed:
    """What one cache entry needs.  kind: "paged_kv", "state" or "none"."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: Optional[torch.dtype] = None   # None: the engine's activation dtype

    @staticmethod
    def paged_kv(n_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        return CacheNeed("paged_kv", n_kv_heads, head_dim, window)

    @staticmethod
    def state(shape: Sequence[int], dtype: Optional[torch.dtype] = None) -> "CacheNeed":
        return CacheNeed("state", state_shape=tuple(int(s) for s in shape), state_dtype=dtype)

    @staticmethod
    def none() -> "CacheNeed":
        return CacheNeed("none")


class PageAllocator:
    """LIFO free list over ``n`` ids; a fresh allocator yields 0, 1, 2, ... and a
    released id is the next one handed out (active_buffer.cpp:71-75, 219-221)."""

    def __init__(self, n: int):
        self.n = int(n)
        self._free: List[int] = list(range(self.n - 1, -1, -1))
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not (0 <= i < self.n) or not self._held[i]:
            raise CacheError(f"page {i} is not held (freed twice or never taken)")
        self._held[i] = False
        self._free.append(i)

    def held(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]


@dataclass
class _Group:
    need: CacheNeed                   # kind paged_kv; window shared by the group
    entries: List[int]                # cache entries that live in this group
    allocator: PageAllocator
    pool: Optional[torch.Tensor] = None   # [entries, 2, pages, Hkv, page, D]


@dataclass
class _Request:
    length: int = 0
    state_slot: int = -1
    tables: List[List[int]] = field(default_factory=list)     # per group: logical page -> page id or -1
    released: List[int] = field(default_factory=list)         # per group: logical pages [0, released) given back


class CacheManager:
    def __init__(self, needs: Sequence[CacheNeed], page_size: int, num_pages, max_requests: int,
                 dtype: torch.dtype = torch.float32, device=None):
        """``needs[i]`` is the need of cache entry i.  ``num_pages`` is an int (every
        group gets that many) or a list per group in order of first appearance.
        ``device=None`` keeps the accounting only (no tensors)."""
        if page_size <= 0:
            raise CacheError("page_size must be > 0")
        self.page_size = int(page_size)
        self.needs = list(needs)
        self.dtype, self.device = dtype, device
        self.groups: List[_Group] = []
        self.group_of_entry: Dict[int, int] = {}
        self.index_in_group: Dict[int, int] = {}
        key_to_group: Dict[Tuple, int] = {}
        for e, need in enumerate(self.needs):
            if need.kind != "paged_kv":
                continue
            key = (need.n_kv_heads, need.head_dim, need.window)
            if key not in key_to_group:
                key_to_group[key] = len(self.groups)
                self.groups.append(_Group(need, [], None))
            g = key_to_group[key]
            self.group_of_entry[e] = g
            self.index_in_group[e] = len(self.groups[g].entries)
            self.groups[g].entries.append(e)
        counts = [int(num_pages)] * len(self.groups) if isinstance(num_pages, int) else [int(n) for n in num_pages]
        if len(counts) != len(self.groups) or any(c <= 0 for c in counts):
            raise CacheError(f"num_pages must give a positive count for each of the {len(self.groups)} groups")
        for grp, c in zip(self.groups, counts):
            grp.allocator = PageAllocator(c)
            if device is not None:
                grp.pool = torch.zeros((len(grp.entries), 2, c, grp.need.n_kv_heads, self.page_size, grp.need.head_dim),
                                       dtype=dtype, device=device)
        self._windowed = any(grp.need.window is not None for grp in self.groups)
        self.max_requests = int(max_requests)
        self._slots = PageAllocator(self.max_requests)
        self.state: Dict[int, torch.Tensor] = {}
        for e, need in enumerate(self.needs):
            if need.kind == "state" and device is not None:
                self.state[e] = torch.zeros((self.max_requests, *need.state_shape),
                                            dtype=need.state_dtype or dtype, device=device)
        self._requests: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ requests
    def open(self, rid: Hashable) -> int:
        """Register a request and give it a state slot.  Holds no pages yet."""
        if rid in self._requests:
            raise CacheError(f"request {rid!r} is already open")
        try:
            slot = self._slots.take()
        except OutOfPages:
            raise OutOfPages(f"no free state slot (max_requests = {self.max_requests})") from None
        self._requests[rid] = _Request(0, slot, [[] for _ in self.groups], [0 for _ in self.groups])
        for e, t in self.state.items():      # fresh state starts at zero
            t[slot].zero_()
        return slot

    def has(self, rid: Hashable) -> bool:
        return rid in self._requests

    def _req(self, rid: Hashable) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise CacheError(f"unknown request {rid!r}") from None

    def length(self, rid: Hashable) -> int:
        return self._req(rid).length

    def n_logical_pages(self, rid: Hashable) -> int:
        """Logical pages the request's tables cover (the fewest over the groups)."""
        r = self._req(rid)
        return min(len(t) for t in r.tables) if r.tables else 0

    def state_slot(self, rid: Hashable) -> int:
        return self._req(rid).state_slot

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, grp: _Group, length: int) -> int:
        """Logical pages below this hold only keys that no query at position >= length sees."""
        if grp.need.window is None:
            return 0
        first_key = length - grp.need.window + 1        # oldest key the query at `length` sees
        return max(0, first_key) // self.page_size

    def pages_to_append(self, rid: Hashable, n_new: int) -> List[int]:
        """New pages each group must take so that the request can grow by ``n_new``
        tokens, after giving back what its windows have passed."""
        r = self._req(rid)
        out = []
        for g, grp in enumerate(self.groups):
            have = len(r.tables[g])
            need = -(-(r.length + n_new) // self.page_size)
            out.append(max(0, need - have))
        return out

    def reclaimable(self, rid: Hashable) -> List[int]:
        r = self._req(rid)
        return [max(0, min(self._first_needed_page(grp, r.length), len(r.tables[g])) - r.released[g])
                for g, grp in enumerate(self.groups)]

    def can_append(self, rid: Hashable, n_new: int) -> bool:
        need = self.pages_to_append(rid, n_new)
        back = self.reclaimable(rid)
        return all(n <= grp.allocator.n_free + b for n, b, grp in zip(need, back, self.groups))

    def can_admit(self, n_tokens: int) -> bool:
        """Could a request that holds nothing yet take ``n_tokens`` tokens (and a slot)?"""
        pages = -(-n_tokens // self.page_size)
        return self._slots.n_free > 0 and all(pages <= grp.allocator.n_free for grp in self.groups)

    def release_passed(self, rid: Hashable) -> int:
        """Give back the pages of windowed groups that every future query has passed."""
        if not self._windowed:
            return 0
        r = self._req(rid)
        n = 0
        for g, grp in enumerate(self.groups):
            upto = min(self._first_needed_page(grp, r.length), len(r.tables[g]))
            for lp in range(r.released[g], upto):
                grp.allocator.give(r.tables[g][lp])
                r.tables[g][lp] = -1
                n += 1
            r.released[g] = max(r.released[g], upto)
        return n

    def append(self, rid: Hashable, n_new: int) -> int:
        """Grow the request by ``n_new`` tokens; returns the position of the first one.
        Either every group gets its pages or nothing changes (OutOfPages)."""
        if n_new <= 0:
            raise CacheError("append needs n_new > 0")
        r = self._req(rid)
        if not self._windowed:
            # no group gives pages back early: one pass, check every group before taking anything
            need = -(-(r.length + n_new) // self.page_size)
            for g, grp in enumerate(self.groups):
                if need - len(r.tables[g]) > grp.allocator.n_free:
                    raise OutOfPages(f"request {rid!r}: {self.pages_to_append(rid, n_new)} new pages needed, "
                                     f"{[x.allocator.n_free for x in self.groups]} free")
            for g, grp in enumerate(self.groups):
                table = r.tables[g]
                for _ in range(need - len(table)):
                    table.append(grp.allocator.take())
            start = r.length
            r.length += n_new
            return start
        if not self.can_append(rid, n_new):
            raise OutOfPages(f"request {rid!r}: {self.pages_to_append(rid, n_new)} new pages needed, "
                             f"{[g.allocator.n_free for g in self.groups]} free")
        self.release_passed(rid)
        for g, need in enumerate(self.pages_to_append(rid, n_new)):
            for _ in range(need):
                r.tables[g].append(self.groups[g].allocator.take())
        start = r.length
        r.length += n_new
        return start

    def close(self, rid: Hashable) -> None:
        """Give back everything the request holds."""
        r = self._req(rid)
        for g, grp in enumerate(self.groups):
            for page in r.tables[g]:
                if page >= 0:
                    grp.allocator.give(page)
        self._slots.give(r.state_slot)
        del self._requests[rid]

    # ------------------------------------------------------------------ views for a step
    def table(self, rid: Hashable, group: int) -> List[int]:
        return self._req(rid).tables[group]

    def slots(self, rid: Hashable, group: int, start: int, n: int) -> List[int]:
        """slot = page * page_size + offset for positions [start, start + n)
        (active_buffer.cpp:255-279)."""
        table = self._req(rid).tables[group]
        ps = self.page_size
        out = []
        for p in range(start, start + n):
            page = table[p // ps]
            if page < 0:
                raise CacheError(f"request {rid!r}: position {p} lies in a released page")
            out.append(page * ps + p % ps)
        return out

    def kv_pools(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        g = self.group_of_entry[entry]
        pool = self.groups[g].pool[self.index_in_group[entry]]
        return pool[0], pool[1]

    def n_free_pages(self) -> List[int]:
        return [g.allocator.n_free for g in self.groups]

    def n_free_slots(self) -> int:
        return self._slots.n_free

    def check_consistency(self) -> None:
        """Every page is free or held by exactly one request; used by tests."""
        for g, grp in enumerate(self.groups):
            seen: Dict[int, Hashable] = {}
            for rid, r in self._requests.items():
                for page in r.tables[g]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"group {g}: page {page} held by {seen[page]!r} and {rid!r}")
                    seen[page] = rid
            if sorted(seen) != grp.allocator.held():
                raise CacheError(f"group {g}: held pages {grp.allocator.held()} != pages in tables {sorted(seen)}")
            if len(seen) + grp.allocator.n_free != grp.allocator.n:
                raise CacheError(f"group {g}: a page was lost")
        slots = sorted(r.state_slot for r in self._requests.values())
        if slots != self._slots.held():
            raise CacheError("state slots out of step with the live requests")
