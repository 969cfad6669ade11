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

The accounting lives in the host runtime (C++, csrc/host/cache.cpp) and is tested without a GPU
(``PageAllocator``, ``CacheManager`` with ``device=None``).

A mixer declares the tensors it caches per token (``CachedTensor``: a name, heads, a width per
head); keys and values of equal shape are the usual case, a mixer may as well cache keys and
values of different widths, or one tensor only.  Every declared tensor has a pool of its own,
``[entries, pages, heads, page_size, width]``, so that one (page, head) tile is contiguous
(``page_size * width`` elements) for bulk copies; the tensors of a group share page ids and
block tables.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from .. import host


class OutOfPages(RuntimeError):
    """No free page (or state slot) is left for what was asked."""


class CacheError(RuntimeError):
    """The manager was used wrongly (unknown request, double free, ...)."""


@dataclass(frozen=True)
class CachedTensor:
    """One tensor a mixer caches for every token: ``heads`` rows of ``width`` elements."""
    name: str
    heads: int
    width: int
    dtype: Optional[torch.dtype] = None         # None: the engine's activation dtype


@dataclass(frozen=True)
class CacheNeed:
    """What one cache entry needs.  kind: "paged_kv" (``tensors`` per token, in pages), "state" or "none"."""
    kind: str
    tensors: Tuple[CachedTensor, ...] = ()
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: Optional[torch.dtype] = None   # None: the engine's activation dtype

    @staticmethod
    def paged(tensors: Sequence[CachedTensor], window: Optional[int] = None) -> "CacheNeed":
        tensors = tuple(tensors)
        names = [t.name for t in tensors]
        if not tensors or len(set(names)) != len(names) or any(t.heads <= 0 or t.width <= 0 for t in tensors):
            raise ValueError(f"a paged cache entry needs tensors with distinct names and positive sizes, found {tensors}")
        return CacheNeed("paged_kv", tensors, window)

    @staticmethod
    def paged_kv(n_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        """Keys and values of one shape: tensors "k" and "v"."""
        return CacheNeed.paged((CachedTensor("k", n_kv_heads, head_dim), CachedTensor("v", n_kv_heads, head_dim)), window)

    def bytes_per_token(self, default_dtype: torch.dtype) -> int:
        return sum(t.heads * t.width * (t.dtype or default_dtype).itemsize for t in self.tensors)

    @staticmethod
    def state(shape: Sequence[int], dtype: Optional[torch.dtype] = None) -> "CacheNeed":
        return CacheNeed("state", state_shape=tuple(int(s) for s in shape), state_dtype=dtype)

    @staticmethod
    def none() -> "CacheNeed":
        return CacheNeed("none")


class PageAllocator:
    """LIFO free list over ``n`` ids; a fresh allocator yields 0, 1, 2, ... and a
    released id is the next one handed out (active_buffer.cpp:71-75, 219-221).  The list
    lives in the host runtime (csrc/host/cache.h: FreeList)."""

    def __init__(self, n: int):
        self.n = int(n)
        self._lib = host.lib()
        self._h = self._lib.ph_freelist_new(self.n)
        if not self._h:
            raise CacheError(f"a free list needs a size >= 0, found {n}")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ph_freelist_delete(h)

    @property
    def n_free(self) -> int:
        return self._lib.ph_freelist_n_free(self._h)

    def take(self) -> int:
        i = self._lib.ph_freelist_take(self._h)
        if i < 0:
            raise OutOfPages("no free page")
        return i

    def give(self, i: int) -> None:
        if self._lib.ph_freelist_give(self._h, int(i)) != 0:
            raise CacheError(f"page {i} is not held (freed twice or never taken)")

    def held(self) -> List[int]:
        return [i for i in range(self.n) if self._lib.ph_freelist_held(self._h, i)]


class _GroupPages:
    """The free list of one group inside the native cache, as far as callers look at it."""

    def __init__(self, manager: "CacheManager", group: int):
        self._m, self._g = manager, group
        self.n = manager._lib.ph_n_pages(manager._h, group)

    @property
    def n_free(self) -> int:
        return self._m._lib.ph_n_free_pages(self._m._h, self._g)

    def held(self) -> List[int]:
        return [i for i in range(self.n) if self._m._lib.ph_page_held(self._m._h, self._g, i)]


@dataclass
class _Group:
    need: CacheNeed                   # kind paged_kv; window shared by the group
    entries: List[int]                # cache entries that live in this group
    allocator: Optional[_GroupPages]
    pools: Optional[Dict[str, torch.Tensor]] = None   # tensor name -> [entries, pages, heads, page, width]


class CacheManager:
    """The tensors of the cache (pools, state arenas) and the request names live here; pages, block
    tables, lengths and slots are kept by the host runtime (csrc/host/cache.cpp), which this class
    calls.  Requests are named by any hashable value; the runtime knows them by a number."""

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
            key = (need.tensors, need.window)
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
        self.max_requests = int(max_requests)
        self._lib = host.lib()
        windows = [int(grp.need.window) if grp.need.window is not None else -1 for grp in self.groups]
        self._h = self._lib.ph_cache_new(len(self.groups), host.ints(windows), host.ints(counts), self.page_size,
                                         self.max_requests)
        if not self._h:
            raise CacheError("the host runtime refused the cache's sizes")
        self._n_groups = len(self.groups)
        self._scratch = (ctypes.c_int * max(1, self._n_groups))()
        for g, (grp, c) in enumerate(zip(self.groups, counts)):
            grp.allocator = _GroupPages(self, g)
            if device is not None:
                grp.pools = {t.name: torch.zeros((len(grp.entries), c, t.heads, self.page_size, t.width),
                                                 dtype=t.dtype or dtype, device=device) for t in grp.need.tensors}
        self.state: Dict[int, torch.Tensor] = {}
        for e, need in enumerate(self.needs):
            if need.kind == "state" and device is not None:
                self.state[e] = torch.zeros((self.max_requests, *need.state_shape),
                                            dtype=need.state_dtype or dtype, device=device)
        # Resident block tables (device): one row per state slot and group; a step sends only the page ids that its
        # requests gained (the step function turns this on and asks for the tensors).
        self.resident: Dict[int, torch.Tensor] = {}
        self._ids: Dict[Hashable, int] = {}         # request name -> the runtime's number for it
        self._names: Dict[int, Hashable] = {}
        self._pinned: set = set()                   # names that keep their number while they hold nothing
        self._next_id = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ph_cache_delete(h)

    # ------------------------------------------------------------------ requests
    def native_id(self, rid: Hashable, create: bool = False) -> int:
        """The runtime's number for a request name.  Names are numbered at their first mention
        (``create``), which may be before the request is opened: the scheduler knows waiting
        requests by the same numbers."""
        nid = self._ids.get(rid)
        if nid is None:
            if not create:
                raise CacheError(f"unknown request {rid!r}")
            nid = self._ids[rid] = self._next_id
            self._names[nid] = rid
            self._next_id += 1
        return nid

    def name_of(self, native_id: int) -> Hashable:
        return self._names[native_id]

    def pin(self, rid: Hashable) -> int:
        """Keep the name's number although the request holds nothing (it waits in the scheduler)."""
        nid = self.native_id(rid, create=True)
        self._pinned.add(rid)
        return nid

    def unpin(self, rid: Hashable) -> None:
        self._pinned.discard(rid)
        self._forget_if_idle(rid)

    def _forget_if_idle(self, rid: Hashable) -> None:
        nid = self._ids.get(rid)
        if nid is not None and rid not in self._pinned and not self._lib.ph_has(self._h, nid):
            del self._ids[rid]
            del self._names[nid]

    def _raise(self, code: int, rid: Hashable, what: str = ""):
        if code == host.UNKNOWN_REQUEST:
            raise CacheError(f"unknown request {rid!r}")
        if code == host.ALREADY_OPEN:
            raise CacheError(f"request {rid!r} is already open")
        if code == host.OUT_OF_PAGES:
            raise OutOfPages(f"request {rid!r}: {what or 'no free page'}; {self.n_free_pages()} pages are free")
        if code == host.OUT_OF_SLOTS:
            raise OutOfPages(f"no free state slot (max_requests = {self.max_requests})")
        if code == host.RELEASED_PAGE:
            raise CacheError(f"request {rid!r}: {what or 'a position'} lies in a released page")
        if code == host.NOT_HELD:
            raise CacheError(f"request {rid!r}: a page or slot is not held (freed twice or never taken)")
        raise CacheError(f"request {rid!r}: the host runtime answered {code} {what}")

    def open(self, rid: Hashable) -> int:
        """Register a request and give it a state slot.  Holds no pages yet."""
        if self.has(rid):
            raise CacheError(f"request {rid!r} is already open")
        slot = self._lib.ph_open(self._h, self.native_id(rid, create=True))
        if slot < 0:
            self._forget_if_idle(rid)
            self._raise(slot, rid)
        self._fresh_state(slot)
        return slot

    def opened_by_runtime(self, rid: Hashable) -> None:
        """The step packer opened the request: its state starts at zero."""
        self._fresh_state(self._lib.ph_state_slot(self._h, self.native_id(rid)))

    def _fresh_state(self, slot: int) -> None:
        for e, t in self.state.items():
            t[slot].zero_()

    def has(self, rid: Hashable) -> bool:
        nid = self._ids.get(rid)
        return nid is not None and self._lib.ph_has(self._h, nid) == 1

    def _open_id(self, rid: Hashable) -> int:
        nid = self._ids.get(rid)
        if nid is None or not self._lib.ph_has(self._h, nid):
            raise CacheError(f"unknown request {rid!r}")
        return nid

    def length(self, rid: Hashable) -> int:
        return self._lib.ph_length(self._h, self._open_id(rid))

    def n_logical_pages(self, rid: Hashable) -> int:
        """Logical pages the request's tables cover (the fewest over the groups)."""
        return self._lib.ph_n_logical_pages(self._h, self._open_id(rid))

    def state_slot(self, rid: Hashable) -> int:
        return self._lib.ph_state_slot(self._h, self._open_id(rid))

    def live_requests(self) -> List[Hashable]:
        return [rid for rid, nid in self._ids.items() if self._lib.ph_has(self._h, nid)]

    # ------------------------------------------------------------------ pages
    def pages_to_append(self, rid: Hashable, n_new: int) -> List[int]:
        """New pages each group must take so that the request can grow by ``n_new``
        tokens, after giving back what its windows have passed."""
        self._lib.ph_pages_to_append(self._h, self._open_id(rid), int(n_new), self._scratch)
        return list(self._scratch[:self._n_groups])

    def reclaimable(self, rid: Hashable) -> List[int]:
        self._lib.ph_reclaimable(self._h, self._open_id(rid), self._scratch)
        return list(self._scratch[:self._n_groups])

    def can_append(self, rid: Hashable, n_new: int) -> bool:
        return self._lib.ph_can_append(self._h, self._open_id(rid), int(n_new)) == 1

    def can_admit(self, n_tokens: int) -> bool:
        """Could a request that holds nothing yet take ``n_tokens`` tokens (and a slot)?"""
        return self._lib.ph_can_admit(self._h, int(n_tokens)) == 1

    def release_passed(self, rid: Hashable) -> int:
        """Give back the pages of windowed groups that every future query has passed."""
        n = self._lib.ph_release_passed(self._h, self._open_id(rid))
        if n < 0:
            self._raise(n, rid)
        return n

    def append(self, rid: Hashable, n_new: int) -> int:
        """Grow the request by ``n_new`` tokens; returns the position of the first one.
        Either every group gets its pages or nothing changes (OutOfPages)."""
        if n_new <= 0:
            raise CacheError("append needs n_new > 0")
        start = self._lib.ph_append(self._h, self._open_id(rid), int(n_new))
        if start < 0:
            self._raise(start, rid, f"{n_new} more tokens do not fit")
        return start

    def close(self, rid: Hashable) -> None:
        """Give back everything the request holds."""
        rc = self._lib.ph_close(self._h, self._open_id(rid))
        self._forget_if_idle(rid)
        if rc < 0:
            self._raise(rc, rid)

    # ------------------------------------------------------------------ views for a step
    def table(self, rid: Hashable, group: int) -> List[int]:
        nid = self._open_id(rid)
        cap = 64
        while True:
            out = (ctypes.c_int * cap)()
            n = self._lib.ph_table(self._h, nid, int(group), out, cap)
            if n <= cap:
                return list(out[:n])
            cap = n

    def slots(self, rid: Hashable, group: int, start: int, n: int) -> List[int]:
        """slot = page * page_size + offset for positions [start, start + n)
        (active_buffer.cpp:255-279)."""
        out = (ctypes.c_int * max(1, n))()
        rc = self._lib.ph_slots(self._h, self._open_id(rid), int(group), int(start), int(n), out)
        if rc < 0:
            self._raise(rc, rid, f"a position in [{start}, {start + n})")
        return list(out[:n])

    def pools(self, entry: int) -> Dict[str, torch.Tensor]:
        """The entry's pools by tensor name, each ``[pages, heads, page_size, width]``."""
        g, i = self.group_of_entry[entry], self.index_in_group[entry]
        return {name: pool[i] for name, pool in self.groups[g].pools.items()}

    def kv_pools(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        pools = self.pools(entry)
        return pools["k"], pools["v"]

    def n_free_pages(self) -> List[int]:
        return [self._lib.ph_n_free_pages(self._h, g) for g in range(self._n_groups)]

    def n_free_slots(self) -> int:
        return self._lib.ph_n_free_slots(self._h)

    def set_resident_tables(self, on: bool) -> None:
        """Whether the step packer sends whole block tables (off) or only the page ids that requests gained since
        they were last sent, for tables that stay on the device (on).  Switching forgets what was sent."""
        self._lib.ph_set_resident_tables(self._h, 1 if on else 0)
        self.resident.clear()

    def resident_table(self, group: int, width: int) -> Tuple[torch.Tensor, bool]:
        """The device's resident table of a group, ``[max_requests, stride]`` with stride >= ``width``; grown (its
        contents kept) when a request needs a wider row.  Second value: whether the tensor was (re)allocated."""
        t = self.resident.get(group)
        if t is not None and t.shape[1] >= width:
            return t, False
        stride = max(64, width)
        if t is not None:
            stride = max(stride, 2 * t.shape[1])
        new = torch.full((self.max_requests, stride), -1, dtype=torch.int32, device=self.device)
        if t is not None:
            new[:, :t.shape[1]] = t
        self.resident[group] = new
        return new, True

    def check_consistency(self) -> None:
        """Every page is free or held by exactly one request, every slot likewise; used by tests."""
        if self._lib.ph_check(self._h) != 0:
            raise CacheError("the cache's accounting is inconsistent: a page or slot is lost, held twice or freed twice")
        live = sorted(self._lib.ph_state_slot(self._h, nid) for nid in self._ids.values() if self._lib.ph_has(self._h, nid))
        held = [s for s in range(self.max_requests) if self._lib.ph_slot_held(self._h, s)]
        if live != held:
            raise CacheError("state slots out of step with the live requests")
