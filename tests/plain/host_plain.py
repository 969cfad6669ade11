"""Plain host runtime: the cache accounting and the scheduler in straightforward Python, one
statement per rule.  The oracle of the tests that drive the C++ host runtime (csrc/host) with
random sequences of requests: same calls on both, same answers expected.  Shares no code with the
product package.

Rules and where the reference has them: LIFO free list and block tables
(pulsar-core/src/runtime/kv/active_buffer.cpp:71-75, 152-228), slot mapping (:255-279); scheduling
order decode, prompts in progress, first-in first-out admission
(pulsar-core/src/runtime/scheduler.cpp:76-222); stop rule (pulsar-core/src/runtime/engine.cpp:727-729).
What differs from the reference by decision (whole-step budget, whole-prompt admission with pages
held back, preemption of the youngest, refusal at submit, windows that give pages back, tokens that
are still unread) is described in the product's scheduler and cache sources.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

UNREAD = -1


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
    state_dtype: object = None

    @staticmethod
    def paged_kv(n_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        return CacheNeed("paged_kv", n_kv_heads, head_dim, window)

    @staticmethod
    def state(shape: Sequence[int], dtype=None) -> "CacheNeed":
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


@dataclass
class _Request:
    length: int = 0
    state_slot: int = -1
    tables: List[List[int]] = field(default_factory=list)     # per group: logical page -> page id or -1
    released: List[int] = field(default_factory=list)         # per group: logical pages [0, released) given back


class CacheManager:
    def __init__(self, needs: Sequence[CacheNeed], page_size: int, num_pages, max_requests: int):
        """``needs[i]`` is the need of cache entry i.  ``num_pages`` is an int (every
        group gets that many) or a list per group in order of first appearance.
        ``device=None`` keeps the accounting only (no tensors)."""
        if page_size <= 0:
            raise CacheError("page_size must be > 0")
        self.page_size = int(page_size)
        self.needs = list(needs)
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
        self._windowed = any(grp.need.window is not None for grp in self.groups)
        self.max_requests = int(max_requests)
        self._slots = PageAllocator(self.max_requests)
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


class SchedulerError(RuntimeError):
    pass


@dataclass
class SequenceState:
    """Scheduling state of one request: all its tokens so far and how many are cached."""
    rid: Hashable
    tokens: List[int]
    max_new_tokens: int
    n_cached: int = 0
    n_generated: int = 0
    admitted_at: int = -1           # admission counter value; larger = admitted later
    preemptions: int = 0
    unread: int = 0                 # trailing tokens that are still UNREAD
    spent: bool = False             # the turn's budget is used up: nothing more is scheduled for it

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.n_cached


@dataclass
class Scheduled:
    """One entry of a step: feed ``tokens`` of request ``rid``; ``sample`` tells whether the
    logits of the last token are wanted (the portion completes what the request knows)."""
    rid: Hashable
    tokens: List[int]
    sample: bool


class Scheduler:
    def __init__(self, cache, max_running: int, max_chunk_size: int):
        if max_running <= 0 or max_chunk_size <= 0:
            raise SchedulerError("max_running and max_chunk_size must be > 0")
        self.cache = cache
        self.max_running = min(int(max_running), cache.max_requests)
        self.max_chunk_size = int(max_chunk_size)
        self.waiting: Deque[Hashable] = deque()
        self.running: List[Hashable] = []
        self.seqs: Dict[Hashable, SequenceState] = {}
        self._admissions = 0
        self.n_preemptions = 0

    # ------------------------------------------------------------------ bookkeeping
    def _pages(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _capacity_pages(self) -> int:
        return min(g.allocator.n for g in self.cache.groups) if self.cache.groups else 1 << 30

    def _free_pages(self) -> int:
        return min(self.cache.n_free_pages()) if self.cache.groups else 1 << 30

    def _held_back(self) -> int:
        """Pages that running prompts still need to reach their last known token plus one."""
        total = 0
        for rid in self.running:
            s = self.seqs[rid]
            have = self._pages(s.n_cached)
            total += max(0, self._pages(len(s.tokens) + 1) - have)
        return total

    def add_request(self, rid: Hashable, tokens: List[int], max_new_tokens: int) -> None:
        if rid in self.seqs:
            raise SchedulerError(f"request {rid!r} is already known")
        if len(tokens) == 0:
            raise SchedulerError("a request needs at least one prompt token")
        if self._pages(len(tokens) + max(0, max_new_tokens)) > self._capacity_pages():
            raise SchedulerError(f"request {rid!r}: {len(tokens)} prompt tokens + {max_new_tokens} new tokens can never "
                                 f"fit the pool of {self._capacity_pages()} pages of {self.cache.page_size}")
        self.seqs[rid] = SequenceState(rid, list(tokens), int(max_new_tokens))
        self.waiting.append(rid)

    def extend_request(self, rid: Hashable, tokens: List[int], max_new_tokens: int) -> None:
        """More tokens for a known request that is not running (a further turn): it keeps
        its pages and waits for admission again."""
        s = self.seqs.get(rid)
        if s is None:
            raise SchedulerError(f"unknown request {rid!r}")
        if rid in self.running:
            raise SchedulerError(f"request {rid!r} is running; feed it when its turn is over")
        if self._pages(len(s.tokens) + len(tokens) + max(0, max_new_tokens)) > self._capacity_pages():
            raise SchedulerError(f"request {rid!r} would outgrow the pool")
        if s.unread:
            raise SchedulerError(f"request {rid!r} still has a sampled token that was not read")
        s.tokens.extend(tokens)
        s.max_new_tokens = int(max_new_tokens)
        s.n_generated = 0
        s.spent = False
        if rid not in self.waiting:
            self.waiting.append(rid)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step
    def _preempt(self, rid: Hashable) -> None:
        s = self.seqs[rid]
        if self.cache.has(rid):
            self.cache.close(rid)
        s.n_cached = 0
        s.preemptions += 1
        self.n_preemptions += 1
        self.running.remove(rid)
        self.waiting.appendleft(rid)

    def schedule(self, allow_preempt: bool = True) -> Optional[List[Scheduled]]:
        """When nothing at all can run although there is work, the holder of pages furthest back in the queue
        gives them up; if no waiting request holds any, the running request admitted last is preempted; then
        the step is decided again."""
        while True:
            out = self._plan_once(allow_preempt)
            if out is None or out or not allow_preempt or not self.has_work():
                return out
            holders = [r for r in reversed(self.waiting) if self.cache.has(r)]
            if holders:
                if len(self.waiting) == 1 and not self.running:
                    return out
                victim = holders[0]
                self.cache.close(victim)
                self.seqs[victim].n_cached = 0
                self.seqs[victim].preemptions += 1
                self.n_preemptions += 1
                continue
            if len(self.running) + len(self.waiting) < 2 or not self.running:
                return out
            youngest = max(self.running, key=lambda r: self.seqs[r].admitted_at)
            if not self.cache.has(youngest):
                return out
            self._preempt(youngest)

    def _plan_once(self, allow_preempt: bool = True) -> Optional[List[Scheduled]]:
        """Decide the next step.  Changes nothing in the cache except by preemption; the
        step function takes the pages when it runs the entries.  With ``allow_preempt``
        false (a step is still in flight, so some tokens are UNREAD and nothing may be
        recomputed from them) the answer is None where a request would have to be preempted."""
        budget = self.max_chunk_size
        out: List[Scheduled] = []
        planned: set = set()         # requests that already have an entry in this step
        planned_pages = 0            # pages this step's entries will take
        ps = self.cache.page_size

        def pages_for(rid, n_new) -> int:
            if self.cache.has(rid) and self.cache.groups:
                # pages to reach the new length, beyond the logical pages the request already has
                return max(0, -(-(self.cache.length(rid) + n_new) // ps) - self.cache.n_logical_pages(rid))
            return self._pages(n_new)

        def room_for(rid, n_new) -> bool:
            return pages_for(rid, n_new) <= self._free_pages() - planned_pages

        def take(rid, n_new) -> None:
            nonlocal planned_pages
            planned_pages += pages_for(rid, n_new)

        def fits(rid) -> int:
            """Most new tokens of ``rid`` that the free pages allow in this step."""
            avail = max(0, self._free_pages() - planned_pages)
            in_last = (-self.cache.length(rid)) % self.cache.page_size if self.cache.has(rid) else 0
            return avail * self.cache.page_size + in_last

        # 1. decode tokens, oldest admission first; preempt the youngest when pages run out.
        decoders = [r for r in self.running
                    if self.seqs[r].pending == 1 and self.seqs[r].n_cached > 0 and not self.seqs[r].spent]
        for rid in sorted(decoders, key=lambda r: self.seqs[r].admitted_at):
            if rid not in self.running:
                continue                      # preempted below
            if budget <= 0:
                break
            while not room_for(rid, 1):
                if not allow_preempt:
                    return None
                victim = max(self.running, key=lambda r: self.seqs[r].admitted_at)
                was_planned = [e for e in out if e.rid == victim]
                for e in was_planned:          # its planned entry (and pages) leave the step
                    out.remove(e)
                    planned.discard(victim)
                    budget += len(e.tokens)
                    planned_pages -= pages_for(victim, len(e.tokens))
                self._preempt(victim)
                if victim == rid:
                    break
            if rid not in self.running:
                continue
            s = self.seqs[rid]
            out.append(Scheduled(rid, [s.tokens[-1]], True))
            planned.add(rid)
            take(rid, 1)
            budget -= 1

        # 2. prompts in progress, in running order.
        for rid in list(self.running):
            s = self.seqs[rid]
            if budget <= 0:
                break
            if rid in planned or s.pending == 0 or s.spent:
                continue
            if s.pending == 1 and s.n_cached > 0:
                continue                      # a decoder that found no budget above
            n = min(s.pending, budget, fits(rid))     # pages are held back for it, so it rarely shrinks
            if n <= 0:
                continue
            out.append(Scheduled(rid, s.tokens[s.n_cached:s.n_cached + n], n == s.pending))
            planned.add(rid)
            take(rid, n)
            budget -= n

        # 3. admission, first-in first-out.
        while self.waiting and len(self.running) < self.max_running and budget > 0:
            rid = self.waiting[0]
            s = self.seqs[rid]
            have = self._pages(s.n_cached) if self.cache.has(rid) else 0
            need_all = self._pages(len(s.tokens) + 1) - have
            # what running requests still need (this step's pages included) stays theirs
            if need_all > self._free_pages() - self._held_back():
                break                          # head of the queue waits; nobody overtakes it
            if not self.cache.has(rid) and self.cache.n_free_slots() - sum(1 for e in out if not self.cache.has(e.rid)) <= 0:
                break
            planned.add(rid)
            self.waiting.popleft()
            self.running.append(rid)
            s.admitted_at = self._admissions
            self._admissions += 1
            n = min(s.pending, budget)
            out.append(Scheduled(rid, s.tokens[s.n_cached:s.n_cached + n], n == s.pending))
            take(rid, n)
            budget -= n
        return out

    def on_step(self, entries: List[Scheduled]) -> None:
        """The entries ran: their tokens are cached now."""
        for e in entries:
            self.seqs[e.rid].n_cached += len(e.tokens)

    def on_sampled(self, rid: Hashable) -> None:
        """A token was sampled for ``rid`` on the device and is not read yet."""
        s = self.seqs[rid]
        s.tokens.append(UNREAD)
        s.unread += 1
        s.n_generated += 1
        if s.n_generated >= s.max_new_tokens:
            s.spent = True

    def on_token(self, rid: Hashable, token: int, eos_id: int) -> bool:
        """The oldest unread token of ``rid`` has arrived (or, if none was announced by
        ``on_sampled``, a token was sampled and read at once).  Returns True when the
        request's turn is over (stop token or budget,
        pulsar-core/src/runtime/engine.cpp:727-729)."""
        s = self.seqs[rid]
        if s.unread == 0:
            self.on_sampled(rid)
        s.tokens[len(s.tokens) - s.unread] = int(token)
        s.unread -= 1
        spent_by_now = s.n_generated - s.unread >= s.max_new_tokens
        return (eos_id >= 0 and int(token) == eos_id) or spent_by_now

    def drop_unread(self, rid: Hashable) -> None:
        """The newest unread token of ``rid`` is void: the request had ended with the token
        before it.  (The step that sampled it has cached that last token, which is all it leaves.)"""
        s = self.seqs[rid]
        if s.unread <= 0 or s.tokens[-1] != UNREAD:
            raise SchedulerError(f"request {rid!r} has no unread token to drop")
        s.tokens.pop()
        s.unread -= 1
        s.n_generated -= 1

    def park(self, rid: Hashable) -> None:
        """The turn is over; the request leaves the running set and keeps its pages."""
        if rid in self.running:
            self.running.remove(rid)

    def finish(self, rid: Hashable) -> None:
        """Forget the request and give back what it holds."""
        if rid in self.running:
            self.running.remove(rid)
        if rid in self.waiting:
            self.waiting.remove(rid)
        if self.cache.has(rid):
            self.cache.close(rid)
        self.seqs.pop(rid, None)
