"""Continuous batching above the step function: admission, prompt portions under a token
budget, decoding, finishing, and what happens when pages run out.

Order of one step, as in the reference (pulsar-core/src/runtime/scheduler.cpp:76-222):
first every running request that is past its prompt gets one decode token, then prompts
in progress continue in running order, then waiting requests are admitted first-in
first-out, the head of the queue blocking those behind it.

Decisions that differ from the reference:
  * the budget ``max_chunk_size`` counts every token of the step, decoded ones included
    (the reference counts prompt tokens only, scheduler.cpp:100);
  * admission looks at the whole prompt plus one token, not at the first portion
    (scheduler.cpp:154-170), and the pages a running prompt still needs are held back
    from later admissions, so two half-fed prompts can never starve each other;
  * when a decoding request cannot get its next page the request admitted last is
    preempted: its pages go back, it returns to the head of the queue and is recomputed
    from its tokens later.  The reference throws "out of pages" here
    (pulsar-core/src/runtime/kv/active_buffer.cpp:153-160);
  * when nothing at all can run because pages are held by requests that wait for a further turn on
    kept pages, the holder furthest back in the queue gives its pages up and is recomputed (if no
    waiting request holds any, the running request admitted last is preempted);
  * a request that could never fit the pool alone is refused when it is submitted.

A step may be decided while the tokens of the step before are still on the device: a
sampled token that the host has not read yet stands in the request's token list as
``UNREAD`` (``on_sampled``), is filled in by ``on_token`` when it arrives, and is taken
back by ``drop_unread`` if the request turned out to have ended one token earlier.

The decisions are taken by the host runtime (C++, csrc/host/scheduler.cpp) over the cache's accounting;
this class names the requests, moves token lists across and turns status codes into exceptions.  It runs
without a GPU.
"""
from __future__ import annotations

import ctypes
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Hashable, Iterator, List, Optional

from .. import host
from ..cache.manager import CacheManager

UNREAD = -1        # stands in a token list for a sampled token that has not been read from the device yet

_NEVER_FITS, _STILL_RUNNING, _HAS_UNREAD, _NO_UNREAD, _NEEDS_PREEMPTION = -20, -21, -22, -23, -24

_SIGNATURES = {
    "ph_sched_new": (ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]),
    "ph_sched_delete": (None, [ctypes.c_void_p]),
    "ph_sched_add": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, host._IP, ctypes.c_int, ctypes.c_int]),
    "ph_sched_extend": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, host._IP, ctypes.c_int, ctypes.c_int]),
    "ph_sched_has_work": (ctypes.c_int, [ctypes.c_void_p]),
    "ph_sched_schedule": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "ph_sched_plan": (ctypes.c_int, [ctypes.c_void_p, host._LP, host._IP, host._IP, host._IP]),
    "ph_sched_plan_tokens": (ctypes.c_int, [ctypes.c_void_p, host._IP]),
    "ph_sched_on_step": (None, [ctypes.c_void_p]),
    "ph_sched_on_sampled": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64]),
    "ph_sched_on_token": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int]),
    "ph_sched_drop_unread": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64]),
    "ph_sched_park": (None, [ctypes.c_void_p, ctypes.c_int64]),
    "ph_sched_finish": (None, [ctypes.c_void_p, ctypes.c_int64]),
    "ph_sched_knows": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64]),
    "ph_sched_info": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, host._LP]),
    "ph_sched_tokens": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, host._IP, ctypes.c_int]),
    "ph_sched_n_preemptions": (ctypes.c_int, [ctypes.c_void_p]),
    "ph_sched_max_running": (ctypes.c_int, [ctypes.c_void_p]),
    "ph_sched_list": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, host._LP, ctypes.c_int]),
}


class SchedulerError(RuntimeError):
    pass


@dataclass
class SequenceState:
    """A snapshot of one request's scheduling state: all its tokens so far and how many are cached."""
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


class _Sequences(Mapping):
    """``scheduler.seqs``: the requests the scheduler knows, by name; a lookup takes a snapshot."""

    def __init__(self, owner: "Scheduler"):
        self._o = owner

    def __contains__(self, rid) -> bool:
        return rid in self._o._known

    def __iter__(self) -> Iterator[Hashable]:
        return iter(list(self._o._known))

    def __len__(self) -> int:
        return len(self._o._known)

    def __getitem__(self, rid) -> SequenceState:
        o = self._o
        if rid not in o._known:
            raise KeyError(rid)
        nid = o.cache.native_id(rid)
        info = (ctypes.c_int64 * 8)()
        o._lib.ph_sched_info(o._h, nid, info)
        n = int(info[0])
        buf = (ctypes.c_int * max(1, n))()
        o._lib.ph_sched_tokens(o._h, nid, buf, n)
        return SequenceState(rid, list(buf[:n]), int(info[1]), int(info[2]), int(info[3]), int(info[4]), int(info[5]),
                             int(info[6]), bool(info[7]))


class Scheduler:
    def __init__(self, cache: CacheManager, max_running: int, max_chunk_size: int):
        if max_running <= 0 or max_chunk_size <= 0:
            raise SchedulerError("max_running and max_chunk_size must be > 0")
        self.cache = cache
        self._lib = host.lib()
        for name, (res, args) in _SIGNATURES.items():
            f = getattr(self._lib, name)
            f.restype, f.argtypes = res, args
        self._h = self._lib.ph_sched_new(cache._h, int(max_running), int(max_chunk_size))
        if not self._h:
            raise SchedulerError("the host runtime refused the scheduler's sizes")
        self.max_running = self._lib.ph_sched_max_running(self._h)
        self.max_chunk_size = int(max_chunk_size)
        self._known: set = set()
        self.seqs = _Sequences(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ph_sched_delete(h)

    # ------------------------------------------------------------------ bookkeeping
    def _pages(self, n_tokens: int) -> int:
        return -(-n_tokens // self.cache.page_size)

    def _capacity_pages(self) -> int:
        return min(g.allocator.n for g in self.cache.groups) if self.cache.groups else 1 << 30

    def _names(self, which: int) -> List[Hashable]:
        cap = 64
        while True:
            out = (ctypes.c_int64 * cap)()
            n = self._lib.ph_sched_list(self._h, which, out, cap)
            if n <= cap:
                return [self.cache.name_of(int(v)) for v in out[:n]]
            cap = n

    @property
    def waiting(self) -> List[Hashable]:
        return self._names(0)

    @property
    def running(self) -> List[Hashable]:
        return self._names(1)

    @property
    def n_preemptions(self) -> int:
        return self._lib.ph_sched_n_preemptions(self._h)

    def add_request(self, rid: Hashable, tokens: List[int], max_new_tokens: int) -> None:
        if rid in self._known:
            raise SchedulerError(f"request {rid!r} is already known")
        if len(tokens) == 0:
            raise SchedulerError("a request needs at least one prompt token")
        nid = self.cache.pin(rid)
        rc = self._lib.ph_sched_add(self._h, nid, host.ints([int(t) for t in tokens]), len(tokens), int(max_new_tokens))
        if rc < 0:
            self.cache.unpin(rid)
            if rc == _NEVER_FITS:
                raise SchedulerError(f"request {rid!r}: {len(tokens)} prompt tokens + {max_new_tokens} new tokens can never "
                                     f"fit the pool of {self._capacity_pages()} pages of {self.cache.page_size}")
            raise SchedulerError(f"request {rid!r}: the host runtime answered {rc}")
        self._known.add(rid)

    def extend_request(self, rid: Hashable, tokens: List[int], max_new_tokens: int) -> None:
        """More tokens for a known request that is not running (a further turn): it keeps
        its pages and waits for admission again."""
        if rid not in self._known:
            raise SchedulerError(f"unknown request {rid!r}")
        rc = self._lib.ph_sched_extend(self._h, self.cache.native_id(rid), host.ints([int(t) for t in tokens] or [0]),
                                       len(tokens), int(max_new_tokens))
        if rc == _STILL_RUNNING:
            raise SchedulerError(f"request {rid!r} is running; feed it when its turn is over")
        if rc == _NEVER_FITS:
            raise SchedulerError(f"request {rid!r} would outgrow the pool")
        if rc == _HAS_UNREAD:
            raise SchedulerError(f"request {rid!r} still has a sampled token that was not read")
        if rc == host.BAD_ARGUMENT:
            raise SchedulerError(f"request {rid!r}: a further turn needs at least one token to run")
        if rc < 0:
            raise SchedulerError(f"request {rid!r}: the host runtime answered {rc}")

    def has_work(self) -> bool:
        return self._lib.ph_sched_has_work(self._h) == 1

    # ------------------------------------------------------------------ one step
    def schedule(self, allow_preempt: bool = True) -> Optional[List[Scheduled]]:
        """Decide the next step.  Changes nothing in the cache except by preemption; the
        step function takes the pages when it runs the entries.  With ``allow_preempt``
        false (a step is still in flight, so some tokens are UNREAD and nothing may be
        recomputed from them) the answer is None where a request would have to be preempted."""
        n = self._lib.ph_sched_schedule(self._h, 1 if allow_preempt else 0)
        if n == _NEEDS_PREEMPTION:
            return None
        if n < 0:
            raise SchedulerError(f"the host runtime answered {n}")
        if n == 0:
            return []
        rids, first = (ctypes.c_int64 * n)(), (ctypes.c_int * n)()
        count, sample = (ctypes.c_int * n)(), (ctypes.c_int * n)()
        total = self._lib.ph_sched_plan(self._h, rids, first, count, sample)
        tokens = (ctypes.c_int * max(1, total))()
        self._lib.ph_sched_plan_tokens(self._h, tokens)
        out, at = [], 0
        for i in range(n):
            c = count[i]
            out.append(Scheduled(self.cache.name_of(int(rids[i])), list(tokens[at:at + c]), bool(sample[i])))
            at += c
        self._last = out
        return out

    def on_step(self, entries: List[Scheduled]) -> None:
        """The entries of the step decided last ran: their tokens are cached now."""
        last = getattr(self, "_last", None)
        if entries is not last and [(e.rid, len(e.tokens)) for e in entries] != [(e.rid, len(e.tokens)) for e in last or []]:
            raise SchedulerError("on_step takes the step that schedule() decided last")
        self._lib.ph_sched_on_step(self._h)

    def on_sampled(self, rid: Hashable) -> None:
        """A token was sampled for ``rid`` on the device and is not read yet."""
        self._lib.ph_sched_on_sampled(self._h, self.cache.native_id(rid))

    def on_token(self, rid: Hashable, token: int, eos_id: int) -> bool:
        """The oldest unread token of ``rid`` has arrived (or, if none was announced by
        ``on_sampled``, a token was sampled and read at once).  Returns True when the
        request's turn is over (stop token or budget,
        pulsar-core/src/runtime/engine.cpp:727-729)."""
        rc = self._lib.ph_sched_on_token(self._h, self.cache.native_id(rid), int(token), int(eos_id))
        if rc < 0:
            raise SchedulerError(f"unknown request {rid!r}")
        return rc == 1

    def drop_unread(self, rid: Hashable) -> None:
        """The newest unread token of ``rid`` is void: the request had ended with the token
        before it.  (The step that sampled it has cached that last token, which is all it leaves.)"""
        rc = self._lib.ph_sched_drop_unread(self._h, self.cache.native_id(rid))
        if rc < 0:
            raise SchedulerError(f"request {rid!r} has no unread token to drop")

    def park(self, rid: Hashable) -> None:
        """The turn is over; the request leaves the running set and keeps its pages."""
        if rid in self._known:
            self._lib.ph_sched_park(self._h, self.cache.native_id(rid))

    def finish(self, rid: Hashable) -> None:
        """Forget the request and give back what it holds."""
        if rid in self._known:
            self._lib.ph_sched_finish(self._h, self.cache.native_id(rid))
            self._known.discard(rid)
            self.cache.unpin(rid)
        elif self.cache.has(rid):
            self.cache.close(rid)
