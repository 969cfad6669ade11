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
  * a request that could never fit the pool alone is refused when it is submitted.

A step may be decided while the tokens of the step before are still on the device: a
sampled token that the host has not read yet stands in the request's token list as
``UNREAD`` (``on_sampled``), is filled in by ``on_token`` when it arrives, and is taken
back by ``drop_unread`` if the request turned out to have ended one token earlier.

The scheduler is host code over the cache manager's accounting and runs without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional

from ..cache.manager import CacheManager


UNREAD = -1        # stands in a token list for a sampled token that has not been read from the device yet


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
    def __init__(self, cache: CacheManager, max_running: int, max_chunk_size: int):
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
