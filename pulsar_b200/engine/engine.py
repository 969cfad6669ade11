"""The engine: sessions, scheduler, step function and sampler in one loop.

Mirrors the surface of the reference's ``Engine`` (pulsar-core/inc/pulsar/runtime/engine.hpp:452-533;
pulsar-core/src/runtime/engine.cpp:312-451 create/feed, :731-817 step_once/step,
:472-486 release): ``create_session`` registers tokens without scheduling, ``feed`` adds
tokens and schedules, ``step(n)`` runs forwards until ``n`` tokens were emitted or
nothing is active, a finished sequence is parked with its pages kept until ``release``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch

from .. import ops, profiling
from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..sampling.sampler import GenerationParams, Sampler, make_generator
from .loading import load_model, torch_dtype
from .runner import ModelRunner, StepEntry
from .scheduler import UNREAD, Scheduled, Scheduler, SchedulerError


@dataclass
class _Session:
    params: GenerationParams
    generator: torch.Generator
    pending: List[int]            # tokens registered but not yet handed to the scheduler
    budget: int                   # new tokens allowed in the current turn
    state: str = "idle"           # "idle", "active", "parked"
    scheduled: bool = False       # known to the scheduler
    ended_on_stop: bool = False   # the last turn ended with the stop token


class EngineFailed(RuntimeError):
    """The engine met a failure it cannot step past (a kernel gave up a bounded wait, so what the device computed
    is not to be trusted) and refuses further work; ``__cause__`` is the failure.  The reference's Python layer
    poisons its engine the same way (pulsar/src/pulsar/rt/sync.py:21-34; rt/streaming.py:9-18)."""


@dataclass
class _Inflight:
    """A forward pass whose sampled ids are on their way to the host."""
    sampled: List[int]                     # sequences sampled in it, in the order of its rows
    row_of: Dict[int, int]
    host: torch.Tensor                     # pinned; filled when ``event`` has passed
    event: torch.cuda.Event
    generator_states: Dict[int, torch.Tensor]      # of stochastic sequences, before their draw
    status: Optional[torch.Tensor] = None          # pinned; the kernels' wait error words behind this pass
    void: set = field(default_factory=set)         # sequences that had ended before this pass: its token is dropped


class Engine:
    """``Engine(model_dir, config)`` loads a model folder; ``Engine.from_model`` takes a
    model that already has weights.  ``config`` is an ``EngineConfig`` or its flat dict
    (unknown keys are rejected)."""

    def __init__(self, model_dir: str, config: Union[EngineConfig, Dict[str, Any], None] = None):
        cfg = self._config(config)
        self._check_device(cfg)
        model_config, model = load_model(model_dir, cfg.dtype, cfg.device)
        self._init(model_config, model, cfg)

    @classmethod
    def from_model(cls, model_config, model, config: Union[EngineConfig, Dict[str, Any], None] = None) -> "Engine":
        self = cls.__new__(cls)
        cfg = cls._config(config)
        cls._check_device(cfg)
        if model.dtype != torch_dtype(cfg.dtype):
            raise ValueError(f"the model computes in {model.dtype}, the engine was configured for {cfg.dtype}")
        self._init(model_config, model, cfg)
        return self

    @staticmethod
    def _config(config) -> EngineConfig:
        if config is None:
            config = {}
        if isinstance(config, dict):
            return EngineConfig.from_dict(config)
        config.validate()
        return config

    @staticmethod
    def _check_device(cfg: EngineConfig) -> None:
        if not str(cfg.device).startswith("cuda") or not torch.cuda.is_available():
            raise RuntimeError(f"the engine needs a CUDA device (configured '{cfg.device}', "
                               f"cuda available: {torch.cuda.is_available()}); there is no CPU path")
        torch.cuda.set_device(cfg.device)

    def _init(self, model_config, model, cfg: EngineConfig) -> None:
        self.config, self.model_config, self.model = cfg, model_config, model
        if cfg.max_running > cfg.max_sessions:        # engine.cpp:121-140
            raise ValueError("max_running must not exceed max_sessions")
        self.cache = CacheManager(model.cache_needs(), cfg.page_size, cfg.num_pages, cfg.max_sessions, model.dtype, cfg.device)
        self.runner = ModelRunner(model, self.cache, cfg.device, cuda_graphs=cfg.cuda_graphs)
        self.scheduler = Scheduler(self.cache, cfg.max_running, cfg.max_chunk_size)
        self.sampler = Sampler(cfg.device)
        self.eos_id = cfg.eos_id
        self._sessions: Dict[int, _Session] = {}
        self._next_id = 0
        self.forwards = 0
        self._mailbox: Dict[int, list] = {}     # events of other sessions seen while one session streams
        self._inflight: Optional[_Inflight] = None          # the pass whose tokens have not been read yet
        self._unclaimed: List[Tuple[int, int, bool]] = []   # events booked outside ``step``
        self._host_ids: List[Optional[torch.Tensor]] = [None, None, None]
        self._host_status = [torch.zeros(8, dtype=torch.int32, pin_memory=True) for _ in self._host_ids]
        self._status_dev = torch.zeros(8, dtype=torch.int32, device=cfg.device)
        self._host_next = 0
        self._failed: Optional[BaseException] = None

    # ------------------------------------------------------------------ sessions
    def _params(self, overrides: Optional[Dict[str, Any]]) -> GenerationParams:
        c = self.config
        p = GenerationParams(c.temperature, c.top_p, c.top_k, c.seed)
        for k, v in (overrides or {}).items():
            if k not in ("temperature", "top_p", "top_k", "seed"):
                raise ValueError(f"unknown session override '{k}' (known: seed, temperature, top_k, top_p)")
            setattr(p, k, v)
        p.validate()
        return p

    def _alive(self) -> None:
        if self._failed is not None:
            raise EngineFailed(f"the engine failed earlier and refuses further work: {self._failed}") from self._failed

    def create_session(self, tokens: Sequence[int] = (), overrides: Optional[Dict[str, Any]] = None) -> int:
        """A new sequence with its first tokens (they are not scheduled before ``feed``)."""
        self._alive()
        if len(self._sessions) >= self.config.max_sessions:
            raise RuntimeError(f"max_sessions ({self.config.max_sessions}) reached")
        params = self._params(overrides)
        sid = self._next_id
        self._next_id += 1
        self._sessions[sid] = _Session(params, make_generator(params.seed), [int(t) for t in tokens], 0)
        return sid

    def set_decode_budget(self, seq_id: int, max_tokens: Optional[int] = None) -> None:
        """New tokens allowed in the turns that follow; None: only the stop token ends a turn
        (engine.cpp:453-456)."""
        self._session(seq_id).budget = 0 if max_tokens is None else int(max_tokens)

    def active_sequence_count(self) -> int:
        """Sequences that are running or waiting to run (engine.cpp:458-460)."""
        return len(self.scheduler.running) + len(self.scheduler.waiting)

    def active_tokens_count(self, seq_id: int) -> int:
        """Tokens of the sequence whose keys and values are in the cache (engine.cpp:492-494)."""
        self._drain()
        return self.cache.length(seq_id) if self.cache.has(seq_id) else 0

    def context_page_ids(self, seq_id: int) -> List[int]:
        """The pages that attention reads for this sequence, in the order of their tokens (of the first group
        of cache entries; pages that a window has passed are given back and not listed) (engine.cpp:533-540)."""
        self._drain()
        if not self.cache.has(seq_id) or not self.cache.groups:
            return []
        return [p for p in self.cache.table(seq_id, 0) if p >= 0]

    def context_pages(self, seq_id: int) -> List[List[int]]:
        """The token ids held by each of those pages (engine.cpp:542-549)."""
        self._drain()
        if not self.cache.has(seq_id) or not self.cache.groups:
            return []
        size, held = self.cache.page_size, self.cache.length(seq_id)
        tokens = [t for t in self.scheduler.seqs[seq_id].tokens[:held]] if seq_id in self.scheduler.seqs else []
        out = []
        for logical, page in enumerate(self.cache.table(seq_id, 0)):
            if page >= 0 and logical * size < held:
                out.append(tokens[logical * size:min(held, (logical + 1) * size)])
        return out

    def _session(self, seq_id: int) -> _Session:
        try:
            return self._sessions[seq_id]
        except KeyError:
            raise KeyError(f"unknown sequence {seq_id}") from None

    def feed(self, seq_id: int, tokens: Sequence[int], max_tokens: Optional[int] = None) -> None:
        """Add tokens to the sequence and schedule it; it will emit up to ``max_tokens``
        new tokens (default: the budget set before, else unlimited until eos)."""
        self._alive()
        s = self._session(seq_id)
        self._drain()                   # a pass in flight may still owe this sequence a token
        if s.state == "active":
            raise RuntimeError(f"sequence {seq_id} is still generating")
        if max_tokens is not None:
            s.budget = int(max_tokens)
        budget = s.budget if s.budget > 0 else (1 << 30 if self.eos_id >= 0 else 0)
        if budget <= 0:
            raise ValueError("a decode budget (max_tokens) is needed when no eos_id is configured")
        new = s.pending + [int(t) for t in tokens]
        for t in new:
            if not (0 <= t < self.model.spec.vocab_size):
                raise ValueError(f"token id {t} outside the vocabulary [0, {self.model.spec.vocab_size})")
        cap = budget if budget < (1 << 30) else 0
        if s.scheduled and not new and s.ended_on_stop:
            # Stepping one pass ahead has cached the stop token by now, stepping one pass at a time has not: a
            # turn without tokens would run nothing in the one mode and the stop token in the other.  Refused in both.
            raise ValueError(f"sequence {seq_id} ended on the stop token: a further turn needs at least one token")
        if s.scheduled:
            self.scheduler.extend_request(seq_id, new, cap if cap else self._room_left(seq_id, len(new)))
        else:
            if not new:
                raise ValueError("a sequence needs at least one token before it can generate")
            self.scheduler.add_request(seq_id, new, cap if cap else self._room_left(None, len(new)))
            s.scheduled = True
        s.pending = []
        s.state = "active"
        s.ended_on_stop = False

    def _room_left(self, seq_id, n_new: int) -> int:
        """Largest decode budget the pool allows (used when only eos stops a sequence)."""
        held = len(self.scheduler.seqs[seq_id].tokens) if seq_id is not None else 0
        pages = min(g.allocator.n for g in self.cache.groups) if self.cache.groups else 1 << 20
        return max(1, pages * self.cache.page_size - held - n_new)

    def session_state(self, seq_id: int) -> str:
        s = self._sessions.get(seq_id)
        return "unknown" if s is None else ("parked" if s.state == "parked" else "active")

    def release(self, seq_id: int) -> None:
        """Cancel the sequence and give back its pages (engine.cpp:472-486)."""
        if seq_id in self._sessions:
            self.scheduler.finish(seq_id)
            del self._sessions[seq_id]

    # ------------------------------------------------------------------ stepping
    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None or bool(self._unclaimed)

    def _launch(self, plan: List[Scheduled]) -> "_Inflight":
        """Put one forward pass and its sampling on the device and ask for the sampled ids;
        nothing here waits for the device.  Tokens that the pass before it sampled, and that the
        host has not read yet, are taken from that pass's ids on the device."""
        before = self._inflight
        entries = []
        for e in plan:
            src = None
            tokens = e.tokens
            if tokens[-1] == UNREAD:
                if before is None or e.rid not in before.row_of or len(tokens) != 1:
                    raise RuntimeError(f"sequence {e.rid}: an unread token outside a single-token entry")
                src, tokens = before.row_of[e.rid], [0]
            entries.append(StepEntry(e.rid, tokens, [len(tokens) - 1] if e.sample else [], src))
        logits = self.runner.step(entries, self.sampler.last_ids if before is not None else None)
        self.forwards += 1
        self.scheduler.on_step(plan)
        sampled = [e.rid for e in plan if e.sample]
        sessions = [self._sessions[r] for r in sampled]
        states = {r: s.generator.get_state() for r, s in zip(sampled, sessions) if not s.params.greedy}
        with profiling.scope("launch (sampling)"):
            ids = self.sampler.sample_on_device(logits, [s.params for s in sessions], [s.generator for s in sessions])
        slot = self._host_ids[self._host_next]
        if slot is None or slot.numel() < len(sampled):
            slot = self._host_ids[self._host_next] = torch.empty(max(64, len(sampled)), dtype=torch.int32, pin_memory=True)
        status = self._host_status[self._host_next]
        self._host_next = (self._host_next + 1) % len(self._host_ids)
        host = slot[:len(sampled)]
        if sampled:
            host.copy_(ids, non_blocking=True)
        # the error words of the kernels with bounded waits travel with the ids: no synchronisation of their own
        ops.gather_wait_words(self._status_dev)
        status.copy_(self._status_dev, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        for r in sampled:
            self.scheduler.on_sampled(r)
        return _Inflight(sampled, {r: i for i, r in enumerate(sampled)}, host, event, states, status)

    def _collect(self, flight: "_Inflight") -> List[Tuple[int, int, bool]]:
        """Wait for a pass's sampled ids and book them: events ``(seq_id, token, finished)``."""
        with profiling.scope("read (wait for the sampled ids)"):
            flight.event.synchronize()
        if flight.status is not None:
            what = ops.describe_wait_words(flight.status[:ops.N_WAIT_WORDS].tolist())
            if what is not None:
                # the pass's tokens come from a kernel that gave up: none of them is booked, and nothing runs after it
                self._failed = ops.DeviceWaitError(what)
                self._inflight = None
                raise EngineFailed(f"a forward pass did not complete: {what}") from self._failed
        events = []
        for rid, tok in zip(flight.sampled, flight.host.tolist()):
            if rid not in self.scheduler.seqs:
                continue                            # released while the pass was in flight
            if rid in flight.void:
                # the sequence had ended with the token before: this pass only cached that token
                self.scheduler.drop_unread(rid)
                if rid in flight.generator_states and rid in self._sessions:
                    self._sessions[rid].generator.set_state(flight.generator_states[rid])
                continue
            finished = self.scheduler.on_token(rid, tok, self.eos_id)
            if finished:
                self.scheduler.park(rid)            # pages stay until release (engine.cpp:770-788)
                self._sessions[rid].state = "parked"
                self._sessions[rid].ended_on_stop = self.eos_id >= 0 and int(tok) == self.eos_id
                nxt = self._inflight
                if nxt is not None and nxt is not flight and rid in nxt.row_of:
                    nxt.void.add(rid)
            events.append((rid, int(tok), finished))
        return events

    def _drain(self) -> None:
        """Book the pass in flight, if any; its events wait for the next ``step``."""
        if self._inflight is not None:
            flight, self._inflight = self._inflight, None
            self._unclaimed.extend(self._collect(flight))

    def step_once(self) -> List[Tuple[int, int, bool]]:
        """One forward pass.  Returns the events ``(seq_id, token, finished)`` of the
        sequences whose logits were sampled in it."""
        self._alive()
        self._drain()
        if self._unclaimed:
            events, self._unclaimed = self._unclaimed, []
            return events
        with profiling.scope("plan (the scheduler's decision)"):
            plan = self.scheduler.schedule()
        if not plan:
            return []
        return self._collect(self._launch(plan))

    def step(self, n: int = 1, lookahead: bool = True) -> List[Tuple[int, int, bool]]:
        """Run forwards until ``n`` tokens were emitted or nothing is active; may overshoot
        by the number of active sequences minus one (engine.hpp:490-498).  A scheduler
        that has work but can run nothing is an error (engine.cpp:809-814).

        With ``lookahead`` the next pass is put on the device before the tokens of the last
        one are read (its inputs are those tokens, taken on the device), so the device does
        not idle while the host books tokens and decides the next step; one pass may then
        still be in flight when the call returns, and the next call picks it up.  A sequence
        that ends on a stop token has by then run one token too far; that token is discarded."""
        self._alive()
        events: List[Tuple[int, int, bool]] = self._unclaimed
        self._unclaimed = []
        while len(events) < n:
            if self._inflight is None:
                with profiling.scope("plan (the scheduler's decision)"):
                    plan = self.scheduler.schedule()
                if not plan:
                    if self.scheduler.has_work():
                        raise RuntimeError("the scheduler has work but nothing can run: the pool is held by parked "
                                           "sequences or is too small; release a sequence")
                    break
                self._inflight = self._launch(plan)
            flight = self._inflight
            nxt = None
            if lookahead:
                with profiling.scope("plan (the scheduler's decision)"):
                    plan = self.scheduler.schedule(allow_preempt=False)
                if plan:
                    nxt = self._launch(plan)
            self._inflight = nxt
            events.extend(self._collect(flight))
        if not lookahead:
            self._drain()
            events.extend(self._unclaimed)
            self._unclaimed = []
        return events

    # ------------------------------------------------------------------ the simple entry point
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: Optional[int] = None
                 ) -> List[List[int]]:
        """Generate for each prompt (token ids in, token ids out).  Requests beyond
        ``max_sessions`` wait their turn; every sequence is released at its end."""
        overrides = {k: v for k, v in dict(temperature=temperature, top_k=top_k, top_p=top_p).items() if v is not None}
        results: List[List[int]] = [[] for _ in prompts]
        todo = list(range(len(prompts)))
        owner: Dict[int, int] = {}
        while todo or owner:
            while todo and len(self._sessions) < self.config.max_sessions:
                i = todo.pop(0)
                ov = dict(overrides)
                if seed is not None:
                    ov["seed"] = seed + i if seed >= 0 else seed
                sid = self.create_session(prompts[i], ov)
                self.feed(sid, [], max_new_tokens)
                owner[sid] = i
            for sid, tok, finished in self.step(1):          # one forward at a time: a finished
                if sid in owner:                              # sequence gives its pages back at once
                    results[owner[sid]].append(tok)
                    if finished:
                        self.release(sid)
                        del owner[sid]
        return results
