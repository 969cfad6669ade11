"""The engine: sessions, scheduler, step function and sampler in one loop.

Mirrors the surface of the reference's ``Engine`` (pulsar-core/inc/pulsar/runtime/engine.hpp:452-533;
pulsar-core/src/runtime/engine.cpp:312-451 create/feed, :731-817 step_once/step,
:472-486 release): ``create_session`` registers tokens without scheduling, ``feed`` adds
tokens and schedules, ``step(n)`` runs forwards until ``n`` tokens were emitted or
nothing is active, a finished sequence is parked with its pages kept until ``release``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..cache.manager import CacheManager
from ..config.engine_config import EngineConfig
from ..sampling.sampler import GenerationParams, Sampler, make_generator
from .loading import load_model, torch_dtype
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler, SchedulerError


@dataclass
class _Session:
    params: GenerationParams
    generator: torch.Generator
    pending: List[int]            # tokens registered but not yet handed to the scheduler
    budget: int                   # new tokens allowed in the current turn
    state: str = "idle"           # "idle", "active", "parked"
    scheduled: bool = False       # known to the scheduler


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

    def create_session(self, tokens: Sequence[int] = (), overrides: Optional[Dict[str, Any]] = None) -> int:
        """A new sequence with its first tokens (they are not scheduled before ``feed``)."""
        if len(self._sessions) >= self.config.max_sessions:
            raise RuntimeError(f"max_sessions ({self.config.max_sessions}) reached")
        params = self._params(overrides)
        sid = self._next_id
        self._next_id += 1
        self._sessions[sid] = _Session(params, make_generator(params.seed), [int(t) for t in tokens], 0)
        return sid

    def set_decode_budget(self, seq_id: int, max_tokens: int) -> None:
        self._session(seq_id).budget = int(max_tokens)

    def _session(self, seq_id: int) -> _Session:
        try:
            return self._sessions[seq_id]
        except KeyError:
            raise KeyError(f"unknown sequence {seq_id}") from None

    def feed(self, seq_id: int, tokens: Sequence[int], max_tokens: Optional[int] = None) -> None:
        """Add tokens to the sequence and schedule it; it will emit up to ``max_tokens``
        new tokens (default: the budget set before, else unlimited until eos)."""
        s = self._session(seq_id)
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
        if s.scheduled:
            self.scheduler.extend_request(seq_id, new, cap if cap else self._room_left(seq_id, len(new)))
        else:
            if not new:
                raise ValueError("a sequence needs at least one token before it can generate")
            self.scheduler.add_request(seq_id, new, cap if cap else self._room_left(None, len(new)))
            s.scheduled = True
        s.pending = []
        s.state = "active"

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
        return self.scheduler.has_work()

    def step_once(self) -> List[Tuple[int, int, bool]]:
        """One forward pass.  Returns the events ``(seq_id, token, finished)`` of the
        sequences whose logits were sampled in it."""
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = [StepEntry(e.rid, e.tokens, [len(e.tokens) - 1] if e.sample else []) for e in plan]
        logits = self.runner.step(entries)
        self.forwards += 1
        self.scheduler.on_step(plan)
        sampled = [e.rid for e in plan if e.sample]
        tokens = self.sampler.sample(logits, [self._sessions[r].params for r in sampled],
                                     [self._sessions[r].generator for r in sampled])
        events = []
        for rid, tok in zip(sampled, tokens):
            finished = self.scheduler.on_token(rid, tok, self.eos_id)
            if finished:
                self.scheduler.park(rid)            # pages stay until release (engine.cpp:770-788)
                self._sessions[rid].state = "parked"
            events.append((rid, int(tok), finished))
        return events

    def step(self, n: int = 1) -> List[Tuple[int, int, bool]]:
        """Run forwards until ``n`` tokens were emitted or nothing is active; may overshoot
        by the number of active sequences minus one (engine.hpp:490-498).  A scheduler
        that has work but can run nothing is an error (engine.cpp:809-814)."""
        events: List[Tuple[int, int, bool]] = []
        while len(events) < n and self.scheduler.has_work():
            before = self.forwards
            events.extend(self.step_once())
            if self.forwards == before:
                raise RuntimeError("the scheduler has work but nothing can run: the pool is held by parked "
                                   "sequences or is too small; release a sequence")
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
            before = self.forwards
            for sid, tok, finished in self.step_once():      # one forward at a time: a finished
                if sid in owner:                              # sequence gives its pages back at once
                    results[owner[sid]].append(tok)
                    if finished:
                        self.release(sid)
                        del owner[sid]
            if self.forwards == before and self.scheduler.has_work():
                raise RuntimeError("the scheduler has work but nothing can run: the pool is too small for it")
        return results
