"""Python entry point in the reference's manner.

The reference's package gives ``Pulsar(weights, config, tokenizer, dtype=...)``,
``create_session(sink)`` and a ``Session`` with ``send`` / ``recv`` / ``destroy`` over an
asyncio worker (pulsar/src/pulsar/rt/pulsar.py:12-43; pulsar/src/pulsar/rt/session.py:11-63;
pulsar/src/pulsar/rt/streaming.py:38-99).  This engine keeps those names on a synchronous
surface (token ids in, token ids out; tokenizers and chat framing are out of scope) and
adds ``generate`` for the common case.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Sequence

import torch

from .engine.engine import Engine


class Session:
    """One sequence of the engine.  ``send`` adds tokens, ``recv`` streams the new ones."""

    def __init__(self, seq_id: int, engine: Engine):
        self._seq_id, self._engine = seq_id, engine

    @property
    def seq_id(self) -> int:
        return self._seq_id

    def send(self, tokens: Sequence[int], max_tokens: Optional[int] = None) -> None:
        self._engine.feed(self._seq_id, tokens, max_tokens)

    def recv(self) -> Iterator[int]:
        """Token ids of this turn, as they are decoded (other sessions advance too)."""
        done = False
        while not done:
            events = self._engine.step(1)
            if not events and not self._engine.has_work():
                return
            for sid, tok, finished in events:
                if sid == self._seq_id:
                    yield tok
                    done = done or finished
                else:
                    self._engine._mailbox.setdefault(sid, []).append((tok, finished))
            for tok, finished in self._engine._mailbox.pop(self._seq_id, []):
                yield tok
                done = done or finished

    def get_state(self) -> str:
        return self._engine.session_state(self._seq_id)

    def get_context(self):
        """``(page ids, token ids of each page)`` of what attention reads for this sequence
        (pulsar/src/pulsar/rt/session.py:37-43, without the reference's recall layer)."""
        return self._engine.context_page_ids(self._seq_id), self._engine.context_pages(self._seq_id)

    def destroy(self) -> None:
        self._engine.release(self._seq_id)


class Pulsar:
    """``Pulsar(model_dir, config, dtype=torch.bfloat16)``: ``config`` is the flat engine
    dictionary of the reference (``page_size``, ``max_sessions``, ``active_buffer_size``,
    ``max_running``, ``max_chunk_size``, ``eos_id``, ``temperature``, ``top_p``, ``top_k``,
    ``seed``, ``device``; unknown keys are rejected) plus ``num_pages``."""

    def __init__(self, model_dir: str, config: Optional[Dict[str, Any]] = None, *, dtype=torch.bfloat16):
        cfg = dict(config or {})
        cfg["dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, dtype)
        self._engine = Engine(model_dir, cfg)

    @property
    def engine(self) -> Engine:
        return self._engine

    def create_session(self, sink: Sequence[int] = (), *, overrides: Optional[Dict[str, Any]] = None) -> Session:
        return Session(self._engine.create_session(sink, overrides), self._engine)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, seed: Optional[int] = None
                 ) -> List[List[int]]:
        return self._engine.generate(prompts, max_new_tokens, temperature, top_k, top_p, seed)

    def close(self) -> None:
        for sid in list(self._engine._sessions):
            self._engine.release(sid)


def generate(model_dir: str, prompts: Sequence[Sequence[int]], max_new_tokens: int, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = -1, dtype: str = "bfloat16",
             **engine_config) -> List[List[int]]:
    """Load ``model_dir`` and generate ``max_new_tokens`` tokens for each prompt."""
    cfg = dict(engine_config)
    cfg.update(dtype=dtype, temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
    return Engine(model_dir, cfg).generate(prompts, max_new_tokens)
