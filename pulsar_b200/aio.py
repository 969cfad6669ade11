"""The Python entry point on asyncio, as the reference's runtime offers it.

The reference's ``Pulsar`` is used from coroutines: ``await pulsar.create_session(sink)``,
``await session.send(ids)``, ``stream = await session.recv()``, ``async for token in stream``,
``await session.destroy()``, ``await pulsar.aclose()``; one background task steps the engine while
any turn is open and hands every token to the stream of its sequence, and an engine failure ends
every open stream with an error (pulsar/src/pulsar/rt/pulsar.py:12-43; rt/session.py:11-63;
rt/streaming.py:22-99; rt/sync.py:19-33).

Here the same names sit on the synchronous ``Engine``.  All engine calls, the constructor
included, run on one worker thread, in the order in which they were asked for: the CUDA device and
stream of the engine belong to that thread, and no lock is needed.  Token ids in, token ids out.
"""
from __future__ import annotations

import asyncio
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Dict, Optional, Sequence

from .engine.engine import EngineFailed       # the engine raised while stepping: every open stream ends with this,
                                              # and the instance refuses further work

_END = object()


class TokenStream:
    """The tokens of one turn, in order: ``async for token in stream``."""

    def __init__(self) -> None:
        self._queue: asyncio.Queue = asyncio.Queue()
        self._closed = False

    def __aiter__(self) -> "TokenStream":
        return self

    async def __anext__(self) -> int:
        if self._closed:
            raise StopAsyncIteration
        item = await self._queue.get()
        if item is _END:
            self._closed = True
            raise StopAsyncIteration
        if isinstance(item, BaseException):
            self._closed = True
            raise EngineFailed("the engine failed during this turn") from item
        return item


class AsyncSession:
    """One sequence.  A turn is ``send`` then ``recv``; a second ``recv`` before the first turn has
    ended is an error, as in the reference."""

    def __init__(self, seq_id: int, owner: "AsyncPulsar"):
        self._seq_id, self._owner = seq_id, owner

    @property
    def seq_id(self) -> int:
        return self._seq_id

    async def send(self, tokens: Sequence[int], max_tokens: Optional[int] = None) -> None:
        """Add tokens to the sequence and schedule it for up to ``max_tokens`` new tokens."""
        await self._owner._call(lambda e: e.feed(self._seq_id, list(tokens), max_tokens))

    async def recv(self) -> TokenStream:
        return self._owner._open(self._seq_id)

    async def get_state(self) -> str:
        return await self._owner._call(lambda e: e.session_state(self._seq_id))

    async def get_context(self):
        """``(page ids, token ids of each page)`` of what attention reads for this sequence
        (the reference's ``get_context``, pulsar/src/pulsar/rt/session.py:37-43, without its recall layer)."""
        return await self._owner._call(lambda e: (e.context_page_ids(self._seq_id), e.context_pages(self._seq_id)))

    async def destroy(self) -> None:
        """End the turn in flight, if any, and give the sequence's pages back."""
        self._owner._discard(self._seq_id)
        await self._owner._call(lambda e: e.release(self._seq_id))


class AsyncPulsar:
    """``pulsar = await AsyncPulsar.load(model_dir, config, dtype="bfloat16")``.  ``config`` is the
    flat engine dictionary (see ``pulsar_b200.api.Pulsar``); ``decode_chunk_size`` is the number of
    tokens one background step asks the engine for (the reference's argument of that name)."""

    def __init__(self, engine, executor: ThreadPoolExecutor, decode_chunk_size: int = 1):
        self._engine = engine
        self._executor = executor
        self._chunk = max(1, int(decode_chunk_size))
        self._streams: Dict[int, TokenStream] = {}
        self._backlog: Dict[int, list] = {}       # tokens of sequences whose stream is not open yet
        self._pump: Optional[asyncio.Task] = None
        self._failed: Optional[BaseException] = None
        self._closed = False

    @classmethod
    async def load(cls, model_dir: str, config: Optional[Dict[str, Any]] = None, *, dtype: str = "bfloat16",
                   decode_chunk_size: int = 1) -> "AsyncPulsar":
        from .engine.engine import Engine
        cfg = dict(config or {})
        cfg["dtype"] = dtype
        executor = ThreadPoolExecutor(max_workers=1, thread_name_prefix="pulsar-engine")
        loop = asyncio.get_running_loop()
        try:
            engine = await loop.run_in_executor(executor, lambda: Engine(model_dir, cfg))
        except BaseException:
            executor.shutdown(wait=False)
            raise
        return cls(engine, executor, decode_chunk_size)

    @classmethod
    def from_engine(cls, engine, decode_chunk_size: int = 1) -> "AsyncPulsar":
        """Around an engine that exists already; from now on it must be used through this object only."""
        return cls(engine, ThreadPoolExecutor(max_workers=1, thread_name_prefix="pulsar-engine"), decode_chunk_size)

    # ------------------------------------------------------------------ engine calls, one at a time
    async def _call(self, what: Callable[[Any], Any]):
        if self._closed:
            raise RuntimeError("this AsyncPulsar was closed")
        if self._failed is not None:
            raise EngineFailed("the engine failed earlier") from self._failed
        return await asyncio.get_running_loop().run_in_executor(self._executor, what, self._engine)

    async def create_session(self, sink: Sequence[int] = (), *, overrides: Optional[Dict[str, Any]] = None) -> AsyncSession:
        seq_id = await self._call(lambda e: e.create_session(list(sink), overrides))
        return AsyncSession(seq_id, self)

    # ------------------------------------------------------------------ streams and the background task
    def _open(self, seq_id: int) -> TokenStream:
        if self._failed is not None:
            raise EngineFailed("the engine failed earlier") from self._failed
        if seq_id in self._streams:
            raise RuntimeError(f"session {seq_id} already has a turn in flight; it must end before the next recv()")
        stream = self._streams[seq_id] = TokenStream()
        if self._pump is None or self._pump.done():
            self._pump = asyncio.get_running_loop().create_task(self._run())
        return stream

    def _discard(self, seq_id: int) -> None:
        stream = self._streams.pop(seq_id, None)
        if stream is not None:
            stream._queue.put_nowait(_END)

    async def _run(self) -> None:
        """Steps the engine while a turn is open.  Tokens of sequences without an open stream (a turn
        whose ``recv`` has not been called yet) are kept for that stream."""
        backlog = self._backlog
        try:
            while self._streams:
                self._flush()                               # what arrived before a stream was opened
                if not self._streams:
                    break
                events = await self._call(lambda e: e.step(self._chunk))
                if not events:
                    idle = await self._call(lambda e: not e.has_work())
                    if idle:                                    # nothing scheduled: the open turns are over
                        for seq_id in list(self._streams):
                            self._discard(seq_id)
                        break
                for seq_id, token, finished in events:       # through the backlog, so that the order holds for a
                    backlog.setdefault(seq_id, []).append((token, finished))     # stream opened during the step
                self._flush()
        except asyncio.CancelledError:
            raise
        except BaseException as exc:
            self._failed = exc
            for stream in self._streams.values():
                stream._queue.put_nowait(exc)
            self._streams.clear()

    def _flush(self) -> None:
        """Hand the kept tokens to the streams that are open; a turn's last token closes its stream, and what
        follows it (a later turn of the same sequence) waits for the next stream."""
        for seq_id in list(self._streams):
            items = self._backlog.pop(seq_id, [])
            stream = self._streams[seq_id]
            for i, (token, finished) in enumerate(items):
                stream._queue.put_nowait(int(token))
                if finished:
                    stream._queue.put_nowait(_END)
                    del self._streams[seq_id]
                    if items[i + 1:]:
                        self._backlog[seq_id] = items[i + 1:]
                    break

    async def aclose(self) -> None:
        """Stop stepping, end the open streams and release every sequence."""
        if self._closed:
            return
        if self._pump is not None and not self._pump.done():
            self._pump.cancel()
            try:
                await self._pump
            except (asyncio.CancelledError, Exception):
                pass
        for seq_id in list(self._streams):
            self._discard(seq_id)
        if self._failed is None:
            try:
                await self._call(lambda e: [e.release(s) for s in list(getattr(e, "_sessions", {}))])
            except Exception:
                pass
        self._closed = True
        self._executor.shutdown(wait=True)
