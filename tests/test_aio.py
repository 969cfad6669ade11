"""The asyncio entry point: the background task's bookkeeping against a scripted engine (no GPU), and the
real engine behind it against the synchronous entry point (GPU)."""
import asyncio

import pytest

from pulsar_b200.aio import AsyncPulsar, EngineFailed


class ScriptedEngine:
    """Emits, for every fed sequence, the tokens 100*seq + 0, 1, 2, ... one per step, round robin."""

    def __init__(self, fail_at=None):
        self._sessions, self.active, self.steps, self.fail_at, self.released = {}, {}, 0, fail_at, []
        self.calls = []

    def create_session(self, tokens, overrides=None):
        sid = len(self._sessions)
        self._sessions[sid] = list(tokens)
        return sid

    def feed(self, sid, tokens, max_tokens=None):
        if sid in self.active:
            raise RuntimeError("still generating")
        self._sessions[sid] += list(tokens)
        self.active[sid] = [0, int(max_tokens)]

    def has_work(self):
        return bool(self.active)

    def step(self, n=1):
        self.steps += 1
        if self.fail_at is not None and self.steps >= self.fail_at:
            raise RuntimeError("device lost")
        events = []
        for sid in sorted(self.active):
            done, budget = self.active[sid]
            events.append((sid, 100 * sid + done, done + 1 == budget))
            self.active[sid][0] += 1
        for sid, _, fin in events:
            if fin:
                del self.active[sid]
        return events

    def session_state(self, sid):
        return "active" if sid in self.active else ("parked" if sid in self._sessions else "unknown")

    def release(self, sid):
        self.active.pop(sid, None)
        if self._sessions.pop(sid, None) is not None:
            self.released.append(sid)


async def _collect(stream):
    return [t async for t in stream]


def test_two_sessions_stream_their_own_tokens():
    async def main():
        eng = ScriptedEngine()
        p = AsyncPulsar.from_engine(eng)
        a = await p.create_session([1, 2, 3])
        b = await p.create_session([4])
        await a.send([], max_tokens=5)
        await b.send([9], max_tokens=3)
        sa, sb = await a.recv(), await b.recv()
        ta, tb = await asyncio.gather(_collect(sa), _collect(sb))
        assert ta == [0, 1, 2, 3, 4] and tb == [100, 101, 102]
        assert await a.get_state() == "parked"
        with pytest.raises(StopAsyncIteration):
            await sa.__anext__()
        # a further turn on the same session; the background task starts again
        await a.send([7], max_tokens=2)
        assert await _collect(await a.recv()) == [0, 1]
        await p.aclose()
        assert sorted(eng.released) == [0, 1]
        with pytest.raises(RuntimeError):
            await p.create_session([1])
    asyncio.run(main())


def test_tokens_before_recv_are_kept_and_a_second_recv_is_refused():
    async def main():
        eng = ScriptedEngine()
        p = AsyncPulsar.from_engine(eng)
        a = await p.create_session([1])
        b = await p.create_session([2])
        await a.send([], max_tokens=4)
        await b.send([], max_tokens=6)
        sb = await b.recv()                   # only b listens: a's tokens wait for its stream
        first = [await sb.__anext__(), await sb.__anext__()]
        assert first == [100, 101]
        with pytest.raises(RuntimeError):
            await b.recv()
        sa = await a.recv()
        ta, tb = await asyncio.gather(_collect(sa), _collect(sb))
        assert ta == [0, 1, 2, 3] and tb == [102, 103, 104, 105]
        await p.aclose()
    asyncio.run(main())


def test_destroy_ends_the_turn_and_an_engine_failure_ends_every_stream():
    async def main():
        eng = ScriptedEngine()
        p = AsyncPulsar.from_engine(eng)
        a = await p.create_session([1])
        await a.send([], max_tokens=1000)
        sa = await a.recv()
        assert await sa.__anext__() == 0
        await a.destroy()
        rest = await _collect(sa)             # ends instead of waiting for ever
        assert len(rest) < 1000 and 0 in eng.released
        await p.aclose()

        eng = ScriptedEngine(fail_at=3)
        p = AsyncPulsar.from_engine(eng)
        a = await p.create_session([1])
        b = await p.create_session([2])
        await a.send([], max_tokens=10)
        await b.send([], max_tokens=10)
        sa, sb = await a.recv(), await b.recv()
        for s in (sa, sb):
            with pytest.raises(EngineFailed):
                await _collect(s)
        with pytest.raises(EngineFailed):
            await a.send([1], max_tokens=1)
        await p.aclose()
    asyncio.run(main())


@pytest.mark.gpu
def test_async_entry_point_gives_the_tokens_of_the_synchronous_one(tmp_path):
    import helpers
    import pulsar_b200
    folder = helpers.make_folder(str(tmp_path / "m"), helpers.TINY_B, 3)
    prompts = [[5, 17, 3, 200, 41], [9, 8, 7], [300, 2, 2, 2, 2, 2, 2, 11]]
    cfg = dict(page_size=8, num_pages=64, max_sessions=4, max_running=4)
    want = pulsar_b200.generate(folder, prompts, 12, dtype="float32", **cfg)

    async def main():
        p = await AsyncPulsar.load(folder, cfg, dtype="float32")
        sessions = [await p.create_session(pr) for pr in prompts]
        for s in sessions:
            await s.send([], max_tokens=12)
        streams = [await s.recv() for s in sessions]
        got = await asyncio.gather(*[_collect(st) for st in streams])
        assert [await s.get_state() for s in sessions] == ["parked"] * 3
        await p.aclose()
        return got
    assert asyncio.run(main()) == want
