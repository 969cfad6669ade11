"""Generation through the entry points: greedy tokens against the plain implementation,
long decoding, the first tokens of a sequence, sampling that a seed reproduces, preemption
when pages run out, several turns on kept pages (GPU)."""
import json
import os
import random
import subprocess
import sys

import pytest
import torch

import helpers
from helpers import TINY, TOL
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (raw, seed, page) in TINY.items():
        d = tmp_path_factory.mktemp(f"eng{name}")
        helpers.make_folder(d, raw, seed)
        out[name] = str(d)
    return out


def _engine(folder, dtype, page, **kw):
    from pulsar_b200.engine.engine import Engine
    cfg = dict(dtype=dtype, page_size=page, num_pages=64, max_sessions=4, max_running=4, max_chunk_size=16, eos_id=-1)
    cfg.update(kw)
    return Engine(folder, cfg)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_equals_the_plain_implementation(folders, name):
    raw, seed, page = TINY[name]
    cfg, weights = helpers.read_folder(folders[name])
    rng = random.Random(seed)
    prompts = [helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (1, 23, 40, 7, 18)]
    eng = _engine(folders[name], "float32", page, max_chunk_size=11)       # prompts are cut into portions, 4 at a time
    got = eng.generate(prompts, 9)
    want = [plain.greedy_generate(cfg, weights, p, 9) for p in prompts]
    assert got == want
    assert eng.cache.live_requests() == [] and all(f == 64 for f in eng.cache.n_free_pages())


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_generation_bfloat16_follows_the_plain_logits(folders, name):
    """Rounding may flip near-ties, so each emitted token is checked against the plain logits
    of its own prefix: it must be (nearly) the most probable one."""
    raw, seed, page = TINY[name]
    cfg, weights = helpers.read_folder(folders[name])
    w16 = helpers.as_bf16_matrices(weights)
    prompts = [helpers.random_tokens(random.Random(3), 19, raw["vocab_size"])]
    out = _engine(folders[name], "bfloat16", page).generate(prompts, 8)[0]
    seq = list(prompts[0])
    for tok in out:
        row = plain.forward(cfg, w16, seq, torch.float64)[-1]
        assert float(row.max() - row[tok]) <= TOL["bfloat16"] * float(row.abs().max())
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_long_decoding(folders, name, dtype):
    """300 tokens one by one after a short prompt: page edges and (in C) the window's edge are
    crossed many times; every position's logits are compared."""
    from pulsar_b200.replay import Replay
    raw, seed, page = TINY[name]
    cfg, weights = helpers.read_folder(folders[name])
    if dtype == "bfloat16":
        weights = helpers.as_bf16_matrices(weights)
    toks = helpers.random_tokens(random.Random(9), 305, raw["vocab_size"])
    ref = plain.forward(cfg, weights, toks, torch.float64)
    rp = Replay(folders[name], dtype, 320, page_size=page)
    rows = [rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks[:5], "want": [0, 1, 2, 3, 4]}]})]
    for i in range(5, len(toks)):
        rows.append(rp.run_step({"step": i, "entries": [{"id": "a", "tokens": [toks[i]], "want": [0]}]}))
    got = torch.cat(rows)
    worst = 0.0
    for pos in range(len(toks)):
        err = helpers.rel_err(got[pos], ref[pos])
        worst = max(worst, err)
        assert err < TOL[dtype], f"position {pos}: {err:.2e}"
    helpers.report(f"long_decoding[{name}]", worst, dtype)
    assert rp.runner.graph_replays > 200           # the decode steps ran as captured graphs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    from pulsar_b200.replay import Replay
    raw, seed, page = TINY["B"]
    cfg, weights = helpers.read_folder(folders["B"])
    if dtype == "bfloat16":
        weights = helpers.as_bf16_matrices(weights)
    rp = Replay(folders["B"], dtype, 128, page_size=page)
    for toks in ([5], [5, 9], [400, 1, 2]):
        ref = plain.forward(cfg, weights, toks, torch.float64)
        got = rp.run_step({"step": 0, "entries": [{"id": "x", "tokens": toks, "want": list(range(len(toks)))}], "end": ["x"]})
        assert helpers.rel_err(got, ref) < TOL[dtype]
        # the same, token by token from position 0
        rows = [rp.run_step({"step": i, "entries": [{"id": "y", "tokens": [t], "want": [0]}],
                             "end": ["y"] if i == len(toks) - 1 else []}) for i, t in enumerate(toks)]
        assert helpers.rel_err(torch.cat(rows), ref) < TOL[dtype]


def test_sampling_is_reproducible_per_request_and_obeys_top_k(folders):
    raw, seed, page = TINY["B"]
    cfg, weights = helpers.read_folder(folders["B"])
    rng = random.Random(4)
    p1, p2, p3 = (helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (12, 5, 20))
    eng = _engine(folders["B"], "float32", page)
    a = eng.generate([p1], 12, temperature=0.9, top_k=8, top_p=0.95, seed=11)[0]
    b = eng.generate([p1], 12, temperature=0.9, top_k=8, top_p=0.95, seed=11)[0]
    assert a == b                                                         # same seed, same tokens
    batch = eng.generate([p1, p2, p3], 12, temperature=0.9, top_k=8, top_p=0.95, seed=11)
    assert batch[0] == a                                                  # whatever else is in the batch
    c = eng.generate([p1], 12, temperature=0.9, top_k=8, top_p=0.95, seed=12)[0]
    assert c != a
    seq = list(p1)
    for tok in a:                                                         # every draw lies in the surviving set
        row = plain.forward(cfg, weights, seq, torch.float64)[-1]
        _, keep = plain.sample_filter(row, 0.9, 8, 0.95)
        assert tok in keep.tolist()
        seq.append(tok)
    g1 = eng.generate([p2], 6, temperature=0.0, top_k=3, seed=5)[0]       # temperature 0 is greedy whatever the rest
    assert g1 == plain.greedy_generate(cfg, weights, p2, 6)


def test_pages_run_out_preempts_and_the_tokens_stay_the_same(folders):
    raw, seed, page = TINY["A"]                                           # page 16
    cfg, weights = helpers.read_folder(folders["A"])
    rng = random.Random(6)
    prompts = [helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (30, 20, 28)]
    want = [plain.greedy_generate(cfg, weights, p, 40) for p in prompts]
    eng = _engine(folders["A"], "float32", page, num_pages=9, max_chunk_size=64)    # 144 tokens of cache for 218 needed
    got = eng.generate(prompts, 40)
    assert eng.scheduler.n_preemptions >= 1
    assert got == want
    assert all(f == 9 for f in eng.cache.n_free_pages())
    from pulsar_b200.engine.scheduler import SchedulerError
    with pytest.raises(SchedulerError, match="never"):
        eng.generate([list(range(100))], 60)                              # could never fit: refused at submit


def test_sessions_turn_by_turn_on_kept_pages(folders):
    from pulsar_b200.api import Pulsar
    raw, seed, page = TINY["B"]
    cfg, weights = helpers.read_folder(folders["B"])
    p = Pulsar(folders["B"], dict(page_size=page, num_pages=64, max_sessions=2, max_running=2, max_chunk_size=16),
               dtype=torch.float32)
    s = p.create_session([3, 4, 5])
    s.send([6, 7], 4)
    first = list(s.recv())
    assert first == plain.greedy_generate(cfg, weights, [3, 4, 5, 6, 7], 4)
    assert s.get_state() == "parked" and p.engine.cache.has(s.seq_id)     # finished turn: pages are kept
    s.send([9, 9, 8], 3)
    second = list(s.recv())
    assert second == plain.greedy_generate(cfg, weights, [3, 4, 5, 6, 7] + first + [9, 9, 8], 3)
    # what the engine tells about a sequence (engine.cpp:458-460, 492-494, 533-549): cached tokens, their pages
    eng = p.engine
    everything = [3, 4, 5, 6, 7] + first + [9, 9, 8] + second
    held = eng.active_tokens_count(s.seq_id)
    assert held == len(everything) - 1                   # the last sampled token has not been fed yet
    ids, pages = eng.context_page_ids(s.seq_id), eng.context_pages(s.seq_id)
    assert len(ids) == len(set(ids)) == -(-held // page) == len(pages)
    assert [t for pg in pages for t in pg] == everything[:held] and all(len(pg) <= page for pg in pages)
    assert eng.active_sequence_count() == 0
    eng.set_decode_budget(s.seq_id, 2)
    s.send([1])
    assert eng.active_sequence_count() == 1
    assert len(list(s.recv())) == 2
    s.destroy()
    assert p.engine.cache.live_requests() == [] and s.get_state() == "unknown"
    assert eng.active_tokens_count(s.seq_id) == 0 and eng.context_page_ids(s.seq_id) == [] and eng.context_pages(s.seq_id) == []
    with pytest.raises(Exception, match="unknown keys"):
        Pulsar(folders["B"], dict(pagesize=8))


def test_a_malformed_session_override_throws_at_create_session(folders):
    """pulsar-core/tests/runtime/test_engine.cpp:165-194: a bad knob fails when the session is made, opens nothing,
    and the next good session is the first one."""
    raw, seed, page = TINY["B"]
    eng = _engine(folders["B"], "float32", page)
    for bad in (dict(top_p=0.0), dict(top_p=1.5), dict(top_k=-1), dict(block_radius=4), dict(temprature=0.7)):
        with pytest.raises(ValueError):
            eng.create_session([1, 2, 3], bad)
    assert eng.active_sequence_count() == 0 and eng.session_state(0) == "unknown"
    sid = eng.create_session([1, 2, 3], dict(temperature=0.7, top_k=5, top_p=0.9, seed=3))
    assert sid == 0
    eng.feed(sid, [], 2)
    assert eng.active_sequence_count() == 1
    with pytest.raises(ValueError, match="vocabulary"):
        eng.feed(eng.create_session([1]), [10 ** 9], 2)
    eng.release(sid)


def _drive(eng, prompts, budgets, lookahead, overrides=None, second_turn=None):
    """Feed the prompts and step until nothing is left; the events per sequence, in order."""
    sids = [eng.create_session(p, overrides(i) if overrides else None) for i, p in enumerate(prompts)]
    for sid, b in zip(sids, budgets):
        eng.feed(sid, [], b)
    seen = {sid: [] for sid in sids}

    def run():
        guard = 0
        while eng.has_work():
            events = eng.step(1) if lookahead else eng.step_once()
            for sid, tok, fin in events:
                seen[sid].append((tok, fin))
            guard += 1
            assert guard < 10000
    run()
    if second_turn:
        for sid, extra in zip(sids, second_turn):
            eng.feed(sid, extra, 5)
        run()
    eng.cache.check_consistency()
    for sid in sids:
        eng.release(sid)
    assert eng.cache.live_requests() == [] and all(f == eng.config.num_pages for f in eng.cache.n_free_pages())
    return [seen[sid] for sid in sids]


def test_a_turn_without_tokens_after_the_stop_token_is_refused_in_both_stepping_modes(folders):
    """Stepping one pass ahead has cached the stop token when the turn ends, stepping one pass at a time has not.
    A further turn without a token is refused in both (nothing is queued, the engine goes on working); a further
    turn with a token gives the same tokens in both; a turn that a budget ended may go on without a token."""
    raw, seed, page = TINY["B"]
    rng = random.Random(4)
    prompt = helpers.random_tokens(rng, 21, raw["vocab_size"])
    free = _drive(_engine(folders["B"], "float32", page), [prompt], [12], lookahead=False)[0]
    eos = free[5][0]
    first_stop = [t for t, _ in free].index(eos)
    runs = []
    for lookahead in (False, True):
        eng = _engine(folders["B"], "float32", page, eos_id=eos)
        sid = eng.create_session(prompt)
        eng.feed(sid, [], 12)
        seen = []
        while eng.has_work():
            seen += eng.step(1) if lookahead else eng.step_once()
        assert [t for _, t, _ in seen] == [t for t, _ in free[:first_stop + 1]] and seen[-1][2]
        with pytest.raises(ValueError, match="stop token"):
            eng.feed(sid, [])
        assert not eng.has_work() and eng.session_state(sid) == "parked"
        eng.feed(sid, [5], 4)
        more = []
        while eng.has_work():
            more += eng.step(1) if lookahead else eng.step_once()
        # that turn ended on its budget (or on the stop token): without the stop token it may go on without a token
        if more[-1][1] != eos:
            eng.feed(sid, [], 3)
            while eng.has_work():
                more += eng.step(1) if lookahead else eng.step_once()
        runs.append([(t, f) for _, t, f in more])
        eng.cache.check_consistency()
        eng.release(sid)
    assert runs[0] == runs[1] and len(runs[0]) >= 2


def test_a_wait_that_runs_out_sets_its_error_word():
    """The give-up path of the kernels with bounded waits, alone: one thread waits on a barrier that nobody arrives on,
    with the limit set to a millisecond; the kernel returns, the error word says so, the context stays usable."""
    from pulsar_b200 import ops
    assert ops.gemm_tcgen05_error() == 0
    try:
        ops.set_wait_limit(2_000_000)
        ops.wait_selftest()
        torch.cuda.synchronize()
        assert ops.gemm_tcgen05_error() == 9
        words = torch.zeros(8, dtype=torch.int32, device="cuda")
        ops.gather_wait_words(words)
        assert words.tolist()[:ops.N_WAIT_WORDS] == [9, 0, 0, 0, 0]
        assert "wait self-test" in ops.describe_wait_words(words.tolist()[:ops.N_WAIT_WORDS])
        with pytest.raises(ops.DeviceWaitError):
            ops.check_wait_words()
    finally:
        ops.set_wait_limit(4_000_000_000)
        ops.set_wait_words(0)
    assert ops.gemm_tcgen05_error() == 0 and ops.prefill_tcgen05_error() == 0
    a = torch.randn(64, 64, device="cuda")
    assert torch.isfinite(a @ a).all()                  # the context still works


@pytest.mark.parametrize("lookahead", [False, True])
def test_an_error_word_behind_a_pass_becomes_an_exception_and_the_engine_refuses_further_work(folders, lookahead):
    """A kernel that gave up a bounded wait leaves its error word set; the engine reads the words with the pass's
    sampled ids, books none of its tokens, raises, and refuses everything after it."""
    from pulsar_b200 import ops
    from pulsar_b200.engine.engine import EngineFailed
    raw, seed, page = TINY["A"]
    eng = _engine(folders["A"], "bfloat16", page)
    sid = eng.create_session(helpers.random_tokens(random.Random(1), 9, raw["vocab_size"]))
    eng.feed(sid, [], 20)
    got = eng.step(2, lookahead=lookahead)
    assert len(got) >= 2
    try:
        ops.set_wait_words(3)               # as if the MMA issuer of a block had given up
        with pytest.raises(EngineFailed, match="MMA issuer") as info:
            for _ in range(3):
                eng.step(1, lookahead=lookahead)
        assert isinstance(info.value.__cause__, ops.DeviceWaitError)
    finally:
        ops.set_wait_words(0)
    for call in (lambda: eng.step(1), lambda: eng.step_once(), lambda: eng.feed(sid, [1]), lambda: eng.create_session([1])):
        with pytest.raises(EngineFailed, match="refuses further work"):
            call()
    eng.release(sid)                            # giving pages back still works
    assert eng.cache.live_requests() == []
    eng2 = _engine(folders["A"], "bfloat16", page)          # and a new engine on the same device runs
    assert len(eng2.generate([[1, 2, 3]], 4)[0]) == 4


@pytest.mark.parametrize("lookahead", [False, True])
@pytest.mark.parametrize("name", ["D", "E"])
def test_bfloat16_tokens_of_the_schedulers_own_mixed_steps_follow_the_plain_logits(folders, name, lookahead):
    """Four requests fed at once with a token budget far below their prompts: the scheduler's own steps hold the
    decoded tokens of the requests that are through their prompts first and portions of the others behind them
    (the order in which the attention dispatch splits a step between its decode and its prompt kernels).  Every
    row of logits that a token is sampled from is compared with the plain logits at its position, and the token
    with the plain logits' choice."""
    raw, seed, page = TINY[name]
    cfg, weights = helpers.read_folder(folders[name])
    w16 = helpers.as_bf16_matrices(weights)
    rng = random.Random(77)
    prompts = [helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (9, 150, 61, 230)]
    budgets = [30, 12, 22, 9]
    eng = _engine(folders[name], "bfloat16", page, max_chunk_size=40, num_pages=256)
    shapes, rows, fed = [], [], {}
    run_step = eng.runner.step

    def spy(entries, sampled_ids=None):
        shapes.append([len(e.tokens) for e in entries])
        logits = run_step(entries, sampled_ids)
        i = 0
        for e in entries:
            fed[e.rid] = fed.get(e.rid, 0) + len(e.tokens)
            for w in e.want:
                rows.append((e.rid, fed[e.rid] - len(e.tokens) + w, logits[i].to("cpu", copy=True)))
                i += 1
        return logits
    eng.runner.step = spy
    sids = [eng.create_session(p) for p in prompts]
    for sid, b in zip(sids, budgets):
        eng.feed(sid, [], b)
    out = {sid: [] for sid in sids}
    while eng.has_work():
        for sid, tok, _ in eng.step(1, lookahead=lookahead):
            out[sid].append(tok)
    assert [len(out[s]) for s in sids] == budgets
    mixed = [q for q in shapes if q[0] == 1 and max(q) > 1]
    assert len(mixed) >= 4, shapes                       # decoded tokens first, portions behind them
    for q in mixed:
        n_dec = next(i for i, n in enumerate(q) if n > 1)
        assert all(n > 1 for n in q[n_dec:]), q
    # the logits every token was sampled from, against the plain logits of the sequence as it came out
    ref = {sid: plain.forward(cfg, w16, list(p) + out[sid], torch.float64) for sid, p in zip(sids, prompts)}
    assert len(rows) == sum(budgets)
    worst = 0.0
    for sid, pos, row in rows:
        err = helpers.rel_err(row, ref[sid][pos])
        worst = max(worst, err)
        assert err < TOL["bfloat16"], f"sequence {sid} position {pos}: error {err:.3e}"
    for sid, prompt in zip(sids, prompts):               # and each token is the plain logits' choice up to rounding
        for i, tok in enumerate(out[sid]):
            row = ref[sid][len(prompt) + i - 1]
            gap = float(row.max() - row[tok]) / float(row.abs().max())
            assert gap <= TOL["bfloat16"], f"sequence {sid}: token {tok} is {gap:.2e} below the best"
    helpers.report(f"mixed_steps[{name}]", worst, "bfloat16")


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16")])
def test_stepping_one_pass_ahead_gives_the_same_tokens(folders, name, dtype):
    """Engine.step launches the next pass before it reads the last one's tokens (they are fed on the
    device).  Same events as one pass at a time: prompts in portions beside decoding sequences, budgets that
    end at different steps, a stop token that ends sequences one pass after they were scheduled again, and a
    second turn behind the stop token."""
    raw, seed, page = TINY[name]
    rng = random.Random(21)
    prompts = [helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (5, 30, 17, 9)]
    budgets = [12, 7, 20, 15]
    free = _drive(_engine(folders[name], dtype, page, max_chunk_size=12), prompts, budgets, lookahead=False)
    assert [len(ev) for ev in free] == budgets
    # a stop token that some sequence emits in the middle of its turn
    eos = free[2][6][0]
    extra = [[3, 1], [4], [5, 9, 2], [8]]
    runs = []
    for lookahead in (False, True):
        eng = _engine(folders[name], dtype, page, max_chunk_size=12, eos_id=eos)
        runs.append(_drive(eng, prompts, budgets, lookahead, second_turn=extra))
        if lookahead:
            assert eng._inflight is None and not eng._unclaimed
    assert runs[0] == runs[1]
    assert any(ev[-1] == (eos, True) for ev in runs[0][2:3] + runs[0]) and len(runs[0][2]) < budgets[2] + 5


def test_stepping_one_pass_ahead_keeps_the_random_streams(folders):
    """A sequence that stops on a stop token has drawn one number too many when the next pass was already
    in flight; its generator is set back, so a seeded sequence continues in its next turn as it would have."""
    raw, seed, page = TINY["B"]
    rng = random.Random(22)
    prompts = [helpers.random_tokens(rng, n, raw["vocab_size"]) for n in (6, 14, 10)]
    budgets = [16, 16, 16]
    ov = lambda i: dict(temperature=0.9, top_k=12, top_p=0.9, seed=100 + i)
    free = _drive(_engine(folders["B"], "float32", page), prompts, budgets, lookahead=False, overrides=ov)
    eos = free[1][4][0]
    extra = [[1], [2, 3], [4]]
    runs = [_drive(_engine(folders["B"], "float32", page, eos_id=eos), prompts, budgets, la, overrides=ov, second_turn=extra)
            for la in (False, True)]
    assert runs[0] == runs[1]
    assert runs[0][1][4] == (eos, True)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_arrivals_one_pass_ahead_and_one_pass_at_a_time(folders, seed):
    """Requests of random lengths and budgets arrive while others run, a stop token ends some early, and the pool is
    so small that requests are preempted and recomputed: the engine that steps one pass ahead emits what the one
    that steps one pass at a time emits, token for token."""
    raw, model_seed, page = TINY["A"]
    rng = random.Random(100 + seed)
    arrivals = []
    for i in range(10):
        arrivals.append((rng.randint(0, 25), helpers.random_tokens(rng, rng.randint(1, 45), raw["vocab_size"]), rng.randint(1, 24)))
    arrivals.sort(key=lambda a: a[0])
    eos = rng.randrange(raw["vocab_size"])

    def drive(lookahead):
        eng = _engine(folders["A"], "float32", page, num_pages=10, max_sessions=4, max_running=3, max_chunk_size=13, eos_id=eos)
        seen, owner, todo, tick = {}, {}, list(arrivals), 0
        while todo or owner:
            while todo and todo[0][0] <= tick and len(owner) < 4:
                _, prompt, budget = todo.pop(0)
                sid = eng.create_session(prompt)
                eng.feed(sid, [], budget)
                owner[sid] = len(seen)
                seen[owner[sid]] = []
            events = (eng.step(1) if lookahead else eng.step_once()) if eng.has_work() else []
            for sid, tok, fin in events:
                seen[owner[sid]].append((tok, fin))
                if fin:
                    eng.release(sid)
                    del owner[sid]
            tick += 1
            assert tick < 5000
        eng.cache.check_consistency()
        assert eng.cache.live_requests() == [] and all(f == 10 for f in eng.cache.n_free_pages())
        return seen, eng.scheduler.n_preemptions

    a, pre_a = drive(False)
    b, pre_b = drive(True)
    assert a == b
    assert all(ev and ev[-1][1] for ev in a.values())


@pytest.mark.parametrize("name,seed", [("A", 1), ("C", 5), ("E", 1), ("F", 1)])
def test_random_arrivals_second_turns_and_preemption_give_the_plain_tokens(folders, name, seed):
    """Requests of random lengths and budgets arrive while others run, in a pool so small that some are preempted
    and recomputed; a stop token ends some early, and some get a second turn of new tokens behind what they
    generated.  Every turn's tokens are the plain implementation's greedy tokens for that turn's whole prefix
    (float32), in either stepping mode."""
    from pulsar_b200.engine.engine import Engine
    raw, model_seed, page = TINY[name]
    cfg, weights = helpers.read_folder(folders[name])
    rng = random.Random(7000 + seed)
    arrivals = sorted(((rng.randint(0, 20), helpers.random_tokens(rng, rng.randint(1, 40), raw["vocab_size"]), rng.randint(1, 12),
                        rng.random() < 0.5) for _ in range(7)), key=lambda a: a[0])
    eos = rng.randrange(raw["vocab_size"])
    n_preempted = 0
    for lookahead in (False, True):
        turn_rng = random.Random(seed)
        eng = Engine(folders[name], dict(dtype="float32", page_size=page, num_pages=-(-72 // page) + 1, max_sessions=4, max_running=3,
                                         max_chunk_size=13, eos_id=eos))
        todo, live, tick = list(arrivals), {}, 0
        while todo or live:
            while todo and todo[0][0] <= tick and len(live) < 4:
                _, prompt, budget, second = todo.pop(0)
                sid = eng.create_session(prompt)
                eng.feed(sid, [], budget)
                live[sid] = dict(seq=list(prompt), got=[], budget=budget, second=second)
            events = (eng.step(1) if lookahead else eng.step_once()) if eng.has_work() else []
            for sid, tok, fin in events:
                r = live[sid]
                r["got"].append(tok)
                if not fin:
                    continue
                assert r["got"] == plain.greedy_generate(cfg, weights, r["seq"], r["budget"], eos_id=eos), (lookahead, len(r["seq"]))
                if r["second"]:
                    extra = helpers.random_tokens(turn_rng, turn_rng.randint(1, 6), raw["vocab_size"])
                    r["seq"] = r["seq"] + r["got"] + extra
                    r["got"], r["second"], r["budget"] = [], False, turn_rng.randint(1, 8)
                    eng.feed(sid, extra, r["budget"])
                else:
                    eng.release(sid)
                    del live[sid]
            tick += 1
            assert tick < 5000
        eng.cache.check_consistency()
        assert eng.cache.live_requests() == []
        n_preempted += eng.scheduler.n_preemptions
    assert n_preempted > 0, "the pool was meant to be too small for all requests at once"


def test_engine_refuses_a_cpu_device(folders):
    from pulsar_b200.engine.engine import Engine
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine(folders["A"], dict(device="cpu"))


def test_command_line(folders, tmp_path):
    raw, seed, page = TINY["A"]
    cfg, weights = helpers.read_folder(folders["A"])
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "pulsar-generate"), "--model", folders["A"], "--dtype",
                          "float32", "--prompt_ids", "1,2,3,4", "--prompt_ids", "9 8 7", "--gen_tokens", "5", "--max_pages",
                          "32", "--eos_id", "-1", "--json"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = json.loads(out.stdout.strip().splitlines()[-1])["outputs"]
    assert got == [plain.greedy_generate(cfg, weights, p, 5) for p in ([1, 2, 3, 4], [9, 8, 7])]


def test_profile_of_a_run_names_kernel_classes_and_host_phases(folders):
    """PULSAR_PROF=1: the same generation, and at exit a table of device time per kernel class (CUDA events) and of
    host time per phase on standard error; the tokens are those of the run without it."""
    raw, seed, page = TINY["D"]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "pulsar-generate"), "--model", folders["D"], "--dtype", "bfloat16",
           "--prompt_ids", "1,2,3,4,5,6,7", "--gen_tokens", "6", "--max_pages", "32", "--eos_id", "-1", "--json"]
    plain_run = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    prof_run = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, PULSAR_PROF="1"))
    assert plain_run.returncode == 0 and prof_run.returncode == 0, prof_run.stderr
    assert json.loads(prof_run.stdout.strip().splitlines()[-1])["outputs"] == json.loads(plain_run.stdout.strip().splitlines()[-1])["outputs"]
    err = prof_run.stderr
    assert "device time per kernel class" in err and "host time per phase" in err
    for name in ("gemm_skinny", "paged_attention_decode", "qk_norm_rope_write", "argmax", "plan (", "pack (", "launch (", "read ("):
        assert name in err, (name, err)
    assert "device time per kernel class" not in plain_run.stderr


LAYER_SIZES = {      # hidden, intermediate, query heads (8 kv heads of 128 each): the dense sizes of the family
    "8b": (4096, 12288, 32), "14b": (5120, 17408, 40), "32b": (5120, 25600, 64)}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("shape", ["8b", "14b", "32b"])
def test_layer_sizes_of_the_family(tmp_path_factory, shape, dtype):
    """Two layers with the real layer sizes (8B: hidden 4096, 32/8 heads of 128, intermediate 12288; 14B: hidden
    5120, groups of 5 query heads, intermediate 17408; 32B: groups of 8, intermediate 25600) and a vocabulary
    that is no power of two: the sizes at which the weight-streaming, tcgen05 and tensor-core attention kernels
    run in the benchmark.  A prompt in portions, then single tokens, beside a second request; then twenty short
    requests that bring one token each in the same step (more rows than the weight-streaming product takes).
    Logits against the plain implementation (float32 on the CPU here)."""
    from pulsar_b200.replay import Replay
    hidden, inter, heads = LAYER_SIZES[shape]
    raw = dict(helpers.TINY_B, vocab_size=15193, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
               num_attention_heads=heads, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0, rms_norm_eps=1e-6,
               max_window_layers=2, initializer_range=0.02)
    folder = helpers.make_folder(tmp_path_factory.mktemp("layers" + shape), raw, 5, store_dtype=torch.bfloat16)
    cfg, weights = helpers.read_folder(folder)
    weights = {n: t.to(torch.float32) for n, t in weights.items()}
    rng = random.Random(12)
    reqs = {"a": helpers.random_tokens(rng, 150, 15193), "b": helpers.random_tokens(rng, 41, 15193)}
    for i in range(20):
        reqs[f"s{i}"] = helpers.random_tokens(rng, 3 + (i * 7) % 11, 15193)
    ref = {rid: plain.forward(cfg, weights, toks, torch.float32) for rid, toks in reqs.items()}
    rp = Replay(folder, dtype, 256 + 20 * 64, page_size=16, max_running=24)
    got = {}
    fed = {rid: 0 for rid in reqs}

    def run(step, entries, end=()):
        logits = rp.run_step({"step": step, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in entries],
                              "end": list(end)})
        i = 0
        for r, t in entries:
            for k in range(len(t)):
                got[(r, fed[r] + k)] = logits[i]
                i += 1
            fed[r] += len(t)
    a, b = reqs["a"], reqs["b"]
    run(0, [("a", a[:100])])
    run(1, [("a", a[100:130]), ("b", b[:33])])                  # a later portion beside a first portion
    for i in range(8):                                          # single tokens of both
        run(2 + i, [("a", a[130 + i:131 + i]), ("b", b[33 + i:34 + i])])
    run(10, [("a", a[138:150])], end=["a", "b"])
    short = [f"s{i}" for i in range(20)]
    run(11, [(r, reqs[r][:-2]) for r in short])                 # twenty first portions in one step
    run(12, [(r, reqs[r][-2:-1]) for r in short])               # twenty single tokens in one step
    run(13, [(r, reqs[r][-1:]) for r in short], end=short)
    assert len(got) == sum(len(t) for t in reqs.values())
    worst = max(helpers.rel_err(row, ref[rid][pos]) for (rid, pos), row in got.items())
    helpers.report(f"layer_sizes[{shape}]", worst, dtype)
    assert worst < helpers.TOL_LARGE[dtype], f"worst relative error {worst:.3e}"
