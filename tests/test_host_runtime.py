"""The C++ host runtime (cache accounting, scheduler, step packer) against the plain Python one
under random sequences of requests: the same calls on both must give the same steps, block tables,
page counts and token lists.  No GPU."""
import ctypes
import random

import pytest

from plain import host_plain as plain
from pulsar_b200 import host
from pulsar_b200.cache import CacheManager, CacheNeed, OutOfPages
from pulsar_b200.engine.scheduler import UNREAD, Scheduler, SchedulerError


def pair(pages, page, max_running, budget, window=None, max_requests=6):
    needs = [CacheNeed.paged_kv(2, 16), CacheNeed.paged_kv(2, 16, window)]
    pneeds = [plain.CacheNeed.paged_kv(2, 16), plain.CacheNeed.paged_kv(2, 16, window)]
    cache = CacheManager(needs, page, pages, max_requests)
    pcache = plain.CacheManager(pneeds, page, pages, max_requests)
    return (cache, Scheduler(cache, max_running, budget)), (pcache, plain.Scheduler(pcache, max_running, budget))


def same_state(native, oracle, rids):
    (cache, sched), (pcache, psched) = native, oracle
    assert cache.n_free_pages() == pcache.n_free_pages() and cache.n_free_slots() == pcache.n_free_slots()
    assert sched.waiting == list(psched.waiting) and sched.running == psched.running
    assert sched.n_preemptions == psched.n_preemptions
    for rid in rids:
        assert (rid in sched.seqs) == (rid in psched.seqs)
        assert cache.has(rid) == pcache.has(rid)
        if rid in psched.seqs:
            a, b = sched.seqs[rid], psched.seqs[rid]
            assert (a.tokens, a.n_cached, a.n_generated, a.unread, a.spent, a.preemptions, a.admitted_at) == \
                   (b.tokens, b.n_cached, b.n_generated, b.unread, b.spent, b.preemptions, b.admitted_at)
        if pcache.has(rid):
            assert cache.length(rid) == pcache.length(rid) and cache.state_slot(rid) == pcache.state_slot(rid)
            for g in range(len(pcache.groups)):
                assert cache.table(rid, g) == pcache.table(rid, g)
    cache.check_consistency()
    pcache.check_consistency()


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("window", [None, 9])
def test_scheduler_and_cache_follow_the_plain_ones(seed, window):
    """Random arrivals, lookahead steps with unread tokens, stop tokens that void a token, turns that
    continue, releases, and so few pages that requests are preempted and recomputed."""
    rng = random.Random(1000 * seed + (window or 0))
    native, oracle = pair(pages=rng.choice([6, 10, 24]), page=4, max_running=rng.choice([2, 4]), budget=rng.choice([5, 16]),
                          window=window)
    both = (native, oracle)
    rids, parked, next_id, eos = [], set(), 0, 7
    inflight = None                       # rids sampled by the step whose tokens are unread
    for _ in range(400):
        op = rng.random()
        if op < 0.15 and len(rids) < 6:
            rid = f"r{next_id}"
            next_id += 1
            toks = [rng.randrange(20) for _ in range(rng.randint(1, 14))]
            new = rng.randint(1, 9)
            outcomes = []
            for cache, sched in both:
                try:
                    sched.add_request(rid, toks, new)
                    outcomes.append("ok")
                except (SchedulerError, plain.SchedulerError) as e:
                    outcomes.append("never" if "never" in str(e) else "other")
            assert outcomes[0] == outcomes[1]
            if outcomes[0] == "ok":
                rids.append(rid)
        elif op < 0.22 and parked and inflight is None:
            rid = rng.choice(sorted(parked))
            extra = [rng.randrange(20) for _ in range(rng.randint(1, 5))]
            outcomes = []
            for cache, sched in both:
                try:
                    sched.extend_request(rid, extra, 3)
                    outcomes.append("ok")
                except (SchedulerError, plain.SchedulerError):
                    outcomes.append("refused")
            assert outcomes[0] == outcomes[1]
            if outcomes[0] == "ok":
                parked.discard(rid)
        elif op < 0.30 and rids and inflight is None:
            rid = rids.pop(rng.randrange(len(rids)))
            parked.discard(rid)
            for cache, sched in both:
                sched.finish(rid)
        else:
            lookahead = inflight is not None
            plans = [sched.schedule(allow_preempt=not lookahead) for cache, sched in both]
            assert (plans[0] is None) == (plans[1] is None)
            tokens = None
            if plans[0] is not None:
                assert [(e.rid, e.tokens, e.sample) for e in plans[0]] == [(e.rid, e.tokens, e.sample) for e in plans[1]]
            # the tokens of the step in flight arrive (before a step that needs preemption, after one that does not)
            if lookahead:
                tokens = {rid: rng.choice([eos, 1, 2, 3, 4]) for rid in inflight}
            if plans[0]:
                for (cache, sched), plan in zip(both, plans):
                    for e in plan:
                        if not cache.has(e.rid):
                            cache.open(e.rid)
                        cache.append(e.rid, len(e.tokens))
                    sched.on_step(plan)
                    for e in plan:
                        if e.sample:
                            sched.on_sampled(e.rid)
            new_inflight = [e.rid for e in plans[0] if e.sample] if plans[0] else None
            if tokens is not None:
                for rid, tok in tokens.items():
                    fin = [sched.on_token(rid, tok, eos) for cache, sched in both]
                    assert fin[0] == fin[1]
                    if fin[0]:
                        for cache, sched in both:
                            sched.park(rid)
                        parked.add(rid)
                        if new_inflight and rid in new_inflight:          # it ran one token too far
                            for cache, sched in both:
                                sched.drop_unread(rid)
                            new_inflight.remove(rid)
            inflight = new_inflight or None
        same_state(native, oracle, rids)
    for rid in list(rids):
        for cache, sched in both:
            sched.finish(rid)
    assert native[0].n_free_pages() == oracle[0].n_free_pages() == [g.allocator.n for g in native[0].groups]


def test_step_packer_writes_what_the_tables_say():
    """ph_step_plan / ph_step_pack against the arrays built by hand from the plain cache: prompt portions,
    single tokens, a token that comes from the device, wanted rows, two groups (one with a window)."""
    rng = random.Random(3)
    needs = [CacheNeed.paged_kv(2, 16), CacheNeed.paged_kv(2, 16, 6)]
    cache = CacheManager(needs, 4, 64, 4)
    pcache = plain.CacheManager([plain.CacheNeed.paged_kv(2, 16), plain.CacheNeed.paged_kv(2, 16, 6)], 4, 64, 4)
    lib = host.lib()
    history = {"a": 0, "b": 0, "c": 0}
    for step in range(12):
        entries = []
        for rid in sorted(history):
            if rng.random() < 0.8:
                n = 1 if step > 3 and rng.random() < 0.6 else rng.randint(1, 7)
                toks = [rng.randrange(50) for _ in range(n)]
                want = sorted(rng.sample(range(n), rng.randint(0, n)))
                src = rng.randrange(3) if n == 1 and rng.random() < 0.5 else -1
                entries.append((rid, toks, want, src))
        if not entries:
            continue
        s = len(entries)
        rids = host.longs([cache.native_id(e[0], create=True) for e in entries])
        n_tok, want_n = host.ints([len(e[1]) for e in entries]), host.ints([len(e[2]) for e in entries])
        tokens = host.ints([t for e in entries for t in e[1]])
        wants = host.ints([w for e in entries for w in e[2]] or [0])
        src = host.ints([e[3] for e in entries])
        starts, slots, widths, bad = (ctypes.c_int * s)(), (ctypes.c_int * s)(), (ctypes.c_int * 2)(), ctypes.c_int()
        total = lib.ph_step_plan(cache._h, s, rids, n_tok, tokens, want_n, wants, src, 3, 50, 64, starts, slots, widths,
                                 ctypes.byref(bad))
        assert total > 0
        buf = (ctypes.c_int * total)()
        moved = any(e[3] >= 0 for e in entries)
        k = 7 + 4 + (2 if moved else 0)          # seven arrays, two per group, two for tokens from the device
        off, ln = (ctypes.c_int * k)(), (ctypes.c_int * k)()
        assert lib.ph_step_pack(cache._h, s, rids, n_tok, tokens, want_n, wants, src, starts, slots, widths,
                                ctypes.cast(buf, ctypes.c_void_p), total, off, ln) == total
        arr = lambda i: list(buf[off[i]:off[i] + ln[i]])
        # the same step on the plain cache, arrays by hand
        tok, pos, seq, cu, kv, lrow, at = [], [], [], [0], [], [], 0
        for i, (rid, toks, want, _) in enumerate(entries):
            if not pcache.has(rid):
                pcache.open(rid)
            else:
                pcache.release_passed(rid)
        for i, (rid, toks, want, _) in enumerate(entries):
            start = pcache.append(rid, len(toks))
            assert start == starts[i] == history[rid]
            history[rid] += len(toks)
            tok += toks
            pos += list(range(start, start + len(toks)))
            seq += [i] * len(toks)
            lrow += [at + w for w in want]
            at += len(toks)
            cu.append(at)
            kv.append(start + len(toks))
        assert (arr(0), arr(1), arr(2), arr(3), arr(4), arr(6)) == (tok, pos, seq, cu, kv, lrow)
        assert arr(5) == [pcache.state_slot(e[0]) for e in entries]
        single = all(len(e[1]) == 1 for e in entries)
        for g in range(2):
            w = max(1, max(len(pcache.table(e[0], g)) for e in entries))
            if single:
                w = -(-w // 64) * 64
            assert widths[g] == w
            want_slots = [sl for i, e in enumerate(entries) for sl in pcache.slots(e[0], g, starts[i], len(e[1]))]
            assert arr(7 + 2 * g) == want_slots
            table = arr(8 + 2 * g)
            for i, e in enumerate(entries):
                row = pcache.table(e[0], g)
                assert table[i * w:(i + 1) * w] == row + [-1] * (w - len(row))
        if moved:
            assert arr(11) == [cu[i] for i, e in enumerate(entries) if e[3] >= 0]
            assert arr(12) == [e[3] for e in entries if e[3] >= 0]
        cache.check_consistency()


def test_step_packer_refuses_without_changing_anything():
    cache = CacheManager([CacheNeed.paged_kv(2, 16)], 4, 3, 2)
    lib = host.lib()
    cache.open("a")
    cache.append("a", 7)

    def plan(entries, vocab=50):
        s = len(entries)
        rids = host.longs([cache.native_id(r, create=True) for r, _ in entries])
        n_tok = host.ints([len(t) for _, t in entries])
        tokens = host.ints([x for _, t in entries for x in t])
        zeros, minus = host.ints([0] * s), host.ints([-1] * s)
        out = [(ctypes.c_int * s)(), (ctypes.c_int * s)(), (ctypes.c_int * 1)(), ctypes.c_int()]
        return lib.ph_step_plan(cache._h, s, rids, n_tok, tokens, zeros, host.ints([0]), minus, 0, vocab, 64, out[0], out[1],
                                out[2], ctypes.byref(out[3]))
    before = (cache.n_free_pages(), cache.length("a"), cache.table("a", 0))
    assert plan([("a", [1] * 2), ("b", [2] * 4)]) == host.OUT_OF_PAGES          # 1 + 1 pages for 1 free
    assert plan([("a", [1]), ("a", [2])]) == host.ALREADY_OPEN                  # twice in one step
    assert plan([("a", [77])]) == host.BAD_ARGUMENT                            # outside the vocabulary
    assert plan([("b", [1]), ("c", [1]), ("d", [1])]) == host.OUT_OF_SLOTS
    assert (cache.n_free_pages(), cache.length("a"), cache.table("a", 0)) == before and not cache.has("b")
    assert plan([("a", [1]), ("b", [2] * 4)]) > 0 and cache.has("b") and cache.length("a") == 8
    cache.check_consistency()


def test_resident_tables_hold_what_the_host_tables_say():
    """With resident tables a step brings only the page ids that its requests gained since they were last sent.
    A stand-in for the device applies them to one row per state slot; after every step each request's row equals
    its table on the host wherever a kernel may read it (pages that a window released are never read), also for
    requests that were closed and opened again on a used row, and the packed array of a step of single tokens
    keeps its length."""
    rng = random.Random(9)
    needs = [CacheNeed.paged_kv(2, 16), CacheNeed.paged_kv(2, 16, 6)]
    cache = CacheManager(needs, 4, 96, 4)
    lib = host.lib()
    lib.ph_set_resident_tables(cache._h, 1)
    resident = [[[-7] * 64 for _ in range(4)] for _ in range(2)]           # [group][row][logical page]
    live, sent_words, table_words = {}, 0, 0
    for step in range(60):
        for rid in list(live):                                             # some requests end, their rows are used again
            if rng.random() < 0.08:
                cache.close(rid)
                del live[rid]
        names = [f"r{i}" for i in range(4)]
        entries = []
        for rid in names:
            if rng.random() < 0.7 and (rid in live or len(live) + len([e for e in entries if e[0] not in live]) < 4):
                n = 1 if rid in live and rng.random() < 0.7 else rng.randint(1, 9)
                entries.append((rid, [rng.randrange(50) for _ in range(n)]))
        if not entries:
            continue
        s = len(entries)
        rids = host.longs([cache.native_id(e[0], create=True) for e in entries])
        n_tok = host.ints([len(e[1]) for e in entries])
        tokens = host.ints([t for e in entries for t in e[1]])
        zeros, minus = host.ints([0] * s), host.ints([-1] * s)
        starts, slots, widths, bad = (ctypes.c_int * s)(), (ctypes.c_int * s)(), (ctypes.c_int * 2)(), ctypes.c_int()
        total = lib.ph_step_plan(cache._h, s, rids, n_tok, tokens, zeros, host.ints([0]), minus, 0, 50, 64, starts, slots,
                                 widths, ctypes.byref(bad))
        assert total > 0, total
        for e in entries:
            live[e[0]] = live.get(e[0], 0) + len(e[1])
        buf = (ctypes.c_int * total)()
        off, ln = (ctypes.c_int * 11)(), (ctypes.c_int * 11)()
        assert lib.ph_step_pack(cache._h, s, rids, n_tok, tokens, zeros, host.ints([0]), minus, starts, slots, widths,
                                ctypes.cast(buf, ctypes.c_void_p), total, off, ln) == total
        single = all(len(e[1]) == 1 for e in entries)
        for g in range(2):
            upd = list(buf[off[8 + 2 * g]:off[8 + 2 * g] + ln[8 + 2 * g]])
            if single:
                assert len(upd) == 1 + 3 * s                               # the same length every such step
            assert upd[0] * 3 + 1 <= len(upd)
            for u in range(upd[0]):
                row, lp, page = upd[1 + 3 * u:4 + 3 * u]
                assert row in list(slots) and page >= 0
                resident[g][row][lp] = page
            sent_words += len(upd)
            table_words += s * widths[g]
            window = needs[g].window
            for i, e in enumerate(entries):
                table = cache.table(e[0], g)
                length = cache.length(e[0])
                first_read = 0 if window is None else max(0, starts[i] - window + 1) // 4     # pages a query of this step reads
                for lp in range(first_read, -(-length // 4)):
                    assert resident[g][slots[i]][lp] == table[lp], (step, g, e[0], lp)
        cache.check_consistency()
    assert sent_words * 4 < table_words                                    # far fewer words travel
