"""The scheduler's decisions without a GPU: a fake step function takes the pages and
"samples" token 1.  Mirrors pulsar-core/tests/runtime/test_scheduler.cpp:2256-2334
(prefill then decode, mixed step, portions 16+16+8, admission within the page budget, free
on finish) and adds what this engine decides differently (whole-step budget, preemption)."""
import pytest

from pulsar_b200.cache import CacheManager, CacheNeed
from pulsar_b200.engine.scheduler import UNREAD, Scheduler, SchedulerError


def make(pages=16, page=4, max_running=4, budget=16, max_requests=8):
    cache = CacheManager([CacheNeed.paged_kv(2, 16)], page, pages, max_requests)
    return cache, Scheduler(cache, max_running, budget)


def run_step(cache, sched, eos=-1, token=1):
    """What Engine.step_once does around the model: take pages, note progress, sample."""
    plan = sched.schedule()
    for e in plan:
        if not cache.has(e.rid):
            cache.open(e.rid)
        cache.append(e.rid, len(e.tokens))
    sched.on_step(plan)
    finished = []
    for e in plan:
        if e.sample and sched.on_token(e.rid, token, eos):
            sched.finish(e.rid)
            finished.append(e.rid)
    cache.check_consistency()
    return plan, finished


def shape(plan):
    return [(e.rid, len(e.tokens), e.sample) for e in plan]


def test_prefill_then_decode():
    cache, s = make()
    s.add_request("a", list(range(10)), 3)
    assert shape(run_step(cache, s)[0]) == [("a", 10, True)]
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("a", 1, True)] and plan[0].tokens == [1]        # the sampled token is fed next
    plan, fin = run_step(cache, s)
    assert fin == ["a"] and not s.has_work() and cache.n_free_pages() == [16]


def test_portions_under_the_budget():
    cache, s = make(budget=16)
    s.add_request("a", list(range(40)), 2)
    assert shape(run_step(cache, s)[0]) == [("a", 16, False)]
    assert shape(run_step(cache, s)[0]) == [("a", 16, False)]
    assert shape(run_step(cache, s)[0]) == [("a", 8, True)]                  # 16 + 16 + 8
    assert shape(run_step(cache, s)[0]) == [("a", 1, True)]


def test_mixed_step_decodes_first_and_counts_them_in_the_budget():
    cache, s = make(budget=8, pages=32)
    s.add_request("a", list(range(5)), 10)
    run_step(cache, s)
    s.add_request("b", list(range(20)), 10)
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("a", 1, True), ("b", 7, False)]                  # 1 decoded token + 7 prompt tokens = 8
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("a", 1, True), ("b", 7, False)]
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("a", 1, True), ("b", 6, True)]
    plan, _ = run_step(cache, s)
    assert sorted(shape(plan)) == [("a", 1, True), ("b", 1, True)]


def test_two_prompts_share_a_step_in_fifo_order():
    cache, s = make(budget=16, pages=32)
    s.add_request("a", list(range(10)), 2)
    s.add_request("b", list(range(10)), 2)
    assert shape(run_step(cache, s)[0]) == [("a", 10, True), ("b", 6, False)]
    assert shape(run_step(cache, s)[0]) == [("a", 1, True), ("b", 4, True)]


def test_admission_waits_for_pages_and_the_head_blocks_the_queue():
    cache, s = make(pages=6, page=4, budget=64)
    s.add_request("a", list(range(15)), 4)          # 15 + 1 -> 4 pages
    s.add_request("b", list(range(11)), 2)          # 11 + 1 -> 3 pages: does not fit beside a
    s.add_request("c", [1, 2], 2)                   # would fit, but waits behind b
    assert shape(run_step(cache, s)[0]) == [("a", 15, True)]
    assert list(s.waiting) == ["b", "c"]
    for _ in range(3):
        plan, fin = run_step(cache, s)
        assert [e.rid for e in plan] == ["a"]
    assert fin == ["a"]                              # a finished: pages are free again
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("b", 11, True), ("c", 2, True)]


def test_max_running_bounds_admission():
    cache, s = make(max_running=2, pages=64, budget=64)
    for r in "abc":
        s.add_request(r, [1, 2, 3], 2)
    assert [e.rid for e in run_step(cache, s)[0]] == ["a", "b"]
    plan, fin = run_step(cache, s)
    assert sorted(fin) == ["a", "b"]
    assert [e.rid for e in run_step(cache, s)[0]] == ["c"]


def test_pages_run_out_while_decoding_the_youngest_is_preempted_and_recomputed():
    cache, s = make(pages=4, page=4, budget=64)
    with pytest.raises(SchedulerError, match="never"):      # 10 + 12 tokens need 6 pages: refused at submit
        s.add_request("huge", list(range(10)), 12)
    s.add_request("old", list(range(7)), 9)          # 16 tokens at most: the whole pool
    s.add_request("young", list(range(3)), 9)        # 12 tokens at most
    run_step(cache, s)                               # both admitted: 2 + 1 pages, 1 free
    assert s.running == ["old", "young"]
    preempted_at = None
    outputs = {"old": 0, "young": 0}
    for step in range(40):
        plan, fin = run_step(cache, s)
        for e in plan:
            if e.sample:
                outputs[e.rid] += 1
        if s.n_preemptions and preempted_at is None:
            preempted_at = step
            assert "young" in s.waiting and "old" in s.running       # the request admitted last gives way
            assert not cache.has("young")
        if not s.has_work():
            break
    assert preempted_at is not None and not s.has_work()
    assert cache.n_free_pages() == [4]
    assert s.n_preemptions >= 1


def test_preempted_request_is_recomputed_from_all_its_tokens():
    cache, s = make(pages=4, page=4, budget=64)
    s.add_request("old", list(range(7)), 9)
    s.add_request("young", list(range(3)), 9)
    seen_prefill = []
    for _ in range(40):
        plan, _ = run_step(cache, s)
        seen_prefill += [(e.rid, len(e.tokens)) for e in plan if len(e.tokens) > 1]
        if not s.has_work():
            break
    young = [n for rid, n in seen_prefill if rid == "young"]
    assert young[0] == 3 and len(young) >= 2 and young[1] > 3        # prompt, later prompt + what it had generated


def test_finish_gives_pages_back_and_eos_stops():
    cache, s = make()
    s.add_request("a", [5, 6, 7], 50)
    run_step(cache, s, eos=9, token=4)
    plan, fin = run_step(cache, s, eos=9, token=9)
    assert fin == ["a"] and cache.n_free_pages() == [16] and not cache.has("a")


def test_park_keeps_pages_and_a_further_turn_continues_from_them():
    cache, s = make(pages=16)
    s.add_request("a", [1, 2, 3, 4, 5], 2)
    run_step(cache, s)
    plan = s.schedule()
    cache.append("a", 1); s.on_step(plan)
    assert s.on_token("a", 1, -1) is True
    s.park("a")
    assert not s.has_work() and cache.has("a") and cache.length("a") == 6
    s.extend_request("a", [7, 8, 9], 2)
    plan, _ = run_step(cache, s)
    assert shape(plan) == [("a", 4, True)] and plan[0].tokens == [1, 7, 8, 9]    # last sampled token + the new turn
    assert cache.length("a") == 10


def test_refusals():
    cache, s = make()
    with pytest.raises(SchedulerError):
        s.add_request("a", [], 3)
    s.add_request("a", [1], 3)
    with pytest.raises(SchedulerError, match="already"):
        s.add_request("a", [1], 3)
    with pytest.raises(SchedulerError):
        Scheduler(cache, 0, 8)


def take(cache, plan):
    for e in plan:
        if not cache.has(e.rid):
            cache.open(e.rid)
        cache.append(e.rid, len(e.tokens))


def test_next_step_is_decided_before_the_last_tokens_are_read():
    """A sampled token that the host has not read stands in the token list as UNREAD; the next
    step feeds it (the engine takes it on the device); on_token fills it in later."""
    cache, s = make()
    s.add_request("a", list(range(6)), 3)
    plan = s.schedule()
    take(cache, plan)
    s.on_step(plan)
    s.on_sampled("a")                                     # step 1 sampled, not read
    nxt = s.schedule(allow_preempt=False)
    assert [(e.rid, e.tokens, e.sample) for e in nxt] == [("a", [UNREAD], True)]
    take(cache, nxt)
    s.on_step(nxt)
    s.on_sampled("a")                                     # step 2 sampled: two unread now
    assert s.seqs["a"].tokens[-2:] == [UNREAD, UNREAD]
    assert s.on_token("a", 41, eos_id=-1) is False        # step 1's token arrives: the older one is filled
    assert s.seqs["a"].tokens[-2:] == [41, UNREAD]
    third = s.schedule(allow_preempt=False)
    take(cache, third)
    s.on_step(third)
    s.on_sampled("a")                                     # the third and last token of the budget
    assert s.schedule(allow_preempt=False) == []          # budget spent: nothing more is planned for it
    assert s.on_token("a", 42, -1) is False and s.on_token("a", 43, -1) is True
    assert s.seqs["a"].tokens[-3:] == [41, 42, 43] and s.seqs["a"].unread == 0
    cache.check_consistency()


def test_a_stop_token_voids_the_token_sampled_after_it():
    cache, s = make()
    s.add_request("a", list(range(5)), 10)
    for _ in range(2):                                    # two steps ahead of the host
        plan = s.schedule(allow_preempt=False)
        take(cache, plan)
        s.on_step(plan)
        s.on_sampled("a")
    assert s.on_token("a", 9, eos_id=9) is True           # the first token was the stop token
    s.park("a")
    s.drop_unread("a")                                    # what was sampled after it never happened
    st = s.seqs["a"]
    assert st.tokens == list(range(5)) + [9] and st.unread == 0 and st.n_generated == 1
    assert st.n_cached == len(st.tokens) == cache.length("a")       # the step that ran too far cached the stop token
    with pytest.raises(SchedulerError, match="no unread"):
        s.drop_unread("a")
    s.extend_request("a", [4, 4], 2)                      # a further turn continues behind the stop token
    plan = s.schedule()
    assert [(e.rid, e.tokens, e.sample) for e in plan] == [("a", [4, 4], True)]


def test_no_preemption_while_tokens_are_unread():
    cache, s = make(pages=4, page=4, max_running=2)       # 16 tokens of cache
    s.add_request("a", list(range(7)), 8)
    s.add_request("b", list(range(7)), 8)
    plan = s.schedule()
    take(cache, plan)
    s.on_step(plan)
    s.on_sampled("a")
    s.on_sampled("b")
    nxt = s.schedule(allow_preempt=False)                 # position 7 of each: still inside their second pages
    assert len(nxt) == 2
    take(cache, nxt)
    s.on_step(nxt)
    s.on_sampled("a")
    s.on_sampled("b")
    assert s.schedule(allow_preempt=False) is None        # position 8 needs a third page each: one must be preempted
    for rid in ("a", "b"):
        s.on_token(rid, 1, -1)
        s.on_token(rid, 1, -1)
    plan = s.schedule()                                   # everything read: now the youngest is preempted
    assert [e.rid for e in plan] == ["a"] and s.n_preemptions == 1


def test_waiting_requests_that_hold_pages_give_them_up_when_nothing_can_run():
    """Two requests finished a turn and kept their pages; both come back for a further turn that no longer fits
    beside the other's pages.  Nothing runs, so nothing above could preempt: the one further back in the queue
    gives its pages up and is recomputed after the first."""
    cache, s = make(pages=6, page=4, max_running=2, budget=64)      # 24 tokens of cache
    for rid in ("a", "b"):
        s.add_request(rid, list(range(9)), 1)                       # 9 + 1 tokens: 3 pages each
    plan = s.schedule()                                             # both prompts in one step
    take(cache, plan)
    s.on_step(plan)
    for rid in ("a", "b"):
        assert s.on_token(rid, 1, -1) is True                       # the one token of the turn
        s.park(rid)                                                 # pages are kept for a further turn
    assert not s.running and cache.n_free_pages() == [0]
    s.extend_request("a", [5] * 6, 2)                               # 10 + 6 + 2 tokens: needs 5 pages, holds 3, none free
    s.extend_request("b", [6] * 6, 2)
    plan = s.schedule()
    assert [e.rid for e in plan] == ["a"] and s.n_preemptions == 1 and not cache.has("b")
    assert s.seqs["b"].n_cached == 0 and s.waiting == ["b"]
    take(cache, plan)
    s.on_step(plan)
    cache.check_consistency()


@pytest.mark.parametrize("seed", range(4))
def test_random_arrivals_and_further_turns_never_stall(seed):
    """Requests of random lengths keep arriving on a small pool with a windowed group; finished ones are released or
    come back for a further turn on their kept pages.  Whenever there is work a step can be decided (somebody gives
    pages up if need be), every request ends, and the accounting stays consistent."""
    import random
    from pulsar_b200.cache import CacheManager, CacheNeed
    rng = random.Random(seed)
    cache = CacheManager([CacheNeed.paged_kv(2, 16), CacheNeed.paged_kv(2, 16, 150)], 8, 160, 12)
    s = Scheduler(cache, 8, 96)
    live, next_id, done = {}, 0, 0
    for _ in range(6000):
        while len(live) < 12 and rng.random() < 0.5:
            s.add_request(next_id, [1] * rng.randint(1, 300), rng.randint(1, 80))
            live[next_id] = 0
            next_id += 1
        if not s.has_work():
            continue
        plan = s.schedule()
        assert plan, (s.waiting, s.running, cache.n_free_pages())
        take(cache, plan)
        s.on_step(plan)
        for e in plan:
            if e.sample and s.on_token(e.rid, rng.choice([9, 1, 2, 3, 4, 5, 6, 7]), 9):
                s.park(e.rid)
                if rng.random() < 0.3 and live[e.rid] < 2:
                    live[e.rid] += 1
                    s.extend_request(e.rid, [2] * rng.randint(1, 20), rng.randint(1, 30))
                else:
                    s.finish(e.rid)
                    del live[e.rid]
                    done += 1
        cache.check_consistency()
    assert done > 100
    for rid in list(live):
        s.finish(rid)
    assert cache.n_free_pages() == [160, 160] and cache.live_requests() == []
