"""The scheduler's decisions (no GPU): admission, portions under the token budget, decode
rows, finishing, abort, and what happens when pages run out.  A fake model stands in for
the step: the next token is a function of the request's tokens, so that outputs can be
compared across schedules (after the reference's tests/batching.rs:74-174)."""
import pytest

from dlm_b200.build import load_host


@pytest.fixture(scope="module")
def host():
    return load_host()


def make(host, pages=64, page=16, slots=8, budget=32, rows=8, ctx=512, vocab=100, window=0):
    cache = host.CacheManager([host.GroupSpec(page, window, pages)], slots)
    sched = host.Scheduler(cache, host.SchedulerConfig(budget, rows, ctx, vocab))
    return cache, sched


def fake_next(tokens):
    return (sum(tokens) * 31 + len(tokens)) % 97


def drive(cache, sched, prompts, max_new, eos=(), trace=None):
    """Runs to completion; the 'model' sees each request's full token list (prompt + output)."""
    hist = {i: list(p) for i, p in enumerate(prompts)}
    for i, p in enumerate(prompts):
        sched.submit(i, p, max_new, list(eos))
    results = {}
    guard = 0
    while sched.has_work():
        guard += 1
        assert guard < 10000
        plan = sched.plan()
        if trace is not None:
            trace.append(plan)
        for pid in plan.preempted:
            pass
        sampled = []
        for it in plan.items:
            # the tokens fed must be exactly the request's tokens from `start`
            assert hist[it.id][it.start:it.start + len(it.tokens)] == it.tokens
            assert cache.length(it.slot) == it.start + len(it.tokens)
            if it.sample:
                assert it.start + len(it.tokens) == len(hist[it.id])
                tok = fake_next(hist[it.id])
                hist[it.id].append(tok)
                sampled.append(tok)
        for f in sched.commit(plan, sampled):
            results[f.id] = (f.output, f.reason)
        assert cache.check() == ""
    return results


def alone(prompt, max_new, eos=()):
    toks, out = list(prompt), []
    for _ in range(max_new):
        t = fake_next(toks)
        toks.append(t)
        out.append(t)
        if t in eos:
            break
    return out


def test_batched_equals_isolated(host):
    prompts = [[1, 2, 3], list(range(40)), [5] * 17, [7], list(range(3, 70)), [9, 9]]
    cache, sched = make(host, rows=2, budget=16)            # two rows, as tests/batching.rs:74-101
    res = drive(cache, sched, prompts, 12)
    for i, p in enumerate(prompts):
        assert res[i] == (alone(p, 12), "length")
    st = sched.stats()
    assert st.finished == 6 and st.decode_tokens == 72 and st.prompt_tokens == sum(map(len, prompts))
    assert cache.stats(0).used_pages == 0 and cache.free_slots == 8


def test_budget_rows_and_portions(host):
    cache, sched = make(host, budget=10, rows=3)
    trace = []
    drive(cache, sched, [list(range(25)), list(range(7)), [1, 2, 3, 4]], 3, trace=trace)
    for plan in trace:
        assert sum(len(it.tokens) for it in plan.items) <= 10 and len(plan.items) <= 3
    first = trace[0]
    assert [len(it.tokens) for it in first.items] == [10] and not first.items[0].sample     # FIFO: oldest first
    second = trace[1]                                          # portions vary: 10 more of request 0
    assert [(it.id, len(it.tokens)) for it in second.items] == [(0, 10)]
    third = trace[2]                                           # the last 5, then room for request 1's 5 first tokens
    assert [(it.id, len(it.tokens), it.sample) for it in third.items] == [(0, 5, True), (1, 5, False)]
    fourth = trace[3]                                          # decode row first, then prompts
    assert fourth.items[0].id == 0 and len(fourth.items[0].tokens) == 1 and fourth.items[0].sample
    assert [(it.id, len(it.tokens)) for it in fourth.items[1:]] == [(1, 2), (2, 4)]


def test_eos_is_emitted_and_stops(host):
    p = [4, 4, 4]
    full = alone(p, 20)
    eos = full[5]
    cache, sched = make(host)
    res = drive(cache, sched, [p], 20, eos=[eos])
    out, reason = res[0]
    assert reason == "eos" and out == full[:full.index(eos) + 1]      # src/batching.rs:353-360


def test_submit_refusals_and_zero_tokens(host):
    cache, sched = make(host, ctx=20, vocab=50)
    with pytest.raises(ValueError, match="empty"):
        sched.submit(0, [], 4, [])                            # src/batching.rs:248-250
    with pytest.raises(ValueError, match="vocabulary"):
        sched.submit(0, [1, 50], 4, [])                       # src/generate.rs:317-322
    with pytest.raises(ValueError, match="no room"):
        sched.submit(0, [1] * 20, 4, [])                      # src/server/engine.rs:725-735
    sched.submit(1, [1, 2], 0, [])                            # src/batching.rs:287-290
    fin = sched.drain_finished()
    assert [(f.id, f.output, f.reason) for f in fin] == [(1, [], "length")] and not sched.has_work()
    sched.submit(2, [1] * 15, 100, [])                        # clamped to what the context leaves
    with pytest.raises(ValueError, match="in use"):
        sched.submit(2, [1], 1, [])
    res = drive_existing(cache, sched, {2: [1] * 15})
    assert len(res[2][0]) == 5


def drive_existing(cache, sched, hist):
    results = {}
    while sched.has_work():
        plan = sched.plan()
        sampled = []
        for it in plan.items:
            if it.sample:
                tok = fake_next(hist[it.id])
                hist[it.id].append(tok)
                sampled.append(tok)
        for f in sched.commit(plan, sampled):
            results[f.id] = (f.output, f.reason)
    return results


def test_abort(host):
    cache, sched = make(host)
    sched.submit(0, [1, 2, 3], 50, [])
    sched.submit(1, [4, 5], 50, [])
    hist = {0: [1, 2, 3], 1: [4, 5]}
    for _ in range(3):
        plan = sched.plan()
        sampled = []
        for it in plan.items:
            if it.sample:
                tok = fake_next(hist[it.id]); hist[it.id].append(tok); sampled.append(tok)
        sched.commit(plan, sampled)
    assert sched.abort(0) and not sched.abort(0) and not sched.abort(42)      # src/batching.rs:264-269
    fin = sched.drain_finished()
    assert [(f.id, f.reason, len(f.output)) for f in fin] == [(0, "abort", 3)]
    assert cache.free_slots == 7 and cache.check() == ""
    res = drive_existing(cache, sched, hist)
    assert res[1][1] == "length" and len(res[1][0]) == 50


def test_preemption_when_pages_run_out(host):
    """Four requests whose final lengths need 20 pages in a pool of 10: the youngest running
    request is sent back and recomputed; every output equals the isolated one."""
    prompts = [[i + 1] * 30 for i in range(4)]
    cache, sched = make(host, pages=10, budget=64, rows=4)
    trace = []
    res = drive(cache, sched, prompts, 40, trace=trace)
    for i, p in enumerate(prompts):
        assert res[i] == (alone(p, 40), "length")
    assert sched.stats().preemptions > 0
    pre = [p for plan in trace for p in plan.preempted]
    assert pre and 0 not in pre                                # the oldest request is never the victim
    # a pre-empted request starts over from position 0 with all its tokens so far
    seen_restart = False
    for plan in trace:
        for it in plan.items:
            if it.id in pre and it.start == 0 and len(it.tokens) > 30:
                seen_restart = True
    assert seen_restart


def test_a_prompt_waits_until_all_of_it_fits(host):
    """Beside a running request a prompt is admitted only when the free pages hold all of it (it would get a
    first portion and lose it again otherwise); alone it is admitted whatever its length."""
    # pool of 10 pages of 16 tokens; request 0: prompt of 64 tokens (4 pages), decodes 40 more (up to 7 pages);
    # request 1: prompt of 100 tokens = 7 pages, which do not fit beside request 0's 4 + 1 spare
    cache, sched = make(host, pages=10, budget=32, rows=4)
    trace = []
    res = drive(cache, sched, [[3] * 64, [5] * 100], 40, trace=trace)
    assert res[0] == (alone([3] * 64, 40), "length") and res[1] == (alone([5] * 100, 40), "length")
    assert sched.stats().preemptions == 0
    first_of_1 = next(i for i, plan in enumerate(trace) if any(it.id == 1 for it in plan.items))
    last_of_0 = max(i for i, plan in enumerate(trace) if any(it.id == 0 for it in plan.items))
    assert first_of_1 > last_of_0                    # request 1 started only when request 0 had left
    # a prompt that does fit whole is admitted beside the running request, portion by portion
    cache2, sched2 = make(host, pages=16, budget=32, rows=4)
    trace2 = []
    res2 = drive(cache2, sched2, [[3] * 64, [5] * 100], 40, trace=trace2)
    assert res2[0] == (alone([3] * 64, 40), "length") and res2[1] == (alone([5] * 100, 40), "length")
    assert any(len({it.id for it in plan.items}) == 2 for plan in trace2)


def test_request_that_can_never_fit_fails_alone(host):
    cache, sched = make(host, pages=2, budget=64)
    res = drive(cache, sched, [[1] * 20, [2] * 10], 30)
    # request 0 needs 50 tokens = 4 pages of a pool of 2: it ends with reason "cache" once it is alone;
    # request 1 (40 tokens = 3 pages) cannot fit either
    assert res[0][1] == "cache" and res[1][1] == "cache"
    assert len(res[0][0]) > 0                                   # it produced what the pool allowed
    assert cache.check() == "" and cache.stats(0).used_pages == 0
    cache2, sched2 = make(host, pages=3, budget=64)
    res2 = drive(cache2, sched2, [[1] * 20, [2] * 10], 30)
    assert res2[1] == (alone([2] * 10, 30), "length") and res2[0][1] == "cache"


def test_windowed_group_lets_long_requests_run_in_few_pages(host):
    cache, sched = make(host, pages=4, window=16, budget=16, ctx=2048)
    res = drive(cache, sched, [[3] * 40], 300)
    assert res[0] == (alone([3] * 40, 300), "length")
    assert cache.stats(0).high_water <= 3
