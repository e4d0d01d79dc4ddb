"""The cache manager's bookkeeping (no GPU): sizing, lazy growth, reuse, atomic failure,
windows, state slots; and under random orders of requests no page is lost, held twice or
freed twice.  Hand-derivable cases restate the reference's (src/cache/paged.rs:244-334)."""
import random

import pytest

from dlm_b200.build import load_host


@pytest.fixture(scope="module")
def host():
    return load_host()


def mgr(host, pages=8, page=16, window=0, slots=4, groups=None):
    specs = groups or [(page, window, pages)]
    return host.CacheManager([host.GroupSpec(p, w, n) for p, w, n in specs], slots)


def test_lazy_growth_and_low_ids_first(host):
    m = mgr(host)
    s = m.open()
    m.append([(s, 16)])                     # src/cache/paged.rs:270-282: 16 tokens fit one page,
    assert m.table(s, 0) == [0]
    m.append([(s, 1)])                      # the 17th takes a second
    assert m.table(s, 0) == [0, 1] and m.length(s) == 17
    assert m.stats(0).used_pages == 2 and m.stats(0).free_pages == 6


def test_free_gives_everything_back_and_pages_are_used_again(host):
    m = mgr(host, pages=4)
    a = m.open()
    m.append([(a, 64)])
    assert m.stats(0).free_pages == 0
    m.close(a)                              # src/cache/paged.rs:286-295
    assert m.stats(0).free_pages == 4
    b = m.open()
    m.append([(b, 20)])
    assert len(m.table(b, 0)) == 2 and set(m.table(b, 0)) <= {0, 1, 2, 3}
    assert m.check() == ""


def test_exhaustion_is_atomic(host):
    m = mgr(host, pages=3)                  # src/cache/paged.rs:299-314: 3 pages, ask for more
    a, b = m.open(), m.open()
    m.append([(a, 16)])
    with pytest.raises(host.CacheExhausted) as ei:
        m.append([(a, 16), (b, 33)])        # needs 1 + 3 pages, 2 are free
    assert "requested 4" in str(ei.value) and "2 free of 3" in str(ei.value)
    assert m.length(a) == 16 and m.length(b) == 0 and m.table(b, 0) == [] and m.stats(0).free_pages == 2
    assert not m.can_append([(a, 16), (b, 33)]) and m.can_append([(a, 16), (b, 16)])
    assert m.max_appendable(b, 100) == 32 and m.max_appendable(b, 100, reserve=1) == 16
    assert m.check() == ""


def test_window_gives_pages_back_while_the_request_runs(host):
    m = mgr(host, pages=4, page=16, window=16)
    s = m.open()
    m.append([(s, 40)])                     # a 40-token portion needs pages 0..2 at once
    assert m.table(s, 0) == [0, 1, 2]
    m.append([(s, 1)])                      # next query at 40 sees keys 25..40: page 0 has passed
    assert m.table(s, 0) == [-1, 1, 2] and m.stats(0).free_pages == 2
    for _ in range(200):                    # decoding never needs more than two live pages
        m.append([(s, 1)])
        assert m.stats(0).used_pages <= 2 and m.check() == ""
    assert m.length(s) == 241 and m.stats(0).high_water == 3
    m.close(s)
    assert m.stats(0).free_pages == 4 and m.check() == ""


def test_groups_have_pools_of_their_own(host):
    m = mgr(host, groups=[(16, 0, 8), (16, 16, 3)], slots=2)
    s = m.open()
    m.append([(s, 33)])
    assert m.table(s, 0) == [0, 1, 2] and m.table(s, 1) == [0, 1, 2]
    for _ in range(60):
        m.append([(s, 1)])
    assert m.stats(0).used_pages == 6 and m.stats(1).used_pages <= 2
    with pytest.raises(host.CacheExhausted):
        m.append([(s, 100)])                # the full group cannot hold it; nothing changes in either
    assert m.length(s) == 93 and m.check() == ""


def test_state_slots(host):
    m = mgr(host, slots=2)
    a, b = m.open(), m.open()
    assert {a, b} == {0, 1} and m.open() == -1 and m.free_slots == 0
    m.close(a)
    assert m.open() == a
    with pytest.raises(ValueError):
        m.close(5)
    with pytest.raises(ValueError):
        m.length(5)


def test_step_metadata(host):
    import numpy as np
    m = mgr(host, pages=8, page=4)
    a, b = m.open(), m.open()
    m.append([(a, 6)])
    m.append([(a, 1), (b, 3)])
    items = [host.StepItem(a, [9], [0]), host.StepItem(b, [5, 6, 7], [0, 2])]
    lay = m.plan_layout(items)
    buf = np.zeros(lay.total, dtype=np.int32)
    m.pack(items, lay, buf.ctypes.data, buf.size)
    assert (lay.num_tokens, lay.num_requests, lay.num_wanted, lay.max_q_len, lay.max_kv_len) == (4, 2, 3, 3, 7)
    sl = lambda off, n: buf[off:off + n].tolist()
    assert sl(lay.off_tokens, 4) == [9, 5, 6, 7] and sl(lay.off_positions, 4) == [6, 0, 1, 2]
    assert sl(lay.off_token_req, 4) == [0, 1, 1, 1] and sl(lay.off_cu_q, 3) == [0, 1, 4]
    assert sl(lay.off_kv_len, 2) == [7, 3] and sl(lay.off_logit_rows, 3) == [0, 1, 3]
    ta, tb = m.table(a, 0), m.table(b, 0)
    assert sl(lay.off_slots[0], 4) == [ta[1] * 4 + 2, tb[0] * 4, tb[0] * 4 + 1, tb[0] * 4 + 2]
    w = lay.table_width[0]
    assert sl(lay.off_table[0], w)[:2] == ta and sl(lay.off_table[0] + w, w)[0] == tb[0]
    with pytest.raises(ValueError):
        m.plan_layout([host.StepItem(a, [1] * 9, [])])       # more tokens than the request holds


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [0, 24])
def test_random_orders_lose_no_page(host, seed, window):
    rng = random.Random(seed)
    m = mgr(host, groups=[(16, 0, 24), (16, window, 24)] if window else [(16, 0, 24)], slots=5)
    live = {}
    for step in range(600):
        r = rng.random()
        if r < 0.15 and len(live) < 5:
            s = m.open()
            assert s >= 0 and s not in live
            live[s] = 0
        elif r < 0.25 and live:
            s = rng.choice(list(live))
            m.close(s)
            del live[s]
            with pytest.raises(ValueError):
                m.close(s)                                  # a second close is refused, nothing is freed twice
        elif live:
            group = rng.sample(list(live), k=min(len(live), rng.randint(1, 3)))
            ask = [(s, rng.choice([1, 1, 1, 2, 7, 16, 40])) for s in group]
            before = {s: (m.length(s), [list(m.table(s, g)) for g in range(m.num_groups)]) for s in live}
            free_before = [m.free_pages(g) for g in range(m.num_groups)]
            try:
                m.append(ask)
                for s, n in ask:
                    live[s] += n
            except host.CacheExhausted:
                assert {s: (m.length(s), [list(m.table(s, g)) for g in range(m.num_groups)]) for s in live} == before
                assert [m.free_pages(g) for g in range(m.num_groups)] == free_before
        assert m.check() == ""
        for s, n in live.items():
            assert m.length(s) == n
            assert len(m.table(s, 0)) == -(-n // 16) and all(p >= 0 for p in m.table(s, 0))
            if window and n:
                t = m.table(s, 1)
                first_needed = max(0, n - window) // 16     # pages the last token's window still touches
                assert all(p >= 0 for p in t[first_needed:])
    for s in list(live):
        m.close(s)
    assert m.check() == "" and all(m.stats(g).used_pages == 0 for g in range(m.num_groups))


def test_padded_rows_belong_to_nobody():
    """A layout with more rows than requests: the extra rows bring one token each, hold one key on the sink
    page (the page after the pool's last), use the sink state slot and want their logits; the real rows
    are packed as without padding."""
    import numpy as np
    host = load_host()
    m = host.CacheManager([host.GroupSpec(16, 0, 10), host.GroupSpec(16, 24, 6)], 4)
    a, b = m.open(), m.open()
    m.append([(a, 40), (b, 3)])
    m.append([(a, 1), (b, 1)])
    items = [host.StepItem(a, [7], [0]), host.StepItem(b, [9], [0])]
    plain = m.plan_layout(items, 8)
    lay = m.plan_layout(items, 8, 4)
    assert (lay.num_requests, lay.num_tokens, lay.num_wanted, lay.num_single) == (4, 4, 4, 4)
    buf = np.zeros(lay.total, dtype=np.int32)
    m.pack(items, lay, buf.ctypes.data, buf.size)
    ref = np.zeros(plain.total, dtype=np.int32)
    m.pack(items, plain, ref.ctypes.data, ref.size)

    def part(l, arr, off, n):
        return arr[off:off + n].tolist()
    assert part(lay, buf, lay.off_tokens, 4) == [7, 9, 0, 0]
    assert part(lay, buf, lay.off_positions, 4) == [40, 3, 0, 0]
    assert part(lay, buf, lay.off_cu_q, 5) == [0, 1, 2, 3, 4]
    assert part(lay, buf, lay.off_kv_len, 4) == [41, 4, 1, 1]
    assert part(lay, buf, lay.off_state_slot, 4) == [a, b, 4, 4]
    assert part(lay, buf, lay.off_logit_rows, 4) == [0, 1, 2, 3]
    for g, (pages, ps) in enumerate([(10, 16), (6, 16)]):
        assert part(lay, buf, lay.off_slots[g], 2) == part(plain, ref, plain.off_slots[g], 2)
        assert part(lay, buf, lay.off_slots[g] + 2, 2) == [pages * ps, pages * ps]
        w = lay.table_width[g]
        rows = buf[lay.off_table[g]:lay.off_table[g] + 4 * w].reshape(4, w)
        assert rows[:2].tolist() == ref[plain.off_table[g]:plain.off_table[g] + 2 * w].reshape(2, w).tolist()
        assert rows[2].tolist() == [pages] + [-1] * (w - 1) and rows[3].tolist() == rows[2].tolist()
    assert m.check() == ""
    # a pure decode step packed from two arrays gives the same words, and refuses what the layout cannot hold
    fast = np.full(lay.total, -7, dtype=np.int32)
    m.pack_decode([a, b], [7, 9], lay, fast.ctypes.data, fast.size)
    assert fast.tolist() == buf.tolist()
    assert m.max_length([a, b]) == 41 and m.max_length([b]) == 4
    with pytest.raises(ValueError):
        m.pack_decode([a, b], [7], lay, fast.ctypes.data, fast.size)
    narrow = m.plan_layout(items, 0, 4)
    assert narrow.table_width[0] == 4
    c = m.open()
    for _ in range(4):
        m.append([(c, 20)])                    # 80 tokens in portions (the windowed group gives pages back):
    with pytest.raises(ValueError):            # five pages, wider than the layout planned without it (four)
        m.pack_decode([a, c], [7, 9], narrow, fast.ctypes.data, fast.size)
    with pytest.raises(ValueError):
        m.pack_decode([a, b], [7, 9], lay, fast.ctypes.data, 3)


def test_row_buckets():
    from dlm_b200.engine.engine import _row_bucket
    assert sorted({_row_bucket(r, 64) for r in range(1, 65)}) == [1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64]
    assert [_row_bucket(r, 64) for r in (1, 5, 7, 9, 33, 49, 64)] == [1, 6, 8, 12, 48, 64, 64]
    assert _row_bucket(5, 5) == 5 and _row_bucket(40, 40) == 40
