"""The cache manager on the CPU: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from iitj_llm_coopt_b200.cache import CacheError, CacheManager, OutOfPages
from iitj_llm_coopt_b200.config.specs import CacheNeed

FULL = CacheNeed(kind="paged_kv", kv_heads=2, head_dim=16, window=0)
WIN = CacheNeed(kind="paged_kv", kv_heads=1, head_dim=32, window=20)
STATE = CacheNeed(kind="state", state_shape=(8,), state_dtype="float32")


def test_slots_follow_the_table():
    cm = CacheManager([FULL, FULL], page_size=4, num_pages=8, max_requests=4)
    cm.admit("a")
    cm.ensure("a", 6)
    t = cm.table(0, "a")
    assert len(t) == 2 and cm.slots(0, "a", 0, 6) == [t[0] * 4 + i for i in range(4)] + [t[1] * 4, t[1] * 4 + 1]
    cm.advance("a", 6)
    assert cm.num_tokens("a") == 6 and cm.num_free == 6
    cm.ensure("a", 8)            # still two pages
    assert cm.num_free == 6
    assert cm.release("a") == 2 and cm.num_free == 8
    cm.check()


def test_layers_with_equal_needs_share_a_group():
    cm = CacheManager([FULL, WIN, FULL, STATE, CacheNeed()], page_size=8, num_pages=4, max_requests=2)
    assert cm.entry_group[0][0] == cm.entry_group[2][0] != cm.entry_group[1][0]
    assert cm.entry_group[4] == (None, 0)
    assert len(cm.paged) == 2 and len(cm.groups) == 3
    assert cm.view(4) == (None, None)


def test_ensure_allocates_nothing_when_it_fails():
    cm = CacheManager([FULL, WIN], page_size=4, num_pages=3, max_requests=4)
    cm.admit("a")
    cm.ensure("a", 8)
    cm.admit("b")
    with pytest.raises(OutOfPages):
        cm.ensure("b", 8)
    assert cm.table(0, "b") == [] and cm.table(1, "b") == []
    assert not cm.can_fit("b", 8) and cm.can_fit("b", 4) and cm.extra_pages_needed("b", 8) == 2
    cm.check()


def test_double_free_and_unknown_requests_are_errors():
    cm = CacheManager([FULL], page_size=4, num_pages=4, max_requests=2)
    cm.admit("a")
    with pytest.raises(CacheError):
        cm.admit("a")
    cm.release("a")
    with pytest.raises(CacheError):
        cm.release("a")
    with pytest.raises(CacheError):
        cm.ensure("zz", 4)
    cm.admit("b"), cm.admit("c")
    with pytest.raises(CacheError):
        cm.admit("d")            # no state slot left
    with pytest.raises(CacheError):
        cm.groups[0].pool.give(3)


def test_window_pages_are_given_back_while_the_request_lives():
    cm = CacheManager([WIN], page_size=8, num_pages=10, max_requests=2)    # window 20
    cm.admit("a")
    n = 0
    for step in [30, 2, 1, 1, 9, 1, 40, 1]:
        n += step
        cm.ensure("a", n)
        cm.advance("a", n)
        cm.check()
        table = cm.table(0, "a")
        first_visible = max(0, n - 20 + 1)       # oldest key the next query (position n) can see
        for lp, p in enumerate(table):
            wholly_passed = (lp + 1) * 8 <= first_visible
            assert (p < 0) == wholly_passed, (n, lp, table)
        live = [p for p in table if p >= 0]
        assert len(live) <= 20 // 8 + 2
    # far more tokens went through than the pool holds
    assert n > 10 * 8 - 8 and cm.num_free >= 6
    with pytest.raises(CacheError):
        cm.slots(0, "a", 0, 1)                   # that page is gone
    cm.release("a")
    assert cm.num_free == 10
    cm.check()


def test_truncate_gives_back_trailing_pages():
    cm = CacheManager([FULL], page_size=4, num_pages=8, max_requests=2)
    cm.admit("a")
    cm.ensure("a", 14)
    cm.advance("a", 14)
    cm.truncate("a", 5)
    assert cm.num_tokens("a") == 5 and len(cm.table(0, "a")) == 2 and cm.num_free == 6
    cm.check()


def test_state_slots_are_unique_and_reused():
    cm = CacheManager([STATE], page_size=4, num_pages=2, max_requests=3)
    slots = {r: cm.admit(r) for r in "abc"}
    assert sorted(slots.values()) == [0, 1, 2]
    cm.release("b")
    assert cm.admit("d") == slots["b"]
    cm.check()


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2**32 - 1), st.sampled_from([(4, 12), (8, 9), (16, 5)]), st.booleans())
def test_random_orders_never_lose_or_share_a_page(seed, geometry, windowed):
    page, pages = geometry
    needs = [FULL, WIN, FULL] if windowed else [FULL, FULL]
    cm = CacheManager(needs, page_size=page, num_pages=pages, max_requests=4)
    rng = random.Random(seed)
    live, next_id = {}, 0
    for _ in range(200):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            cm.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 5, page, 3 * page])
            try:
                cm.ensure(r, live[r] + grow)
            except OutOfPages:
                before = {g: list(cm.table(g, r)) for g in cm.paged}
                assert before == {g: cm.table(g, r) for g in cm.paged}
                victim = rng.choice(list(live))
                cm.release(victim)
                del live[victim]
            else:
                live[r] += grow
                cm.advance(r, live[r])
        elif live:
            r = rng.choice(list(live))
            cm.release(r)
            del live[r]
        cm.check()
        for g in cm.paged:
            held = sum(1 for r in live for p in cm.table(g, r) if p >= 0)
            assert held + cm.groups[g].pool.num_free == pages
    for r in list(live):
        cm.release(r)
    cm.check()
    assert cm.num_free == pages and len(cm.free_slots) == 4


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2**32 - 1), st.sampled_from([(4, 40, 12), (8, 30, 24), (16, 12, 16)]))
def test_pools_of_their_own_size_and_the_questions_the_scheduler_asks(seed, geometry):
    """A group with a window gets a pool sized for windows and one step's tokens; `can_admit` and `can_grow_all` must
    say exactly what `ensure` then does, group by group, under random orders of requests whose steps stay within
    the declared bound."""
    page, pages, step_tokens = geometry
    needs = [FULL, WIN, FULL]
    cm = CacheManager(needs, page_size=page, num_pages=pages, max_requests=3, max_step_tokens=step_tokens)
    g_full, g_win = cm.entry_group[0][0], cm.entry_group[1][0]
    sizes = {g: cm.groups[g].pool.num_pages for g in cm.paged}
    assert sizes[g_full] == pages
    assert sizes[g_win] == min(pages, 3 * (-(-WIN.window // page) + 2) + -(-step_tokens // page) + 3)
    assert CacheManager.bytes_for(needs, page, pages, 2, 3, step_tokens) == \
        2 * (2 * FULL.kv_heads * FULL.head_dim * page * 2) * (pages + 1) + (2 * WIN.kv_heads * WIN.head_dim * page * 2) * (sizes[g_win] + 1)
    rng = random.Random(seed)
    live, next_id = {}, 0
    for _ in range(150):
        op = rng.random()
        if op < 0.3 and len(live) < 3:
            first = rng.randint(1, step_tokens)
            fits = all(cm.groups[g].pages_for(first) <= cm.groups[g].pool.num_free for g in cm.paged)
            assert cm.can_admit(first) == fits
            if fits:
                cm.admit(next_id)
                cm.ensure(next_id, first)
                cm.advance(next_id, first)
                live[next_id] = first
                next_id += 1
        elif op < 0.85 and live:
            # one step: some of the live requests grow, together by no more than the step's bound
            grow, left = [], step_tokens
            for r in rng.sample(list(live), rng.randint(1, len(live))):
                n = rng.randint(1, max(1, min(left, page + 3)))
                if n > left:
                    break
                grow.append((r, live[r] + n))
                left -= n
            need = {g: sum(cm.groups[g].extra_pages(r, t) for r, t in grow) for g in cm.paged}
            fits = all(need[g] <= cm.groups[g].pool.num_free for g in cm.paged)
            assert cm.can_grow_all(grow) == fits
            if fits:
                for r, t in grow:
                    cm.ensure(r, t)
                for r, t in grow:
                    cm.advance(r, t)
                    live[r] = t
            else:
                victim = rng.choice(list(live))
                cm.release(victim)
                del live[victim]
        elif live:
            r = rng.choice(list(live))
            cm.release(r)
            del live[r]
        cm.check()
        for g in cm.paged:
            held = sum(1 for r in live for p in cm.table(g, r) if p >= 0)
            assert held + cm.groups[g].pool.num_free == sizes[g]
        # the windowed group never holds more than its windows and the last step's tokens
        assert sizes[g_win] - cm.groups[g_win].pool.num_free <= 3 * (-(-WIN.window // page) + 2) + -(-step_tokens // page) + 3
    for r in list(live):
        cm.release(r)
    cm.check()
    assert all(cm.groups[g].pool.num_free == sizes[g] for g in cm.paged)
