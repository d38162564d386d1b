"""The ten tests of crates/qubivex-kv-cache/src/lib.rs:224-364, restated against the library's
prefix index, and a randomized comparison with the Python restatement."""
import numpy as np

from oracle.hostlogic import RefPrefixCache
from qubivex_b200.kvpool import PrefixCache

MIN_REUSE = PrefixCache.MIN_REUSE
N = MIN_REUSE * 2


def run(start, n):
    return list(range(start, start + n))


def reuse(c, scope, prompt):
    hit = c.lookup(scope, prompt)
    if hit is None:
        return None
    value, n, h = hit
    c.release(h)
    return value, n


def test_min_reuse_is_the_references():
    assert MIN_REUSE == 32


def test_the_longest_shared_prefix_wins():
    c = PrefixCache(100)
    long = run(0, N)
    short = long[:N - 4] + [9999]
    assert c.insert(None, short, 1, "short")
    assert c.insert(None, long, 1, "long")
    assert reuse(c, None, long + [7, 8]) == ("long", N)
    other = long[:N - 8] + [1, 2, 3]
    assert reuse(c, None, other)[1] == N - 8


def test_the_last_token_always_runs():
    c = PrefixCache(100)
    t = run(0, N)
    c.insert(None, t, 1, ())
    assert reuse(c, None, t)[1] == N - 1
    assert reuse(c, None, t[:N - 3])[1] == N - 4
    assert c.lookup(None, []) is None


def test_short_matches_are_not_worth_a_copy():
    c = PrefixCache(100)
    assert not c.insert(None, run(0, MIN_REUSE - 1), 1, ())
    assert c.stats().entries == 0
    c.insert(None, run(0, N), 1, ())
    assert c.lookup(None, run(0, MIN_REUSE - 1) + [9999, 9998]) is None
    assert reuse(c, None, run(0, MIN_REUSE) + [9999])[1] == MIN_REUSE


def test_scopes_never_see_each_other():
    c = PrefixCache(100)
    t = run(0, N)
    c.insert("a", t, 1, "a")
    assert c.lookup("b", t) is None
    assert c.lookup(None, t) is None
    assert c.insert("b", t, 1, "b")
    assert c.insert(None, t, 1, "none")
    assert c.stats().entries == 3
    assert reuse(c, "b", t)[0] == "b"
    assert reuse(c, None, t)[0] == "none"


def test_the_budget_holds_and_the_least_recently_used_goes_first():
    c = PrefixCache(3)
    a, b, d = run(0, N), run(1000, N), run(2000, N)
    c.insert(None, a, 1, "a")
    c.insert(None, b, 1, "b")
    c.insert(None, run(3000, N), 1, "c")
    assert reuse(c, None, a) is not None  # touching a leaves b the oldest
    c.insert(None, d, 1, "d")
    assert c.cost() == 3
    assert c.lookup(None, b) is None
    assert reuse(c, None, a) is not None
    assert reuse(c, None, d) is not None
    assert c.insert(None, run(4000, N), 3, "e")
    assert c.stats().entries == 1
    assert c.stats().evicted == 4


def test_a_value_over_budget_is_refused_and_evicts_nothing():
    c = PrefixCache(3)
    a = run(0, N)
    c.insert(None, a, 3, ())
    assert not c.insert(None, run(1000, N), 4, ())
    assert reuse(c, None, a) is not None
    assert c.stats().evicted == 0


def test_a_conversation_holds_one_entry():
    c = PrefixCache(10)
    long = run(0, N + 10)
    assert c.insert(None, long[:N], 2, 1)
    assert c.insert(None, long, 3, 2)
    s = c.stats()
    assert (s.entries, c.cost(), s.evicted) == (1, 3, 0)
    assert not c.insert(None, long[:N], 2, 3)
    assert reuse(c, None, long)[0] == 2
    assert c.insert(None, long[:N] + [9999], 2, 4)
    assert c.stats().entries == 2


def test_a_replaced_value_makes_room_before_anything_older_is_evicted():
    c = PrefixCache(4)
    old, turn = run(1000, N), run(0, N + 4)
    c.insert(None, old, 2, ())
    c.insert(None, turn[:N], 2, ())
    assert c.insert(None, turn, 2, ())
    assert reuse(c, None, old) is not None


def test_a_hit_outlives_its_eviction():
    released = []
    c = PrefixCache(10, on_release=released.append)
    t = run(0, N)
    c.insert(None, t, 1, [1, 2, 3])
    value, n, hit = c.lookup(None, t)
    c.clear()
    assert c.cost() == 0
    assert value == [1, 2, 3] and released == []   # the hit still holds it
    c.release(hit)
    assert released == [[1, 2, 3]]


def test_counters_add_up():
    c = PrefixCache(10)
    t = run(0, N)
    assert c.lookup(None, t) is None
    c.insert(None, t, 2, ())
    assert reuse(c, None, t) is not None
    s = c.stats()
    assert (s.lookups, s.hits, s.tokens_reused, s.inserted) == (2, 1, N - 1, 1)
    c.clear()
    assert c.stats().evicted == 1
    assert not c.evict_oldest()


def test_random_traffic_matches_the_restatement():
    rng = np.random.default_rng(5)
    ref, got = RefPrefixCache(12), PrefixCache(12)
    bases = [run(b * 1000, 200) for b in range(4)]
    for step in range(600):
        scope = [None, "a", "b"][int(rng.integers(0, 3))]
        base = bases[int(rng.integers(0, 4))]
        n = int(rng.integers(20, 120))
        toks = base[:n]
        if rng.random() < 0.3:
            toks = toks + [int(rng.integers(5000, 6000))]
        if rng.random() < 0.5:
            cost = int(rng.integers(1, 6))
            assert ref.insert(scope, toks, cost, step) == got.insert(scope, toks, cost, step)
        elif rng.random() < 0.9:
            r, g = ref.lookup(scope, toks), reuse(got, scope, toks)
            assert (r is None) == (g is None)
            if r is not None:
                assert tuple(r) == tuple(g)
        else:
            assert ref.evict_oldest() == got.evict_oldest()
        s = got.stats()
        assert {k: getattr(s, k) for k in ref.stats} == ref.stats
