"""Device-resident CCOS pool vs the oracle's ElasticKvCache: same slots, states,
tile bytes and byte accounting after the same sequence of operations."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def assert_same(pool, cache, importance_tol=0.0):
    st = pool.stats()
    h, w, c = cache.counts()
    assert (st["len"], st["live_bytes"], st["hot"], st["warm"], st["cold"]) == (len(cache), cache.live_bytes(), h, w, c)
    assert st["nocorr"] == cache.nocorr_count() and st["reclaimed_correction_bytes"] == cache.reclaimed_correction_bytes()
    tiles, state, imp, seq = pool.read()
    assert np.array_equal(state, cache.states())
    live = state != ora.COLD
    want = cache.tiles()
    if len(want):
        assert tiles[live].tobytes() == want[live].tobytes()
    wi = np.array([cache.importance(s) for s in range(len(cache))], F)
    assert np.all(np.abs(imp[live] - wi[live]) <= importance_tol)
    assert np.array_equal(seq[live], np.array([cache.seq(s) for s in range(len(cache))], np.uint64)[live])


def test_insert_page_drop_evict_and_lifo_reuse():
    tiles = H.random_tiles(40, 4, seed=1, warm_every=6)
    pool, cache = S.TilePool(64, 2**40), ora.Cache(2**40)
    slots = pool.insert(tiles)
    assert list(slots) == [cache.insert(tiles[i:i + 1]) for i in range(40)]
    for s in (3, 9, 3):
        pool.page_out(s)
        cache.page_out(s)
    for s in (3, 4, 4, 12):
        assert pool.drop_correction(s) == cache.drop_correction(s)
    for s in (7, 2, 30, 7):
        assert pool.evict(s) == cache.evict(s)
    assert_same(pool, cache)
    more = H.random_tiles(5, 4, seed=2)
    assert list(pool.insert(more)) == [cache.insert(more[i:i + 1]) for i in range(5)]  # 30, 2, 7 then fresh slots
    assert_same(pool, cache)


@pytest.mark.parametrize("host_phases", [False, True], indirect=True)
@pytest.mark.parametrize("trial", range(24))
def test_randomised_enforce_budget_matches_oracle(trial, host_phases):
    # construction of scirust/tests/ccos.rs:36-76 with codecs and policies varied
    rng = ora.Rng(1000 + trial)
    n = 1 + rng.next_u64() % 200
    codec = [1, 4, 5, 3][trial % 4]
    budget = rng.next_u64() % (n * 128 + 1)
    page, evict = trial % 2, (trial // 2) % 2
    sink = 3 if evict else 0
    recent = 5 if trial % 8 == 7 else 0
    pool = S.TilePool(2 * n + 8, budget, page, evict, sink, recent)
    cache = ora.Cache(budget, page, evict, sink, recent)
    tiles = H.random_tiles(n, codec, seed=trial)
    tiles["position"] = np.arange(n)
    i = 0
    while i < n:
        b = 1 + rng.next_u64() % 9
        chunk = tiles[i:i + b]
        assert list(pool.insert(chunk)) == [cache.insert(chunk[j:j + 1]) for j in range(len(chunk))]
        i += len(chunk)
        if evict and rng.next_u64() % 2 == 0:
            live = np.nonzero(cache.states() != ora.COLD)[0].astype(np.uint32)
            sc = ora.Rng(i).gaussian(len(live)) * 3
            pool.observe_scores(live, sc, 0.7)
            cache.observe_scores(live, sc, 0.7)
        if rng.next_u64() % 3 == 0:
            assert pool.enforce_budget() == cache.enforce_budget()
            assert_same(pool, cache, 1e-5)
    assert pool.enforce_budget() == cache.enforce_budget()
    assert pool.live_bytes() <= budget
    assert_same(pool, cache, 1e-5)
    again = tiles[: min(n, 20)]
    assert list(pool.insert(again)) == [cache.insert(again[j:j + 1]) for j in range(len(again))]
    assert_same(pool, cache, 1e-5)


def test_reference_sink_and_heavy_hitter_scenario():
    # scirust/tests/ccos.rs:308-389
    z = H.scenario_projection(41)
    pool = S.TilePool(16, 3 * 96, evict_policy=S.EVICT_IMPORTANCE, sink_window=2)
    slots = []
    for i in range(8):
        _, toks = H.scenario_generate(50 + i, 1, 0.3)
        slots.append(int(pool.insert(H.scenario_tile(z, toks[0], i))[0]))
    sc = np.array([10.0 if s == slots[2] else 0.0 for s in slots], F)
    for _ in range(5):
        pool.observe_scores(np.array(slots, np.uint32), sc, 0.5)
    assert pool.read()[2][slots[2]] > 4.0
    assert pool.enforce_budget()
    state = pool.read()[1]
    assert all(state[s] != ora.COLD for s in (0, 1, 2)) and all(state[s] == ora.COLD for s in (3, 4, 5, 6, 7))


def test_score_all_topk_and_observe_query_skip_cold():
    n = 3000
    tiles = H.random_tiles(n, 3, seed=8)
    pool, cache = S.TilePool(n, 2**40), ora.Cache(2**40)
    pool.insert(tiles)
    for i in range(n):
        cache.insert(tiles[i:i + 1])
    for s in range(0, n, 3):
        pool.evict(s), cache.evict(s)
    for s in range(1, n, 7):
        pool.page_out(s), cache.page_out(s)
    qc, qs = H.random_queries(2, 9)
    gs, gv = pool.score_all(qc[0], qs[0])
    ws, wv = cache.score_all(qc[0], qs[0])
    assert np.array_equal(gs, ws) and np.all(np.abs(gv - wv) <= 1e-3)
    ti, tv, tc = pool.score_topk(qc, qs, 2, 50)
    for j in range(2):
        s_, v_ = cache.score_all(qc[j], qs[j])
        oi, ov = ora.topk(v_, 50)
        assert tc[j] == 50 and np.all(np.abs(tv[j] - ov) <= 1e-3)
        assert len(set(ti[j]) - set(s_)) == 0
    pool.observe_query(qc[0], qs[0], 2.0)
    cache.observe_scores(ws, wv, 2.0)
    assert_same(pool, cache, 1e-5)


def test_append_keys_encodes_into_the_pool():
    om, p = H.make_model_pair(128, seed=3)
    gm = S.Model.from_projection(p, 128, 3)
    keys = H.gaussian_keys(4, 100, 128)
    pool, cache = S.TilePool(128, 60 * 128, evict_policy=S.EVICT_CAUSAL), ora.Cache(60 * 128)
    heads = (np.arange(100) % 8).astype(np.uint16)
    slots = pool.append_keys(gm, keys, S.CODEC_MIXED, position_base=10, head_ids=heads)
    want = om.encode_batch(keys, 3, pos=np.arange(10, 110, dtype=np.uint32), head=heads)
    assert list(slots) == [cache.insert(want[i:i + 1]) for i in range(100)]
    assert_same(pool, cache)
    assert pool.enforce_budget() == cache.enforce_budget()
    assert_same(pool, cache)
    with pytest.raises(S.SlhaError) as e:
        pool.append_keys(gm, np.tile(keys, (2, 1)), S.CODEC_MIXED)
    assert e.value.code == S.ERR_CAPACITY


@pytest.fixture
def host_phases(request):
    """With the parameter set, enforce_budget runs its phases one by one from the host (the path an attached
    event log or an unbounded phase takes) instead of in the single cooperative launch."""
    if request.param:
        S.debug_force_generic_score(True)
    yield request.param
    S.debug_force_generic_score(False)


@pytest.mark.parametrize("host_phases", [False, True], indirect=True)
@pytest.mark.parametrize("codec,page,evict", [(4, 0, 1), (3, 1, 1), (1, 1, 0)])
def test_large_pool_enforce_budget_with_long_candidate_lists(codec, page, evict, host_phases):
    # phases with tens of thousands of candidates: the pool compacts them and sorts only those that can
    # be reached before the deficit is covered; states, free-list order (slot reuse) and byte accounting
    # must still equal the oracle's full ordered walk.  First a large deficit (everything is paged, many
    # tiles evicted), then small deficits after a few more inserts (a handful of operations per phase).
    n = 90000
    budget = int(0.6 * 128 * n)
    pool = S.TilePool(n + 512, budget, page, evict, 4 * evict, 64 * evict)
    cache = ora.Cache(budget, page, evict, 4 * evict, 64 * evict)
    tiles = H.random_tiles(n + 256, codec, seed=77 + codec)
    tiles["position"] = np.arange(n + 256)
    for b in range(0, n, 30000):
        chunk = tiles[b:b + 30000]
        assert list(pool.insert(chunk)) == [cache.insert(chunk[j:j + 1]) for j in range(len(chunk))]
    live = np.arange(n, dtype=np.uint32)
    sc = ora.Rng(5).gaussian(n) * 4
    pool.observe_scores(live, sc, 0.9)
    cache.observe_scores(live, sc, 0.9)
    assert pool.enforce_budget() == cache.enforce_budget()
    assert_same(pool, cache, 1e-3)  # (the oracle sums 90 000 softmax terms sequentially in f32, the pool in a tree)
    for r in range(4):
        more = tiles[n + 64 * r:n + 64 * (r + 1)]
        assert list(pool.insert(more)) == [cache.insert(more[j:j + 1]) for j in range(64)]  # reuses evicted slots in LIFO order
        assert pool.enforce_budget() == cache.enforce_budget()
        assert pool.live_bytes() <= budget
    assert_same(pool, cache, 1e-3)  # (the oracle sums 90 000 softmax terms sequentially in f32, the pool in a tree)


def test_scoring_a_pool_whose_oldest_slots_are_cold_stays_on_the_tensor_core_kernel():
    # One long stream scored by every CTA, with nothing to score at its start (the oldest third of the slots is COLD):
    # the first thresholds must still form early, otherwise the rows' candidate buffers overflow and the rows are handed
    # to the generic kernel (correct, but several times slower) -- the statistics call shows which happened.
    n, k = 300000, 64
    base = H.random_tiles(5000, 3, seed=55)
    tiles = np.tile(base, n // 5000)
    tiles["dynamic_lambda"] *= (1 + np.random.default_rng(2).random(n)).astype(F)
    pool = S.TilePool(n, 2**40, S.PAGE_OLDEST_FIRST, S.EVICT_CAUSAL)
    for b in range(0, n, 50000):
        pool.insert(tiles[b:b + 50000])
    pool.set_budget(96 * (n - 100000))
    assert pool.enforce_budget()  # every tile is paged out (96 live bytes each), then causal eviction takes exactly the oldest 100000
    now, state = pool.read()[:2]
    assert np.all(state[:100000] == ora.COLD) and np.all(state[100000:] == ora.WARM)
    qc, qs = H.random_queries(4, 56)
    ti, tv, tc = pool.score_topk(qc, qs, 4, k)
    stats = S.last_score_stats()
    assert stats["rows_handed_to_generic_kernel"] == 0, stats
    assert stats["candidates_appended"] < 4 * 100000, stats  # (the first, unfiltered round of 148 CTAs x 24 warps alone brings 57 000 per row)
    for j in range(4):
        want = ora.score_tiles(now[100000:], qc[j], qs[j])
        oi, ov = ora.topk(want, k)
        assert tc[j] == k and np.all(np.abs(tv[j] - ov) <= 1e-3)
        assert np.all(ti[j] >= 100000)
