"""The reference's elastic-cache tests (scirust/tests/ccos.rs) as cases over a small cache interface.

Each case restates one reference test (cited) with the reference's seeds, budgets and expectations. It takes a
`make(budget, evict_policy=0, sink_window=0)` factory returning an object with the methods below, so the same
case runs on the oracle's ElasticKvCache restatement (CPU) and on the device pool through the C ABI (GPU).
Where the reference draws keys from `gen_keys` + `LearnedModel::fit` (codec_cache, ccos.rs:467-477) the cases use
oracle-encoded tiles of seeded Gaussian keys: the byte accounting they assert does not depend on the key values.

Interface: insert(tile) -> slot, state(slot), flags(slot), importance(slot), live_bytes(), counts() -> (hot, warm,
cold), nocorr_count(), reclaimed_correction_bytes(), observe_scores(slots, scores, temperature), evict(slot),
enforce_budget() -> bool, score_all(q, q_sign) -> (slots, scores).
"""
import numpy as np

from oracle import pyoracle as ora
from . import helpers as H

F = np.float32
HOT_BYTES, WARM_BYTES, TQ3_CORR_BYTES, MIX3_CORR_BYTES = 128, 96, 16, 14
BIG = 2 ** 62


def assert_invariants(cache, budget):
    """ccos.rs:13-30: h*128 + w*96 - reclaimed == live_bytes <= budget."""
    h, w, _ = cache.counts()
    assert h * HOT_BYTES + w * WARM_BYTES - cache.reclaimed_correction_bytes() == cache.live_bytes()
    assert cache.live_bytes() <= budget


def _scenario_tiles(proj_seed, gen_seed, n, rho=0.3, warm=False):
    z = H.scenario_projection(proj_seed)
    q, toks = H.scenario_generate(gen_seed, n, rho)
    return z, q, [H.scenario_tile(z, t, i, warm) for i, t in enumerate(toks)]


def _codec_cache(make, n, budget, codec):
    cache = make(budget)
    tiles = H.random_tiles(n, codec, seed=7)
    tiles["position"] = np.arange(n, dtype=np.uint32)
    for i in range(n):
        cache.insert(tiles[i:i + 1])
    return cache


def insert_preserves_encoded_warm_state(make):
    """ccos.rs:209-220"""
    _, _, tiles = _scenario_tiles(0xC01D, 0xC01D, 1, warm=True)
    cache = make(BIG)
    slot = cache.insert(tiles[0])
    assert cache.state(slot) == ora.WARM
    assert cache.flags(slot) & ora.FLAG_WARM
    assert cache.live_bytes() == WARM_BYTES


def cold_and_absent_slots_are_never_scored(make):
    """ccos.rs:222-240 (try_score), through score_all"""
    z, q, tiles = _scenario_tiles(0xC01E, 0xC01E, 1)
    q_sign = H.scenario_sign_bits(z, q)
    cache = make(BIG)
    slot = cache.insert(tiles[0])
    slots, scores = cache.score_all(q, q_sign)
    assert list(slots) == [slot] and abs(scores[0] - ora.score_tiles(tiles[0], q, q_sign)[0]) <= 1e-3
    assert cache.evict(slot)
    assert len(cache.score_all(q, q_sign)[0]) == 0


def observe_scores_rejects_invalid_numeric_inputs(make):
    """ccos.rs:242-259"""
    _, _, tiles = _scenario_tiles(0xC01F, 0xC01F, 1)
    cache = make(BIG)
    slot = cache.insert(tiles[0])
    for temperature in (0.0, -1.0, float("nan"), float("inf")):
        cache.observe_scores([slot], [1.0], temperature)
        assert cache.importance(slot) == 0.0
    for score in (float("nan"), float("inf"), float("-inf")):
        cache.observe_scores([slot], [score], 1.0)
        assert cache.importance(slot) == 0.0
    cache.observe_scores([slot, 10 ** 6], [1.0, 5.0], 1.0)  # an absent slot takes no share of the mass (ccos.rs:280-286)
    assert abs(cache.importance(slot) - 1.0) <= 1e-6


def observe_scores_accumulates_importance(make):
    """ccos.rs:263-301"""
    _, _, tiles = _scenario_tiles(31, 32, 4)
    cache = make(BIG)
    slots = [cache.insert(t) for t in tiles]
    scores = [10.0 if s == slots[2] else 0.0 for s in slots]
    cache.observe_scores(slots, scores, 0.5)
    assert abs(sum(cache.importance(s) for s in slots) - 1.0) <= 1e-4
    assert cache.importance(slots[2]) > 0.9 and cache.importance(slots[0]) < 0.1
    cache.observe_scores(slots, scores, 0.5)
    assert cache.importance(slots[2]) > 1.8


def importance_eviction_with_no_sinks_is_pure_h2o(make):
    """ccos.rs:396-463"""
    z = H.scenario_projection(61)
    n = 6
    cache = make(2 * WARM_BYTES, evict_policy=1, sink_window=0)
    slots = []
    for i in range(n):
        _, toks = H.scenario_generate(70 + i, 1, 0.3)
        slots.append(cache.insert(H.scenario_tile(z, toks[0], i)))
        assert slots[i] == i
    cache.observe_scores(slots, [float(n - i) for i in range(n)], 0.25)
    assert abs(sum(cache.importance(s) for s in slots) - 1.0) <= 1e-4
    for i in range(n - 1):
        assert cache.importance(slots[i]) > cache.importance(slots[i + 1])
    cache.enforce_budget()
    assert cache.counts()[2] == n - 2
    assert cache.state(slots[0]) != ora.COLD and cache.state(slots[1]) != ora.COLD
    assert all(cache.state(s) == ora.COLD for s in slots[2:])


def tq3_correction_rung_comes_before_paging(make):
    """ccos.rs:484-497"""
    n = 32
    budget = n * (HOT_BYTES - TQ3_CORR_BYTES)
    cache = _codec_cache(make, n, budget, 4)
    assert cache.live_bytes() == n * HOT_BYTES
    cache.enforce_budget()
    assert_invariants(cache, budget)
    assert cache.counts() == (n, 0, 0)
    assert cache.nocorr_count() == n and cache.live_bytes() == budget


def tq3_single_drop_reclaims_exactly_one_plane(make):
    """ccos.rs:499-509"""
    n = 16
    budget = n * HOT_BYTES - TQ3_CORR_BYTES
    cache = _codec_cache(make, n, budget, 4)
    cache.enforce_budget()
    assert_invariants(cache, budget)
    assert cache.counts() == (n, 0, 0) and cache.nocorr_count() == 1


def tq3_ladder_reaches_warm_after_corrections(make):
    """ccos.rs:511-529"""
    n = 32
    budget = n * 96
    cache = _codec_cache(make, n, budget, 4)
    cache.enforce_budget()
    assert_invariants(cache, budget)
    h, w, c = cache.counts()
    assert c == 0 and h + w == n and w > 0
    assert cache.nocorr_count() == n


def non_tq3_tiles_skip_the_correction_rung(make):
    """ccos.rs:531-548"""
    n = 16
    budget = n * 112
    _, _, tiles = _scenario_tiles(0xB0D, 3, n)
    cache = make(budget)
    for t in tiles:
        cache.insert(t)
    cache.enforce_budget()
    assert_invariants(cache, budget)
    assert cache.nocorr_count() == 0
    h, w, _ = cache.counts()
    assert w > 0 and h + w == n


def tq3_ladder_is_deterministic(make):
    """ccos.rs:550-566"""
    n = 24
    budget = n * 100
    a, b = _codec_cache(make, n, budget, 4), _codec_cache(make, n, budget, 4)
    a.enforce_budget()
    b.enforce_budget()
    assert a.live_bytes() == b.live_bytes()
    assert [(a.state(s), a.flags(s)) for s in range(n)] == [(b.state(s), b.flags(s)) for s in range(n)]


def mix3_correction_rung_reclaims_fourteen_bytes(make):
    """ccos.rs:568-583"""
    n = 32
    budget = n * (HOT_BYTES - MIX3_CORR_BYTES)
    cache = _codec_cache(make, n, budget, 5)
    assert cache.live_bytes() == n * HOT_BYTES
    cache.enforce_budget()
    assert_invariants(cache, budget)
    assert cache.counts() == (n, 0, 0) and cache.nocorr_count() == n
    assert cache.reclaimed_correction_bytes() == n * MIX3_CORR_BYTES and cache.live_bytes() == budget


def mixed_codec_has_no_correction_rung(make):
    """ccos.rs:585-597"""
    n = 16
    budget = n * (HOT_BYTES - MIX3_CORR_BYTES)
    cache = _codec_cache(make, n, budget, 3)
    cache.enforce_budget()
    assert_invariants(cache, budget)
    assert cache.nocorr_count() == 0
    h, w, _ = cache.counts()
    assert w > 0 and h + w == n


CASES = [
    insert_preserves_encoded_warm_state,
    cold_and_absent_slots_are_never_scored,
    observe_scores_rejects_invalid_numeric_inputs,
    observe_scores_accumulates_importance,
    importance_eviction_with_no_sinks_is_pure_h2o,
    tq3_correction_rung_comes_before_paging,
    tq3_single_drop_reclaims_exactly_one_plane,
    tq3_ladder_reaches_warm_after_corrections,
    non_tq3_tiles_skip_the_correction_rung,
    tq3_ladder_is_deterministic,
    mix3_correction_rung_reclaims_fourteen_bytes,
    mixed_codec_has_no_correction_rung,
]
