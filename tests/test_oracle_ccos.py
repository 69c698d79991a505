"""Pins the oracle's ElasticKvCache against the scenarios the reference's
scirust/tests/ccos.rs states in text (expected states are theirs)."""
import numpy as np

from oracle import pyoracle as ora
from tests import helpers as H

HOT_B, WARM_B = 128, 96


def _invariants(c, budget):
    # scirust/tests/ccos.rs:13-30
    assert c.live_bytes() <= budget
    h, w, _ = c.counts()
    assert h * HOT_B + w * WARM_B - c.reclaimed_correction_bytes() == c.live_bytes()


def test_randomised_budget_invariant_and_recycling():
    # scirust/tests/ccos.rs:36-76 (60 of the 300 trials, same construction)
    z = H.scenario_projection(0xB0D)
    for trial in range(60):
        rng = ora.Rng(trial)
        n = 1 + rng.next_u64() % 48
        budget = rng.next_u64() % (n * HOT_B + 1)
        c = ora.Cache(budget, page_policy=trial % 2)
        _, toks = H.scenario_generate(trial + 1, n, 0.3)
        for i, t in enumerate(toks):
            c.insert(H.scenario_tile(z, t, i))
            if rng.next_u64() % 3 == 0:
                c.enforce_budget()
                _invariants(c, budget)
        c.enforce_budget()
        _invariants(c, budget)
        total = sum(c.counts())
        for i, t in enumerate(toks):
            c.insert(H.scenario_tile(z, t, i))
        assert sum(c.counts()) <= total + n


def test_page_out_masks_residual():
    # scirust/tests/ccos.rs:78-100
    z = H.scenario_projection(1)
    q, toks = H.scenario_generate(2, 1, 0.5)
    qs = H.scenario_sign_bits(z, q)
    c = ora.Cache(2**62)
    s = c.insert(H.scenario_tile(z, toks[0], 0))
    hot = c.score_all(q, qs)[1][0]
    c.page_out(s)
    assert c.state(s) == ora.WARM
    warm = c.score_all(q, qs)[1][0]
    ref = ora.score_tiles(H.scenario_tile(z, toks[0], 0, warm=True), q, qs)[0]
    assert abs(warm - ref) <= 1e-4 * (1 + abs(warm)) and hot != warm
    t = c.tile(s)
    assert not t["residual_bitmap"].any() and t["dynamic_lambda"][0] == 0 and t["flags"][0] & 1


def test_evict_recycles_slots_lifo():
    # scirust/tests/ccos.rs:122-134
    z = H.scenario_projection(4)
    _, toks = H.scenario_generate(5, 4, 0.3)
    c = ora.Cache(2**62, page_policy=1)
    s0 = c.insert(H.scenario_tile(z, toks[0], 0))
    c.insert(H.scenario_tile(z, toks[1], 1))
    c.evict(s0)
    assert c.state(s0) == ora.COLD
    s2 = c.insert(H.scenario_tile(z, toks[2], 2))
    assert s2 == s0 and c.state(s2) == ora.HOT


def _fill_rhos(c, z, seed0):
    for i, r in enumerate([0.9, 0.7, 0.5, 0.3, 0.1]):
        _, toks = H.scenario_generate(seed0 + i, 1, r)
        c.insert(H.scenario_tile(z, toks[0], i))


def test_page_out_policies_differ():
    # scirust/tests/ccos.rs:136-165
    z = H.scenario_projection(6)
    budget = 5 * HOT_B - 1
    lo, old = ora.Cache(budget, page_policy=0), ora.Cache(budget, page_policy=1)
    _fill_rhos(lo, z, 100)
    _fill_rhos(old, z, 100)
    lo.enforce_budget()
    old.enforce_budget()
    assert old.state(0) == ora.WARM and old.state(4) == ora.HOT
    assert lo.state(4) == ora.WARM and lo.state(0) == ora.HOT


def test_hybrid_evicts_oldest_not_lowest_impact():
    # scirust/tests/ccos.rs:167-192
    z = H.scenario_projection(11)
    c = ora.Cache(4 * 96)
    _fill_rhos(c, z, 200)
    c.enforce_budget()
    assert c.counts()[2] == 1 and c.state(0) == ora.COLD and c.state(4) == ora.WARM


def test_score_all_skips_cold():
    # scirust/tests/ccos.rs:194-207
    z = H.scenario_projection(7)
    q, toks = H.scenario_generate(8, 6, 0.3)
    qs = H.scenario_sign_bits(z, q)
    c = ora.Cache(2**62, page_policy=1)
    for i, t in enumerate(toks):
        c.insert(H.scenario_tile(z, t, i))
    c.evict(2)
    slots, _ = c.score_all(q, qs)
    assert list(slots) == [0, 1, 3, 4, 5]


def test_informed_eviction_preserves_sinks_and_heavy_hitters():
    # scirust/tests/ccos.rs:308-389: exact expected COLD sets
    z = H.scenario_projection(41)
    budget = 3 * WARM_B
    causal = ora.Cache(budget, evict_policy=0)
    informed = ora.Cache(budget, evict_policy=1, sink_window=2)
    slots = []
    for i in range(8):
        _, toks = H.scenario_generate(50 + i, 1, 0.3)
        causal.insert(H.scenario_tile(z, toks[0], i))
        slots.append(informed.insert(H.scenario_tile(z, toks[0], i)))
    hh = slots[2]
    sc = [10.0 if s == hh else 0.0 for s in slots]
    for _ in range(5):
        informed.observe_scores(slots, sc, 0.5)
    assert informed.importance(hh) > 4.0
    causal.enforce_budget()
    informed.enforce_budget()
    assert causal.live_bytes() <= budget and informed.live_bytes() <= budget
    assert causal.counts()[2] == 5 and informed.counts()[2] == 5
    assert [causal.state(s) for s in (0, 1, 2)] == [ora.COLD] * 3
    assert all(informed.state(s) != ora.COLD for s in (0, 1, 2))
    assert all(informed.state(s) == ora.COLD for s in (3, 4, 5, 6, 7))


def test_tq3_ladder_drops_correction_before_paging():
    # scirust/tests/ccos.rs:484-601: 128 -> 112 -> 96 -> 80 -> 0 for TQ3
    p = H.orthogonal_projection(9, 160)
    m = ora.Model(p, 160, seed=3)
    keys = H.gaussian_keys(10, 4, 160)
    c = ora.Cache(4 * 128 - 1)
    for i in range(4):
        c.insert(m.encode(keys[i], i, codec=4))
    c.enforce_budget()
    assert c.nocorr_count() == 1 and c.counts() == (4, 0, 0) and c.live_bytes() == 4 * 128 - 16
    c2 = ora.Cache(4 * 80)
    for i in range(4):
        c2.insert(m.encode(keys[i], i, codec=4))
    c2.enforce_budget()
    assert c2.counts() == (0, 4, 0) and c2.live_bytes() == 320 and c2.nocorr_count() == 4
    t = c2.tile(0)
    assert not t["latent_kv"][0][48:].any() and t["flags"][0] == (8 | 16 | 1)
