"""The reference's codec unit tests, run on the oracle with the reference's seeds and thresholds.

Every test restates one test of scirust/src/attention/slha_v2/tests.rs (named in its docstring) on inputs
drawn from the oracle's restatement of scirust/src/rng.rs, so an oracle quantiser or decoder that departs
from the reference's fails the reference's own bounds.
"""
import numpy as np
import pytest

from oracle import pyoracle as ora
from . import reference_fixtures as rf

F = np.float32


def _eff(scale, gs, g):
    return F(F(scale) * F(F(gs[g]) / F(255.0)))


def test_int4_dequant_round_trips_signed_values():
    """tests.rs:48-74"""
    v = rf.signed_ramp()
    latent, scale, _ = ora.quantize(v, rf.INT4)
    dq = ora.dequant(ora.make_tile(latent, scale, np.full(8, 255, np.uint8)))
    assert (dq < 0).any()
    assert (np.abs(dq - v) <= scale + 1e-6).all()


def test_grouped_int4_beats_single_on_spread_variance():
    """tests.rs:76-101"""
    rng = ora.Rng(5)
    v = np.zeros(128, F)
    for g in range(8):
        amp = F(10.0) ** -g
        for d in range(g * 16, (g + 1) * 16):
            v[d] = F(F(amp) * F(rng.next_gaussian()))
    latent, scale, _ = ora.quantize(v, rf.INT4)
    e_single = rf.sq_err(ora.make_tile(latent, scale, np.full(8, 255, np.uint8)), v)
    e_grouped = rf.sq_err(rf.tile_of(v, rf.GROUPED)[0], v)
    assert e_grouped < e_single * 0.5


def test_nf4_beats_uniform_int4_on_gaussian_latent():
    """tests.rs:103-129"""
    v = rf.gaussian_latent(8)
    assert rf.sq_err(rf.tile_of(v, rf.NF4)[0], v) < rf.sq_err(rf.tile_of(v, rf.GROUPED)[0], v)


@pytest.mark.parametrize("codec,seed", [(rf.MIXED, 11), (rf.MIX3, 41)])
def test_mixed_and_mix3_dequant_roundtrip_and_drop_tail(codec, seed):
    """tests.rs:143-175 (mixed), :386-420 (mix3)"""
    v = rf.steep_latent(seed)
    tile, scale, gs = rf.tile_of(v, codec)
    dq = ora.dequant(tile)
    assert (np.abs(dq[:8] - v[:8]) <= _eff(scale, gs, 0) + 1e-6).all()
    for d in range(rf.MIXED_HI_DIMS, rf.MIXED_DIMS):
        g = 1 + (d - rf.MIXED_HI_DIMS) // rf.GROUP_DIM
        assert abs(dq[d] - v[d]) <= _eff(scale, gs, g) + 1e-6, d
    assert (dq[rf.MIXED_DIMS:] == 0.0).all()


def test_mixed_beats_uniform_int4_on_steep_spectrum():
    """tests.rs:177-204"""
    for seed in range(8):
        v = rf.steep_latent(100 + seed)
        assert rf.sq_err(rf.tile_of(v, rf.MIXED)[0], v) < rf.sq_err(rf.tile_of(v, rf.GROUPED)[0], v) * 0.5, seed


def test_tq3_dequant_roundtrips_within_quarter_step():
    """tests.rs:206-235"""
    rng = ora.Rng(17)
    pattern = np.array([rng.next_gaussian() for _ in range(16)], F)
    v = np.tile(pattern, 8)
    tile, scale, gs = rf.tile_of(v, rf.TQ3)
    assert (gs == 255).all()
    assert (np.abs(ora.dequant(tile) - v) <= rf.TQ3_CORRECTION * F(scale) + 1e-5).all()


def test_tq3_roundtrips_on_steep_spectrum():
    """tests.rs:237-256"""
    v = rf.steep_latent(19)
    tile, scale, gs = rf.tile_of(v, rf.TQ3)
    dq = ora.dequant(tile)
    for d in range(128):
        assert abs(dq[d] - v[d]) <= _eff(scale, gs, d // 16) + 1e-6, d


def test_tq3_positive_values_do_not_collapse():
    """tests.rs:258-284"""
    v = rf.signed_ramp()
    tile, scale, gs = rf.tile_of(v, rf.TQ3)
    dq = ora.dequant(tile)
    pos = 0
    for d in range(128):
        eff = _eff(scale, gs, d // 16)
        if v[d] >= eff:
            assert dq[d] > 0
            pos += 1
        if v[d] <= -eff:
            assert dq[d] < 0
    assert pos > 0


def test_tq3_error_matches_int4_grouped_resolution():
    """tests.rs:286-315"""
    for seed in range(8):
        v = rf.gaussian_latent(200 + seed)
        assert rf.sq_err(rf.tile_of(v, rf.TQ3)[0], v) <= rf.sq_err(rf.tile_of(v, rf.GROUPED)[0], v) * 2.0, seed


@pytest.mark.parametrize("codec,seed,corr_off,first,last", [(rf.TQ3, 29, rf.TQ3_CODE_BYTES, 0, 128),
                                                            (rf.MIX3, 43, rf.MIX3_CORR_OFF, rf.MIXED_HI_DIMS, rf.MIXED_DIMS)])
def test_nocorr_decodes_the_bare_grid(codec, seed, corr_off, first, last):
    """tests.rs:317-349 (tq3), :456-494 (mix3): with the NOCORR flag the (zeroed) correction plane is ignored."""
    v = rf.steep_latent(seed)
    with_corr, scale, gs = rf.tile_of(v, codec)
    nocorr = with_corr.copy()
    nocorr["flags"] |= ora.FLAG_TQ3_NOCORR
    nocorr["latent_kv"][0][corr_off:] = 0
    dc, db = ora.dequant(with_corr), ora.dequant(nocorr)
    e_corr = e_bare = F(0.0)
    for d in range(first, last):
        g = d // 16 if codec == rf.TQ3 else 1 + (d - rf.MIXED_HI_DIMS) // rf.GROUP_DIM
        assert abs(db[d] - v[d]) <= F(0.5) * _eff(scale, gs, g) + 1e-5, d
        e_corr = F(e_corr + F(F(dc[d] - v[d]) ** 2))
        e_bare = F(e_bare + F(F(db[d] - v[d]) ** 2))
    assert dc[:first].tobytes() == db[:first].tobytes()
    assert e_corr < e_bare


def test_mix3_stays_in_the_mixed_error_class_and_beats_uniform():
    """tests.rs:422-454"""
    for seed in range(8):
        v = rf.steep_latent(300 + seed)
        e_uniform = rf.sq_err(rf.tile_of(v, rf.GROUPED)[0], v)
        e_mixed = rf.sq_err(rf.tile_of(v, rf.MIXED)[0], v)
        e_mix3 = rf.sq_err(rf.tile_of(v, rf.MIX3)[0], v)
        assert e_mix3 < e_uniform and e_mix3 <= e_mixed * 2.0, seed


@pytest.mark.parametrize("name", sorted(rf.FIXTURES))
def test_score_paths_agree_on_the_equivalence_fixtures(name):
    """tests.rs:529-547, :609-627, :717-734, :824-842, :904-953: every vector path within 1e-3 (1 + |s|) of scalar."""
    q, q_sign, tiles = rf.FIXTURES[name]()
    assert len(tiles) == {"int4": 64, "nf4": 40, "mixed": 16, "tq3": 40, "mix3": 32}[name]
    scalar = ora.score_tiles(tiles, q, q_sign)
    assert np.isfinite(scalar).all() and np.ptp(scalar) > 0
    for which in (1, 2, -1):
        if which > ora.simd_level():
            continue
        for i in range(len(tiles)):
            a = ora.score_simd(tiles[i:i + 1], q, q_sign, which)
            assert abs(scalar[i] - a) <= 1e-3 * (1.0 + abs(scalar[i])), (name, which, i)


def test_hamming_distance_matches_bruteforce():
    """tests.rs:974-997 (4000 draws of Rng 0x4D31)"""
    rng = ora.Rng(0x4D31)
    for _ in range(4000):
        a = [rng.next_u64() for _ in range(4)]
        b = [rng.next_u64() for _ in range(4)]
        assert ora.hamming(a, b) == sum(bin(x ^ y).count("1") for x, y in zip(a, b))


# ---- scirust/tests/properties.rs, same seeds ---------------------------------------------------------------------
def test_prop_simd_restatement_equals_scalar():
    """properties.rs:60-86"""
    tiles, qc, qs = rf.property_triples(0xF00D, 1000, lambda it: it % 3 == 0)
    for i in range(1000):
        s = ora.score_tiles(tiles[i:i + 1], qc[i], qs[i])[0]
        for which in (1, 2):
            if which <= ora.simd_level():
                assert abs(s - ora.score_simd(tiles[i:i + 1], qc[i], qs[i], which)) <= 1e-3 * (1.0 + abs(s)), (i, which)


def test_prop_score_is_always_finite():
    """properties.rs:88-100"""
    tiles, qc, qs = rf.property_triples(0xBEEF, 3000, lambda it: it % 5 == 0, lambda it: it % 2 == 0)
    assert all(np.isfinite(ora.score_tiles(tiles[i:i + 1], qc[i], qs[i])[0]) for i in range(3000))


def test_prop_warm_equals_coarse_only_and_residual_term_is_bounded():
    """properties.rs:102-118, :226-240"""
    for seed in (7, 4):
        hot, qc, qs = rf.property_triples(seed, 500, lambda it: False)
        warm, hot0 = hot.copy(), hot.copy()
        warm["flags"] |= ora.FLAG_WARM
        hot0["dynamic_lambda"] = 0.0
        for i in range(500):
            sh, sw, s0 = (ora.score_tiles(t[i:i + 1], qc[i], qs[i])[0] for t in (hot, warm, hot0))
            assert abs(sw - s0) <= 1e-4 * (1.0 + abs(sw))
            assert abs(sh - sw) <= abs(hot["dynamic_lambda"][i]) * 256.0 + 1e-2


def test_prop_dequant_error_within_bound():
    """properties.rs:138-180"""
    rng = ora.Rng(99)
    for _ in range(300):
        v = np.array([F(F(rng.next_gaussian()) * F(F(rng.next_unit()) * F(5.0) + F(0.1))) for _ in range(128)], F)
        for codec, factor in ((rf.GROUPED, 1.0), (rf.NF4, 0.16)):
            tile, scale, gs = rf.tile_of(v, codec)
            eff = np.repeat(F(scale) * (gs.astype(F) / F(255.0)), 16)
            assert np.all(np.abs(ora.dequant(tile) - v) <= factor * eff + 1e-5)


def test_prop_rng_is_deterministic_and_sign_bits_flip_under_negation():
    """properties.rs:184-224"""
    a, b = ora.Rng(42), ora.Rng(42)
    assert all(a.next_u64() == b.next_u64() for _ in range(256))
    from .helpers import scenario_projection, scenario_sign_bits
    z = scenario_projection(2)
    rng = ora.Rng(3)
    for _ in range(200):
        v = rng.gaussian(128)
        assert ora.hamming(scenario_sign_bits(z, v), scenario_sign_bits(z, -v)) == 256
