"""scirust/tests/properties.rs on the GPU library: the reference's randomised invariants, from its own generator and seeds.

Iteration i of a reference loop scores tile i with query i; here the n tiles form one arena, the n queries one batch,
and the full n x n score matrix comes from one call (the diagonal is the reference's loop, the rest is checked against
the oracle as well).
"""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H
from tests import reference_fixtures as rf

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def _gpu_matrix(tiles, qc, qs):
    n, nq = len(tiles), len(qc)
    out = np.zeros((nq, n), F)
    S.score_segments(S.to_device(tiles), S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, out, (np.arange(nq) * n).astype(np.uint64), n)
    return out


def test_prop_gpu_path_equals_scalar():
    """properties.rs:60-86 (prop_simd_paths_equal_scalar) with the GPU as the vector path"""
    tiles, qc, qs = rf.property_triples(0xF00D, 1000, lambda it: it % 3 == 0)
    got, want = _gpu_matrix(tiles, qc, qs), H.oracle_scores(tiles, qc, qs)
    assert np.all(np.abs(got - want) <= 1e-3 * (1.0 + np.abs(want)))


def test_prop_score_is_always_finite():
    """properties.rs:88-100"""
    tiles, qc, qs = rf.property_triples(0xBEEF, 3000, lambda it: it % 5 == 0, lambda it: it % 2 == 0)
    got = _gpu_matrix(tiles, qc[:64], qs[:64])
    assert np.isfinite(got).all()
    diag = np.array([S.score_tiles(tiles[i:i + 1], 1, qc[i:i + 1], qs[i:i + 1], 1)[0, 0] for i in range(0, 3000, 50)])
    assert np.isfinite(diag).all()


def test_prop_warm_equals_coarse_only_and_residual_term_is_bounded():
    """properties.rs:102-118, :226-240"""
    for seed in (7, 4):
        hot, qc, qs = rf.property_triples(seed, 500, lambda it: False)
        warm = hot.copy()
        warm["flags"] |= ora.FLAG_WARM
        hot0 = hot.copy()
        hot0["dynamic_lambda"] = 0.0
        idx = np.arange(500)
        sh, sw, s0 = (_gpu_matrix(t, qc, qs)[idx, idx] for t in (hot, warm, hot0))
        assert np.all(np.abs(sw - s0) <= 1e-4 * (1.0 + np.abs(sw)))
        assert np.all(np.abs(sh - sw) <= np.abs(hot["dynamic_lambda"]) * 256.0 + 1e-2)


def test_prop_sign_bits_negation_flips_all_bits_and_encode_is_deterministic():
    """properties.rs:184-224 through slha_b200_prepare_queries / slha_b200_encode_keys"""
    _, p = H.make_model_pair(160, seed=2)
    for rht in (False, True):
        gm = S.Model.from_projection(p, 160, 2, rht=rht)
        v = H.gaussian_keys(3, 200, 160)
        _, a = gm.prepare_queries(v)
        _, b = gm.prepare_queries(-v)
        assert np.all((a ^ b) == np.uint64(0xFFFFFFFFFFFFFFFF))
        for codec in range(6):
            assert gm.encode_keys(v, codec).tobytes() == gm.encode_keys(v, codec).tobytes()


def test_prop_dequant_error_within_bound():
    """properties.rs:138-180: a coordinate projection makes the latent the key itself; encode on the GPU, decode on the GPU"""
    p = np.zeros((128, 160), F)
    p[np.arange(128), np.arange(128)] = 1.0
    gm = S.Model.from_projection(p, 160, 1)
    rng = ora.Rng(99)
    keys = np.zeros((300, 160), F)
    for i in range(300):
        for d in range(128):
            keys[i, d] = F(F(rng.next_gaussian()) * F(F(rng.next_unit()) * F(5.0) + F(0.1)))
    for codec, factor in ((S.CODEC_INT4_GROUPED, 1.0), (S.CODEC_NF4, 0.16)):
        tiles = gm.encode_keys(keys, codec)
        for i in range(0, 300, 7):
            dq = gm.decode_latent(tiles[i:i + 1])[:128]
            eff = tiles["scale"][i] * (tiles["group_scales"][i].astype(F) / F(255.0))
            assert np.all(np.abs(dq - keys[i, :128]) <= factor * np.repeat(eff, 16) + 1e-5)
