"""The reference's score-equivalence matrix with the GPU kernels as further 'instruction sets'.

scirust/src/attention/slha_v2/tests.rs holds, per codec, a fixture of tiles (HOT / WARM, with and without the
TQ3 correction plane, Gaussian scenario tokens and the steep spectrum) on which every vector path must stay
within 1e-3 (1 + |s|) of compute_score_scalar (:529-547, :609-627, :717-734, :824-842, :904-953).  The same
fixtures (tests/reference_fixtures.py restates them with the reference's seeds) go through every scoring
kernel of the library, called through the C ABI: the generic kernel, the streaming tensor-core kernel (top-k
and dense mode), and the tcgen05 kernel for sixteen or more query rows.
"""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H
from tests import reference_fixtures as rf

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32
NAMES = sorted(rf.FIXTURES)


def _within_reference_bound(got, want):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(err <= 1e-3 * (1.0 + np.abs(want))), float((err / (1.0 + np.abs(want))).max())


@pytest.mark.parametrize("name", NAMES)
def test_full_scores_of_the_fixture(name):
    q, q_sign, tiles = rf.FIXTURES[name]()
    want = ora.score_tiles(tiles, q, q_sign)
    _within_reference_bound(S.score_tiles(tiles, len(tiles), q[None], q_sign[None], 1)[0], want)


@pytest.mark.parametrize("name", NAMES)
def test_long_arena_of_fixture_tiles_on_the_streaming_kernel(name):
    # the fixture repeated to more than 32768 tiles (from where full score vectors come from the tensor-core kernel's
    # dense mode, MIX3 from the generic kernel): every copy must meet the bound; then top-k over the same arena
    q, q_sign, tiles = rf.FIXTURES[name]()
    reps = -(-40000 // len(tiles))
    arena = np.tile(tiles, reps)
    want = np.tile(ora.score_tiles(tiles, q, q_sign), reps)
    _within_reference_bound(S.score_tiles(arena, len(arena), q[None], q_sign[None], 1)[0], want)
    k = min(3 * reps, 1024)  # copies of the fixture's three best tiles
    idx, score, cnt = S.score_topk(S.to_device(arena), S.make_segments([(0, len(arena), 0, 1, 0)]), q[None], q_sign[None], 1, k)
    assert cnt[0] == k
    _within_reference_bound(score[0], want[idx[0]])
    assert np.all(np.diff(score[0]) <= 0)
    kth = np.sort(want)[::-1][k - 1]
    assert np.all(want[idx[0]] >= kth - 2e-3 * (1.0 + abs(kth)))  # nothing clearly below the k-th was chosen


@pytest.mark.parametrize("name", ["int4", "mixed", "tq3", "nf4"])
def test_fixture_against_sixteen_or_more_query_rows(name):
    # the fixture's query among other rows: INT4, mixed 8/4 and TQ3 take the tcgen05 kernel (NF4 the generic one)
    q, q_sign, tiles = rf.FIXTURES[name]()
    qc, qs = H.random_queries(24, 71)
    qc[5], qs[5] = q, q_sign
    n = len(tiles)
    out = np.zeros((24, n), F)
    S.score_segments(S.to_device(tiles), S.make_segments([(0, n, 0, 24, 0)]), qc, qs, 24, out, (np.arange(24) * n).astype(np.uint64), n)
    _within_reference_bound(out, H.oracle_scores(tiles, qc, qs))
    idx, score, cnt = S.score_topk(S.to_device(tiles), S.make_segments([(0, n, 0, 24, 0)]), qc, qs, 24, 8)
    want = H.oracle_scores(tiles, qc, qs)
    for j in range(24):
        assert cnt[j] == 8
        _within_reference_bound(score[j], want[j][idx[j]])
        kth = np.sort(want[j])[::-1][7]
        assert np.all(want[j][idx[j]] >= kth - 2e-3 * (1.0 + abs(kth)))


def _degenerate_arena(codec, n):
    """Valid tiles at the edges of the format: scirust/tests/properties.rs:259-273 (zero latent, zero scale, lambda 1e6,
    group scales 1) and scales / lambdas far from the usual range."""
    tiles = H.random_tiles(n, codec, seed=700 + codec, warm_every=11, nocorr_every=3)
    z = slice(0, 100)
    tiles["latent_kv"][z] = 0
    tiles["scale"][z] = 0.0
    tiles["dynamic_lambda"][z] = 1.0e6
    tiles["group_scales"][z] = 1
    tiles["scale"][100:200] = 1e-30
    tiles["scale"][200:300] *= F(1e20)
    tiles["dynamic_lambda"][300:400] = 0.0
    tiles["dynamic_lambda"][400:500] = -3.0
    tiles["group_scales"][500:600] = 0
    tiles["residual_bitmap"][600:700] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return tiles


def _degenerate_queries(nq):
    qc, qs = H.random_queries(nq, 77)
    qc[0], qs[0] = 1.0e3, np.uint64(0xFFFFFFFFFFFFFFFF)  # properties.rs:267-268
    if nq > 2:
        qc[2] *= F(1e5)    # beyond the fp16 split of the tensor-core kernels
    if nq > 3:
        qc[3] *= F(1e-12)
    if nq > 4:
        qc[4], qs[4] = 0.0, 0
    return qc, qs


def _term_magnitudes(tiles, qc):
    """sum_d |dequant_d q_d| + 256 |lambda| per (query, tile): the scale of the rounding error of any summation order."""
    d = np.abs(np.stack([ora.dequant(tiles[i:i + 1]) for i in range(len(tiles))]).astype(np.float64))
    lam = np.where(tiles["flags"] & ora.FLAG_WARM, 0.0, np.abs(tiles["dynamic_lambda"].astype(np.float64)))
    return np.abs(qc.astype(np.float64)) @ d.T + 256.0 * lam[None, :]


def _within_summation_bound(got, want, mags):
    # the reference's bound 1e-3 (1 + |s|) presumes terms of the size of the sum; where they cancel (a constant query of
    # 1e3 against signed levels: the reference's own vector paths leave the bound there too) 32 ulp of the terms' total
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(err <= 1e-3 * (1.0 + np.abs(want)) + 4e-6 * mags), float((err / (1e-3 * (1.0 + np.abs(want)) + 4e-6 * mags)).max())


@pytest.mark.parametrize("codec", [0, 6, 2, 3, 4, 5])
@pytest.mark.parametrize("n,nq", [(3000, 5), (40000, 5), (40000, 20)])
def test_degenerate_tiles_and_queries_stay_finite_and_agree(codec, n, nq):
    tiles = _degenerate_arena(codec, n)
    qc, qs = _degenerate_queries(nq)
    want = H.oracle_scores(tiles, qc, qs)
    mags = _term_magnitudes(tiles, qc)
    assert np.isfinite(want).all()
    dt = S.to_device(tiles)
    if nq <= 5:
        got = S.score_tiles(dt, n, qc, qs, nq)
    else:
        got = np.zeros((nq, n), F)
        S.score_segments(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, got, (np.arange(nq) * n).astype(np.uint64), n)
    assert np.isfinite(got).all()
    _within_summation_bound(got, want, mags)
    k = 300
    idx, score, cnt = S.score_topk(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)
    for j in range(nq):
        assert cnt[j] == k
        _within_summation_bound(score[j], want[j][idx[j]], mags[j][idx[j]])
        assert len(set(idx[j].tolist())) == k
        slack = 2e-3 * (1.0 + np.abs(want[j])) + 8e-6 * mags[j]
        kth = np.sort(want[j])[::-1][k - 1]
        assert np.all(want[j][idx[j]] + slack[idx[j]] >= kth - slack.max())  # nothing clearly below the k-th was chosen


@pytest.mark.parametrize("n,nq", [(4096, 3), (40960, 4), (40960, 16)])
def test_every_flag_combination_is_decoded_as_compute_score_decodes_it(n, nq):
    # Tiles in device memory are not validated (slha_score_tiles validates, slha-c/src/lib.rs:244-286): whatever the six
    # flag bits say, contradictory combinations included, every kernel must decode a tile by the precedence of the
    # reference's dequant_at / compute_score (tile.rs:133-281), which the oracle restates.
    tiles = H.random_tiles(n, 1, seed=800)
    rng = np.random.default_rng(801)
    tiles["latent_kv"] = rng.integers(0, 256, size=(n, 64), dtype=np.uint8)
    tiles["flags"] = (np.arange(n) % 64).astype(np.uint16)
    qc, qs = H.random_queries(nq, 802)
    want = H.oracle_scores(tiles, qc, qs)
    dt = S.to_device(tiles)
    if nq < 16:
        got = S.score_tiles(dt, n, qc, qs, nq)
    else:
        got = np.zeros((nq, n), F)
        S.score_segments(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, got, (np.arange(nq) * n).astype(np.uint64), n)
    _within_summation_bound(got, want, _term_magnitudes(tiles, qc))
    for first in (0, 2, 4, 8, 12):  # the first tile's codec selects the tensor-core instantiation: INT4, NF4, mixed, TQ3, mixed|TQ3
        rolled = np.roll(tiles, -first)
        idx, score, cnt = S.score_topk(S.to_device(rolled), S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, 64)
        w = np.roll(want, -first, axis=1)
        for j in range(nq):
            _within_reference_bound(score[j], w[j][idx[j]])
            kth = np.sort(w[j])[::-1][63]
            assert np.all(w[j][idx[j]] >= kth - 2e-3 * (1.0 + abs(kth)))
