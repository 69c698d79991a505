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
