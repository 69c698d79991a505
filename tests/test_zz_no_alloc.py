"""slha_b200_score_topk_noalloc -- the entry point for callers that cannot call
cudaMalloc (a latency-bound decode loop, a server whose pool owns all of HBM).
Its working memory is a fixed array inside the library, shared by every call, so
the check is: same answer as the allocating entry point and as the CPU oracle,
twice in a row with different inputs (the second call must not see anything the
first one left).  Collected last on purpose: a failure here cannot hide the
other tests."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def _run_both(tiles_dev, segs, qc, qs, nq, k):
    dq, ds = S.to_device(qc), S.to_device(qs)
    oi, osc, oc = S.DeviceBuffer(nq * k * 4), S.DeviceBuffer(nq * k * 4), S.DeviceBuffer(nq * 4)
    S.score_topk_noalloc(tiles_dev, segs, dq, ds, nq, k, oi, osc, oc)
    S.synchronize()
    got = (oi.download(np.uint32, nq * k).reshape(nq, k), osc.download(F, nq * k).reshape(nq, k), oc.download(np.uint32, nq))
    want = S.score_topk(tiles_dev, segs, qc, qs, nq, k)
    return got, want


def _same(got, want, all_scores):
    gi, gs, gc = got
    wi, ws, wc = want
    assert np.array_equal(gc, wc)
    for j in range(len(gc)):
        n = int(gc[j])
        assert np.all(np.abs(gs[j, :n] - ws[j, :n]) <= 1e-3)              # the suite's score tolerance
        assert np.all(np.abs(all_scores[j][gi[j, :n]] - gs[j, :n]) <= 1e-3)  # reported pairs are real
        thr = ws[j, n - 1] if n else 0.0
        for i in set(gi[j, :n]) ^ set(wi[j, :n]):                          # index sets differ only at ties
            assert abs(all_scores[j][i] - thr) <= 2e-3
        assert np.all(gi[j, n:] == 0xFFFFFFFF)


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    n, nq, k = 30000, 8, 512
    tiles = H.random_tiles(n, 2, seed=21, warm_every=11)
    dt = S.to_device(tiles)
    segs = S.make_segments([(0, 17000, 0, 4, 0), (17000, n - 17000, 4, 4, 100)])
    for seed in (31, 32):  # second call: new queries, same shared scratch
        qc, qs = H.random_queries(nq, seed)
        scores = np.concatenate([  # the oracle's scores, laid out by reported index (segment 2: index_base 100)
            np.pad(H.oracle_scores(tiles[:17000], qc[:4], qs[:4]), ((0, 0), (0, n)), constant_values=np.nan)[:, :n + 100],
            np.pad(H.oracle_scores(tiles[17000:], qc[4:], qs[4:]), ((0, 0), (100, 17000)), constant_values=np.nan)[:, :n + 100],
        ])
        got, want = _run_both(dt, segs, qc, qs, nq, k)
        _same(got, want, scores)
    # a smaller problem afterwards: stale candidates of the larger calls must not surface
    small = S.make_segments([(5, 300, 0, 2, 0)])
    qc, qs = H.random_queries(2, 33)
    got, want = _run_both(dt, small, qc, qs, 2, 512)
    sc = np.pad(H.oracle_scores(tiles[5:305], qc, qs), ((0, 0), (0, 1)))
    _same(got, want, sc)


@pytest.mark.parametrize("n,nq,k", [(1048576, 12, 256), (300000, 20, 1024)])
def test_noalloc_long_segment_with_several_query_groups(n, nq, k):
    # one long segment scored by 3 or 5 groups of four queries: the work items must be sized so
    # that items x queries fit the 512 candidate lists of the fixed scratch (these two shapes
    # were once refused although they are well inside the documented limits)
    base = H.random_tiles(65536, 1, seed=n & 0xFFFF)
    tiles = np.tile(base, n // 65536 + 1)[:n].copy()
    tiles["scale"] *= (1.0 + 0.001 * (np.arange(n) % 97)).astype(F)  # the repeats do not tie exactly
    dt = S.to_device(tiles)
    qc, qs = H.random_queries(nq, n + 7)
    segs = S.make_segments([(0, n, 0, nq, 0)])
    got, want = _run_both(dt, segs, qc, qs, nq, k)
    _same(got, want, H.oracle_scores(tiles, qc, qs))


def test_noalloc_rejects_oversize_and_host_buffers():
    tiles = H.random_tiles(64, 1, seed=1)
    dt = S.to_device(tiles)
    qc, qs = H.random_queries(1, 2)
    dq, ds = S.to_device(qc), S.to_device(qs)
    seg = S.make_segments([(0, 64, 0, 1, 0)])
    oi, osc = S.DeviceBuffer(4 * 2048), S.DeviceBuffer(4 * 2048)
    with pytest.raises(S.SlhaError) as e:
        S.score_topk_noalloc(dt, seg, dq, ds, 1, 2048, oi, osc)
    assert e.value.code == S.ERR_CAPACITY and "1024" in e.value.message
    with pytest.raises(S.SlhaError) as e:
        S.score_topk_noalloc(dt, seg, qc, ds, 1, 16, oi, osc)  # host query buffer
    assert e.value.code == S.ERR_DEVICE
    one = S.make_segments([(0, 64, 0, 1, 0)])
    with pytest.raises(S.SlhaError) as e:
        S.score_topk_noalloc(dt, one, dq, ds, 300, 16, oi, osc)  # more than 256 query rows
    assert e.value.code == S.ERR_CAPACITY
    # 130 segments of 4 queries each: 520 (segment, query) pairs exceed the 512 candidate lists
    qc4, qs4 = H.random_queries(4, 3)
    dq4, ds4 = S.to_device(np.tile(qc4, (64, 1))), S.to_device(np.tile(qs4, (64, 1)))
    many = S.make_segments([(0, 64, 4 * (i % 64), 4, 0) for i in range(130)])
    o2 = S.DeviceBuffer(4 * 256 * 16)
    with pytest.raises(S.SlhaError) as e:
        S.score_topk_noalloc(dt, many, dq4, ds4, 256, 16, o2, o2)
    assert e.value.code in (S.ERR_CAPACITY, S.ERR_DIMENSION)
