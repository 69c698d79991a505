"""slha_b200_score_topk_noalloc -- the entry point for callers that cannot call
cudaMalloc (a latency-bound decode loop, a server whose pool owns all of HBM).
Its working memory is a fixed array inside the library, shared by every call, so
the check is: same answer as the allocating entry point, twice in a row with
different inputs (the second call must not see anything the first one left).
Collected last on purpose: a failure here cannot hide the other tests."""
import numpy as np
import pytest

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
        scores = np.concatenate([
            np.pad(S.score_tiles(tiles[:17000], 17000, qc[:4], qs[:4], 4), ((0, 0), (0, n)), constant_values=np.nan)[:, :n + 100],
            np.pad(S.score_tiles(tiles[17000:], n - 17000, qc[4:], qs[4:], 4), ((0, 0), (100, 17000)), constant_values=np.nan)[:, :n + 100],
        ])
        got, want = _run_both(dt, segs, qc, qs, nq, k)
        _same(got, want, scores)
    # a smaller problem afterwards: stale candidates of the larger calls must not surface
    small = S.make_segments([(5, 300, 0, 2, 0)])
    qc, qs = H.random_queries(2, 33)
    got, want = _run_both(dt, small, qc, qs, 2, 512)
    sc = np.pad(S.score_tiles(tiles[5:305], 300, qc, qs, 2), ((0, 0), (0, 1)))
    _same(got, want, sc)


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
    many = S.make_segments([(0, 64, 0, 1, 0)] * 1)
    with pytest.raises(S.SlhaError) as e:
        S.score_topk_noalloc(dt, many, dq, ds, 300, 16, oi, osc)
    assert e.value.code == S.ERR_CAPACITY
