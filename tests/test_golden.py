"""Committed golden vectors (tests/golden/slha_golden.npz, made by
tests/golden/make_golden.py): the oracle must keep reproducing them (CPU), and
the CUDA path must match them (GPU): tile bytes exactly, scores within 1e-3."""
import os

import numpy as np
import pytest

from oracle import pyoracle as ora

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "slha_golden.npz"))
CASES = [(rht, codec) for rht in (0, 1) for codec in range(7)]


@pytest.mark.parametrize("rht,codec", CASES)
def test_oracle_reproduces_golden(rht, codec):
    tag = "rht%d_" % rht
    m = ora.Model(G[tag + "projection"], 160, seed=40 + rht, rht=bool(rht))
    tiles = m.encode_batch(G[tag + "keys"], codec, pos=np.arange(96, dtype=np.uint32) + 11)
    assert np.array_equal(tiles.view(np.uint8).reshape(96, 128), G[tag + "tiles_c%d" % codec])
    for j in range(3):
        qc, qs = m.prepare_query(G[tag + "queries"][j])
        assert np.array_equal(qc, G[tag + "q_coarse"][j]) and np.array_equal(qs, G[tag + "q_sign"][j])
        assert np.array_equal(ora.score_tiles(tiles, qc, qs), G[tag + "scores_c%d" % codec][j])


@pytest.mark.gpu
@pytest.mark.parametrize("rht,codec", CASES)
def test_cuda_matches_golden(rht, codec):
    import slhav2_b200 as S

    tag = "rht%d_" % rht
    m = S.Model.from_projection(G[tag + "projection"], 160, 40 + rht, rht=bool(rht))
    keys = G[tag + "keys"]
    bf16 = (keys.view(np.uint32) >> 16).astype(np.uint16)
    tiles = m.encode_keys(bf16, codec, n=96, key_dtype=S.BF16, position_base=11)
    assert np.array_equal(tiles.view(np.uint8).reshape(96, 128), G[tag + "tiles_c%d" % codec])
    qc, qs = m.prepare_queries(G[tag + "queries"])
    assert np.array_equal(qc, G[tag + "q_coarse"]) and np.array_equal(qs, G[tag + "q_sign"])
    want = G[tag + "scores_c%d" % codec]
    got = S.score_tiles(tiles, 96, qc, qs, 3)
    assert np.all(np.abs(got - want) <= 1e-3)
    dt = S.to_device(tiles)
    gi, gsc, _ = S.score_topk(dt, S.make_segments([(0, 96, 0, 3, 0)]), qc, qs, 3, 16)
    for j in range(3):
        top = G[tag + "top16_c%d" % codec][j]
        thr = want[j][top[-1]]
        assert all(abs(want[j][i] - thr) <= 2e-3 for i in set(top) ^ set(gi[j]))
    m.release()
