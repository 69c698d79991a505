"""Decode tail on the selected tiles (slha_b200_attend_topk) against the oracle's restatement of the
reference's softmax_into + aggregate_v (scirust/src/metrics.rs:338-420,
scirust/examples/benchmark_decode.rs:28-38, :82-95).  Floating point: weights and outputs within
2e-6 absolute + 2e-5 relative (the device sums in another, fixed order and uses float32 exp)."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def close(a, b):
    return np.all(np.abs(a - b) <= 2e-6 + 2e-5 * np.abs(b))


@pytest.mark.parametrize("n,nq,k,d_v,bf16", [(5000, 4, 256, 128, False), (3000, 3, 100, 96, True), (700, 2, 1024, 128, False),
                                             (4096, 5, 64, 300, False)])
def test_attend_after_topk_matches_the_reference_tail(n, nq, k, d_v, bf16):
    tiles = H.random_tiles(n, 1, seed=n)
    qc, qs = H.random_queries(nq, n + 1)
    dt = S.to_device(tiles)
    # two KV heads' worth of value rows; the query rows alternate between them; reported indices start at 50
    heads = 2
    values = ora.Rng(n + 2).gaussian(heads * n * d_v).reshape(heads * n, d_v)
    if bf16:
        values = H.to_bf16_f32(values).reshape(heads * n, d_v)
        dv = S.to_device((values.view(np.uint32) >> 16).astype(np.uint16))
    else:
        dv = S.to_device(values)
    segs = [(0, n, 0, nq, 50)]
    gi, gs, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    base = np.array([(j % heads) * n - 50 for j in range(nq)], np.int64).astype(np.uint64)
    scale = float(1.0 / np.sqrt(128.0))
    w_out = np.zeros((nq, k), F)
    out = S.attend_topk(gi, gs, k, scale, dv, d_v, value_dtype=S.BF16 if bf16 else S.F32, top_count=gc, value_row_base=base,
                        weights_out=w_out)
    want, want_w = ora.attend_topk(gi, gs, scale, values, top_count=gc, row_base=base)
    assert close(w_out, want_w) and close(out, want)
    assert np.all(np.abs(w_out.sum(1) - 1.0) <= 1e-5)
    assert np.all(w_out[:, min(k, n):] == 0)  # padding entries weigh nothing


def test_attend_rows_without_winners_and_bad_arguments():
    d_v, k = 64, 16
    values = ora.Rng(3).gaussian(100 * d_v).reshape(100, d_v)
    dv = S.to_device(values)
    idx = np.full((2, k), 0xFFFFFFFF, np.uint32)
    sc = np.full((2, k), -np.inf, F)
    idx[1, :3] = [5, 7, 99]
    sc[1, :3] = [1.0, 0.5, -2.0]
    out = S.attend_topk(idx, sc, k, 0.25, dv, d_v)
    want, _ = ora.attend_topk(idx, sc, 0.25, values)
    assert np.all(out[0] == 0) and close(out, want)
    with pytest.raises(S.SlhaError) as e:
        S.attend_topk(idx, sc, k, float("nan"), dv, d_v)
    assert e.value.code == S.ERR_NONFINITE
    with pytest.raises(S.SlhaError) as e:
        S.attend_topk(idx, sc, k, 0.25, values, d_v)  # host values
    assert e.value.code == S.ERR_DEVICE
