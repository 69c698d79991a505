"""CUDA scoring vs the CPU oracle (compute_score_scalar), through the C ABI.

Tolerance: scores within 1e-3 absolute of the scalar path and within the
reference's own SIMD-vs-scalar bound 1e-3*(1+|s|)
(scirust/src/attention/slha_v2/tests.rs:542, slhav2-vram/tests/cuda.rs:381);
Hamming distances bit-exact."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def _close(got, want):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(err <= 1e-3), float(err.max())
    assert np.all(err <= 1e-3 * (1 + np.abs(want)))


@pytest.mark.parametrize("codec", range(7))
@pytest.mark.parametrize("nq", [1, 2, 3, 4, 5])
def test_score_tiles_all_codecs(codec, nq):
    n = 1000 + 37 * codec
    tiles = H.random_tiles(n, codec, seed=100 + codec, warm_every=7, nocorr_every=5)
    qc, qs = H.random_queries(nq, 200 + codec)
    got = S.score_tiles(tiles, n, qc, qs, nq)
    _close(got, H.oracle_scores(tiles, qc, qs))


@pytest.mark.parametrize("n", [1, 3, 31, 32, 33, 127, 128, 129, 255, 257, 4095, 4097])
def test_score_tiles_ragged_sizes(n):
    tiles = H.random_tiles(n, 2, seed=n)
    qc, qs = H.random_queries(1, n + 1)
    _close(S.score_tiles(tiles, n, qc, qs, 1), H.oracle_scores(tiles, qc, qs))


def test_empty_input_is_a_noop():
    assert S.score_tiles(np.zeros(0, S.TILE_DTYPE), 0, np.zeros((1, 128), F), np.zeros((1, 4), np.uint64), 1).shape == (1, 0)


def test_hamming_term_is_bit_exact():
    # zero-level INT4 latent (0x88), lambda = 1: score == 256 - 2*hamming exactly
    rng = ora.Rng(0x4D31)
    n = 4000
    tiles = np.zeros(n, S.TILE_DTYPE)
    tiles["latent_kv"] = 0x88
    tiles["scale"] = 1.0
    tiles["group_scales"] = 255
    tiles["dynamic_lambda"] = 1.0
    tiles["residual_bitmap"] = np.array([[rng.next_u64() for _ in range(4)] for _ in range(n)], np.uint64)
    qc, qs = H.random_queries(3, 5)
    got = S.score_tiles(tiles, n, qc, qs, 3)
    for j in range(3):
        ham = np.array([ora.hamming(qs[j], tiles["residual_bitmap"][i]) for i in range(n)])
        assert np.array_equal(got[j], (256 - 2 * ham).astype(F))


@pytest.mark.parametrize("byte,expected", [(0x88, 0.0), (0x00, -1024.0), (0xFF, 896.0)])
def test_int4_known_answers_through_legacy_abi(byte, expected):
    # slhav2-vram/tests/cpu.rs:53-115
    t = np.zeros(1, S.TILE_DTYPE)
    t["latent_kv"] = byte
    t["scale"] = 1.0
    t["group_scales"] = 255
    assert abs(S.process_tile(t, np.ones(128, F), np.zeros(4, np.uint64)) - expected) < 1e-4


def test_readme_basic_usage_through_legacy_abi():
    v = ((np.arange(128, dtype=F) - 64) / 16).astype(F)
    lat, scale, gs = ora.quantize(v, 0)
    t = ora.make_tile(lat, scale, gs, lam=0.5)
    qc = np.zeros(128, F)
    qc[:2] = 1
    s = S.process_tile(t, qc, np.full(4, 0x123456789ABCDEF0, np.uint64))
    assert "%.6f" % s == "-8.000000"


def test_device_resident_inputs_and_outputs():
    n, nq = 5000, 4
    tiles = H.random_tiles(n, 1, seed=3)
    qc, qs = H.random_queries(nq, 4)
    dt, dq, ds = S.to_device(tiles), S.to_device(qc), S.to_device(qs)
    dout = S.DeviceBuffer(n * nq * 4)
    S.score_tiles(dt, n, dq, ds, nq, out=dout)
    S.synchronize()
    _close(dout.download(F, n * nq).reshape(nq, n), H.oracle_scores(tiles, qc, qs))
    assert S.launch_count() > 0


def test_score_segments_writes_a_layer_of_dense_rows_in_one_call():
    # The llama.cpp shim's layout (integration/llama.cpp/shim/slha_llama.cpp:1387-1503): dst[head][token][n_kv] with
    # n_kv padded beyond the tiles that exist; one segment per KV head, its query rows the (token, head) vectors of
    # the GQA group in token-major order.  Codecs differ per KV head; one head has no tiles yet.
    n_kv_head, gqa, n_token, n_kv = 3, 2, 5, 6000
    written = [4099, 0, 5000]
    codecs = [0, 3, 4]
    tiles = np.concatenate([H.random_tiles(max(w, 1), c, seed=40 + c, warm_every=9)[:w] for w, c in zip(written, codecs)])
    dt = S.to_device(tiles)
    n_head = n_kv_head * gqa
    qc, qs = H.random_queries(n_token * n_head, 77)  # query row = t * n_head + h
    # rows of the launch: per KV head, (token, head in group); destination element offset of row (t, h): (h * n_token + t) * n_kv
    order, offsets, segs, begin = [], [], [], 0
    for kvh in range(n_kv_head):
        rows = [(t, kvh * gqa + j) for t in range(n_token) for j in range(gqa)]
        segs.append((begin, written[kvh], len(order), len(rows), 0))
        begin += written[kvh]
        for t, h in rows:
            order.append(t * n_head + h)
            offsets.append((h * n_token + t) * n_kv)
    qc_l, qs_l = qc[order], qs[order]
    out = np.full((n_head, n_token, n_kv), 123.0, F)
    S.score_segments(dt, S.make_segments(segs), qc_l, qs_l, len(order), out, offsets, n_kv, fill=0.0)
    begin = 0
    for kvh in range(n_kv_head):
        seg_tiles = tiles[begin:begin + written[kvh]]
        begin += written[kvh]
        for j in range(gqa):
            h = kvh * gqa + j
            for t in range(n_token):
                q = t * n_head + h
                if written[kvh]:
                    _close(out[h, t, :written[kvh]], H.oracle_scores(seg_tiles, qc[q:q + 1], qs[q:q + 1])[0])
                assert np.all(out[h, t, written[kvh]:] == 0.0)
    # device destination, rows that cover only part of it: the rest stays as it was
    dev = S.to_device(np.full(4 * n_kv, 7.0, F))
    S.score_segments(dt, S.make_segments([(0, written[0], 0, 2, 0)]), qc_l[:2], qs_l[:2], 2, dev, [0, 2 * n_kv], n_kv, fill=-1.0)
    got = dev.download(F, 4 * n_kv).reshape(4, n_kv)
    _close(got[0, :written[0]], H.oracle_scores(tiles[:written[0]], qc_l[:1], qs_l[:1])[0])
    assert np.all(got[0, written[0]:] == -1.0) and np.all(got[2, written[0]:] == -1.0) and np.all(got[1] == 7.0) and np.all(got[3] == 7.0)
    # a row that would reach beyond the destination is refused
    with pytest.raises(S.SlhaError) as e:
        S.score_segments(dt, S.make_segments([(0, 10, 0, 1, 0)]), qc_l[:1], qs_l[:1], 1, dev, [3 * n_kv + 1], n_kv)
    assert e.value.code == S.ERR_DIMENSION


@pytest.mark.parametrize("codec,foreign", [(0, False), (1, False), (6, False), (4, False), (4, True), (0, True), (3, False), (3, True), (2, False)])
def test_score_segments_with_many_query_rows_uses_the_tensor_cores_and_agrees_with_the_oracle(codec, foreign):
    # sixteen or more query rows per segment: INT4 / MX-INT4 / TQ3 / mixed 8/4 tiles are scored by the tcgen05 kernel in its
    # dense mode (other codecs, here NF4, by the generic kernel).  `foreign`: a few tiles of another codec inside a segment --
    # the rows of the work items that meet them are handed to the generic kernel, the results stay the same.
    lens = [5000, 0, 777, 128, 9001]
    nqs = [16, 20, 64, 70, 33]
    tiles = H.random_tiles(sum(lens), codec, seed=60 + codec, warm_every=13, nocorr_every=6)
    if foreign:
        other = H.random_tiles(sum(lens), 2 if codec != 2 else 0, seed=61)
        for i in (4000, 5000 + 777 + 128 + 4500):
            tiles[i] = other[i]
    dt = S.to_device(tiles)
    qc, qs = H.random_queries(sum(nqs), 62 + codec)
    row_len = 9100
    segs, offsets, tb, qb = [], [], 0, 0
    for n, q in zip(lens, nqs):
        segs.append((tb, n, qb, q, 3))
        tb += n
        qb += q
    order = np.random.default_rng(5).permutation(sum(nqs))  # rows lie in the destination in another order than the query rows
    offsets = (order * row_len).astype(np.uint64)
    out = np.full((sum(nqs), row_len), 55.0, F)
    S.score_segments(dt, S.make_segments(segs), qc, qs, sum(nqs), out, offsets, row_len, fill=-2.0)
    for (tb, n, qb, q, base) in segs:
        for j in range(qb, qb + q):
            row = out[order[j]]
            if n:
                _close(row[base:base + n], ora.score_tiles(tiles[tb:tb + n], qc[j], qs[j]))
            assert np.all(row[base + n:] == -2.0)
            assert np.all(row[:base] == 0.0)  # (before the segment's index base: no row covers it, a host destination comes back zero there)


@pytest.mark.parametrize("codec,nq,foreign", [(0, 1, None), (1, 4, None), (2, 5, None), (3, 3, None), (4, 2, None), (6, 9, None), (5, 2, None),
                                              (1, 4, 2), (2, 3, 4), (3, 4, 0)])
def test_score_tiles_of_a_long_arena_runs_on_the_streaming_kernel(codec, nq, foreign):
    # 32768 tiles or more: full score vectors come from the tensor-core kernel's dense mode (MIX3 and tiles of another
    # codec than the first tile's through the generic kernel); same bar as the short arenas above
    n = 70000 + 13 * codec
    tiles = H.random_tiles(n, codec, seed=500 + codec, warm_every=7, nocorr_every=5)
    if foreign is not None:
        tiles[30000:30500] = H.random_tiles(500, foreign, seed=501)
    qc, qs = H.random_queries(nq, 502 + codec)
    got = S.score_tiles(tiles, n, qc, qs, nq)
    _close(got, H.oracle_scores(tiles, qc, qs))
