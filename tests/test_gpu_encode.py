"""CUDA encode / prepare_query vs the oracle: tile bytes bit-exact."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def _models(d, rht, seed=7):
    om, p = H.make_model_pair(d, seed=seed, rht=rht)
    return om, S.Model.from_projection(p, d, seed, rht=rht)


def _diff(a, b):
    bad = np.nonzero(a.view(np.uint8).reshape(-1, 128) != b.view(np.uint8).reshape(-1, 128))
    return "first mismatch tile %d byte %d" % (bad[0][0], bad[1][0]) if len(bad[0]) else ""


@pytest.mark.parametrize("codec", range(7))
@pytest.mark.parametrize("d,rht", [(128, False), (160, False), (160, True), (128, True)])
def test_encode_bit_exact(codec, d, rht):
    om, gm = _models(d, rht)
    n = 300
    keys = H.gaussian_keys(50 + codec, n, d, outlier_channels=(7, 93))
    keys[5] = 0.0  # all-zero key: scale falls back to 1.0
    pos = np.arange(1000, 1000 + n, dtype=np.uint32)
    heads = (np.arange(n) % 8).astype(np.uint16)
    want = om.encode_batch(keys, codec, pos=pos, head=heads)
    got = gm.encode_keys(keys, codec, positions=pos, head_ids=heads)
    assert got.tobytes() == want.tobytes(), _diff(got, want)


@pytest.mark.parametrize("n", [1, 15, 16, 17, 33])
def test_encode_ragged_batches_and_bf16(n):
    om, gm = _models(128, False)
    keys = H.to_bf16_f32(H.gaussian_keys(n, n, 128))
    want = om.encode_batch(keys, 2, pos=np.arange(n, dtype=np.uint32) + 7)
    bf16 = (keys.view(np.uint32) >> 16).astype(np.uint16)
    got = gm.encode_keys(bf16, 2, n=n, key_dtype=S.BF16, position_base=7)
    assert got.tobytes() == want.tobytes(), _diff(got, want)


def test_single_key_abi_matches_batch_and_oracle():
    om, gm = _models(160, False)
    keys = H.gaussian_keys(3, 4, 160)
    for codec in range(6):
        batch = gm.encode_keys(keys, codec)
        for i in range(4):
            one = gm.encode_key(keys[i], position=i, codec=codec)
            assert one.tobytes() == batch[i:i + 1].tobytes() == om.encode(keys[i], i, codec=codec).tobytes()


@pytest.mark.parametrize("d,rht", [(128, False), (160, True)])
def test_prepare_queries_bit_exact(d, rht):
    om, gm = _models(d, rht)
    q = H.gaussian_keys(9, 37, d)
    qc, qs = gm.prepare_queries(q)
    for j in range(len(q)):
        wc, ws = om.prepare_query(q[j])
        assert np.array_equal(qs[j], ws)
        assert np.array_equal(qc[j].view(np.uint32), wc.view(np.uint32))
    c1, s1 = gm.prepare_query(q[0])
    assert np.array_equal(c1, qc[0]) and np.array_equal(s1, qs[0])


def test_whitened_model_and_decode():
    p = H.orthogonal_projection(21, 160)
    scale = (0.5 + np.abs(ora.Rng(22).gaussian(128))).astype(F)
    om = ora.Model(p, 160, seed=5, scale=scale)
    gm = S.Model.from_projection(p, 160, 5, scale=scale)
    keys = H.gaussian_keys(23, 64, 160)
    want = om.encode_batch(keys, 3)
    got = gm.encode_keys(keys, 3)
    assert got.tobytes() == want.tobytes(), _diff(got, want)
    for i in (0, 17):
        assert np.allclose(gm.decode_latent(got[i:i + 1]), om.decode_latent(want[i:i + 1]), atol=1e-5)
        assert np.allclose(gm.decode_key(got[i:i + 1]), om.decode_key(want[i:i + 1]), atol=1e-4)


def test_encode_then_score_end_to_end_config1_shape():
    # configuration 1 (single-head INT4 cache) at reduced length: INT4 single, d=128, outlier channels, top-64
    om, gm = _models(128, False, seed=0)
    n = 2048
    keys = H.gaussian_keys(0, n, 128, outlier_channels=(7, 93))
    dt = S.DeviceBuffer(n * 128)
    gm.encode_keys(keys, 0, out=dt)
    tiles = dt.download(S.TILE_DTYPE, n)
    assert tiles.tobytes() == om.encode_batch(keys, 0).tobytes()
    q = ora.Rng(1).gaussian(128)
    qc, qs = gm.prepare_queries(q[None])
    gi, gsc, gc = S.score_topk(dt, S.make_segments([(0, n, 0, 1, 0)]), qc, qs, 1, 64)
    want = ora.score_tiles(tiles, qc[0], qs[0])
    oi, ov = ora.topk(want, 64)
    assert set(gi[0]) == set(oi) or np.all(np.abs(np.sort(gsc[0])[::-1] - ov) <= 1e-3)


def _edge_keys(d, seed):
    """Keys that sit on the quantisers' decision points: with a coordinate projection the latent is the key itself, so
    half-integer multiples of the step are exact rounding ties, the residual has exact zeros, and whole groups vanish."""
    rng = np.random.default_rng(seed)
    rows = []
    half_steps = (rng.integers(-14, 15, size=(24, d)) * 0.5).astype(F)
    half_steps[:, 0] = 7.0  # absmax 7 -> INT4 step exactly 1
    rows.append(half_steps)
    rows.append(half_steps * F(2.0 ** -20))
    rows.append(half_steps * F(2.0 ** 40))
    rows.append((half_steps * F(1e15)).astype(F))              # (squares stay finite: no overflow in the residual's rms)
    rows.append((half_steps * F(1e-38)).astype(F))           # denormal range
    spike = np.zeros((8, d), F)
    spike[np.arange(8), rng.integers(0, d, 8)] = rng.choice([-1.0, 1.0, 3e18, -1e-45], 8).astype(F)
    rows.append(spike)
    const = np.repeat(rng.choice([1.0, -1.0, 0.3, -2.5e-7], 8).astype(F)[:, None], d, axis=1)
    rows.append(const)
    zeros = np.zeros((2, d), F)
    zeros[1] = -0.0
    rows.append(zeros)
    one_group = np.zeros((8, d), F)
    one_group[:, 16:32] = rng.standard_normal((8, 16)).astype(F)   # all other groups empty
    rows.append(one_group)
    tq3_grid = ((rng.integers(0, 8, size=(16, d)) - 3.5) * 2.0).astype(F)  # exactly the TQ3 levels at half range 7
    rows.append(tq3_grid)
    return np.ascontiguousarray(np.concatenate(rows), F)


@pytest.mark.parametrize("codec", range(7))
@pytest.mark.parametrize("d,rht,coord", [(128, False, True), (256, False, True), (128, True, True), (200, True, False), (128, False, False)])
def test_encode_bit_exact_on_rounding_ties_zeros_and_extreme_magnitudes(codec, d, rht, coord):
    if coord:
        p = np.zeros((128, d), F)
        p[np.arange(128), np.arange(128)] = 1.0  # latent dimension i = key coordinate i
    else:
        p = H.orthogonal_projection(31, d)
    om, gm = ora.Model(p, d, seed=3, rht=rht), S.Model.from_projection(p, d, 3, rht=rht)
    keys = _edge_keys(d, 40 + codec)
    want = om.encode_batch(keys, codec)
    got = gm.encode_keys(keys, codec)
    assert got.tobytes() == want.tobytes(), _diff(got, want)
    qc, qs = gm.prepare_queries(keys)
    for j in range(0, len(keys), 5):
        wc, ws = om.prepare_query(keys[j])
        assert np.array_equal(qs[j], ws) and np.array_equal(qc[j].view(np.uint32), wc.view(np.uint32))


@pytest.mark.parametrize("codec", range(6))
@pytest.mark.parametrize("d,rht", [(160, False), (200, True), (256, False)])
def test_decode_latent_and_key_for_every_codec(codec, d, rht):
    # slha_decode_latent / slha_decode_key (slha-c/src/lib.rs:1034-1191) against the oracle's LearnedModel decode, NOCORR
    # tiles with their plane bytes left in place included; the sums run in another order, hence 1e-5 of the vector's norm.
    # And the reference's own property: the key decode (latent + residual estimate) is closer to the key than the latent alone.
    om, gm = _models(d, rht, seed=11)
    keys = H.gaussian_keys(70 + codec, 40, d, outlier_channels=(3,))
    tiles = om.encode_batch(keys, codec)
    if codec in (4, 5):
        tiles["flags"][::3] |= ora.FLAG_TQ3_NOCORR
    better = 0
    for i in range(len(keys)):
        t = tiles[i:i + 1]
        wl, wk = om.decode_latent(t), om.decode_key(t)
        gl, gk = gm.decode_latent(t), gm.decode_key(t)
        assert np.all(np.abs(gl - wl) <= 1e-5 * (1.0 + np.linalg.norm(wl)))
        assert np.all(np.abs(gk - wk) <= 1e-5 * (1.0 + np.linalg.norm(wk)))
        better += np.linalg.norm(keys[i] - gk) < np.linalg.norm(keys[i] - gl)
    # (with the Hadamard rotation the residual estimate is left out, learned.rs:295-299: both decodes coincide)
    assert better == (0 if rht else len(keys))
