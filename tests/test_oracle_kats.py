"""Pins the CPU oracle against the reference's own known-answer tests.

The reference is Rust and cannot be run here, so every expected value below is
one the reference's test-suite or README states in text; the file:line of each
is given.  These run on CPU (`-m "not gpu"`).
"""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

F = np.float32


def test_tile_layout_offsets():
    # slha-c/include/slha.h:100-110
    want = dict(latent_kv=0, residual_bitmap=64, scale=96, dynamic_lambda=100, residual_sigma=104,
                token_id=108, position=112, head_id=116, flags=118, group_scales=120)
    for name, off in want.items():
        assert ora.TILE_DTYPE.fields[name][1] == off
    assert ora.TILE_DTYPE.itemsize == 128


@pytest.mark.parametrize("byte,expected", [(0x88, 0.0), (0x00, -8.0 * 128), (0xFF, 7.0 * 128)])
def test_int4_zero_point_known_answers(byte, expected):
    # slhav2-vram/tests/cpu.rs:53-115
    t = ora.make_tile(np.full(64, byte, np.uint8), 1.0, np.full(8, 255, np.uint8))
    s = ora.score_tiles(t, np.ones(128, F), np.zeros(4, np.uint64))[0]
    assert abs(s - expected) < 1e-4
    for which in (0, 1, 2):
        if which <= ora.simd_level():
            assert abs(ora.score_simd(t, np.ones(128, F), np.zeros(4, np.uint64), which) - expected) < 1e-4


def test_readme_basic_usage():
    # scirust/examples/basic_usage.rs:9-33, README.md:97-102
    v = ((np.arange(128, dtype=F) - 64) / 16).astype(F)
    lat, scale, gs = ora.quantize(v, 0)
    t = ora.make_tile(lat, scale, gs, lam=0.5)
    qc = np.zeros(128, F)
    qc[0] = qc[1] = 1.0
    qs = np.full(4, 0x123456789ABCDEF0, np.uint64)
    assert "%.6f" % ora.score_tiles(t, qc, qs)[0] == "-8.000000"
    assert list(ora.dequant(t)[:4]) == [-4.0, -4.0, -4.0, -4.0]


def test_hamming_bruteforce_and_sign_dot_identity():
    # scirust/src/attention/slha_v2/tests.rs:976-997, scirust/tests/slha.rs:16-47
    rng = ora.Rng(0x4D31)
    for _ in range(1000):
        a = np.array([rng.next_u64() for _ in range(4)], np.uint64)
        b = np.array([rng.next_u64() for _ in range(4)], np.uint64)
        bits_a = np.unpackbits(a.view(np.uint8), bitorder="little")
        bits_b = np.unpackbits(b.view(np.uint8), bitorder="little")
        brute = int((bits_a ^ bits_b).sum())
        h = ora.hamming(a, b)
        assert h == brute
        sa, sb = 1 - 2 * bits_a.astype(int), 1 - 2 * bits_b.astype(int)
        assert 256 - 2 * h == int((sa * sb).sum())


def test_analytic_lambda_constant():
    # scirust/src/scenario.rs:27-32: sqrt(pi/512) ~= 0.0783
    assert abs(ora.lib.ora_analytic_lambda_c() - 0.0783) < 1e-4


def test_nf4_codebook_nearest_is_antisymmetric_and_monotone():
    # scirust/tests/properties.rs:239-256 + codec/nf4.rs:7-18
    cb = [-1.0, -0.7075, -0.5421, -0.4165, -0.3108, -0.2158, -0.1272, -0.0421,
          0.0421, 0.1272, 0.2158, 0.3108, 0.4165, 0.5421, 0.7075, 1.0]
    for i, c in enumerate(cb):
        assert ora.lib.ora_nf4_nearest(c) == i
    assert ora.lib.ora_nf4_nearest(0.0) == 7  # tie between 7 and 8: first minimum wins
    last = 0
    for t in np.linspace(-1, 1, 4001, dtype=F):
        i = ora.lib.ora_nf4_nearest(float(t))
        assert i >= last
        last = i


def test_int4_roundtrip_within_one_step():
    # scirust/src/attention/slha_v2/tests.rs:48-74, tests/properties.rs:137-179
    rng = ora.Rng(5)
    for _ in range(50):
        v = rng.gaussian(128)
        for codec in (0, 1):
            lat, scale, gs = ora.quantize(v, codec)
            dq = ora.dequant(ora.make_tile(lat, scale, gs))
            eff = scale * gs.astype(F).repeat(16) / 255
            assert np.all(np.abs(dq - v) <= eff * 1.0001 + 1e-6)
        lat, scale, gs = ora.quantize(v, 2)
        dq = ora.dequant(ora.make_tile(lat, scale, gs, flags=ora.FLAG_NF4))
        eff = scale * gs.astype(F).repeat(16) / 255
        assert np.all(np.abs(dq - v) <= 0.16 * eff + 1e-5)


def test_tq3_equal_groups_share_scale_and_quarter_step():
    # scirust/src/attention/slha_v2/tests.rs:206-235
    pattern = ora.Rng(17).gaussian(16)
    v = np.tile(pattern, 8).astype(F)
    lat, glob, gs = ora.quantize(v, 4)
    assert list(gs) == [255] * 8
    dq = ora.dequant(ora.make_tile(lat, glob, gs, flags=ora.FLAG_TQ3))
    assert np.all(np.abs(dq - v) <= 0.25 * glob + 1e-5)
    # without the correction plane the bound degrades to half a step (tests.rs:237-349)
    dq2 = ora.dequant(ora.make_tile(lat, glob, gs, flags=ora.FLAG_TQ3 | ora.FLAG_TQ3_NOCORR))
    assert np.all(np.abs(dq2 - v) <= 0.5 * glob + 1e-5)


@pytest.mark.parametrize("codec,flag", [(3, ora.FLAG_MIXED), (5, ora.FLAG_MIX3)])
def test_mixed_tail_decodes_to_zero(codec, flag):
    # scirust/src/attention/slha_v2/tests.rs:172-174, :417-419
    v = ora.Rng(3).gaussian(128)
    lat, glob, gs = ora.quantize(v, codec)
    dq = ora.dequant(ora.make_tile(lat, glob, gs, flags=flag))
    assert np.all(dq[120:] == 0.0)


def test_simd_restatement_matches_scalar():
    # tolerance of scirust/src/attention/slha_v2/tests.rs:529-972: 1e-3*(1+|s|)
    rng = ora.Rng(99)
    for codec in (0, 1, 2):
        for _ in range(100):
            lat, scale, gs = ora.quantize(rng.gaussian(128), codec)
            res = [rng.next_u64() for _ in range(4)]
            t = ora.make_tile(lat, scale, gs, flags=ora.CODEC_FLAG[codec], lam=0.07, residual=res)
            qc = rng.gaussian(128)
            qs = np.array([rng.next_u64() for _ in range(4)], np.uint64)
            s = ora.score_tiles(t, qc, qs)[0]
            for which in range(1, ora.simd_level() + 1):
                a = ora.score_simd(t, qc, qs, which)
                assert abs(s - a) <= 1e-3 * (1 + abs(s))


def test_score_equation_2_3_and_warm():
    # scirust/tests/slha.rs:50-89
    z = H.scenario_projection(3)
    q, toks = H.scenario_generate(4, 1, 0.4)
    t = H.scenario_tile(z, toks[0], 0)
    qs = H.scenario_sign_bits(z, q)
    got = ora.score_tiles(t, q, qs)[0]
    k = ora.dequant(t)
    coarse = F(0)
    for d in range(128):
        coarse = F(coarse + F(q[d] * k[d]))
    ham = ora.hamming(qs, t["residual_bitmap"][0])
    manual = coarse + t["dynamic_lambda"][0] * F(256 - 2 * ham)
    assert abs(got - manual) < 1e-4
    w = t.copy()
    w["flags"] |= ora.FLAG_WARM
    assert abs(ora.score_tiles(w, q, qs)[0] - coarse) < 1e-4


def test_negated_vector_flips_all_sign_bits_and_encode_is_deterministic():
    # scirust/tests/properties.rs:183-221
    z = H.scenario_projection(11)
    v = ora.Rng(12).gaussian(128)
    a, b = H.scenario_sign_bits(z, v), H.scenario_sign_bits(z, -v)
    assert ora.hamming(a, b) == 256
    p = H.orthogonal_projection(1, 160)
    m = ora.Model(p, 160, seed=7)
    key = ora.Rng(13).gaussian(160)
    assert m.encode(key, 5).tobytes() == m.encode(key, 5).tobytes()


def test_fwht_orthogonal_inverse_and_next_pow2():
    # scirust/src/incoherence.rs:134-176
    v = ora.Rng(11).gaussian(128)
    w = ora.fwht(ora.fwht(v))
    assert np.all(np.abs(w - v) <= 1e-4 * (1 + np.abs(v)))
    assert [ora.lib.ora_next_pow2(n) for n in (1, 2, 160, 257)] == [1, 2, 256, 512]


def test_rht_model_pads_to_pow2_and_preserves_dot():
    # scirust/src/incoherence.rs:178-214
    p = H.orthogonal_projection(2, 160)
    m = ora.Model(p, 160, seed=99, rht=True)
    assert m.d_pad == 256 and m.z.shape == (256, 256)
    assert set(np.unique(m.rht_diag)) <= {-1.0, 1.0}


def test_weights_parser_contract():
    # scirust/src/weights.rs:159-270 and its tests :313-513
    p = H.orthogonal_projection(3, 160)
    blob = ora.weights_to_bytes(p, 160, 42, True)
    m = ora.weights_from_bytes(blob)
    assert m.d == 160 and m.d_pad == 256
    assert ora.weights_from_bytes(ora.weights_to_bytes(p, 160, 42, False, version=1)).d_pad == 160
    bad = bytearray(blob)
    bad[40] ^= 1
    with pytest.raises(ValueError, match="checksum"):
        ora.weights_from_bytes(bad)
    with pytest.raises(ValueError, match="magic"):
        ora.weights_from_bytes(b"XXXX" + blob[4:])
    with pytest.raises(ValueError, match="dimension"):
        ora.weights_from_bytes(ora.weights_to_bytes(np.zeros((128, 128), F), 128, 1, False))
    with pytest.raises(ValueError, match="size"):
        ora.weights_from_bytes(blob[:-4])


def test_validate_tile_rules():
    # slha-c/src/lib.rs:244-286
    t = ora.make_tile(np.zeros(64, np.uint8), 1.0, np.full(8, 255, np.uint8))
    assert ora.validate_tile(t) == 0
    for flags, rc in ((1 << 6, -6), (ora.FLAG_NF4 | ora.FLAG_TQ3, -6), (ora.FLAG_TQ3_NOCORR, -6),
                      (ora.FLAG_TQ3 | ora.FLAG_TQ3_NOCORR, 0), (ora.FLAG_MIX3 | ora.FLAG_WARM, 0)):
        u = t.copy()
        u["flags"] = flags
        assert ora.validate_tile(u) == rc
    u = t.copy()
    u["scale"] = np.nan
    assert ora.validate_tile(u) == -5
    u = t.copy()
    u["dynamic_lambda"] = -1.0
    assert ora.validate_tile(u) == -6


def test_topk_order_ties_to_lower_index():
    # scirust/src/metrics.rs:186-192
    s = np.array([1.0, 3.0, 3.0, -0.0, 0.0, 2.0], F)
    idx, val = ora.topk(s, 6)
    assert list(idx) == [1, 2, 5, 0, 4, 3]  # +0.0 orders above -0.0 under total_cmp
    assert list(val[:4]) == [3.0, 3.0, 2.0, 1.0]


def test_softmax_into_known_answers_of_the_reference():
    # scirust/src/metrics.rs:331-337 (doc test), :444-449, :483-489, :516-538
    inf, nan = np.inf, np.nan
    w = ora.softmax_into([0.0, 0.0, 0.0], 1.0)
    assert abs(w.sum() - 1.0) < 1e-6 and abs(w[0] - 1.0 / 3.0) < 1e-6
    assert len(ora.softmax_into([], 1.0)) == 0
    assert np.array_equal(ora.softmax_into([-inf] * 4, 1.0), np.zeros(4, np.float32))
    assert np.array_equal(ora.softmax_into([0.0, nan], 1.0), [0.0, 0.0])
    assert np.array_equal(ora.softmax_into([0.0, 1.0], inf), [0.0, 0.0])
    assert np.array_equal(ora.softmax_into([1.0, inf, inf, -inf], 1.0), [0.0, 0.5, 0.5, 0.0])
    o = ora.softmax_into([0.0, -inf, 1.0, -inf], 1.0)
    assert o[0] > 0 and o[1] == 0 and o[2] > o[0] and o[3] == 0 and abs(o.sum() - 1.0) < 1e-6
    assert np.all(np.abs(ora.softmax_into([1.0, 2.0, 3.0, 4.0], 0.0) - 0.25) < 1e-6)


def test_attend_topk_is_softmax_then_sequential_weighted_sum():
    # scirust/examples/benchmark_decode.rs:28-38, :82-95 on a hand-checkable case
    v = np.array([[1.0, 0.0], [0.0, 2.0], [4.0, 4.0]], np.float32)
    idx = np.array([[2, 0, 0xFFFFFFFF]], np.uint32)
    sc = np.array([[0.0, 0.0, 5.0]], np.float32)
    out, w = ora.attend_topk(idx, sc, 1.0, v)
    assert np.allclose(w, [[0.5, 0.5, 0.0]]) and np.allclose(out, [[2.5, 2.0]])


def test_eventlog_layout_matches_the_documented_format():
    # scirust/src/eventlog.rs:9-24: 16-byte header, 144-byte records, FNV-1a (offset basis 0x811C9DC5, prime 0x01000193)
    tile = np.zeros(1, ora.TILE_DTYPE)
    tile["token_id"] = 77
    data = ora.eventlog_bytes([(5, 9, tile), (6, 2, tile)])
    assert len(data) == 16 + 2 * 144
    assert data[:16] == bytes.fromhex("474c4c53" "02000000" "80000000" "00000000")
    assert data[16:28] == (5).to_bytes(8, "little") + (9).to_bytes(4, "little")
    h = 0x811C9DC5
    for b in data[16:28] + data[32:160]:
        h = ((h ^ b) * 0x01000193) & 0xFFFFFFFF
    assert int.from_bytes(data[28:32], "little") == h
    version, recs = ora.eventlog_parse(data)
    assert version == 2 and [(r[0], r[1]) for r in recs] == [(5, 9), (6, 2)]
    assert recs[0][2].tobytes() == tile.tobytes()
    # version 1 carries zero in place of the checksum and stays readable
    v1 = ora.eventlog_bytes([(5, 9, tile)], version=1)
    assert v1[28:32] == b"\0\0\0\0" and ora.eventlog_parse(v1)[0] == 1
    for bad in (data[:10], b"XXXX" + data[4:], data[:4] + (3).to_bytes(4, "little") + data[8:], data + b"\1" * 7,
                data[:40] + bytes([data[40] ^ 1]) + data[41:]):
        with pytest.raises(ValueError):
            ora.eventlog_parse(bad)
