"""Error contract of the reference's C ABI (slha-c/src/lib.rs tests :952-1886)."""
import ctypes as C

import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


@pytest.fixture(scope="module")
def model():
    _, p = H.make_model_pair(160, seed=7)
    return S.Model.from_projection(p, 160, 7)


def test_null_nan_dimension_codec_rejections_leave_outputs_untouched(model):
    lib = S.load_library()
    key = H.gaussian_keys(1, 1, 160)[0]
    out = np.full(1, 0xAB, np.uint8).repeat(128).view(S.TILE_DTYPE)
    sentinel = out.tobytes()
    assert lib.slha_encode_key(model.handle, None, 160, 0, 1, S.ptr(out)) == S.ERR_NULL
    assert lib.slha_encode_key(model.handle, S.ptr(key), 159, 0, 1, S.ptr(out)) == S.ERR_DIMENSION
    assert b"expected 160" in lib.slha_last_error_message()
    assert lib.slha_encode_key(model.handle, S.ptr(key), 160, 0, 6, S.ptr(out)) == S.ERR_CODEC
    bad = key.copy()
    bad[3] = np.nan
    assert lib.slha_encode_key(model.handle, S.ptr(bad), 160, 0, 1, S.ptr(out)) == S.ERR_NONFINITE
    assert b"key[3]" in lib.slha_last_error_message()
    assert lib.slha_encode_key(None, S.ptr(key), 160, 0, 1, S.ptr(out)) == S.ERR_NULL
    forged = (C.c_uint64 * 1)(0)
    assert lib.slha_encode_key(C.addressof(forged), S.ptr(key), 160, 0, 1, S.ptr(out)) == S.ERR_INVALID_HANDLE
    assert lib.slha_encode_key(C.addressof(forged) + 1, S.ptr(key), 160, 0, 1, S.ptr(out)) == S.ERR_INVALID_HANDLE
    assert out.tobytes() == sentinel
    assert lib.slha_encode_key(model.handle, S.ptr(key), 160, 0, 1, S.ptr(out)) == S.OK
    assert lib.slha_last_error_message() == b""


def test_score_tiles_contract(model):
    lib = S.load_library()
    tiles = H.random_tiles(64, 1, seed=1)
    qc, qs = H.random_queries(1, 2)
    out = np.full(64, 7.0, F)
    big = (1 << 20) + 1
    assert lib.slha_score_tiles(model.handle, S.ptr(tiles), big, S.ptr(qc), S.ptr(qs), S.ptr(out)) == S.ERR_DIMENSION
    assert lib.slha_score_tiles(model.handle, S.ptr(tiles), 0, S.ptr(qc), S.ptr(qs), S.ptr(out)) == S.OK
    t2 = tiles.copy()
    t2["flags"][40] = 1 << 9
    assert lib.slha_score_tiles(model.handle, S.ptr(t2), 64, S.ptr(qc), S.ptr(qs), S.ptr(out)) == S.ERR_INVALID_TILE
    t2 = tiles.copy()
    t2["scale"][10] = np.inf
    assert lib.slha_score_tiles(model.handle, S.ptr(t2), 64, S.ptr(qc), S.ptr(qs), S.ptr(out)) == S.ERR_NONFINITE
    qn = qc.copy()
    qn[0, 5] = np.nan
    assert lib.slha_score_tiles(model.handle, S.ptr(tiles), 64, S.ptr(qn), S.ptr(qs), S.ptr(out)) == S.ERR_NONFINITE
    assert np.all(out == 7.0)
    # batch == repeated single (lib.rs:1314), also with unaligned storage
    got = model.score_tiles(tiles, qc[0], qs[0])
    raw = np.zeros(64 * 128 + 1, np.uint8)
    raw[1:] = tiles.view(np.uint8)
    one = np.zeros(1, F)
    for i in (0, 13, 63):
        assert lib.slha_score_tile(model.handle, raw.ctypes.data + 1 + 128 * i, S.ptr(qc), S.ptr(qs), S.ptr(one)) == S.OK
        assert one[0] == got[i]
    assert np.all(np.abs(got - ora.score_tiles(tiles, qc[0], qs[0])) <= 1e-3)


def test_weights_load_roundtrip_and_release(tmp_path, model):
    lib = S.load_library()
    p = H.orthogonal_projection(5, 192)
    path = tmp_path / "m.slhw"
    path.write_bytes(ora.weights_to_bytes(p, 192, 99, True))
    m = S.Model.load(str(path))
    assert m.d == 192
    om = ora.Model(p, 192, seed=99, rht=True)
    key = H.gaussian_keys(2, 1, 192)[0]
    assert m.encode_key(key, 4, S.CODEC_TQ3).tobytes() == om.encode(key, 4, codec=4).tobytes()
    blob = bytearray(path.read_bytes())
    blob[100] ^= 0xFF
    (tmp_path / "bad.slhw").write_bytes(blob)
    assert not lib.slha_weights_load(str(tmp_path / "bad.slhw").encode())
    assert b"checksum" in lib.slha_last_error_message()
    assert not lib.slha_weights_load(str(tmp_path / "absent.slhw").encode())
    h = m.handle
    m.release()
    assert lib.slha_model_dim(h) == 0  # stale handle never revives
    assert lib.slha_weights_release(h) == S.ERR_INVALID_HANDLE
    assert lib.slha_weights_release(None) == S.OK


def test_audit_reports_known_answers():
    import json

    rep = json.loads(S.audit())
    assert rep["tile_size"] == 128 and rep["int4_known_answers"] is True and rep["devices"] >= 1


def test_weights_file_contract_of_the_reference(tmp_path):
    # scirust/src/weights.rs tests :352-512 through slha_weights_load: every malformed file is refused with the reference's
    # message, a version-1 file stays readable, and a loaded model encodes like the model it was saved from
    lib = S.load_library()
    d = 129  # the smallest valid dimension (weights.rs:318)
    p = H.orthogonal_projection(8, d)

    def load(blob, name="w.slhw"):
        path = tmp_path / name
        path.write_bytes(bytes(blob))
        h = lib.slha_weights_load(str(path).encode())
        return h, lib.slha_last_error_message()

    v2 = bytearray(ora.weights_to_bytes(p, d, 0xC0FFEE, False))
    v1 = bytearray(ora.weights_to_bytes(p, d, 0x1E6AC001, True, version=1))
    assert int.from_bytes(v2[4:8], "little") == 2
    for blob, seed, rht in ((v2, 0xC0FFEE, False), (v1, 0x1E6AC001, True)):
        h, _ = load(blob)
        assert h and lib.slha_model_dim(h) == d
        key = H.gaussian_keys(4, 1, d)[0]
        out = np.zeros(1, S.TILE_DTYPE)
        assert lib.slha_encode_key(h, S.ptr(key), d, 3, S.CODEC_MIXED, S.ptr(out)) == S.OK
        assert out.tobytes() == ora.Model(p, d, seed=seed, rht=rht).encode(key, 3, codec=3).tobytes()
        assert lib.slha_weights_release(h) == S.OK
    header = len(v2) - 4 * 128 * d
    bad = bytearray(v2)
    bad[header + 17] ^= 0x80                      # payload corruption (:386-400)
    h, msg = load(bad)
    assert not h and b"checksum mismatch" in msg
    bad = bytearray(v2)
    bad[12] ^= 0x01                               # one seed byte: the checksum covers the header (:402-418)
    h, msg = load(bad)
    assert not h and b"checksum mismatch" in msg
    small = bytearray(24)
    small[0:8] = v1[0:8]
    small[8:12] = (128).to_bytes(4, "little")     # d <= D_C (:432-452)
    h, msg = load(small)
    assert not h and b"invalid dimension" in msg
    small[8:12] = (0xFFFFFFFF).to_bytes(4, "little")
    assert not load(small)[0]
    bad = bytearray(v1)
    bad[20] = 2                                   # (:454-474)
    h, msg = load(bad)
    assert not h and b"invalid RHT flag" in msg
    bad = bytearray(v1)
    bad[22] = 1
    h, msg = load(bad)
    assert not h and b"reserved" in msg
    bad = bytearray(v1)
    bad[24:28] = np.array([np.nan], F).tobytes()  # (:476-491)
    h, msg = load(bad)
    assert not h and b"non-finite projection value" in msg
    assert not load(bytes([0, 1, 2]))[0] and not load(bytes(32))[0]  # (:508-512)
