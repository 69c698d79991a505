"""The reference's end-to-end tests of the learned encode path (tests/reference_learned_cases.py) on the GPU library:
encode, prepare_query, scoring and decode all through the C ABI."""
import numpy as np
import pytest

from . import reference_learned_cases as cases

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")


class DeviceModel:
    def __init__(self, p, d, seed, rht):
        self.m = S.Model.from_projection(p, d, seed, rht=rht)

    def encode(self, keys, codec):
        return self.m.encode_keys(np.ascontiguousarray(keys, np.float32), codec, positions=np.arange(len(keys), dtype=np.uint32))

    def prepare(self, q):
        qc, qs = self.m.prepare_queries(np.ascontiguousarray(q, np.float32)[None])
        return qc[0], qs[0]

    def score(self, tiles, qc, qs):
        return S.score_tiles(tiles, len(tiles), qc[None], qs[None], 1)[0]

    def decode_latent(self, tile):
        return self.m.decode_latent(tile)

    def decode_key(self, tile):
        return self.m.decode_key(tile)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.__name__)
def test_reference_case_on_the_device(case):
    case(DeviceModel)
