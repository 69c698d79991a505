"""The reference's end-to-end tests of the learned encode path (tests/reference_learned_cases.py) on the oracle."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from . import reference_learned_cases as cases


class OracleModel:
    def __init__(self, p, d, seed, rht):
        self.m = ora.Model(p, d, seed=seed, rht=rht)

    def encode(self, keys, codec):
        return self.m.encode_batch(np.ascontiguousarray(keys, np.float32), codec)

    def prepare(self, q):
        return self.m.prepare_query(q)

    def score(self, tiles, qc, qs):
        return ora.score_tiles(tiles, qc, qs)

    def decode_latent(self, tile):
        return self.m.decode_latent(tile)

    def decode_key(self, tile):
        return self.m.decode_key(tile)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.__name__)
def test_reference_case_on_the_oracle(case):
    case(OracleModel)
