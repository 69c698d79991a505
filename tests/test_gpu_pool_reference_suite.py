"""scirust/tests/ccos.rs restated (tests/reference_ccos_cases.py) on the device pool, through the C ABI."""
import numpy as np
import pytest

from . import reference_ccos_cases as cases

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")


class DevicePool:
    def __init__(self, budget, evict_policy, sink_window):
        self.pool = S.TilePool(64, budget, S.PAGE_LOWEST_IMPACT_FIRST, evict_policy, sink_window)

    def insert(self, tile):
        return int(self.pool.insert(np.ascontiguousarray(tile))[0])

    def state(self, s):
        return int(self.pool.read(s, 1)[1][0])

    def flags(self, s):
        return int(self.pool.read(s, 1)[0]["flags"][0])

    def importance(self, s):
        return float(self.pool.read(s, 1)[2][0])

    def live_bytes(self):
        return self.pool.live_bytes()

    def counts(self):
        return self.pool.counts()

    def nocorr_count(self):
        return self.pool.stats()["nocorr"]

    def reclaimed_correction_bytes(self):
        return self.pool.stats()["reclaimed_correction_bytes"]

    def observe_scores(self, slots, scores, temperature):
        self.pool.observe_scores(slots, scores, temperature)

    def evict(self, s):
        return self.pool.evict(s)

    def enforce_budget(self):
        return self.pool.enforce_budget()

    def score_all(self, q, q_sign):
        return self.pool.score_all(q, q_sign)


def make(budget, evict_policy=0, sink_window=0):
    return DevicePool(budget, evict_policy, sink_window)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.__name__)
def test_reference_case_on_the_device_pool(case):
    case(make)
