"""scirust/tests/ccos.rs restated (tests/reference_ccos_cases.py) on the oracle's ElasticKvCache."""
import pytest

from oracle import pyoracle as ora
from . import reference_ccos_cases as cases


class OracleCache(ora.Cache):
    def flags(self, s):
        return int(self.tile(s)["flags"][0])


def make(budget, evict_policy=0, sink_window=0):
    return OracleCache(budget, 0, evict_policy, sink_window, 0)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c.__name__)
def test_reference_case_on_the_oracle(case):
    case(make)
