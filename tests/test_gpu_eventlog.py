"""COLD persistence of the device pool: the log file must hold exactly the records (and bytes) the
reference's EventLog would hold for the same evictions (scirust/src/eventlog.rs:9-24,
scirust/src/ccos.rs:404-466; reference tests scirust/tests/ccos.rs:609-785)."""
import os

import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def test_evictions_are_logged_in_order_and_bytes_match_the_reference_format(tmp_path):
    # importance eviction with sinks under a tight budget: enforce_budget evicts in (is_sink, importance, seq) order
    n, budget = 400, 128 * 150
    tiles = H.random_tiles(n, 1, seed=9)
    tiles["position"] = np.arange(n, dtype=np.uint32)
    path = tmp_path / "evicted.sllg"
    pool = S.TilePool(n, budget, S.PAGE_LOWEST_IMPACT_FIRST, S.EVICT_IMPORTANCE, sink_window=4)
    pool.attach_event_log(path)
    cache = ora.Cache(budget, 0, 1, 4, 0)
    slots = pool.insert(tiles)
    assert list(slots) == [cache.insert(tiles[i:i + 1]) for i in range(n)]
    imp = ora.Rng(3).gaussian(n)
    pool.observe_scores(np.arange(n, dtype=np.uint32), imp, 1.0)
    cache.observe_scores(np.arange(n, dtype=np.uint32), imp, 1.0)
    assert pool.enforce_budget() == cache.enforce_budget()
    assert pool.evict(7) == cache.evict(7) and pool.evict(7) == cache.evict(7)  # second time: already COLD, nothing logged
    journal = cache.journal()
    assert len(journal) > 100
    st = pool.event_log_stats()
    assert st == {"records": len(journal), "log_errors": 0, "blocked_evictions": 0}
    data = open(path, "rb").read()
    assert data == ora.eventlog_bytes(journal)  # byte-identical file
    version, recs = ora.eventlog_parse(data)
    assert version == 2 and [r[:2] for r in recs] == [j[:2] for j in journal]
    # rehydrate: a fresh admission of the logged tile (LIFO slot reuse, new seq, HOT / WARM from the tile's flag)
    seq5, slot5, tile5 = journal[5]
    got = pool.rehydrate(seq5)
    want = cache.insert(tile5)  # ElasticKvCache::rehydrate = insert_with_state(record.tile, state from the WARM flag)
    assert got == want
    t, state, _, seqs = pool.read()
    assert t[got].tobytes() == np.ascontiguousarray(tile5).tobytes() and state[got] == cache.state(want)
    assert seqs[got] == cache.seq(want)
    assert pool.rehydrate(10 ** 12) is None
    assert pool.stats()["live_bytes"] == cache.live_bytes()


def test_reopen_strictly_recover_a_torn_tail_and_reject_corruption(tmp_path):
    n = 64
    tiles = H.random_tiles(n, 2, seed=4)
    path = tmp_path / "log.sllg"
    pool = S.TilePool(n, 128 * n, S.PAGE_OLDEST_FIRST, S.EVICT_CAUSAL)
    pool.attach_event_log(path, mode=1)
    with pytest.raises(S.SlhaError) as e:  # create_new refuses to overwrite a journal
        S.TilePool(n, 128 * n).attach_event_log(path, mode=1)
    assert e.value.code == S.ERR_IO
    pool.insert(tiles)
    for s in (3, 9, 11):
        assert pool.evict(s)
    pool.attach_event_log(None)
    good = open(path, "rb").read()
    assert len(good) == 16 + 3 * 144
    # strict open continues the same log
    pool.attach_event_log(path, mode=2)
    assert pool.event_log_stats()["records"] == 3
    assert pool.evict(20) and pool.event_log_stats()["records"] == 4
    pool.attach_event_log(None)
    # a torn tail: strict open refuses, recovery drops the partial record only
    whole = open(path, "rb").read()
    open(path, "wb").write(whole + b"\x01" * 50)
    with pytest.raises(S.SlhaError):
        pool.attach_event_log(path, mode=2)
    pool.attach_event_log(path, mode=3)
    assert pool.event_log_stats()["records"] == 4 and os.path.getsize(path) == len(whole)
    pool.attach_event_log(None)
    # corruption of a complete record stays fatal
    bad = bytearray(whole)
    bad[16 + 144 + 40] ^= 0xFF
    open(path, "wb").write(bytes(bad))
    for mode in (2, 3, 4):
        with pytest.raises(S.SlhaError) as e:
            pool.attach_event_log(path, mode=mode)
        assert e.value.code == S.ERR_IO and b"checksum" in e.value.message.encode()
    # header errors
    open(path, "wb").write(b"XXXX" + whole[4:])
    with pytest.raises(S.SlhaError):
        pool.attach_event_log(path, mode=2)


def test_durable_eviction_refuses_cold_when_the_log_cannot_be_written(tmp_path):
    # scirust/tests/ccos.rs:641-686: with RequireDurable a failed append leaves the slot live
    n = 32
    tiles = H.random_tiles(n, 1, seed=6)
    path = tmp_path / "ro.sllg"
    pool = S.TilePool(n, 128 * 8, S.PAGE_OLDEST_FIRST, S.EVICT_CAUSAL)
    pool.attach_event_log(path)           # creates a valid empty log ...
    pool.attach_event_log(path, mode=4, require_durable=True)  # ... re-attached read-only: appends fail
    pool.insert(tiles)
    assert pool.evict(2) is False
    st = pool.stats()
    assert st["cold"] == 0
    assert pool.event_log_stats() == {"records": 0, "log_errors": 1, "blocked_evictions": 1}
    assert pool.enforce_budget() is False   # paging happens, evictions are all refused
    st = pool.stats()
    assert st["cold"] == 0 and st["warm"] == n and pool.event_log_stats()["blocked_evictions"] == 1 + n
    # best effort: the eviction proceeds and only the error is counted
    pool.attach_event_log(path, mode=4, require_durable=False)
    assert pool.evict(2) is True and pool.event_log_stats()["log_errors"] >= 2
