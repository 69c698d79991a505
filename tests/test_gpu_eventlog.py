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


# ---- the reference's own persistence tests (scirust/tests/ccos.rs:609-785), same seeds and budgets ----------------
def _scenario_tiles(proj_seed, gen_seed, n, rho):
    z = H.scenario_projection(proj_seed)
    _, toks = H.scenario_generate(gen_seed, n, rho)
    return [H.scenario_tile(z, t, i) for i, t in enumerate(toks)]


def test_durable_eviction_persists_before_recycling(tmp_path):
    # ccos.rs:609-639
    path = tmp_path / "durable_success"
    pool = S.TilePool(4, 2 ** 62)
    pool.attach_event_log(path, require_durable=True)
    slot = int(pool.insert(_scenario_tiles(0xD001, 0xD001, 1, 0.3)[0])[0])
    assert pool.evict(slot) and pool.read(slot, 1)[1][0] == ora.COLD
    assert pool.event_log_stats() == {"records": 1, "log_errors": 0, "blocked_evictions": 0}
    pool.destroy()
    assert len(ora.eventlog_parse(open(path, "rb").read())[1]) == 1


def test_durable_eviction_failure_keeps_tile_live(tmp_path):
    # ccos.rs:641-686: budget zero stays unmet, the tile stays live, its slot is not recycled, the log stays empty
    path = tmp_path / "durable_failure"
    first = S.TilePool(1, 0)
    first.attach_event_log(path)  # creates an empty log
    first.destroy()
    pool = S.TilePool(4, 0)
    pool.attach_event_log(path, mode=4, require_durable=True)
    tile = _scenario_tiles(0xD002, 0xD002, 1, 0.3)[0]
    slot = int(pool.insert(tile)[0])
    assert pool.enforce_budget() is False
    assert pool.read(slot, 1)[1][0] != ora.COLD and pool.live_bytes() > 0
    st = pool.event_log_stats()
    assert st["log_errors"] == 1 and st["blocked_evictions"] == 1
    tile["position"] = 1
    assert int(pool.insert(tile)[0]) != slot
    pool.destroy()
    assert len(ora.eventlog_parse(open(path, "rb").read())[1]) == 0


def test_evict_snapshots_to_event_log_then_rehydrates_identically(tmp_path):
    # ccos.rs:688-747
    path = tmp_path / "roundtrip"
    pool = S.TilePool(16, 2 * 128)
    pool.attach_event_log(path)
    tiles = _scenario_tiles(0xE7, 9, 5, 0.4)
    for t in tiles:
        pool.insert(t)
    pool.enforce_budget()
    cold = pool.counts()[2]
    assert cold >= 3 and pool.event_log_stats()["log_errors"] == 0
    _, recs = ora.eventlog_parse(open(path, "rb").read())
    assert len(recs) == cold
    for seq, _slot, tile in recs:
        assert tile["latent_kv"].tobytes() == tiles[seq]["latent_kv"].tobytes()
        assert int(tile["flags"][0]) & ora.FLAG_WARM  # paged WARM before it was evicted
    logged0 = next(r for r in recs if r[0] == 0)[2]
    slot = pool.rehydrate(0)
    assert slot is not None
    t, state, _, _ = pool.read(slot, 1)
    assert state[0] == ora.WARM and t.tobytes() == np.ascontiguousarray(logged0).tobytes()


def test_eviction_order_is_reflected_in_the_log(tmp_path):
    # ccos.rs:749-767: causal eviction, one enforce per insert -> records of seq 0, 1, 2
    path = tmp_path / "order"
    pool = S.TilePool(8, 128)
    pool.attach_event_log(path)
    for t in _scenario_tiles(0xA5, 3, 4, 0.3):
        pool.insert(t)
        pool.enforce_budget()
    assert [r[0] for r in ora.eventlog_parse(open(path, "rb").read())[1]] == [0, 1, 2]


def test_no_event_log_leaves_behavior_and_rehydrate_inert():
    # ccos.rs:769-785
    pool = S.TilePool(8, 128)
    for t in _scenario_tiles(0x11, 2, 3, 0.3):
        pool.insert(t)
    pool.enforce_budget()
    assert pool.event_log_stats()["log_errors"] == 0
    assert pool.rehydrate(0) is None


def test_legacy_version_one_log_stays_readable_and_appendable(tmp_path):
    # scirust/src/eventlog.rs:753-786: a version-1 file (no record checksums) is accepted, and what is appended to it
    # stays in version-1 form (checksum field zero), so the reference's reader accepts the whole file
    path = tmp_path / "legacy_v1"
    tiles = H.random_tiles(3, 1, seed=12)
    path.write_bytes(ora.eventlog_bytes([(1, 4, tiles[0:1])], version=1))
    pool = S.TilePool(8, 2 ** 62)
    pool.attach_event_log(path, mode=2)
    assert pool.event_log_stats()["records"] == 1
    slot = int(pool.insert(tiles[1:2])[0])
    assert pool.evict(slot)
    pool.destroy()
    data = path.read_bytes()
    version, recs = ora.eventlog_parse(data)
    assert version == 1 and len(recs) == 2 and data[16 + 144 + 12:16 + 144 + 16] == bytes(4)
    assert recs[1][2].tobytes() == tiles[1:2].tobytes()


def test_rehydrate_takes_the_latest_record_of_a_sequence_number(tmp_path):
    # eventlog.rs:592-609 (fetch_by_seq returns the newest record of a seq) through slha_b200_pool_rehydrate
    path = tmp_path / "fetch"
    tiles = H.random_tiles(3, 2, seed=13)
    path.write_bytes(ora.eventlog_bytes([(100, 0, tiles[0:1]), (100, 0, tiles[1:2]), (200, 1, tiles[2:3])]))
    pool = S.TilePool(8, 2 ** 62)
    pool.attach_event_log(path, mode=2)
    slot = pool.rehydrate(100)
    assert slot is not None and pool.read(slot, 1)[0].tobytes() == tiles[1:2].tobytes()
    assert pool.rehydrate(999) is None
