"""Fused scoring + top-k vs the oracle (score desc, ties -> lower index)."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def check_topk(tiles, segs, qc, qs, k, got_idx, got_sc, got_cnt):
    """Index sets must match except where scores tie within 1e-3."""
    for (tb, nt, qb, nq, base) in segs:
        seg_tiles = tiles[tb:tb + nt]
        for j in range(qb, qb + nq):
            want = ora.score_tiles(seg_tiles, qc[j], qs[j]) if nt else np.zeros(0, F)
            kk = min(k, nt)
            assert got_cnt[j] == kk
            idx = got_idx[j, :kk].astype(np.int64) - base
            assert np.all((idx >= 0) & (idx < nt)) and len(set(idx)) == kk
            # reported scores are the tile scores, sorted descending
            assert np.all(np.abs(got_sc[j, :kk] - want[idx]) <= 1e-3)
            assert np.all(np.diff(got_sc[j, :kk]) <= 0)
            eq = got_sc[j, :kk][1:] == got_sc[j, :kk][:-1]
            assert np.all(got_idx[j, :kk][1:][eq] > got_idx[j, :kk][:-1][eq])  # ties -> lower index first
            if kk < nt:
                oi, ov = ora.topk(want, kk)
                missing = set(oi) - set(idx)
                extra = set(idx) - set(oi)
                thr = ov[-1]
                assert all(abs(want[i] - thr) <= 2e-3 for i in missing | extra), (len(missing), len(extra))
            assert np.all(got_idx[j, kk:] == 0xFFFFFFFF) and np.all(np.isneginf(got_sc[j, kk:]))


@pytest.mark.parametrize("n,k,nq,codec", [(4096, 64, 1, 0), (5000, 100, 4, 2), (333, 1024, 2, 1), (20000, 1024, 4, 2),
                                           (9000, 2048, 3, 6), (257, 1, 1, 4), (70000, 512, 5, 3)])
def test_single_segment(n, k, nq, codec):
    tiles = H.random_tiles(n, codec, seed=n + k, warm_every=9)
    qc, qs = H.random_queries(nq, k)
    segs = [(0, n, 0, nq, 0)]
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_gqa_segments_ragged_and_empty():
    # several KV heads (segments) of different lengths, 4 query heads each, a
    # global index base per segment, one empty segment
    lens = [3000, 1, 0, 8191, 513]
    tiles = H.random_tiles(sum(lens), 2, seed=77)
    nq = 4 * len(lens)
    qc, qs = H.random_queries(nq, 78)
    segs, off = [], 0
    for i, ln in enumerate(lens):
        segs.append((off, ln, 4 * i, 4, 1000 * i))
        off += ln
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, 128)
    check_topk(tiles, segs, qc, qs, 128, gi, gs_, gc)


def test_ties_resolve_to_lower_index():
    base = H.random_tiles(50, 1, seed=5)
    tiles = np.concatenate([base] * 40)  # every score appears 40 times
    qc, qs = H.random_queries(2, 6)
    n = len(tiles)
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments([(0, n, 0, 2, 0)]), qc, qs, 2, 100)
    for j in range(2):
        want = ora.score_tiles(tiles, qc[j], qs[j])
        gpu_all = S.score_tiles(tiles, n, qc[j:j + 1], qs[j:j + 1], 1)[0]
        oi, _ = ora.topk(gpu_all, 100)  # exact order on the GPU's own scores
        assert np.array_equal(gi[j], oi)
        assert np.all(np.abs(gs_[j] - want[oi]) <= 1e-3)


def test_topk_merge_of_shard_lists():
    # two "shards" score disjoint token ranges; merged result == single pass
    n, k, nq = 6000, 256, 4
    tiles = H.random_tiles(n, 6, seed=9)
    qc, qs = H.random_queries(nq, 10)
    dt = S.to_device(tiles)
    full = S.score_topk(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)
    a = S.score_topk(dt, S.make_segments([(0, 2500, 0, nq, 0)]), qc, qs, nq, k)
    b = S.score_topk(dt, S.make_segments([(2500, n - 2500, 0, nq, 2500)]), qc, qs, nq, k)
    ci = np.stack([a[0], b[0]])
    cs = np.stack([a[1], b[1]])
    mi, ms = S.topk_merge(ci, cs, 2, nq, k, k)
    assert np.array_equal(mi, full[0]) and np.array_equal(ms, full[1])


@pytest.mark.parametrize("n_lists,k,skew", [(2, 256, 1.0), (8, 2048, 1.0), (8, 2048, 4.0), (5, 300, 0.0), (3, 64, 1.0), (3, 8192, 1.0), (16, 4096, 2.0),
                                            (64, 512, 1.0)])
def test_merge_of_sorted_lists_uses_a_proven_floor_and_gives_the_same_answer(n_lists, k, skew):
    # lists ordered best first, as score_topk writes them: the merge gathers only the keys at or above the smallest
    # ceil(k / n_lists)-th entry.  Even shards, a shard that holds most of the winners (skew: its scores are shifted
    # up), equal scores everywhere (skew 0: ties decided by index), short lists with absent entries at their ends.
    from slhav2_b200 import shard

    rng = np.random.default_rng(100 + n_lists)
    nq, k_in = 5, k
    sc = rng.standard_normal((n_lists, nq, k_in)).astype(F) if skew else np.zeros((n_lists, nq, k_in), F)
    sc[0] += F(skew if skew != 1.0 else 0.0)
    idx = rng.permutation(n_lists * nq * k_in).astype(np.uint32).reshape(n_lists, nq, k_in)
    order = np.lexsort((idx, -sc), axis=-1)  # best first, ties to the lower index
    sc, idx = np.take_along_axis(sc, order, -1), np.take_along_axis(idx, order, -1)
    idx[1, 2, k_in // 3:] = 0xFFFFFFFF  # a short list: fewer than ceil(k / n_lists) entries in one row disables the floor there
    idx[n_lists - 1, 4, k_in - 3:] = 0xFFFFFFFF
    wi, ws = shard.merge_reference(idx, sc, k)
    for lists_sorted in (True, False):
        mi, ms = S.topk_merge(idx, sc, n_lists, nq, k_in, k, lists_sorted=lists_sorted)
        assert np.array_equal(mi, wi) and np.array_equal(ms, ws), lists_sorted


def test_merge_with_more_candidates_than_the_shared_buffer():
    # 8 lists x 4096 candidates per query exceeds the in-shared-memory path
    rng = np.random.default_rng(3)
    n_lists, nq, k_in, k_out = 8, 3, 4096, 2048
    sc = rng.standard_normal((n_lists, nq, k_in)).astype(F)
    idx = rng.permutation(n_lists * nq * k_in).astype(np.uint32).reshape(n_lists, nq, k_in)
    idx[2, 1, 100:] = 0xFFFFFFFF  # a short list
    mi, ms = S.topk_merge(idx, sc, n_lists, nq, k_in, k_out)
    from slhav2_b200 import shard

    wi, ws = shard.merge_reference(idx, sc, k_out)
    assert np.array_equal(mi, wi) and np.array_equal(ms, ws)


def test_long_segment_many_items_shares_thresholds():
    # one long segment scanned by many CTAs (config-5 shape at reduced length)
    n, k, nq = 300000, 2048, 4
    base = H.random_tiles(5000, 6, seed=11)
    tiles = np.tile(base, n // 5000)
    tiles["dynamic_lambda"] *= (1 + np.random.default_rng(1).random(n)).astype(F)
    qc, qs = H.random_queries(nq, 12)
    dt = S.to_device(tiles)
    segs = [(0, n, 0, nq, 7)]
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_heavy_ties_longer_than_the_candidate_buffers():
    # every score appears 2000 times and the segment is far longer than the in-kernel candidate
    # buffers: the bucket selection cannot separate equal scores, so the item is handed to the
    # generic kernel; the answer is still the exact order, ties to the lower index
    base = H.random_tiles(50, 1, seed=21)
    tiles = np.concatenate([base] * 2000)
    qc, qs = H.random_queries(2, 22)
    n = len(tiles)
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments([(0, n, 0, 2, 0)]), qc, qs, 2, 100)
    assert np.all(gc == 100)
    for j in range(2):
        gpu_all = S.score_tiles(tiles, n, qc[j:j + 1], qs[j:j + 1], 1)[0]
        oi, _ = ora.topk(gpu_all, 100)
        assert np.array_equal(gi[j], oi)


def test_periodic_tiles_do_not_starve_a_warp():
    # a tile pattern that repeats every 4096 tiles sends the same tiles to the same warps of a CTA
    # unless the set assignment rotates; either way the regions are rebalanced and the answer is exact
    n, k, nq = 262144, 1024, 4
    base = H.random_tiles(4096, 2, seed=23)
    tiles = np.tile(base, n // 4096)
    tiles["dynamic_lambda"] *= (1 + 0.3 * np.random.default_rng(2).random(n)).astype(F)
    qc, qs = H.random_queries(2 * nq, 24)
    dt = S.to_device(tiles)
    segs = [(0, n // 2, 0, nq, 0), (n // 2, n // 2, nq, nq, 0)]
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, 2 * nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_large_queries_are_scored_by_the_generic_kernel():
    # |q| above what the fp16 hi/lo split of the tensor-core kernel can carry
    n, k, nq = 30000, 64, 4
    tiles = H.random_tiles(n, 1, seed=25)
    qc, qs = H.random_queries(nq, 26)
    qc = (qc * F(1.0e4)).astype(F)
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)
    assert np.all(gc == k)
    for j in range(nq):
        want = ora.score_tiles(tiles, qc[j], qs[j])
        tol = 1e-3 * (1 + np.abs(want))
        assert np.all(np.abs(gs_[j] - want[gi[j]]) <= tol[gi[j]])
        oi, ov = ora.topk(want, k)
        assert all(abs(want[i] - ov[-1]) <= 2 * tol[i] for i in set(oi) ^ set(gi[j].tolist()))


def test_generic_kernel_only_mode_matches():
    # slha_b200_debug_force_generic_score switches the tensor-core kernel off for this thread:
    # the generic kernel must give the same answers, and both must match the oracle
    n, nq, k = 20000, 4, 256
    t = H.random_tiles(n, 2, seed=4)
    qc, qs = H.random_queries(nq, 5)
    d = S.to_device(t)
    segs = [(0, n, 0, nq, 0)]
    i1, s1, c1 = S.score_topk(d, S.make_segments(segs), qc, qs, nq, k)
    S.debug_force_generic_score(True)
    try:
        i0, s0, c0 = S.score_topk(d, S.make_segments(segs), qc, qs, nq, k)
    finally:
        S.debug_force_generic_score(False)
    check_topk(t, segs, qc, qs, k, i0, s0, c0)
    check_topk(t, segs, qc, qs, k, i1, s1, c1)
    assert np.all(np.abs(s0 - s1) <= 1e-3)
    assert np.mean(i0 == i1) > 0.98


@pytest.mark.parametrize("n,nq,k,foreign", [(33333, 4, 256, 0), (50001, 3, 1024, 0), (40007, 4, 128, 2)])
def test_mixed_8_4_tiles_on_the_tensor_core_kernel(n, nq, k, foreign):
    # mixed 8/4 tiles (8-bit head group + seven INT4 groups, last eight dims dropped), a ragged last
    # set, some WARM tiles; with `foreign` a stretch of NF4 tiles sits inside the mixed launch, whose
    # work items the tensor-core kernel hands back to the generic kernel
    tiles = H.random_tiles(n, 3, seed=n, warm_every=7)
    if foreign:
        other = H.random_tiles(512, foreign, seed=n + 1)
        tiles[20000:20512] = other
    qc, qs = H.random_queries(nq, n + 2)
    qc[1 % nq, :8] *= 30.0  # weight on the 8-bit head dims
    segs = [(0, n, 0, nq, 5)]
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


@pytest.mark.parametrize("n,nq,k,nocorr_every,foreign", [(33335, 4, 256, 0, None), (50001, 3, 1024, 5, None), (40007, 4, 128, 3, 2)])
def test_tq3_tiles_on_the_tensor_core_kernel(n, nq, k, nocorr_every, foreign):
    # TQ3 tiles are rewritten as nibble rows in shared memory and scored by the INT4 path plus one
    # MMA for the half-level offset; ragged last set, WARM tiles, tiles whose correction plane was
    # dropped (NOCORR), and with `foreign` a stretch of NF4 tiles that is handed back
    tiles = H.random_tiles(n, 4, seed=n, warm_every=11, nocorr_every=nocorr_every)
    if foreign:
        tiles[16000:16640] = H.random_tiles(640, foreign, seed=n + 1)
    qc, qs = H.random_queries(nq, n + 2)
    qc[0] += 0.75  # a query with a large sum over every group weighs the half-level offset
    segs = [(0, n, 0, nq, 9)]
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_rejected_call_shape_leaves_no_plan_behind():
    # a segment table that is refused (query range past n_queries; a query row in two segments) must
    # be refused every time it is presented, and a valid call afterwards must still be right: a plan
    # enters the per-thread cache only once it is complete
    n, nq, k = 6000, 4, 64
    tiles = H.random_tiles(n, 1, seed=77)
    qc, qs = H.random_queries(nq, 78)
    dt = S.to_device(tiles)
    bad_range = S.make_segments([(0, n, 2, 4, 0)])            # rows 2..5 of 4
    twice = S.make_segments([(0, 3000, 0, 4, 0), (3000, 3000, 2, 2, 0)])
    for bad in (bad_range, twice):
        for _ in range(3):
            with pytest.raises(S.SlhaError) as e:
                S.score_topk(dt, bad, qc, qs, nq, k)
            assert e.value.code == S.ERR_DIMENSION
    segs = [(0, n, 0, nq, 0)]
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)
    with pytest.raises(S.SlhaError):
        S.score_topk(dt, bad_range, qc, qs, nq, k)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


@pytest.mark.parametrize("n,nq,k,codec,warm,nocorr,foreign", [
    (5000, 64, 64, 1, 0, 0, None),       # MX-INT4, a full 64-row item, ragged last block
    (33001, 37, 256, 6, 9, 0, None),     # MX-32, 37 rows (a partial item), WARM tiles
    (12800, 16, 128, 4, 7, 5, None),     # TQ3 with WARM tiles and tiles whose correction plane was dropped
    (9000, 100, 32, 4, 0, 0, None),      # TQ3, two items of 64 + 36 rows
    (20000, 24, 100, 0, 0, 0, 2),        # INT4 with a stretch of NF4 tiles: the rows are handed to the generic kernel
    (127, 20, 200, 1, 0, 0, None),       # fewer tiles than k and than one block
    (21000, 40, 128, 3, 8, 0, None),     # mixed 8/4 (8-bit head levels split over two K slots each), WARM tiles
    (7000, 64, 512, 3, 0, 0, 1),         # mixed 8/4 with a stretch of MX-INT4 tiles: handed to the generic kernel
])
def test_wide_scoring_on_the_tcgen05_kernel(n, nq, k, codec, warm, nocorr, foreign):
    # 16 or more queries per segment: score_wide_kernel (128-tile blocks x up to 64 query rows on tcgen05 MMAs)
    tiles = H.random_tiles(n, codec, seed=n + nq, warm_every=warm, nocorr_every=nocorr)
    if foreign:
        tiles[6000:6300] = H.random_tiles(300, foreign, seed=n + 1)
    qc, qs = H.random_queries(nq, n + 3)
    qc[nq // 2] += 0.5  # a query with large group sums weighs the TQ3 half-level term
    segs = [(0, n, 0, nq, 11)]
    dt = S.to_device(tiles)
    gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)
    st = S.last_score_stats()
    assert st["rows"] == nq and st["rows_handed_to_generic_kernel"] == (nq if foreign else 0)


def test_wide_scoring_two_segments_and_repeat():
    # two KV heads with 48 queries each; the second call must not see anything the first left behind
    n, qph, k = 7000, 48, 80
    tiles = H.random_tiles(2 * n, 6, seed=77)
    dt = S.to_device(tiles)
    segs = [(0, n, 0, qph, 0), (n, n, qph, qph, 0)]
    for seed in (1, 2):
        qc, qs = H.random_queries(2 * qph, seed)
        gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, 2 * qph, k)
        check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_outputs_in_page_locked_host_memory_are_written_in_place():
    # the same call with pageable numpy outputs (staging copy) and with page-locked outputs the GPU addresses directly
    torch = pytest.importorskip("torch")
    n, k, nq = 20000, 128, 4
    tiles = H.random_tiles(n, 0, seed=31)
    qc, qs = H.random_queries(nq, 32)
    dt = S.to_device(tiles)
    segs = S.make_segments([(0, n, 0, nq, 0)])
    want = S.score_topk(dt, segs, qc, qs, nq, k)
    pi = torch.full((nq, k), -1, dtype=torch.int32).pin_memory()
    ps = torch.zeros(nq, k, dtype=torch.float32).pin_memory()
    pc = torch.zeros(nq, dtype=torch.int32).pin_memory()
    S.score_topk(dt, segs, qc, qs, nq, k, out_index=pi, out_score=ps, out_count=pc)
    S.synchronize()
    assert np.array_equal(pi.numpy().view(np.uint32), want[0]) and np.array_equal(ps.numpy(), want[1])
    assert np.array_equal(pc.numpy().view(np.uint32), want[2])


@pytest.mark.parametrize("trial", range(16))
def test_random_call_shapes_match_the_oracle(trial):
    # segments of random lengths (some empty, some a single tile, some long enough to be cut over many CTAs), 1 to 9
    # or 20 to 40 query rows each (so the four-query, the generic and the 64-query kernels all get work), random k and
    # index bases, one codec per call; a second identical call exercises the cached plan and the cleared streaming state
    rng = np.random.default_rng(7000 + trial)
    codec = [0, 1, 2, 3, 4, 6][trial % 6]
    wide = trial % 4 == 3 and codec in (0, 1, 3, 4, 6)
    n_seg = int(rng.integers(1, 7))
    lens = [int(rng.choice([0, 1, 17, int(rng.integers(2, 3000)), int(rng.integers(3000, 60000))])) for _ in range(n_seg)]
    nqs = [int(rng.integers(20, 41)) if wide else int(rng.integers(1, 10)) for _ in range(n_seg)]
    k = int(rng.choice([1, 7, 64, 500, 1024, 3000]))
    total = max(sum(lens), 1)
    tiles = H.random_tiles(total, codec, seed=300 + trial, warm_every=11, nocorr_every=7)[:sum(lens)]
    qc, qs = H.random_queries(sum(nqs), 400 + trial)
    segs, tb, qb = [], 0, 0
    for n, q in zip(lens, nqs):
        segs.append((tb, n, qb, q, int(rng.integers(0, 1000))))
        tb += n
        qb += q
    dt = S.to_device(tiles if len(tiles) else np.zeros(1, S.TILE_DTYPE))
    for _ in range(2):
        gi, gs_, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, sum(nqs), k)
        check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


@pytest.mark.parametrize("codec,n,nq,k", [(6, 300000, 4, 1024), (2, 120000, 4, 512), (4, 16384, 64, 256), (5, 50000, 3, 100)])
def test_repeated_calls_are_bitwise_identical(codec, n, nq, k):
    # slhav2-vram/tests/cuda.rs:327 (deterministic scoring) and :405 (a thousand launches) for the fused call: the order in
    # which warps append candidates varies from launch to launch, the winners, their order and their scores must not
    tiles = H.random_tiles(n, codec, seed=90 + codec, warm_every=9, nocorr_every=4)
    dt = S.to_device(np.concatenate([tiles, tiles]))
    segs = S.make_segments([(0, n, 0, nq, 0), (n, n, nq, nq, 7)])
    qc, qs = H.random_queries(2 * nq, 91)
    first = S.score_topk(dt, segs, qc, qs, 2 * nq, k)
    for _ in range(6):
        again = S.score_topk(dt, segs, qc, qs, 2 * nq, k)
        for a, b in zip(first, again):
            assert a.tobytes() == b.tobytes()
    m = min(nq, 4)
    full = S.score_tiles(dt, 2 * n, qc[:m], qs[:m], m)
    assert S.score_tiles(dt, 2 * n, qc[:m], qs[:m], m).tobytes() == full.tobytes()


def test_largest_k_long_and_short_segments():
    # k at its maximum (4096): a long segment on the streaming kernel, one shorter than k, one a little longer than k
    k = 4096
    lens = [150000, 3000, 4100]
    tiles = H.random_tiles(sum(lens), 6, seed=611, warm_every=13)
    qc, qs = H.random_queries(3 * 3, 612)
    segs, tb = [], 0
    for i, n in enumerate(lens):
        segs.append((tb, n, 3 * i, 3, 10 * i))
        tb += n
    gi, gs_, gc = S.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, 9, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)
    with pytest.raises(S.SlhaError) as e:
        S.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, 9, k + 1)
    assert e.value.code == S.ERR_DIMENSION


def test_thousands_of_tiny_segments():
    # 3000 segments of 0..40 tiles with one or two query rows each (a batch of short sequences)
    rng = np.random.default_rng(613)
    lens = rng.integers(0, 41, 3000)
    nqs = rng.integers(1, 3, 3000)
    tiles = H.random_tiles(int(lens.sum()), 2, seed=614, warm_every=5)
    qc, qs = H.random_queries(int(nqs.sum()), 615)
    segs, tb, qb = [], 0, 0
    for n, q in zip(lens, nqs):
        segs.append((tb, int(n), qb, int(q), 0))
        tb += int(n)
        qb += int(q)
    gi, gs_, gc = S.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, qb, 16)
    check_topk(tiles, segs, qc, qs, 16, gi, gs_, gc)


@pytest.mark.parametrize("codec", [0, 3, 4, 2])
def test_hundreds_of_query_rows_on_one_segment(codec):
    # 250 rows against one KV head (a long prompt chunk): several 64-row groups of the tcgen05 kernel, a ragged last one
    n, nq, k = 20000, 250, 96
    tiles = H.random_tiles(n, codec, seed=616 + codec, warm_every=17, nocorr_every=3)
    qc, qs = H.random_queries(nq, 617)
    segs = [(0, n, 0, nq, 5)]
    gi, gs_, gc = S.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs_, gc)


def test_segments_that_share_tiles():
    # two query groups over overlapping tile ranges with different index bases (a sliding window beside the full context)
    n = 60000
    tiles = H.random_tiles(n, 1, seed=618)
    qc, qs = H.random_queries(8, 619)
    segs = [(0, n, 0, 4, 0), (n - 9000, 9000, 4, 4, 1000000), (100, 40000, 0, 0, 0)]
    gi, gs_, gc = S.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, 8, 200)
    check_topk(tiles, segs[:2], qc, qs, 200, gi, gs_, gc)


def test_concurrent_callers_on_their_own_threads_get_their_own_results():
    # Four host threads (the ggml worker pool of the llama.cpp shim calls from several threads, slha_llama.cpp:1387-1503),
    # each with its own tiles, queries and codec, call encode / score + top-k / full scores at the same time; every
    # thread must get what it gets when it runs alone.
    import threading

    jobs = []
    for t, codec in enumerate([6, 2, 4, 3]):
        n = 40000 + 1000 * t
        tiles = H.random_tiles(n, codec, seed=900 + t, warm_every=7, nocorr_every=3)
        qc, qs = H.random_queries(4, 910 + t)
        jobs.append((tiles, qc, qs, n, 100 + 50 * t))
    _, p = H.make_model_pair(160, seed=5)
    model = S.Model.from_projection(p, 160, 5)  # one model shared by all threads
    keys = H.gaussian_keys(920, 500, 160)

    def run(job):
        tiles, qc, qs, n, k = job
        dt = S.to_device(tiles)
        a = S.score_topk(dt, S.make_segments([(0, n, 0, 4, 0)]), qc, qs, 4, k)
        b = S.score_tiles(dt, n, qc, qs, 4)
        c = model.encode_keys(keys, S.CODEC_MIXED)
        return [x.copy() for x in a] + [b, c]

    alone = [run(j) for j in jobs]
    results, errors = [None] * len(jobs), []

    def worker(i):
        try:
            for _ in range(5):
                results[i] = run(jobs[i])
                for x, y in zip(results[i], alone[i]):
                    assert x.tobytes() == y.tobytes()
        except BaseException as e:  # surfaced in the main thread below
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(jobs))]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


def test_a_thousand_launches_alternating_between_call_shapes():
    # slhav2-vram/tests/cuda.rs:405 (a thousand launches): three call shapes that share the thread's streaming state and
    # plan cache, interleaved 334 times each; every call must return what its first call returned
    shapes = []
    for i, (codec, n, nq, k) in enumerate([(6, 90000, 4, 512), (2, 50000, 7, 1000), (4, 40000, 32, 64)]):
        tiles = H.random_tiles(n, codec, seed=930 + i, warm_every=9, nocorr_every=4)
        qc, qs = H.random_queries(nq, 940 + i)
        # (second segment of each table: no query rows -- a head nobody asks about in this call)
        shapes.append((S.to_device(tiles), S.make_segments([(0, n // 2, 0, nq, 0), (n // 2, n - n // 2, 0, 0, 5)]), qc, qs, nq, k))
    first = [None] * len(shapes)
    for it in range(1002):
        j = it % len(shapes)
        dt, segs, qc, qs, nq, k = shapes[j]
        got = S.score_topk(dt, segs, qc, qs, nq, k)
        if first[j] is None:
            first[j] = [x.copy() for x in got]
        else:
            for a, b in zip(first[j], got):
                assert a.tobytes() == b.tobytes(), (it, j)
    st = S.last_score_stats()
    assert st["rows_handed_to_generic_kernel"] == 0
