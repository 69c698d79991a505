"""The sharded step behind the C ABI (slha_b200_shard_*) on two real GPUs: two processes, one per
GPU, exchange the NCCL unique id through a file, score their token ranges and must both end up
with the top-k of the whole context (computed on one GPU and by the CPU oracle).  Skipped on a
machine with fewer than two GPUs."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")

WORKER = r"""
import os, sys, time
import numpy as np
rank, world, tmp = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
import slhav2_b200 as S
from slhav2_b200 import shard
from tests import helpers as H
from tests.test_gpu_topk import check_topk
S.set_device(rank)
n, nq, k = 60000, 8, 512
tiles = H.random_tiles(n, 1, seed=91, warm_every=13)
qc, qs = H.random_queries(nq, 92)
idf = os.path.join(tmp, "nccl_id.npy")
if rank == 0:
    np.save(idf + ".tmp.npy", S.shard_unique_id())
    os.replace(idf + ".tmp.npy", idf)
else:
    for _ in range(600):
        if os.path.exists(idf):
            break
        time.sleep(0.05)
sh = S.Shard(np.load(idf), rank, world)
start, count = shard.shard_range(n, rank, world)
dt = S.to_device(tiles[start:start + count])
# two segments of 4 queries each over this rank's token range; indices are global token positions
segs = S.make_segments([(0, count, 0, 4, start), (0, count, 4, 4, start)])
sh.set_timing(True)
for _ in range(3):
    gi, gs = sh.score_topk(dt, segs, qc, qs, nq, k)
ms = sh.last_times()
assert np.all(ms >= 0) and ms[0] > 0
full = [(0, n, 0, 4, 0), (0, n, 4, 4, 0)]
check_topk(tiles, full, qc, qs, k, gi, gs, np.full(nq, k))
# the repeated step without timing: captured into a graph per buffer parity and replayed; every step must give the same
sh.set_timing(False)
gi2, gs2 = np.zeros_like(gi), np.zeros_like(gs)
dq, ds = S.to_device(qc), S.to_device(qs)
for _ in range(7):
    gi2[:] = 0
    sh.score_topk(dt, segs, dq, ds, nq, k, out_index=gi2, out_score=gs2)
    assert np.array_equal(gi2, gi) and np.array_equal(gs2, gs)
st = sh.status()
assert st["exchange"] in ("peer-memory loads", "nccl all-gather") and not st["wait_ran_out"] and st["steps"] == 10, st
np.save(os.path.join(tmp, "out%d.npy" % rank), np.stack([gi.astype(np.float64), gs.astype(np.float64)]))
# other shapes on the same handle, through both exchanges: shards shorter than k (lists with absent entries at their
# ends), a context shorter than k (padded result), an uneven split, another codec
for mode in ("nccl", "peer", "nccl"):
    sh.set_exchange(mode)
    for n2, k2 in ((300, 256), (200, 256), (5001, 64)):
        t2 = H.random_tiles(n2, 3, seed=93 + n2)
        s2, c2 = shard.shard_range(n2, rank, world)
        d2 = S.to_device(t2[s2:s2 + c2])
        for _ in range(3):
            g = sh.score_topk(d2, S.make_segments([(0, c2, 0, 3, s2)]), qc[:3], qs[:3], 3, k2)
        check_topk(t2, [(0, n2, 0, 3, 0)], qc[:3], qs[:3], k2, g[0], g[1], np.full(3, min(k2, n2)))
assert not sh.status()["wait_ran_out"]
sh.destroy()
print("rank", rank, "ok", ms, st)
"""


def test_two_gpu_sharded_step_through_the_c_abi():
    if S.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tmp = tempfile.mkdtemp()
    env = dict(os.environ, PYTHONPATH=root, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, str(r), "2", tmp], env=env, cwd=root, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    a, b = np.load(os.path.join(tmp, "out0.npy")), np.load(os.path.join(tmp, "out1.npy"))
    assert np.array_equal(a, b)  # every rank holds the same merged result


def test_single_rank_shard_handle_needs_no_nccl():
    from tests import helpers as H
    from tests.test_gpu_topk import check_topk

    n, nq, k = 9000, 3, 100
    tiles = H.random_tiles(n, 2, seed=5)
    qc, qs = H.random_queries(nq, 6)
    sh = S.Shard(None, 0, 1)
    segs = [(0, n, 0, nq, 7)]
    gi, gs = sh.score_topk(S.to_device(tiles), S.make_segments(segs), qc, qs, nq, k)
    check_topk(tiles, segs, qc, qs, k, gi, gs, np.full(nq, k))
    with pytest.raises(S.SlhaError):
        S.Shard(None, 0, 2)  # more than one rank needs the unique id
    with pytest.raises(S.SlhaError):
        S.Shard(None, 3, 2)
    sh.destroy()
