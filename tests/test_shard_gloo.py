"""world_size-2 gloo run of the token-range sharding plumbing on CPU: shard
ranges, segment tables, the [2][nq][k] candidate block, one all-gather, merge.
The device steps are replaced by the oracle (scoring) and the numpy statement of
the merge rule, so what is tested is the host logic every rank runs."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total_tokens, q, k_short=0, skew=False):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from oracle import pyoracle as ora
    from slhav2_b200 import shard
    from tests import helpers as H

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    heads, group, k = 2, 2, 32
    nq = heads * group
    all_tiles = H.random_tiles(heads * total_tokens, 2, seed=5).reshape(heads, total_tokens)
    if skew:  # the best candidates all sit in the first rank's token range
        all_tiles["scale"][:, : total_tokens // world] *= 50.0
    qc, qs = H.random_queries(nq, 6)
    start, count = shard.shard_range(total_tokens, rank, world)
    local = np.ascontiguousarray(all_tiles[:, start:start + count]).reshape(-1)
    segs = shard.shard_segments(1, heads, count, group, start)

    cand = torch.zeros(2, nq, k, dtype=torch.int32)
    gathered = torch.zeros(world, 2, nq, k, dtype=torch.int32)
    out = torch.zeros(2, nq, k, dtype=torch.int32)

    class CpuScorer(shard.ShardedScorer):
        def local_topk(self, tiles, segments, q_coarse, q_sign):
            ci = np.full((nq, k), 0xFFFFFFFF, np.uint32)
            cs = np.full((nq, k), -np.inf, np.float32)
            for seg in segments:
                t = tiles[int(seg["tile_begin"]):int(seg["tile_begin"]) + int(seg["n_tiles"])]
                for j in range(int(seg["query_begin"]), int(seg["query_begin"]) + int(seg["n_queries"])):
                    sc = ora.score_tiles(t, q_coarse[j], q_sign[j])
                    i, v = ora.topk(sc, k)
                    ci[j, :len(i)], cs[j, :len(i)] = i + int(seg["index_base"]), v
            self.cand[0].copy_(torch.from_numpy(ci.view(np.int32)))
            self.cand[1].copy_(torch.from_numpy(cs.view(np.int32)))

        def merge(self, out_index=None, out_score=None, gathered=None, k_in=None):
            g = (self.gathered if gathered is None else gathered).numpy()
            oi, osc = shard.merge_reference(g[:, 0].view(np.uint32), g[:, 1].view(np.float32), self.k)
            self.out[0].copy_(torch.from_numpy(oi.view(np.int32)))
            self.out[1].copy_(torch.from_numpy(osc.view(np.int32)))

    short = None
    if k_short:
        send = torch.zeros(2, nq, k_short, dtype=torch.int32)
        gathered_short = torch.zeros(world, 2, nq, k_short, dtype=torch.int32)

        def overflow(c, o):
            mine = shard.short_exchange_overflows(c[0].numpy().view(np.uint32), c[1].numpy().view(np.float32),
                                                  o[1].numpy().view(np.float32), k_short)
            flag = torch.tensor([int(mine)])
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            return bool(flag.item())

        short = shard.ShortExchange(k_short, send, gathered_short, lambda s_, c: s_.copy_(c[:, :, :k_short]), overflow)
    sc = CpuScorer(world, nq, k, cand, gathered, out, lambda g, c: dist.all_gather(list(g.unbind(0)), c.contiguous()), short=short)
    res = sc.step(local, segs, qc, qs).numpy()
    ok = True
    for h in range(heads):
        for g_ in range(group):
            j = h * group + g_
            want_i, want_v = ora.topk(ora.score_tiles(all_tiles[h], qc[j], qs[j]), k)
            ok &= np.array_equal(res[0, j].view(np.uint32), want_i) and np.array_equal(res[1, j].view(np.float32), want_v)
    # the pipelined scorer (exchange of step i beside the scoring of step i+1) gives the same results
    class NoStreams:
        def use_score(self): pass
        def use_exchange(self): pass
        def record(self, tag): return object()
        def wait_event(self, ev): pass
        def sync(self, ev): pass

    ag = lambda g, c: dist.all_gather(list(g.unbind(0)), c.contiguous())
    slots = [CpuScorer(world, nq, k, torch.zeros(2, nq, k, dtype=torch.int32), torch.zeros(world, 2, nq, k, dtype=torch.int32),
                       torch.zeros(2, nq, k, dtype=torch.int32), ag) for _ in range(2)]
    pipe = shard.PipelinedScorer(slots, NoStreams())
    for _ in range(3):
        slot = pipe.submit(local, segs, qc, qs)
        ok &= np.array_equal(pipe.wait(slot).numpy(), res)
    pipe.drain()
    q.put((rank, bool(ok), (start, count), sc.full_exchanges))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total_tokens", [257, 1000])
def test_two_rank_gloo_sharded_topk(total_tokens):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total_tokens, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in results)
    ranges = sorted(r for _, _, r, _ in results)
    assert ranges[0][0] == 0 and ranges[0][0] + ranges[0][1] == ranges[1][0] and ranges[1][0] + ranges[1][1] == total_tokens


def test_shard_ranges_cover_without_overlap():
    sys.path.insert(0, ROOT)
    from slhav2_b200 import shard

    for total in (0, 1, 7, 1048576, 1000003):
        for world in (1, 2, 3, 4, 8):
            pos = 0
            for r in range(world):
                s, c = shard.shard_range(total, r, world)
                assert s == pos
                pos += c
            assert pos == total


@pytest.mark.parametrize("skew", [False, True])
def test_four_rank_short_exchange(skew):
    # k = 32 over 4 ranks with a first round of 14 candidates per rank: evenly spread winners need no
    # second round; winners concentrated in one rank's range make the collective check ask for the full lists
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, 1200, q, 14, skew)) for r in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in results)
    full = {f for _, _, _, f in results}
    assert full == ({1} if skew else {0})


def test_short_exchange_rule():
    sys.path.insert(0, ROOT)
    from slhav2_b200 import shard

    assert shard.short_exchange_len(1024, 2) == 1024 and shard.short_exchange_len(1024, 8) == 384
    idx = np.arange(8, dtype=np.uint32).reshape(1, 8)
    sc = np.array([[9, 8, 7, 6, 5, 4, 3, 2]], np.float32)
    merged = np.array([[9, 9, 8, 8, 7, 7, 6.5, 6.5]], np.float32)
    assert not shard.short_exchange_overflows(idx, sc, merged, 4)      # first unsent 5 < merged k-th 6.5
    merged[0, 7] = 5.0
    assert shard.short_exchange_overflows(idx, sc, merged, 4)          # a tie counts
    idx[0, 4:] = 0xFFFFFFFF
    assert not shard.short_exchange_overflows(idx, sc, merged, 4)      # nothing was held back
