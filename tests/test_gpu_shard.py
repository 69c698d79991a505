"""Token-range sharding on the device, several ranks emulated on one GPU: the library's own scoring
and strided merge, the short first exchange round and its fall-back to the full lists."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
torch = pytest.importorskip("torch")
F = np.float32


def assert_same_topk(got_i, got_s, want_i, want_s):
    """Sharded and single-pass results name the same tiles.  Scores agree to a few ulps (a row the
    tensor-core kernel hands to the generic kernel is summed in another order), and where the order
    of two entries differs their scores are that close."""
    assert np.allclose(got_s, want_s, rtol=4e-6, atol=2e-5)
    for r in range(len(want_i)):
        diff = got_i[r] != want_i[r]
        assert set(got_i[r].tolist()) == set(want_i[r].tolist()) or np.all(np.abs(want_s[r][diff] - want_s[r, -1]) <= 1e-4)
        if diff.any():
            pos = np.nonzero(diff)[0]
            assert np.all(np.abs(got_s[r][pos] - want_s[r][pos]) <= 2e-5 + 4e-6 * np.abs(want_s[r][pos]))


@pytest.mark.parametrize("skew", [False, True])
def test_short_exchange_matches_single_pass(skew):
    from slhav2_b200 import shard

    world, n, nq, k, k_short = 4, 48000, 4, 256, 160
    tiles = H.random_tiles(n, 2, seed=31)
    if skew:  # the best candidates all sit in rank 0's token range: the short round must be rejected
        tiles["scale"][: n // world] *= 50.0
    qc, qs = H.random_queries(nq, 32)
    dev = torch.device("cuda", 0)
    dt = torch.from_numpy(tiles.view(np.uint8).reshape(-1)).to(dev)
    torch.cuda.synchronize()
    want_i, want_s, _ = S.score_topk(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)

    blocks = []
    for r in range(world):
        start, count = shard.shard_range(n, r, world)
        c = torch.empty(2, nq, k, dtype=torch.int32, device=dev)
        S.score_topk(dt[start * 128:(start + count) * 128], S.make_segments([(0, count, 0, nq, start)]), qc, qs, nq, k,
                     out_index=c[0], out_score=c[1])
        blocks.append(c)
    torch.cuda.synchronize()

    for r in range(world):
        out = torch.empty(2, nq, k, dtype=torch.int32, device=dev)
        gathered = torch.empty(world, 2, nq, k, dtype=torch.int32, device=dev)
        send = torch.empty(2, nq, k_short, dtype=torch.int32, device=dev)
        gathered_short = torch.empty(world, 2, nq, k_short, dtype=torch.int32, device=dev)

        def all_gather(g, c):
            for w in range(world):  # what the collective would deliver: rank w's block, cut like `c`
                g[w].copy_(blocks[w][:, :, : c.shape[2]])

        def overflow(c, o):  # the collective decision: any rank held back a candidate that matters
            torch.cuda.synchronize()
            merged = o[1].cpu().numpy().view(F)
            return any(shard.short_exchange_overflows(b[0].cpu().numpy().view(np.uint32), b[1].cpu().numpy().view(F), merged, k_short)
                       for b in blocks)

        class Emulated(shard.ShardedScorer):
            def local_topk(self, *a):
                self.cand.copy_(blocks[r])

        sc = Emulated(world, nq, k, torch.empty_like(blocks[r]), gathered, out, all_gather,
                      short=shard.ShortExchange(k_short, send, gathered_short, lambda s_, c: s_.copy_(c[:, :, :k_short]), overflow))
        res = sc.step(None, None, None, None)
        torch.cuda.synchronize()
        assert sc.full_exchanges == (1 if skew else 0)
        got_i = res[0].cpu().numpy().view(np.uint32)
        got_s = res[1].cpu().numpy().view(F)
        assert_same_topk(got_i, got_s, want_i, want_s)


def test_pipelined_schedule_matches_single_pass():
    """The overlapped schedule on real streams: rank 0 of four scores its own shard with the library on
    one stream while the exchange (peers' blocks delivered by copy) and the strided merge of the previous
    step run on another; every step's result equals the single-pass top-k of the whole context."""
    from slhav2_b200 import shard

    world, n, nq, k, steps = 4, 40000, 4, 128, 7
    tiles = H.random_tiles(n, 1, seed=41)
    dev = torch.device("cuda", 0)
    dt = torch.from_numpy(tiles.view(np.uint8).reshape(-1)).to(dev)
    queries = [H.random_queries(nq, 50 + i) for i in range(steps)]
    dq = [(torch.from_numpy(qc).to(dev), torch.from_numpy(qs.view(np.int64).reshape(nq, 4)).to(dev)) for qc, qs in queries]
    torch.cuda.synchronize()
    want, peers = [], []
    for qc, qs in queries:
        want.append(S.score_topk(dt, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)[:2])
        blocks = []
        for r in range(1, world):
            start, count = shard.shard_range(n, r, world)
            c = torch.empty(2, nq, k, dtype=torch.int32, device=dev)
            S.score_topk(dt[start * 128:(start + count) * 128], S.make_segments([(0, count, 0, nq, start)]), qc, qs, nq, k,
                         out_index=c[0], out_score=c[1])
            blocks.append(c)
        peers.append(blocks)
    torch.cuda.synchronize()

    score_stream, exchange_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev, priority=-1)

    class Streams:
        def use_score(self):
            torch.cuda.set_stream(score_stream)
            S.set_stream(score_stream.cuda_stream)

        def use_exchange(self):
            torch.cuda.set_stream(exchange_stream)
            S.set_stream(exchange_stream.cuda_stream)

        def record(self, tag):
            ev = torch.cuda.Event()
            ev.record()
            return ev

        def wait_event(self, ev):
            torch.cuda.current_stream().wait_event(ev)

        def sync(self, ev):
            ev.synchronize()

    step_of_slot = {}

    def make(slot):
        def all_gather(g, c):  # what the collective would deliver for the step this slot holds
            g[0].copy_(c)
            for w in range(1, world):
                g[w].copy_(peers[step_of_slot[slot]][w - 1])

        return shard.ShardedScorer(world, nq, k, torch.empty(2, nq, k, dtype=torch.int32, device=dev),
                                   torch.empty(world, 2, nq, k, dtype=torch.int32, device=dev),
                                   torch.empty(2, nq, k, dtype=torch.int32, device=dev), all_gather)

    slots = [make(0), make(1)]
    pipe = shard.PipelinedScorer(slots, Streams())
    start0, count0 = shard.shard_range(n, 0, world)
    segs0 = S.make_segments([(0, count0, 0, nq, start0)])
    hout = [torch.empty(2, nq, k, dtype=torch.int32).pin_memory() for _ in range(steps)]
    try:
        handles = []
        for i in range(steps):
            step_of_slot[i % 2] = i
            slot = pipe.submit(dt[: count0 * 128], segs0, dq[i][0], dq[i][1],
                               download=lambda s_, i=i: hout[i].copy_(slots[s_].out, non_blocking=True))
            handles.append(slot)
            if i >= 1:  # the previous step's result is read while this one is in flight
                pipe.wait(handles[i - 1])
        pipe.drain()
        torch.cuda.synchronize()
    finally:
        torch.cuda.set_stream(torch.cuda.default_stream(dev))
        S.set_stream(None)
    for i in range(steps):
        assert_same_topk(hout[i][0].numpy().view(np.uint32), hout[i][1].numpy().view(F), want[i][0], want[i][1])
