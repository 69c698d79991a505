"""Token-range sharding on the device, several ranks emulated on one GPU: the library's own scoring
and strided merge, the short first exchange round and its fall-back to the full lists."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
torch = pytest.importorskip("torch")
F = np.float32


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
        assert np.array_equal(got_i, want_i) and np.array_equal(got_s, want_s)
