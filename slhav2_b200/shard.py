"""Token-range sharding of a tile context over the GPUs of one node.

Every rank owns a contiguous token range of every KV head, scores only its own
tiles (resident in its own HBM) and keeps its own top-k per query head; the
per-rank candidates are exchanged with ONE all-gather and merged by every rank
with the same deterministic rule (score descending, ties towards the lower
global index).  With three or more ranks a shorter first exchange (the best
2k/world + 128 candidates per rank) usually suffices; a collective check decides
whether the full lists are needed after all.  The reference has no multi-device path; the per-tile
independence this relies on is ElasticKvCache::score_all
(scirust/src/ccos.rs:346-355).

The collective is torch.distributed's (NCCL on GPUs, gloo in the CPU tests);
local scoring and the merge are the C-ABI calls slha_b200_score_topk and
slha_b200_topk_merge_strided.
"""
import numpy as np

from . import api


def shard_range(total_tokens, rank, world):
    """Contiguous token range [start, start+count) of `rank`; ranges differ by at most one token."""
    base, rem = divmod(total_tokens, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def shard_segments(n_layers, kv_heads, tokens_local, group, position_base):
    """Segment table of one rank: tiles laid out [layer][kv_head][token]; the
    queries of (layer, kv_head) are rows (layer*kv_heads + kv_head)*group + g.
    Reported indices are global token positions (position_base + local token)."""
    rows = []
    for l in range(n_layers):
        for h in range(kv_heads):
            s = l * kv_heads + h
            rows.append((s * tokens_local, tokens_local, s * group, group, position_base))
    return api.make_segments(rows)


def short_exchange_len(k, world):
    """Candidates per rank the short exchange sends: twice a rank's fair share of the top-k plus a
    margin, or k when that is no shorter."""
    return min(k, (2 * k + world - 1) // world + 128)


class ShortExchange:
    """Optional first round of ShardedScorer.step for world >= 3: every rank sends only its best
    k_short candidates per query.  The merged top-k is exact unless some rank holds an unsent candidate
    whose score reaches the merged k-th score; `overflow` decides that for all ranks together (it is a
    collective), and the full exchange then runs as if the short one had not happened.

      send      [2][nq][k_short]          this rank's best k_short (indices, then score bits)
      gathered  [world][2][nq][k_short]
      pack      callable(send, cand): send[:, :, :] = cand[:, :, :k_short]
      overflow  callable(cand, out) -> bool, the same value on every rank
    """

    def __init__(self, k_short, send, gathered, pack, overflow):
        self.k_short, self.send, self.gathered, self.pack, self.overflow = k_short, send, gathered, pack, overflow


def short_exchange_overflows(cand_index, cand_score, merged_score, k_short):
    """numpy statement of one rank's part of ShortExchange.overflow: cand_* are this rank's [nq][k]
    lists (sorted, index 0xFFFFFFFF = absent), merged_score the [nq][k] result of the short exchange.
    True when a candidate this rank did not send could belong to the top-k (ties count: an equal score
    with a lower index would win)."""
    k = cand_index.shape[1]
    if k_short >= k:
        return False
    unsent = cand_index[:, k_short] != 0xFFFFFFFF
    return bool(np.any(unsent & (cand_score[:, k_short] >= merged_score[:, k - 1])))


class ShardedScorer:
    """One decode-step scorer of a rank.

    Buffers (anything with data_ptr(), int32 storage):
      cand     [2][nq][k]         this rank's indices, then score bits
      gathered [world][2][nq][k]  every rank's block after the all-gather
      out      [2][nq][k]         merged indices, then score bits
    """

    def __init__(self, world, nq, k, cand, gathered, out, all_gather, count=None, short=None):
        self.world, self.nq, self.k = world, nq, k
        self.cand, self.gathered, self.out, self.count = cand, gathered, out, count
        self.all_gather = all_gather  # callable(gathered, cand)
        self.block = 2 * nq * k       # int32 elements per rank in `gathered`
        self.short = short if (short is not None and short.k_short < k) else None
        self.full_exchanges = 0       # steps that needed the full lists (all steps without a short exchange)
        self._skip, self._penalty = 0, 1  # back-off of the short round after it was rejected

    # the two device steps; the CPU tests substitute checker implementations
    def local_topk(self, tiles, segments, q_coarse, q_sign):
        api.score_topk(tiles, segments, q_coarse, q_sign, self.nq, self.k, out_index=self.cand[0], out_score=self.cand[1],
                       out_count=self.count)

    def merge(self, out_index=None, out_score=None, gathered=None, k_in=None):
        g = self.gathered if gathered is None else gathered
        k_in = self.k if k_in is None else k_in
        api.topk_merge(g, g[0][1], self.world, self.nq, k_in, self.k,
                       out_index=self.out[0] if out_index is None else out_index,
                       out_score=self.out[1] if out_score is None else out_score, list_stride=2 * self.nq * k_in)

    def step(self, tiles, segments, q_coarse, q_sign, out_index=None, out_score=None):
        self.local_topk(tiles, segments, q_coarse, q_sign)
        if self.world == 1:
            return self.cand
        if self.short is not None and self._skip > 0:
            self._skip -= 1  # (the decision below is collective, so every rank skips the same steps)
        elif self.short is not None:
            s = self.short
            s.pack(s.send, self.cand)
            self.all_gather(s.gathered, s.send)
            self.merge(None, None, s.gathered, s.k_short)
            if not s.overflow(self.cand, self.out):
                self._penalty = 1
                if out_index is not None or out_score is not None:
                    self.merge(out_index, out_score, s.gathered, s.k_short)
                return self.out
            # winners concentrated on few ranks (they often stay there from step to step): leave the
            # short round out for a while, twice as long after every rejection
            self._skip = self._penalty
            self._penalty = min(2 * self._penalty, 1024)
        self.full_exchanges += 1
        self.all_gather(self.gathered, self.cand)
        self.merge(out_index, out_score)
        return self.out


class PipelinedScorer:
    """Throughput mode for independent steps (e.g. the layers of a batch scored back to back): the
    exchange and merge of step i run on a second stream while step i+1 is being scored, with `depth`
    sets of candidate / gathered / result buffers.  `submit` returns the slot whose `out` buffers hold
    the step's result once `wait(slot)` has returned; `drain` waits for everything in flight.

      scorers   `depth` ShardedScorer objects, each with buffers of its own
      streams   hooks that keep this module free of any framework:
                  use_score()      make the scoring stream current (framework and library)
                  use_exchange()   make the exchange stream current
                  record(tag)      record an event on the current stream, returns it
                  wait_event(ev)   make the current stream wait for the event
                  sync(ev)         host wait for the event

    The result of a step does not depend on the pipelining: every step runs the same calls in the same
    order on its own buffers (tests/test_shard_gloo.py runs this class against the serial scorer).
    """

    def __init__(self, scorers, streams):
        self.scorers, self.st = list(scorers), streams
        self.scored = [None] * len(self.scorers)     # event: candidates of the slot are complete
        self.exchanged = [None] * len(self.scorers)  # event: merged result of the slot is complete
        self.sent = [None] * len(self.scorers)       # event: the slot's candidates have been gathered (scoring may overwrite them)
        self.n = 0

    def submit(self, tiles, segments, q_coarse, q_sign, upload=None, download=None):
        """Queue one step.  `upload(slot)`, if given, runs on the scoring stream once the slot is free
        and returns the (q_coarse, q_sign) to score with (e.g. after copying host queries into the
        slot's device buffers); `download(slot)` runs on the exchange stream after the merge (e.g. an
        asynchronous copy of the slot's result to host memory) and is covered by `wait(slot)`."""
        slot = self.n % len(self.scorers)
        sc, st = self.scorers[slot], self.st
        st.use_score()
        if self.sent[slot] is not None:
            # the slot's candidate block is free again; its gathered and result buffers are only
            # touched on the exchange stream, in order
            st.wait_event(self.sent[slot])
        if upload is not None:
            q_coarse, q_sign = upload(slot)
        sc.local_topk(tiles, segments, q_coarse, q_sign)
        self.scored[slot] = st.record("scored")
        st.use_exchange()
        st.wait_event(self.scored[slot])
        if sc.world > 1:
            sc.full_exchanges += 1
            sc.all_gather(sc.gathered, sc.cand)
            self.sent[slot] = st.record("sent")
            sc.merge()
        if download is not None:
            download(slot)
        self.exchanged[slot] = st.record("exchanged")
        if sc.world == 1:
            self.sent[slot] = self.exchanged[slot]  # one rank: `download` reads the candidate block itself
        st.use_score()
        self.n += 1
        return slot

    def wait(self, slot):
        if self.exchanged[slot] is not None:
            self.st.sync(self.exchanged[slot])
        sc = self.scorers[slot]
        return sc.out if sc.world > 1 else sc.cand

    def drain(self):
        for slot in range(len(self.scorers)):
            self.wait(slot)


def merge_reference(gathered_index, gathered_score, k):
    """numpy statement of the merge rule for [world][nq][k] candidate blocks
    (index 0xFFFFFFFF = absent): used by the CPU tests as the checker."""
    world, nq, kin = gathered_index.shape
    oi = np.full((nq, k), 0xFFFFFFFF, np.uint32)
    osc = np.full((nq, k), -np.inf, np.float32)
    for j in range(nq):
        idx = gathered_index[:, j, :].reshape(-1)
        sc = gathered_score[:, j, :].reshape(-1)
        keep = idx != 0xFFFFFFFF
        idx, sc = idx[keep], sc[keep]
        order = np.lexsort((idx, -sc.astype(np.float64)))[:k]
        oi[j, : len(order)], osc[j, : len(order)] = idx[order], sc[order]
    return oi, osc
