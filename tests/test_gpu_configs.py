"""The five benchmark configurations as parity cases (reduced lengths where the oracle
would take minutes; full length through size-independent properties)."""
import numpy as np
import pytest

from oracle import pyoracle as ora
from tests import helpers as H
from tests.test_gpu_topk import check_topk

pytestmark = pytest.mark.gpu
S = pytest.importorskip("slhav2_b200")
F = np.float32


def test_config1_single_head_cpu_runnable_reference():
    # 4096 x 128 f32 N(0,1) seed 0, channels 7 and 93 x8, orthogonal 128x128 P, INT4 single, top-64
    n, d, k = 4096, 128, 64
    om, p = H.make_model_pair(d, seed=0, pseed=0)
    gm = S.Model.from_projection(p, d, 0)
    keys = H.gaussian_keys(0, n, d, outlier_channels=(7, 93))
    dt = S.DeviceBuffer(n * 128)
    gm.encode_keys(keys, S.CODEC_INT4_SINGLE, out=dt)
    tiles = dt.download(S.TILE_DTYPE, n)
    assert tiles.tobytes() == om.encode_batch(keys, 0).tobytes()
    q = ora.Rng(1).gaussian(d)
    qc, qs = gm.prepare_queries(q[None])
    segs = [(0, n, 0, 1, 0)]
    gi, gsc, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, 1, k)
    check_topk(tiles, segs, qc, qs, k, gi, gsc, gc)


def llama_decode_keys(seed, heads, tokens, d, pos0=0, theta=500000.0):
    """Config-2 / config-5 key distribution from the oracle PRNG: N(0,1) x per-channel log-normal(0, 0.5),
    RoPE (pairs (2i, 2i+1), theta) at positions pos0.., rounded to bf16 (returned widened to f32)."""
    rng = ora.Rng(seed)
    chan = np.exp(0.5 * rng.gaussian(d).astype(np.float64)).astype(F)
    k = rng.gaussian(heads * tokens * d).reshape(heads, tokens, d) * chan
    pos = np.arange(pos0, pos0 + tokens, dtype=np.float64)
    inv = theta ** (-np.arange(0, d, 2, dtype=np.float64) / d)
    ang = pos[:, None] * inv[None, :]
    c, s_ = np.cos(ang).astype(F), np.sin(ang).astype(F)
    a, b = k[..., 0::2].copy(), k[..., 1::2].copy()
    k[..., 0::2] = a * c - b * s_
    k[..., 1::2] = a * s_ + b * c
    return H.to_bf16_f32(k.astype(F)).reshape(heads * tokens, d)


def test_config2_llama_decode_kv_nf4_gqa4_top1024():
    # the benchmarked workload at 2 layers x 8 KV heads x 4096 tokens: bf16 log-normal-channel RoPE keys,
    # NF4, one model per layer, the [layer][kv_head][token] segment table of the sharded scorer, GQA
    # groups of 4, top-1024 per query head; tile bytes and top-k against the oracle
    L, Hh, T, G, d, k = 2, 8, 4096, 4, 128, 1024
    n = L * Hh * T
    dt = S.DeviceBuffer(n * 128)
    want_tiles = np.zeros(n, S.TILE_DTYPE)
    qc = np.zeros((L * Hh * G, 128), F)
    qs = np.zeros((L * Hh * G, 4), np.uint64)
    pos = np.tile(np.arange(T, dtype=np.uint32), Hh)
    heads = np.repeat(np.arange(Hh, dtype=np.uint16), T)
    for l in range(L):
        om, p = H.make_model_pair(d, seed=100 + l, pseed=200 + l)
        gm = S.Model.from_projection(p, d, 100 + l)
        keys = llama_decode_keys(1234 + l, Hh, T, d)
        bf16 = (keys.view(np.uint32) >> 16).astype(np.uint16)
        lo = l * Hh * T
        gm.encode_keys(bf16, S.CODEC_NF4, n=Hh * T, key_dtype=S.BF16, positions=pos, head_ids=heads, out=dt.view(lo * 128, Hh * T * 128))
        want_tiles[lo:lo + Hh * T] = om.encode_batch(keys, 2, pos=pos, head=heads)
        q = H.gaussian_keys(99 + l, Hh * G, d)
        a, b = gm.prepare_queries(q)
        qc[l * Hh * G:(l + 1) * Hh * G], qs[l * Hh * G:(l + 1) * Hh * G] = a, b
        wc, ws = om.prepare_query(q[5])
        assert np.array_equal(a[5], wc) and np.array_equal(b[5], ws)
        gm.release()
    tiles = dt.download(S.TILE_DTYPE, n)
    assert tiles.tobytes() == want_tiles.tobytes()
    assert np.all(tiles["flags"] == ora.FLAG_NF4)
    from slhav2_b200 import shard

    segs = shard.shard_segments(L, Hh, T, G, 0)
    gi, gsc, gc = S.score_topk(dt, segs, qc, qs, L * Hh * G, k)
    check_topk(tiles, [tuple(int(x) for x in r) for r in segs.tolist()], qc, qs, k, gi, gsc, gc)


def student_t_keys(seed, n, d):
    rng = ora.Rng(seed)
    g = rng.gaussian(n * d * 5).reshape(n, d, 5)
    t = g[..., 0] / np.sqrt((g[..., 1:] ** 2).sum(-1) / 4.0)
    out = np.nonzero(ora.Rng(seed + 1).gaussian(n * d).reshape(n, d) > 2.326)  # ~1 % of the entries
    t[out] *= 20.0
    return H.to_bf16_f32(t.astype(F))


@pytest.mark.parametrize("heads,tokens,k", [(2, 2048, 32), (8, 16384, 256)], ids=["reduced", "full-size"])
def test_config3_tq3_rht_many_queries_per_head(heads, tokens, k):
    # TQ3 + Hadamard RHT, Student-t(4) keys with 1 % x20 outliers, 64 queries per KV head (16 sequences x 4 GQA heads);
    # the second case is the configuration at its full size: 8 KV heads x 16384 tokens, 512 query rows
    d, qph = 128, 64
    om, p = H.make_model_pair(d, seed=3, rht=True, pseed=4)
    gm = S.Model.from_projection(p, d, 3, rht=True)
    keys = student_t_keys(5, heads * tokens, d)
    dt = S.DeviceBuffer(heads * tokens * 128)
    bf16 = (keys.view(np.uint32) >> 16).astype(np.uint16)
    gm.encode_keys(bf16, S.CODEC_TQ3, n=heads * tokens, key_dtype=S.BF16, out=dt)
    tiles = dt.download(S.TILE_DTYPE, heads * tokens)
    assert tiles.tobytes() == om.encode_batch(keys, 4).tobytes()
    q = H.gaussian_keys(6, heads * qph, d)
    qc, qs = gm.prepare_queries(q)
    for j in (0, 77):
        wc, ws = om.prepare_query(q[j])
        assert np.array_equal(qs[j], ws) and np.array_equal(qc[j], wc)
    segs = [(h * tokens, tokens, h * qph, qph, 0) for h in range(heads)]
    gi, gsc, gc = S.score_topk(dt, S.make_segments(segs), qc, qs, heads * qph, k)
    check_topk(tiles, segs, qc, qs, k, gi, gsc, gc)


@pytest.mark.parametrize("steps,recent", [(96, 64), (640, 2048)], ids=["reduced", "recent-window-2048"])
def test_config4_ccos_under_budget_interleaved_appends_and_decode_steps(steps, recent):
    # mixed 8/4 codec, budget 60 % of full-HOT, H2O importance with sink 4 + recent window,
    # appends interleaved with decode-step scoring over the device-resident arena; the second case has the
    # configuration's recent window of 2048 tokens over 5120 appended tokens.
    # Tokens are followed by position, not by slot: the pool's importances equal the reference's to about 1e-7 relative
    # (its softmax sum runs in a fixed tree order), so two evictions of one call with nearly tied importances can leave
    # the free list in the other order, and later appends then land in other slots than the oracle's.
    d, per_step = 128, 8
    om, p = H.make_model_pair(d, seed=8, pseed=9)
    gm = S.Model.from_projection(p, d, 8)
    total = steps * per_step
    budget = int(0.6 * 128 * total)
    pool = S.TilePool(total, budget, S.PAGE_LOWEST_IMPACT_FIRST, S.EVICT_IMPORTANCE, sink_window=4, recent_window=recent)
    cache = ora.Cache(budget, 0, 1, 4, recent)
    keys = H.gaussian_keys(10, total, d)
    q = H.gaussian_keys(11, steps, d)
    qc, qs = gm.prepare_queries(q)
    slot_of = {}   # position -> slot in the device pool
    oslot_of = {}  # position -> slot in the oracle's cache
    for s in range(steps):
        chunk = keys[s * per_step:(s + 1) * per_step]
        pos = np.arange(s * per_step, (s + 1) * per_step, dtype=np.uint32)
        slots = pool.append_keys(gm, chunk, S.CODEC_MIXED, positions=pos)
        want = om.encode_batch(chunk, 3, pos=pos)
        for i in range(per_step):
            slot_of[int(pos[i])] = int(slots[i])
            oslot_of[int(pos[i])] = cache.insert(want[i:i + 1])
        assert len(set(slot_of[int(x)] for x in pos)) == per_step
        # decode step: score the arena, feed the scores back as H2O observations
        gsl, gsv = pool.score_all(qc[s], qs[s])
        wsl, wsv = cache.score_all(qc[s], qs[s])
        tiles_now = pool.read()[0]
        got = {int(tiles_now["position"][sl]): v for sl, v in zip(gsl, gsv)}
        opos = {sl: ps for ps, sl in oslot_of.items()}
        wanted = {opos[int(sl)]: v for sl, v in zip(wsl, wsv)}
        assert got.keys() == wanted.keys() and all(abs(got[k] - wanted[k]) <= 1e-3 for k in got)
        # identical observations on both sides (the oracle's scores, addressed by position) keep the eviction order comparable
        obs_pos = [opos[int(sl)] for sl in wsl]
        pool.observe_scores(np.array([slot_of[ps] for ps in obs_pos], np.uint32), wsv, 1.0)
        cache.observe_scores(wsl, wsv, 1.0)
        if s % 4 == 3:
            assert pool.enforce_budget() == cache.enforce_budget()
            st = pool.stats()
            assert st["live_bytes"] <= budget and st["live_bytes"] == cache.live_bytes()
            assert (st["hot"], st["warm"], st["cold"]) == cache.counts()
            state = pool.read()[1]
            cstate = cache.states()
            for ps in [k for k in slot_of if state[slot_of[k]] == ora.COLD or cstate[oslot_of[k]] == ora.COLD]:
                assert state[slot_of[ps]] == cstate[oslot_of[ps]] == ora.COLD, ps  # the same tokens were evicted
                del slot_of[ps], oslot_of[ps]
    tiles, state, imp, _ = pool.read()
    cstate, ctiles = cache.states(), cache.tiles()
    assert {ora.WARM, ora.COLD} <= set(state.tolist())  # paged and evicted tiles both present (60 % < all-WARM 75 %)
    assert len(slot_of) == len(oslot_of) == int((state != ora.COLD).sum())
    for ps, sl in slot_of.items():
        osl = oslot_of[ps]
        assert state[sl] == cstate[osl] and tiles[sl:sl + 1].tobytes() == ctiles[osl:osl + 1].tobytes()
        assert abs(imp[sl] - cache.importance(osl)) <= 1e-5


def test_config5_full_length_head_fused_topk_against_the_oracle():
    # one KV head of the 1M-token context (134 MB of tiles), MX-32 INT4, 4 queries, top-2048.  The
    # oracle scores every tile of the head (4 M tile-query pairs, a few seconds with its threads);
    # the library's full-score mode is checked against it too, then the fused top-k against both
    n, d, k, nq = 1 << 20, 128, 2048, 4
    _, p = H.make_model_pair(d, seed=12, pseed=13)
    gm = S.Model.from_projection(p, d, 12)
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    keys = torch.randn(n, d, generator=g, device="cuda").to(torch.bfloat16).contiguous()
    tiles = torch.empty(n * 128, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()  # the library runs on its own stream: torch's producers must have finished
    gm.encode_keys(keys, S.CODEC_INT4_GROUPED32, n=n, key_dtype=S.BF16, out=tiles)
    q = H.gaussian_keys(14, nq, d)
    qc, qs = gm.prepare_queries(q)
    full = torch.empty(nq, n, dtype=torch.float32, device="cuda")
    S.score_tiles(tiles, n, qc, qs, nq, out=full)
    gi, gsc, gc = S.score_topk(tiles, S.make_segments([(0, n, 0, nq, 0)]), qc, qs, nq, k)
    full = full.cpu().numpy()
    host_tiles = np.frombuffer(tiles.cpu().numpy().tobytes(), S.TILE_DTYPE)
    want = H.oracle_scores(host_tiles, qc, qs)
    assert np.all(np.abs(full - want) <= 1e-3)
    full = want  # from here on the oracle's scores are the yardstick
    # tile bytes of a sub-range against the oracle's encoder (bf16 keys widen exactly)
    om = ora.Model(p, d, seed=12)
    sub = slice(500000, 500000 + 4096)
    kf = keys[sub].float().cpu().numpy()
    assert host_tiles[sub].tobytes() == om.encode_batch(kf, 6, pos=np.arange(sub.start, sub.stop, dtype=np.uint32)).tobytes()
    assert np.all(gc == k)
    for j in range(nq):
        oi, ov = ora.topk(full[j], k)
        assert np.all(np.abs(gsc[j] - ov) <= 1e-3)
        assert np.all(np.abs(full[j][gi[j]] - gsc[j]) <= 1e-3) and len(set(gi[j])) == k
        thr = ov[-1]
        assert all(abs(full[j][i] - thr) <= 2e-3 for i in set(oi) ^ set(gi[j]))
    # encode -> decode_latent round trip on a sample: reconstruction within one INT4 step per latent dim
    sample = np.frombuffer(tiles[:128 * 4].cpu().numpy().tobytes(), S.TILE_DTYPE)
    assert np.all(sample["position"] == np.arange(4)) and np.all(sample["flags"] == 0)
