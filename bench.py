#!/usr/bin/env python
"""Benchmark of the SLHA v2 tile hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload c1..c5] [--impl reference]

A "step" is one pass of fused eq. 2.3 scoring + top-k over every tile of the context (for
N > 1: every rank scores its token range, one NCCL all-gather, one merge).

Default workload: configuration 5, the long-context case the target is written on -- 1 048 576
tokens x 8 KV heads = 8.4 M INT4 MX-32 tiles (1.07 GB), 32 query heads in GQA groups of 4, top-2048
per query head.  With N GPUs the token range is split over the ranks (strong scaling) and every
step goes through the C ABI's sharded entry point (slha_b200_shard_score_topk).  The JSON line's
`value` is the one-step-at-a-time figure.  At N = 1 the line also carries, under "also", the other
configurations: c2 (Llama-3-8B decode KV, 32 layers x 8 KV heads x 32768 tokens, NF4, top-1024),
c1 (the single-head CPU-runnable case), c3 (TQ3 + RHT, 64 queries per KV head: encode and score
rates) and c4 (the elastic pool under a 60 % budget: appends interleaved with decode steps).

Synthetic data stands in for real activations: seeded N(0,1) keys scaled by per-channel
log-normal(0, 0.5) factors with RoPE (theta = 500000) applied, bf16, encoded on the GPU by this
library; seeded N(0,1) queries.  Part of the timed workload is checked against the CPU oracle after
the timed region ("verified").

Rank 0 prints ONE JSON line.  `--impl reference` times the CPU restatement of the reference's
vectorised compute_score (oracle/) on the host cores instead.
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "c1": dict(name="config1 single head", layers=1, kv_heads=1, tokens=4096, group=1, codec=0, codec_name="int4", k=64,
               scaling="strong", dist="gauss_outlier_channels", f32=True),
    "c2": dict(name="config2 llama3-8b decode KV", layers=32, kv_heads=8, tokens=32768, group=4, codec=2,
               codec_name="nf4", k=1024, scaling="weak"),
    "c3": dict(name="config3 tq3 + rht, 64 queries per KV head", layers=1, kv_heads=8, tokens=16384, group=64, codec=4,
               codec_name="tq3", k=256, scaling="strong", rht=True, dist="student_t"),
    "c5": dict(name="config5 long-context sharded", layers=1, kv_heads=8, tokens=1048576, group=4, codec=6,
               codec_name="int4-mx32", k=2048, scaling="strong"),
}
HEAD_DIM = 128
ROPE_THETA = 500000.0
BLOCKS = 5  # the timed region is BLOCKS blocks of --steps steps; the median block is reported


def workload_config(w, n_gpus):
    return {
        "workload": "%s: %d layers x %d KV heads x %d tokens%s, %s tiles, %d queries per KV head, top-%d per query head"
        % (w["name"], w["layers"], w["kv_heads"], w["tokens"], " per GPU" if w["scaling"] == "weak" else " total",
           w["codec_name"], w["group"], w["k"]),
        "tiles_per_gpu": tiles_per_rank(w, n_gpus),
        "queries_per_tile": w["group"],
        "head_dim": HEAD_DIM,
        "sharding": "token range over the ranks, one NCCL all-gather of the per-rank top-k, merge" if n_gpus > 1 else "single GPU",
        "l2_policy": ("the tile stream of a step (>= 134 MB per GPU) exceeds the 126 MB L2; no explicit flush"
                      if tiles_per_rank(w, n_gpus) * 128 > 126e6 else
                      "this configuration's tiles fit the L2 and are timed as they are (L2-resident); not a bandwidth figure"),
        "timed_region": "%d blocks of --steps steps, median block reported" % BLOCKS,
    }


def tiles_per_rank(w, n_gpus):
    t = w["tokens"] if w["scaling"] == "weak" else w["tokens"] // n_gpus
    return w["layers"] * w["kv_heads"] * t


def seeded_projection(seed):
    """Seeded orthogonal 128x128 projection (QR of a Gaussian), float32."""
    g = np.random.default_rng(seed).standard_normal((HEAD_DIM, HEAD_DIM))
    q, _ = np.linalg.qr(g)
    return np.ascontiguousarray(q.T, np.float32)


def synth_keys_numpy(seed, n_heads, tokens, pos0):
    """CPU twin of the key generator (used by the reference arm)."""
    rng = np.random.default_rng(seed)
    chan = np.exp(0.5 * rng.standard_normal(HEAD_DIM)).astype(np.float32)
    k = rng.standard_normal((n_heads, tokens, HEAD_DIM), dtype=np.float32) * chan
    pos = np.arange(pos0, pos0 + tokens, dtype=np.float64)
    inv = ROPE_THETA ** (-np.arange(0, HEAD_DIM, 2, dtype=np.float64) / HEAD_DIM)
    ang = pos[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    a, b = k[..., 0::2].copy(), k[..., 1::2].copy()
    k[..., 0::2] = a * c - b * s
    k[..., 1::2] = a * s + b * c
    u = k.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16  # round to bf16, widen back
    return r.astype(np.uint32).view(np.float32)


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML (read-only) in a
    background thread while the timed region runs."""

    def __init__(self, gpu_index, period_s=0.002):
        self.gpu, self.period = gpu_index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._ready = threading.Event()
        self._thread = None

    def _run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            uuid = None
            try:
                import torch

                uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            except Exception:
                pass
            h = None
            if uuid:
                for cand in ("GPU-" + uuid, uuid):
                    try:
                        h = nv.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {
                "hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap,
            }
            self._ready.set()
            while not self._stop.is_set():
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
                time.sleep(self.period)
        except Exception as e:  # no NVML: report nothing rather than fail the bench
            self.error = repr(e)
            self._ready.set()

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        self._ready.wait(timeout=10)  # NVML is initialised before the timed region starts

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=5)
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.samples:
            out["sm_mhz"] = float(np.median(self.samples))
        if getattr(self, "error", None):
            out["error"] = self.error
        return out


def measured_peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic(kind, n_tiles, nq):
    """DRAM bytes of one score-kernel launch, scaled from the tracked ncu capture of the same kernel
    (read bytes per tile, written bytes per query row); None when no capture is on record."""
    try:
        t = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))["score_stream_kernel"][kind]
        return t["dram_read_bytes_per_tile"] * n_tiles + t["dram_write_bytes_per_query_row"] * nq
    except Exception:
        return None


# --------------------------------------------------------------------------- CPU arm
def cpu_score_rate(tiles, qc, qs, group, heads, min_seconds, threads):
    """Tiles/s of the CPU port over `tiles` ([heads][tokens] tiles, `group` queries per
    head): every tile is scored against its head's `group` queries."""
    from oracle import pyoracle as ora

    per_head = len(tiles) // heads
    t0, reps = time.perf_counter(), 0
    while True:
        for h in range(heads):
            seg = tiles[h * per_head:(h + 1) * per_head]
            for g in range(group):
                ora.score_sink(seg, qc[h * group + g], qs[h * group + g], -1, threads)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            return reps * len(tiles) / dt, dt, reps


def reference_arm(args, w):
    """The reference's own CPU path for this workload: vectorised compute_score
    (AVX-512 > AVX2 > scalar dispatch) over a contiguous tile array, all host
    threads.  The reference has no top-k step, so none is timed here."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import pyoracle as ora

    threads = os.cpu_count() or 1
    heads, tokens = w["kv_heads"], min(w["tokens"], 32768)
    group = min(w["group"], 4)
    keys = synth_keys_numpy(1234, heads, tokens, 0).reshape(-1, HEAD_DIM)
    model = ora.Model(seeded_projection(100), HEAD_DIM, seed=100)
    tiles = model.encode_batch(keys, w["codec"])
    rng = np.random.default_rng(7)
    q = rng.standard_normal((heads * group, HEAD_DIM), dtype=np.float32)
    prep = [model.prepare_query(x) for x in q]
    qc, qs = np.stack([p[0] for p in prep]), np.stack([p[1] for p in prep])
    for _ in range(max(args.warmup, 1)):
        cpu_score_rate(tiles, qc, qs, group, heads, 0.0, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_score_rate(tiles, qc, qs, group, heads, 0.0, threads)
    dt = time.perf_counter() - t0
    value = args.steps * len(tiles) / dt
    sample = "%d tiles (%d KV heads x %d tokens of the context) x %d queries per step" % (len(tiles), heads, tokens, group)
    line = {
        "impl": "reference", "metric": "tiles_scored_per_s", "value": value, "unit": "tiles/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": w["scaling"], "vs_baseline": None, "dtype": "int4->f32", "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": "tiles/s", "cores": threads, "kind": "port", "sample": sample,
                         "isa": ["scalar", "avx2", "avx512"][ora.simd_level()]},
        "e2e": {"value": value, "unit": "tiles/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference binary unavailable (Rust, no toolchain): C restatement of its AVX-512/AVX2 compute_score; "
                "scoring only (the reference has no top-k)",
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- GPU arm
def build_shard(S, torch, w, rank, world, dev, keep_keys_of_segment=None):
    """Generate this rank's keys on the device, encode them into tiles, prepare the queries.
    Returns (tiles_u8, segments, q_coarse, q_sign, n_tiles, encode_tiles_per_s, extras); extras holds
    what the oracle check needs (projection and seed per layer, the raw queries, the bf16 keys of
    one segment)."""
    L, H, G = w["layers"], w["kv_heads"], w["group"]
    if w["scaling"] == "weak":
        T, pos0 = w["tokens"], rank * w["tokens"]
    else:
        pos0, T = S.shard.shard_range(w["tokens"], rank, world)
    n_tiles = L * H * T
    tiles = torch.empty(n_tiles * 128, dtype=torch.uint8, device=dev)
    nq = L * H * G
    q_coarse = torch.empty(nq, 128, dtype=torch.float32, device=dev)
    q_sign = torch.empty(nq, 4, dtype=torch.int64, device=dev)
    gen = torch.Generator(device=dev)
    pos = torch.arange(pos0, pos0 + T, device=dev, dtype=torch.float64)
    inv = ROPE_THETA ** (-torch.arange(0, HEAD_DIM, 2, device=dev, dtype=torch.float64) / HEAD_DIM)
    ang = pos[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    positions = torch.arange(pos0, pos0 + T, device=dev, dtype=torch.int32).repeat(H).contiguous()
    heads = torch.arange(H, device=dev, dtype=torch.int16).repeat_interleave(T).contiguous()
    enc_ms = 0.0
    chunk_tokens = min(T, 131072)
    extras = {"layers": [], "queries": [], "keys": None, "pos0": pos0, "T": T}
    for l in range(L):
        proj = seeded_projection(100 + l)
        model = S.Model.from_projection(proj, HEAD_DIM, 100 + l, rht=bool(w.get("rht")))
        extras["layers"].append((proj, 100 + l))
        gen.manual_seed(1234 + l)  # the per-channel scale belongs to the layer: the same on every rank
        chan = torch.exp(0.5 * torch.randn(HEAD_DIM, generator=gen, device=dev))
        gen.manual_seed(5678 + l + 7919 * rank)  # every rank holds different tokens
        # one encode call covers a whole layer when its heads fit one chunk, else one head's chunk
        heads_per_call = H if T <= chunk_tokens else 1
        for h in range(0, H, heads_per_call):
            for t0 in range(0, T, chunk_tokens):
                t1 = min(T, t0 + chunk_tokens)
                shape = (heads_per_call, t1 - t0, HEAD_DIM)
                if w.get("dist") == "student_t":
                    # Student-t (nu = 4) with 1 % of the entries x 20 (configuration 3)
                    z = torch.randn(5, *shape, generator=gen, device=dev)
                    k = z[0] / torch.sqrt((z[1:] ** 2).mean(0))
                    k = torch.where(torch.rand(shape, generator=gen, device=dev) < 0.01, 20.0 * k, k)
                elif w.get("dist") == "gauss_outlier_channels":
                    # N(0,1), channels 7 and 93 x 8 (configuration 1)
                    k = torch.randn(shape, generator=gen, device=dev)
                    k[..., 7] *= 8.0
                    k[..., 93] *= 8.0
                else:
                    k = torch.randn(shape, generator=gen, device=dev) * chan
                    a, b = k[..., 0::2].clone(), k[..., 1::2].clone()
                    k[..., 0::2] = a * cos[t0:t1] - b * sin[t0:t1]
                    k[..., 1::2] = a * sin[t0:t1] + b * cos[t0:t1]
                kb = k.contiguous() if w.get("f32") else k.to(torch.bfloat16).contiguous()
                n = heads_per_call * (t1 - t0)
                off = ((l * H + h) * T + t0) * 128
                lo = h * T + t0
                if keep_keys_of_segment is not None and l == keep_keys_of_segment[0] and h <= keep_keys_of_segment[1] < h + heads_per_call \
                        and t0 == 0:
                    extras["keys"] = kb[keep_keys_of_segment[1] - h, : min(t1, 4096)].float().cpu().numpy()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                model.encode_keys(kb, w["codec"], n=n, key_dtype=S.F32 if w.get("f32") else S.BF16, positions=positions[lo:lo + n],
                                  head_ids=heads[lo:lo + n], out=tiles[off:off + n * 128])
                e1.record()
                torch.cuda.synchronize()
                enc_ms += e0.elapsed_time(e1)
        gen.manual_seed(99 + l)  # queries are the same on every rank
        q = torch.randn(H * G, HEAD_DIM, generator=gen, device=dev)
        extras["queries"].append(q.cpu().numpy())
        model.prepare_queries(q, nq=H * G, q_coarse_out=q_coarse[l * H * G:(l + 1) * H * G], q_sign_out=q_sign[l * H * G:(l + 1) * H * G])
        torch.cuda.synchronize()
        model.release()
    return tiles, S.shard.shard_segments(L, H, T, G, pos0), q_coarse, q_sign, n_tiles, n_tiles / (enc_ms * 1e-3), extras


def verify_against_oracle(S, w, tiles, segs, q_coarse, q_sign, out_idx, out_sc, extras, layer, head, world):
    """One (layer, KV head) segment of the timed workload against the CPU oracle, outside the timed
    region: the first 4096 tile records bit for bit against the oracle's encoder, the prepared
    queries of the segment bit for bit, and the top-k of the segment's query rows (at N = 1: scores
    within 1e-3 of the oracle's, index sets equal except where scores tie within 2e-3; at N > 1 the
    merged result mixes ranks, so the reported (index, score) pairs of this rank's token range are
    checked against the oracle's scores of those tiles)."""
    from oracle import pyoracle as ora

    H, G, T, k = w["kv_heads"], w["group"], extras["T"], w["k"]
    seg = layer * H + head
    tb, nt, qb, nq, base = (int(x) for x in segs[seg].tolist())
    host = np.frombuffer(tiles[tb * 128:(tb + nt) * 128].cpu().numpy().tobytes(), S.TILE_DTYPE)
    proj, seed = extras["layers"][layer]
    om = ora.Model(proj, HEAD_DIM, seed=seed, rht=bool(w.get("rht")))
    ok = True
    if extras["keys"] is not None:
        n0 = len(extras["keys"])
        want = om.encode_batch(extras["keys"], w["codec"], pos=np.arange(base, base + n0, dtype=np.uint32),
                               head=np.full(n0, head, np.uint16))
        ok &= host[:n0].tobytes() == want.tobytes()
    qc = q_coarse[qb:qb + nq].cpu().numpy()
    qs = q_sign[qb:qb + nq].cpu().numpy().view(np.uint64)
    for j in (0, nq - 1):
        wc, ws = om.prepare_query(extras["queries"][layer][head * G + j])
        ok &= np.array_equal(qc[j], wc) and np.array_equal(qs[j], ws)
    gi = out_idx[qb:qb + nq].cpu().numpy().view(np.uint32)
    gs = out_sc[qb:qb + nq].cpu().numpy().view(np.float32)
    for j in range(min(nq, 4)):
        want = ora.score_tiles(host, qc[j], qs[j])
        mine = (gi[j] >= base) & (gi[j] < base + nt)
        ok &= bool(np.all(np.abs(want[gi[j][mine] - base] - gs[j][mine]) <= 1e-3))
        if world == 1:
            kk = min(k, nt)
            oi, ov = ora.topk(want, kk)
            ok &= bool(np.all(np.abs(gs[j][:kk] - ov) <= 1e-3))
            ok &= all(abs(want[i] - ov[-1]) <= 2e-3 for i in set(oi) ^ set((gi[j][:kk] - base).tolist()))
    return bool(ok)


def time_blocks(torch, step, steps, barrier):
    """BLOCKS blocks of `steps` steps, CUDA events around every block; returns the per-block ms."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(BLOCKS)]
    barrier()
    for a, b in ev:
        a.record()
        for _ in range(steps):
            step()
        b.record()
    barrier()
    return [a.elapsed_time(b) for a, b in ev]


def run_scoring_workload(args, w, S, torch, dist, rank, local, world, dev, stream, verify=True, cpu_legs=True):
    """Build, time and check one scoring workload; returns the JSON record (rank 0) or None."""
    tiles, segs, q_coarse, q_sign, n_tiles, enc_rate, extras = build_shard(S, torch, w, rank, world, dev, keep_keys_of_segment=(0, 0))
    nq, k = q_coarse.shape[0], w["k"]
    out_idx = torch.empty(nq, k, dtype=torch.int32, device=dev)
    out_sc = torch.empty(nq, k, dtype=torch.float32, device=dev)

    # every rank's handle of the sharded scorer: the NCCL unique id of rank 0 travels by a torch broadcast
    uid = None
    if world > 1:
        t = torch.from_numpy(S.shard_unique_id() if rank == 0 else np.zeros(128, np.uint8)).to(dev)
        dist.broadcast(t, 0)
        uid = t.cpu().numpy()
    shard = S.Shard(uid, rank, world)
    if world > 1 and args.exchange != "peer":
        shard.set_exchange(args.exchange)

    def step():
        shard.score_topk(tiles, segs, q_coarse, q_sign, nq, k, out_index=out_idx, out_score=out_sc)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = S.launch_count()
    torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see the timed region only
    block_ms = time_blocks(torch, step, args.steps, barrier)
    torch.cuda.profiler.stop()
    launches = (S.launch_count() - launches0) // BLOCKS
    clocks = sampler.stop() if rank == 0 else None
    # kernel durations for the roofline: CUDA events inside the library around the score kernel and the merge,
    # over steps of their own (the timed blocks above replay a captured graph, which records no events)
    S.timing_begin(min(args.steps, 20))
    for _ in range(min(args.steps, 20)):
        step()
    score_ms, merge_ms = S.timing_end(min(args.steps, 20))
    # per-component device times of a sharded step (events inside the library), a few steps outside the timed blocks
    comp = np.zeros(3)
    if world > 1:
        shard.set_timing(True)
        acc = []
        for _ in range(10):
            step()
            acc.append(shard.last_times())
        shard.set_timing(False)
        comp = np.median(np.array(acc), axis=0)
    verified = verify_against_oracle(S, w, tiles, segs, q_coarse, q_sign, out_idx, out_sc, extras, 0, 0, world) if verify else None

    # ---- end to end through the C ABI with host buffers (pinned): queries up, top-k down, one call at a time
    hq = q_coarse.cpu().pin_memory()
    hs = q_sign.cpu().pin_memory()
    h_idx = torch.empty(nq, k, dtype=torch.int32).pin_memory()
    h_sc = torch.empty(nq, k, dtype=torch.float32).pin_memory()

    def e2e_step():
        shard.score_topk(tiles, segs, hq, hs, nq, k, out_index=h_idx, out_score=h_sc)

    barrier()  # (the ranks' verification took different times: start the next steps together)
    for _ in range(3):
        e2e_step()
    barrier()
    e2e_blocks = []
    for _ in range(BLOCKS):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_blocks.append(1e3 * (time.perf_counter() - t0))
    barrier()
    e2e_ok = bool(torch.equal(h_idx.to(dev), out_idx))

    # The same end-to-end calls from two host threads (the C ABI is re-entrant; every thread has its own
    # stream and staging buffers inside the library, and the reference's consumers call it from several
    # worker threads): one caller's copies overlap the other caller's kernels.  A named extra, N = 1 only.
    concurrent = None
    if world == 1:
        callers = 2
        per = (args.steps + callers - 1) // callers
        outs = [(torch.empty(nq, k, dtype=torch.int32).pin_memory(), torch.empty(nq, k, dtype=torch.float32).pin_memory())
                for _ in range(callers)]
        go, done = threading.Barrier(callers + 1), threading.Barrier(callers + 1)
        failed = []
        slowest = [0.0] * callers
        n_rounds = 3  # the median round is reported (a round is short: one stalled call would dominate it)
        t_end = [[0.0] * callers for _ in range(n_rounds)]

        def caller(i, n_calls):
            # the thread lives through all rounds: its set-up (stream, staging memory, plan) and its tear-down at thread exit
            # are the library's per-thread state, not part of a call
            try:
                S.set_device(local)  # thread-local in the library; no stream set: the library's own per-thread stream
                for _ in range(2):
                    S.score_topk(tiles, segs, hq, hs, nq, k, out_index=outs[i][0], out_score=outs[i][1])
                for r in range(n_rounds):
                    go.wait()
                    for _ in range(n_calls):
                        t_call = time.perf_counter()
                        S.score_topk(tiles, segs, hq, hs, nq, k, out_index=outs[i][0], out_score=outs[i][1])
                        slowest[i] = max(slowest[i], 1e3 * (time.perf_counter() - t_call))
                    t_end[r][i] = time.perf_counter()  # (host outputs: the call returns when its results have arrived)
                    done.wait()
            except Exception as exc:  # surfaces in the main thread
                failed.append(exc)
                go.abort()
                done.abort()

        threads = [threading.Thread(target=caller, args=(i, per)) for i in range(callers)]
        for th in threads:
            th.start()
        rounds_ms = []
        try:
            for r in range(n_rounds):
                go.wait()
                t0 = time.perf_counter()
                done.wait()
                rounds_ms.append(1e3 * (max(t_end[r]) - t0) / (per * callers))
        except threading.BrokenBarrierError:
            pass
        for th in threads:
            th.join()
        if failed:
            raise failed[0]
        piped_ms = float(np.median(rounds_ms))
        assert torch.equal(outs[0][0], h_idx) and torch.equal(outs[1][0], h_idx), "concurrent callers disagree with the serial result"
        concurrent = {"callers": callers, "ms_per_step": piped_ms, "value": n_tiles / (piped_ms * 1e-3), "rounds_ms_per_step": rounds_ms,
                      "slowest_call_ms": max(slowest)}

    ms_block = float(np.median(block_ms))
    e2e_block = float(np.median(e2e_blocks))
    if world > 1:
        t = torch.tensor([ms_block, e2e_block, max(block_ms), min(block_ms)] + list(comp), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_block, e2e_block = float(t[0]), float(t[1])
        block_ms = [float(t[3]), ms_block, float(t[2])]
        comp = t[4:7].cpu().numpy()
        v = torch.tensor([1 if (verified and e2e_ok) else 0], device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MIN)
        verified = bool(v.item())
    shard_how = shard.status()
    shard.destroy()
    if rank != 0:
        return None

    total_tiles = n_tiles * world
    ms_step = ms_block / args.steps
    value = total_tiles / (ms_step * 1e-3)
    peak, peak_kind = measured_peak_gbs()
    k_ms = float(np.median(score_ms)) if len(score_ms) else float("nan")
    achieved = n_tiles * 128 / (k_ms * 1e-3) / 1e9
    e2e_ms = e2e_block / args.steps
    rec = {
        "metric": "tiles_scored_per_s", "value": value, "unit": "tiles/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": w["scaling"],
        "vs_baseline": None, "dtype": "int4->f32", "data": "synthetic", "config": workload_config(w, world),
        "blocks_ms_per_step": {"min": min(block_ms) / args.steps, "median": ms_step, "max": max(block_ms) / args.steps, "blocks": BLOCKS},
        "scores_per_s": value * w["group"],
        "hbm_gbs_whole_step": total_tiles * 128 / (ms_step * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "kernel": "score_stream_kernel (fused eq. 2.3 score + streaming top-k)", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "frac_of_nominal_8000": achieved / 8000.0, "kernel_ms": k_ms,
                     "merge_kernel_ms": float(np.median(merge_ms)) if len(merge_ms) else None,  # (early-exit pass of the generic kernel, compaction, merge)
                     "algorithmic_bytes_per_launch": n_tiles * 128,
                     "traffic": ncu_traffic(w["codec_name"], n_tiles, nq),
                     "traffic_source": "ncu dram__bytes of the same kernel on this workload shape, per tile and per query row, "
                                       "scaled to this launch"},
        "e2e": {"value": total_tiles / (e2e_ms * 1e-3), "unit": "tiles/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(nq * (512 + 32)), "d2h_bytes_per_step": int(nq * k * 8),
                "schedule": "one call at a time from one host thread", "concurrent_callers": concurrent},
        "gpu_launches": int(launches),
        # which kernel scored the rows of the last step: rows the tensor-core kernel handed to the generic kernel are correct but slow
        "score_stats": S.last_score_stats(),
        "encode_tiles_per_s": enc_rate,
        "verified": bool(verified and e2e_ok),
        "clocks": clocks,
    }
    if world > 1:
        rec["exchange"] = {"entry_point": "slha_b200_shard_score_topk", "how": shard_how, "ms_local_score_topk": float(comp[0]),
                           "ms_all_gather": float(comp[1]), "ms_merge": float(comp[2]),
                           "all_gather_bytes_per_rank": int(2 * nq * k * 4)}
    if world == 1 and cpu_legs:
        n_s = min(n_tiles, w["kv_heads"] * min(w["tokens"], 32768))
        heads, group = w["kv_heads"], min(w["group"], 4)
        per = n_tiles // (w["layers"] * heads)
        host_tiles = np.concatenate([np.frombuffer(tiles[h * per * 128:(h * per + n_s // heads) * 128].cpu().numpy().tobytes(), S.TILE_DTYPE)
                                     for h in range(heads)])
        threads = os.cpu_count() or 1
        rows = [h * w["group"] + g for h in range(heads) for g in range(group)]
        hqc = hq.numpy()[rows]
        hqs = hs.numpy().view(np.uint64)[rows]
        rate, dt, reps = cpu_score_rate(host_tiles, hqc, hqs, group, heads, 3.0, threads)
        from oracle import pyoracle as ora

        rec["cpu_baseline"] = {
            "value": rate, "unit": "tiles/s", "cores": threads, "kind": "port",
            "isa": ["scalar", "avx2", "avx512"][ora.simd_level()],
            "sample": "%d tiles (%d KV heads x %d tokens) x %d queries, %d passes in %.1f s" % (n_s, heads, n_s // heads, group, reps, dt),
        }
        # For context only: the reference's own CUDA scoring kernel (one thread per tile, one launch
        # per query, 256-thread blocks as in its tests) on the same resident tiles, when the built
        # oracle/_ref library travelled with the repository.  It writes full score vectors and has
        # no top-k; the figure is tiles per second with every tile scored against its 4 queries.
        refk = ora.ref_cuda_library()
        if refk is not None:
            pt = n_s // heads
            sc = torch.empty(group * pt, dtype=torch.float32, device=dev)
            ms_out = ctypes.c_float(0.0)
            total_ms = 0.0
            for h in range(heads):
                rc = refk.slha_ref_cuda_time(tiles.data_ptr() + h * per * 128, pt, q_coarse[h * w["group"]:].data_ptr(),
                                             q_sign[h * w["group"]:].data_ptr(), group, sc.data_ptr(), 3, stream.cuda_stream,
                                             ctypes.byref(ms_out))
                assert rc == 0, rc
                total_ms += ms_out.value
            rec["reference_cuda_kernel"] = {
                "value": n_s / (total_ms * 1e-3), "unit": "tiles/s", "ms": total_ms,
                "sample": "slhav2-vram/kernels/slha_score.cu unmodified: %d KV heads x %d tiles x %d queries, full score vectors, no top-k" % (heads, pt, group),
            }
    return rec


def run_pool_workload(args, S, torch, dev):
    """Configuration 4 at full size: one pool of 131072 tokens x 8 KV heads = 1 048 576 slots of mixed
    8/4 tiles under a budget of 60 % of the full-HOT footprint, H2O importance eviction with a sink of
    4 and a recent window of 2048.  A step = append 8 keys (one token x 8 heads), score one GQA group
    with top-64, observe the query (H2O), enforce the budget.  Host-timed through the C ABI."""
    cap, d = 131072 * 8, HEAD_DIM
    budget = int(0.6 * 128 * cap)
    model = S.Model.from_projection(seeded_projection(7), d, 7)
    pool = S.TilePool(cap, budget, S.PAGE_LOWEST_IMPACT_FIRST, S.EVICT_IMPORTANCE, sink_window=4, recent_window=2048)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4242)
    steps, extra = 256, 64
    total = 16 + steps + extra
    fill = cap - 8 * total
    for t0 in range(0, fill, 131072):
        n = min(131072, fill - t0)
        kb = torch.randn(n, d, generator=gen, device=dev).to(torch.bfloat16).contiguous()
        pos = torch.arange(t0, t0 + n, device=dev, dtype=torch.int32) // 8
        torch.cuda.synchronize()
        pool.append_keys(model, kb, S.CODEC_MIXED, n=n, key_dtype=S.BF16, positions=pos)
    q = torch.randn(total, 4, d, generator=gen, device=dev)
    qc, qs = model.prepare_queries(q.reshape(-1, d), nq=4 * total)
    keys = torch.randn(total, 8, d, generator=gen, device=dev).to(torch.bfloat16).contiguous()
    torch.cuda.synchronize()
    pool.enforce_budget()
    parts = {"append_keys": 0.0, "score_topk": 0.0, "observe_query": 0.0, "enforce_budget": 0.0}

    def step(i, timed=False):
        pos = np.full(8, fill // 8 + i, np.uint32)
        calls = (("append_keys", lambda: pool.append_keys(model, keys[i], S.CODEC_MIXED, n=8, key_dtype=S.BF16, positions=pos)),
                 ("score_topk", lambda: pool.score_topk(qc[4 * i:4 * i + 4], qs[4 * i:4 * i + 4], 4, 64)),
                 ("observe_query", lambda: pool.observe_query(qc[4 * i], qs[4 * i], 1.0)),
                 ("enforce_budget", lambda: pool.enforce_budget()))
        for name, call in calls:
            if timed:
                S.synchronize()
                t = time.perf_counter()
            call()
            if timed:
                S.synchronize()
                parts[name] += 1e3 * (time.perf_counter() - t) / extra

    for i in range(16):
        step(i)
    S.synchronize()
    l0 = S.launch_count()
    t0 = time.perf_counter()
    for i in range(16, 16 + steps):
        step(i)
    S.synchronize()
    ms = 1e3 * (time.perf_counter() - t0) / steps
    launches = (S.launch_count() - l0) / steps
    for i in range(16 + steps, total):  # each call alone, a synchronize on both sides: where the step's time goes
        step(i, timed=True)
    st = pool.stats()
    return {"workload": "config4 elastic pool: 1048576 slots, mixed 8/4, budget 60 %, H2O sink 4 + recent 2048; "
                        "step = append 8 keys + score 4 queries top-64 + observe + enforce_budget",
            "ms_per_step": ms, "steps": steps, "launches_per_step": launches, "calls_alone_ms": {k: round(v, 4) for k, v in parts.items()},
            "score_stats": S.last_score_stats(), "hot": st["hot"], "warm": st["warm"], "cold": st["cold"],
            "live_bytes": st["live_bytes"], "budget": budget, "within_budget": bool(st["live_bytes"] <= budget)}


def run_next_rows(S, torch, dev):
    """Timed figures of the rows beside the hot path (one GPU, device-resident inputs, CUDA events on the launching
    stream, 20 calls after 3): the decode tail over a step's winners, a layer's dense scores for the llama.cpp shim,
    and evictions journalled in the reference's event-log format."""
    import tempfile

    out = {}
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    S.set_stream(stream.cuda_stream)
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    # decode tail: softmax over the 2048 winners of 32 query rows + weighted sum of their bf16 value rows (d_v = 128);
    # winners drawn from a 2^20-row value array per KV head as configuration 5's would be
    nq, k, d_v, rows_per_head = 32, 2048, HEAD_DIM, 1 << 20
    values = torch.randn(8 * rows_per_head, d_v, generator=gen, device=dev).to(torch.bfloat16).contiguous()
    top_i = torch.stack([torch.randperm(rows_per_head, generator=gen, device=dev)[:k] for _ in range(nq)]).to(torch.int32).contiguous()
    top_s = (torch.randn(nq, k, generator=gen, device=dev).sort(dim=1, descending=True).values * 4).contiguous()
    base = (torch.arange(nq, device=dev) // 4 * rows_per_head).to(torch.int64)
    o = torch.empty(nq, d_v, dtype=torch.float32, device=dev)
    ms = timed(lambda: S.attend_topk(top_i, top_s, k, 1.0 / np.sqrt(HEAD_DIM), values, d_v, value_dtype=S.BF16, value_row_base=base, out=o))
    out["attend_topk"] = {"workload": "32 query rows x top-2048, bf16 value rows of 128 (gathered from 8 x 2^20 rows)", "ms": ms,
                          "gathered_gb_per_s": nq * k * d_v * 2 / (ms * 1e-3) / 1e9}
    del values

    # a layer's dense scores in one call: 8 KV heads x 32768 tiles, 16 tokens x 4 query heads per KV head; once with the
    # shim's default codec (mixed 8/4) and once with grouped INT4
    heads, tokens, n_tok, gqa = 8, 32768, 16, 4
    model = S.Model.from_projection(seeded_projection(11), HEAD_DIM, 11)
    keys = torch.randn(heads * tokens, HEAD_DIM, generator=gen, device=dev).to(torch.bfloat16).contiguous()
    rows = heads * n_tok * gqa
    q = torch.randn(rows, HEAD_DIM, generator=gen, device=dev)
    qc = torch.empty(rows, 128, dtype=torch.float32, device=dev)
    qs = torch.empty(rows, 4, dtype=torch.int64, device=dev)
    model.prepare_queries(q, nq=rows, q_coarse_out=qc, q_sign_out=qs)
    segs = S.make_segments([(h * tokens, tokens, h * n_tok * gqa, n_tok * gqa, 0) for h in range(heads)])
    offs = np.arange(rows, dtype=np.uint64) * np.uint64(tokens)  # (host descriptors: the call reads them without a stream round trip)
    dst = torch.empty(rows, tokens, dtype=torch.float32, device=dev)
    tiles = S.DeviceBuffer(heads * tokens * 128)
    out["score_segments"] = {"workload": "8 KV heads x 32768 tiles, 64 query rows per head, dense float32 scores (67 MB written per call)"}
    for name, codec in (("mixed-8/4", S.CODEC_MIXED), ("int4-grouped", S.CODEC_INT4_GROUPED)):
        model.encode_keys(keys, codec, n=heads * tokens, key_dtype=S.BF16, out=tiles)
        l0 = S.launch_count()
        ms = timed(lambda: S.score_segments(tiles, segs, qc, qs, rows, dst, offs, tokens), n=10)
        out["score_segments"][name] = {"ms": ms, "scores_per_s": rows * tokens / (ms * 1e-3), "written_gb_per_s": rows * tokens * 4 / (ms * 1e-3) / 1e9,
                                       "launches_per_call": (S.launch_count() - l0) / 13}
    # full score vectors (slha_score_tiles over a device arena): the int4 tiles of above, four queries, one float per tile and query
    full = torch.empty(4, heads * tokens, dtype=torch.float32, device=dev)
    ms = timed(lambda: S.score_tiles(tiles, heads * tokens, qc[:4], qs[:4], 4, out=full))
    out["score_tiles"] = {"workload": "262144 int4-grouped tiles x 4 queries, full float32 score vectors", "ms": ms,
                          "tiles_per_s": heads * tokens / (ms * 1e-3), "tile_gb_per_s": heads * tokens * 128 / (ms * 1e-3) / 1e9}
    del dst, keys, full
    tiles.free()

    # evictions journalled in the reference's event-log format: 262144 HOT tiles, budget for 65536, causal policy
    S.set_stream(None)
    n = 262144
    pool = S.TilePool(n, 128 * n, S.PAGE_OLDEST_FIRST, S.EVICT_CAUSAL)
    kb = torch.randn(n, HEAD_DIM, generator=gen, device=dev).to(torch.bfloat16).contiguous()
    torch.cuda.synchronize()
    pool.append_keys(model, kb, S.CODEC_INT4_GROUPED, n=n, key_dtype=S.BF16, want_slots=False)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "evicted.sllg")
        pool.attach_event_log(path)
        pool.set_budget(96 * (n // 4))  # everything is paged out (96 B per WARM tile), then three quarters are evicted
        S.synchronize()
        t0 = time.perf_counter()
        within = pool.enforce_budget()
        S.synchronize()
        dt = time.perf_counter() - t0
        st = pool.event_log_stats()
        out["event_log"] = {"workload": "262144 tiles, budget for a quarter of them: page-out of all, eviction of 196608 with their records appended",
                            "ms": 1e3 * dt, "records": st["records"], "log_mb": (16 + 144 * st["records"]) / 1e6,
                            "evicted_tiles_per_s": st["records"] / dt, "within_budget": bool(within), "log_errors": st["log_errors"]}
    pool.destroy()
    return out


def pool_arm(args):
    """--workload c4 on its own: the elastic pool's decode step (one GPU; the pool does not shard)."""
    import torch

    import slhav2_b200 as S

    if not torch.cuda.is_available() or S.device_count() == 0:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(0)
    S.set_device(0)
    r = run_pool_workload(args, S, torch, torch.device("cuda", 0))
    line = {"metric": "ccos_pool_decode_steps_per_s", "value": 1e3 / r["ms_per_step"], "unit": "steps/s", "n_gpus": 1,
            "steps": r["steps"], "warmup": 16, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "replicas only",
            "vs_baseline": None, "dtype": "u8/f32", "data": "synthetic", "config": {"workload": r["workload"]}, "pool": r,
            "gpu_launches": int(r["launches_per_step"] * r["steps"])}
    print(json.dumps(line))


def gpu_arm(args, w):
    import torch

    import slhav2_b200 as S

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, "launch with torchrun --nproc-per-node N for --gpus N"
    if not torch.cuda.is_available() or S.device_count() == 0:
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    S.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    # one explicit stream for torch and the library: the library treats a NULL stream as
    # "use my own non-blocking stream", which would not be ordered after torch's default stream
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    S.set_stream(stream.cuda_stream)

    line = run_scoring_workload(args, w, S, torch, dist, rank, local, world, dev, stream)
    also = {}
    if args.also and args.workload == "c5" and not (args.layers or args.tokens):
        light = argparse.Namespace(**vars(args))
        light.steps = max(5, args.steps // 4)
        for name in (["c2", "c1", "c3"] if world == 1 else ["c2"]):
            torch.cuda.empty_cache()
            r = run_scoring_workload(light, dict(WORKLOADS[name]), S, torch, dist, rank, local, world, dev, stream, cpu_legs=False)
            if r is not None:
                also[name] = {kk: r[kk] for kk in ("value", "unit", "ms_per_step", "scaling", "config", "roofline", "e2e", "encode_tiles_per_s",
                                                   "verified", "gpu_launches", "blocks_ms_per_step", "score_stats") if kk in r}
                if "exchange" in r:
                    also[name]["exchange"] = r["exchange"]
        if world == 1:
            torch.cuda.empty_cache()
            S.set_stream(None)
            also["c4"] = run_pool_workload(args, S, torch, dev)
            torch.cuda.empty_cache()
            also["next_rows"] = run_next_rows(S, torch, dev)
    if rank == 0:
        line["also"] = also
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS) + ["c4"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the ranks' top-k lists meet (peer-memory loads by the merge kernel, or an NCCL all-gather)")
    ap.add_argument("--no-also", dest="also", action="store_false", help="only the named workload (no c1..c4 sub-records)")
    ap.add_argument("--layers", type=int, default=0, help="profiling aid: shrink the workload to this many layers")
    ap.add_argument("--tokens", type=int, default=0, help="profiling aid: shrink the workload to this many tokens")
    args = ap.parse_args()
    if args.workload == "c4":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the pool workload has no CPU reference arm; the headline workload is c5"}))
            return
        return pool_arm(args)
    w = dict(WORKLOADS[args.workload])
    if args.layers:
        w["layers"] = args.layers
        w["name"] += " (reduced to %d layers)" % args.layers
    if args.tokens:
        w["tokens"] = args.tokens
        w["name"] += " (reduced to %d tokens)" % args.tokens
    if args.impl == "reference":
        reference_arm(args, w)
    else:
        gpu_arm(args, w)


if __name__ == "__main__":
    main()
