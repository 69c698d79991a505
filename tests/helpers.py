"""Shared test helpers: seeded synthetic inputs built with the oracle's PRNG."""
import numpy as np

from oracle import pyoracle as ora

F = np.float32


def scenario_generate(seed, n, rho):
    """scirust/src/scenario.rs:116-156 (generate): query + (k_coarse, e) tokens."""
    rng = ora.Rng(seed)
    q = rng.gaussian(128)
    rho = F(min(max(rho, 0.0), 0.999))
    alpha = F(rho / np.sqrt(F(1.0) - rho * rho, dtype=F))
    toks = []
    for _ in range(n):
        kc = rng.gaussian(128)
        e = rng.gaussian(128)
        nk = _norm(kc)
        ne = max(_norm(e), F(1.0e-9))
        g = F(F(alpha * nk) / ne)
        e = (e * g).astype(F)
        toks.append((kc, e))
    return q, toks


def _norm(v):
    s = F(0.0)
    for x in v:
        s = F(s + F(x * x))
    return F(np.sqrt(s))


def scenario_tile(z, tok, pos, warm=False):
    t = np.zeros(1, ora.TILE_DTYPE)
    kc, e = tok
    ora.lib.ora_scenario_build_tile(
        z.ctypes.data, np.ascontiguousarray(kc, F).ctypes.data, np.ascontiguousarray(e, F).ctypes.data, pos, int(warm), t.ctypes.data
    )
    return t


def scenario_projection(seed):
    """scirust/src/scenario.rs:56-66: Z = Rng(seed).fill_gaussian(256*128)."""
    return ora.Rng(seed).gaussian(256 * 128)


def scenario_sign_bits(z, v):
    out = np.zeros(4, np.uint64)
    ora.lib.ora_scenario_sign_bits(z.ctypes.data, np.ascontiguousarray(v, F).ctypes.data, out.ctypes.data)
    return out


def orthogonal_projection(seed, d, rows=128):
    """Seeded random matrix with orthonormal rows (rows x d), float32."""
    g = ora.Rng(seed).gaussian(rows * d).astype(np.float64).reshape(rows, d)
    q, _ = np.linalg.qr(g.T)  # d x rows, orthonormal columns
    return np.ascontiguousarray(q.T[:rows], dtype=F)


def gaussian_keys(seed, n, d, outlier_channels=(), outlier_scale=8.0):
    k = ora.Rng(seed).gaussian(n * d).reshape(n, d)
    for c in outlier_channels:
        k[:, c] *= F(outlier_scale)
    return np.ascontiguousarray(k, F)


def to_bf16_f32(x):
    """Round float32 to bfloat16 (nearest even) and widen back: exact in f32."""
    u = np.ascontiguousarray(x, F).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(F)


# ---- configuration-shaped synthetic inputs (seeded, oracle PRNG) -----------------
def make_model_pair(d=128, seed=7, rht=False, pseed=11):
    """(oracle model, projection) for a seeded row-orthonormal projection."""
    p = orthogonal_projection(pseed, d)
    return ora.Model(p, d, seed=seed, rht=rht), p


def random_tiles(n, codec, seed, d=128, warm_every=0, nocorr_every=0, model=None):
    """Oracle-encoded tiles of seeded Gaussian keys (optionally some WARM / NOCORR)."""
    if model is None:
        model, _ = make_model_pair(d)
    keys = gaussian_keys(seed, n, model.d, outlier_channels=(7, 93))
    tiles = model.encode_batch(keys, codec)
    if warm_every:
        idx = np.arange(n) % warm_every == 0
        tiles["flags"][idx] |= ora.FLAG_WARM
        tiles["residual_bitmap"][idx] = 0
        tiles["dynamic_lambda"][idx] = 0
    if nocorr_every and codec in (4, 5):
        idx = np.arange(n) % nocorr_every == 1
        nb = 16 if codec == 4 else 14
        # every second of them keeps the plane's bytes: a decoder must go by the flag (tests.rs:356-384 builds such tiles)
        tiles["latent_kv"][idx & (np.arange(n) % (2 * nocorr_every) == 1), 64 - nb:] = 0
        tiles["flags"][idx] |= ora.FLAG_TQ3_NOCORR
    return tiles


def random_queries(nq, seed):
    rng = ora.Rng(seed)
    qc = rng.gaussian(nq * 128).reshape(nq, 128)
    qs = np.array([[rng.next_u64() for _ in range(4)] for _ in range(nq)], np.uint64)
    return qc, qs


def oracle_scores(tiles, qc, qs):
    return np.stack([ora.score_tiles(tiles, qc[j], qs[j]) for j in range(len(qc))])
