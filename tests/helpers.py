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
