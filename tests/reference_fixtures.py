"""The reference's own codec test inputs, restated with the oracle's PRNG (same seeds, same construction).

scirust/src/attention/slha_v2/tests.rs builds every codec test from `Rng::new(seed)` draws: the steep
GPT-2-like latent (:133-141), the signed ramp (:52-55, :263-266) and the per-codec score-equivalence
fixtures (tq3 :356-384, mix3 :501-527, nf4 :693-715, mixed :800-822, int4 :912-919). The functions here
return the same tiles and queries, so the tests that use them are the reference's tests run on the oracle
and, for the scores, on the GPU library.
"""
import numpy as np

from oracle import pyoracle as ora
from .helpers import scenario_generate, scenario_projection, scenario_sign_bits, scenario_tile

F = np.float32
ALL_ONES = 0xFFFFFFFFFFFFFFFF
INT4, GROUPED, NF4, MIXED, TQ3, MIX3 = 0, 1, 2, 3, 4, 5
MIXED_HI_DIMS, MIXED_DIMS, GROUP_DIM = 8, 120, 16
TQ3_CODE_BYTES, MIX3_CORR_OFF, TQ3_CORRECTION = 48, 50, F(0.25)


def steep_latent(seed):
    """tests.rs:133-141: per-dimension std 37 (d+1)^-0.9."""
    rng = ora.Rng(seed)
    v = np.zeros(128, F)
    for d in range(128):
        amp = F(37.0) * F(np.power(F(d + 1), F(-0.9), dtype=F))
        v[d] = F(amp * F(rng.next_gaussian()))
    return v


def signed_ramp():
    """tests.rs:52-55: (i - 64) / 16."""
    return ((np.arange(128, dtype=F) - F(64.0)) / F(16.0)).astype(F)


def gaussian_latent(seed):
    rng = ora.Rng(seed)
    return np.array([rng.next_gaussian() for _ in range(128)], F)


def tile_of(v, codec, flags=0):
    """tests.rs:29-46 (tile_from) over quantize_latent_<codec>; returns (tile, scale, group_scales)."""
    latent, scale, gs = ora.quantize(v, codec)
    return ora.make_tile(latent, scale, gs, flags=ora.CODEC_FLAG[codec] | flags), scale, gs


def sq_err(tile, v):
    dq = ora.dequant(tile)
    e = F(0.0)
    for d in range(128):
        e = F(e + F(F(dq[d] - v[d]) ** 2))
    return e


def _fixture_tile(v, codec, bitmap, pos, flags):
    latent, scale, gs = ora.quantize(v, codec)
    return ora.make_tile(latent, scale, gs, flags=flags, lam=0.37, residual=bitmap, pos=pos)


def _scenario_fixture(codec, flags_of):
    z = scenario_projection(9)
    q, toks = scenario_generate(123, 32, 0.4)
    q_sign = scenario_sign_bits(z, q)
    tiles = []
    for i, (kc, e) in enumerate(toks):
        tiles.append(_fixture_tile(kc, codec, tuple(int(x) for x in scenario_sign_bits(z, e)), i, flags_of(i)))
    return q, q_sign, tiles


def tq3_equivalence_fixture():
    """tests.rs:356-384: scenario tokens + steep latents, HOT/WARM x corr/nocorr by index."""
    def flags_of(i):
        return ora.FLAG_TQ3 | (ora.FLAG_WARM if i % 2 == 0 else 0) | (ora.FLAG_TQ3_NOCORR if (i // 2) % 2 == 0 else 0)
    q, q_sign, tiles = _scenario_fixture(TQ3, flags_of)
    for seed in range(8):
        tiles.append(_fixture_tile(steep_latent(300 + seed), TQ3, (ALL_ONES, 0, ALL_ONES, 0), seed, flags_of(seed)))
    return q, q_sign, np.concatenate(tiles)


def nf4_equivalence_fixture():
    """tests.rs:693-715."""
    def flags_of(i):
        return ora.FLAG_NF4 | (ora.FLAG_WARM if i % 2 == 0 else 0)
    q, q_sign, tiles = _scenario_fixture(NF4, flags_of)
    for seed in range(8):
        tiles.append(_fixture_tile(steep_latent(400 + seed), NF4, (ALL_ONES, 0, ALL_ONES, 0), seed, flags_of(seed)))
    return q, q_sign, np.concatenate(tiles)


def _steep_fixture(rng_seed, latent_seed, codec, base_flag, with_nocorr):
    rng = ora.Rng(rng_seed)
    q = rng.gaussian(128)
    q_sign = np.array([rng.next_u64() for _ in range(4)], np.uint64)
    tiles = []
    for seed in range(8):
        v = steep_latent(latent_seed + seed)
        for warm in (False, True):
            for nocorr in ((False, True) if with_nocorr else (False,)):
                bitmap = (ALL_ONES, rng.next_u64(), ALL_ONES, rng.next_u64())
                flags = base_flag | (ora.FLAG_WARM if warm else 0) | (ora.FLAG_TQ3_NOCORR if nocorr else 0)
                tiles.append(_fixture_tile(v, codec, bitmap, 0, flags))
    return q, q_sign, np.concatenate(tiles)


def mix3_equivalence_fixture():
    """tests.rs:501-527."""
    return _steep_fixture(53, 600, MIX3, ora.FLAG_MIX3, True)


def mixed_equivalence_fixture():
    """tests.rs:800-822."""
    return _steep_fixture(33, 500, MIXED, ora.FLAG_MIXED, False)


def int4_equivalence_fixture():
    """tests.rs:912-919: 64 scenario tiles built by scenario::build_tile, alternating HOT / WARM."""
    z = scenario_projection(9)
    q, toks = scenario_generate(123, 64, 0.4)
    q_sign = scenario_sign_bits(z, q)
    tiles = [scenario_tile(z, t, i, warm=(i % 2 == 0)) for i, t in enumerate(toks)]
    return q, q_sign, np.concatenate(tiles)


FIXTURES = {
    "int4": int4_equivalence_fixture,
    "nf4": nf4_equivalence_fixture,
    "mixed": mixed_equivalence_fixture,
    "tq3": tq3_equivalence_fixture,
    "mix3": mix3_equivalence_fixture,
}


# ---- scirust/tests/properties.rs: randomised tiles and queries from the reference's generator -----------------------
def rand_q(rng):
    """properties.rs:21-25"""
    return rng.gaussian(128)


def rand_q_sign(rng):
    """properties.rs:27-33"""
    return np.array([rng.next_u64() for _ in range(4)], np.uint64)


def rand_int4_tile(rng, warm):
    """properties.rs:36-58: random latent bytes, group scales 1..255 (odd), scale in [0.01, 2.01), lambda ~ 0.1 N(0,1)."""
    latent = np.array([rng.next_u64() & 0xFF for _ in range(64)], np.uint8)
    gs = np.array([(rng.next_u64() & 0xFF) | 1 for _ in range(8)], np.uint8)
    bitmap = tuple(int(x) for x in rand_q_sign(rng))
    scale = F(F(rng.next_unit()) * F(2.0) + F(0.01))
    lam = F(F(rng.next_gaussian()) * F(0.1))
    sigma = F(rng.next_unit())
    return ora.make_tile(latent, scale, gs, flags=ora.FLAG_WARM if warm else 0, lam=lam, sigma=sigma, residual=bitmap)


def property_triples(seed, n, warm_of, nf4_of=lambda it: False):
    """n iterations of (tile, q, q_sign) drawn in the order the reference's loops draw them."""
    rng = ora.Rng(seed)
    tiles, qc, qs = [], [], []
    for it in range(n):
        t = rand_int4_tile(rng, warm_of(it))
        if nf4_of(it):
            t["flags"] |= ora.FLAG_NF4
        tiles.append(t)
        qc.append(rand_q(rng))
        qs.append(rand_q_sign(rng))
    return np.concatenate(tiles), np.stack(qc), np.stack(qs)
