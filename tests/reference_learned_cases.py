"""The reference's end-to-end tests of the learned encode path (scirust/src/learned.rs:574-1000, slha-c/src/lib.rs:1034-1191)
as cases over a small model interface, so that they run on the oracle (CPU) and on the GPU library.

The reference fits its projection by PCA (`LearnedModel::fit`: the leading D_C eigenvectors of the uncentered covariance of
the training keys, learned.rs:64-97).  PCA fitting is not part of the encode path; the cases take the same eigenvectors from
numpy (float64 `eigh`) and build the model with `from_projection`, which is what `fit` does after its eigendecomposition
(unit scale, same seed).  Keys come from a restatement of `gen_keys` (learned.rs:455-484) on the reference's PRNG.  The
assertions are the reference's, with its thresholds.

Interface: make(p, d, seed, rht) -> model with encode(keys, codec) -> tiles, prepare(q) -> (q_coarse, q_sign),
score(tiles, q_coarse, q_sign) -> scores, decode_latent(tile), decode_key(tile).
"""
import numpy as np

from oracle import pyoracle as ora

F = np.float32


def gen_keys(seed, n, d, r, decay, noise):
    """learned.rs:455-484: r unit factor directions with strengths decay^i, plus isotropic noise."""
    rng = ora.Rng(seed)
    factors = np.zeros((r, d), F)
    for i in range(r):
        f = rng.gaussian(d)
        nrm = max(F(np.sqrt(np.sum(f * f, dtype=F))), F(1e-9))
        factors[i] = f / nrm
    strengths = np.array([F(decay) ** i for i in range(r)], F)
    keys = np.zeros((n, d), F)
    for j in range(n):
        g = rng.gaussian(r) * strengths
        k = (g[:, None] * factors).sum(0, dtype=F)
        keys[j] = k + F(noise) * rng.gaussian(d)
    return keys


def pca_projection(train, d):
    """Leading 128 eigenvectors (rows) of the uncentered covariance, and the energy they capture (learned.rs:64-97, :430-449)."""
    x = train.astype(np.float64)
    cov = x.T @ x / max(len(x), 1)
    w, v = np.linalg.eigh(cov)
    order = np.argsort(w)[::-1]
    p = np.ascontiguousarray(v[:, order[:128]].T, F)
    return p, float(w[order[:128]].sum() / w.sum())


def ranks(x):
    """metrics.rs: average ranks (ties share the mean rank)."""
    x = np.asarray(x, np.float64)
    order = np.argsort(x, kind="stable")
    r = np.empty(len(x))
    i = 0
    while i < len(x):
        j = i
        while j + 1 < len(x) and x[order[j + 1]] == x[order[i]]:
            j += 1
        r[order[i:j + 1]] = 0.5 * (i + j)
        i = j + 1
    return r


def spearman(a, b):
    ra, rb = ranks(a), ranks(b)
    ra, rb = ra - ra.mean(), rb - rb.mean()
    return float((ra * rb).sum() / np.sqrt((ra * ra).sum() * (rb * rb).sum()))


def _hot_warm_spearman(make, decay, codec=1, rht=False):
    d = 160
    p, captured = pca_projection(gen_keys(1, 600, d, 200, decay, 0.02), d)
    model = make(p, d, 7, rht)
    ev = gen_keys(2, 256, d, 200, decay, 0.02)
    q = gen_keys(3, 1, d, 200, decay, 0.02)[0]
    qc, qs = model.prepare(q)
    hot = model.encode(ev, codec)
    warm = hot.copy()
    warm["flags"] |= ora.FLAG_WARM
    s_true = ev.astype(np.float64) @ q.astype(np.float64)
    return captured, spearman(model.score(hot, qc, qs), s_true), spearman(model.score(warm, qc, qs), s_true)


def pca_captures_dominant_subspace_and_hot_beats_warm(make):
    """learned.rs:610-617"""
    captured, sp_hot, sp_warm = _hot_warm_spearman(make, 0.95)
    assert captured > 0.8 and sp_hot > 0.8 and sp_hot + 0.03 >= sp_warm, (captured, sp_hot, sp_warm)


def grouped_int4_does_not_hurt_end_to_end(make):
    """learned.rs:634-668"""
    single = _hot_warm_spearman(make, 0.93, codec=0)[1]
    grouped = _hot_warm_spearman(make, 0.93, codec=1)[1]
    assert grouped + 0.02 >= single, (grouped, single)


def attention_output_is_high_fidelity_and_hot_ge_warm(make):
    """learned.rs:670-733"""
    d, dv, n = 160, 48, 200
    p, _ = pca_projection(gen_keys(1, 600, d, 200, 0.9, 0.02), d)
    model = make(p, d, 7, False)
    keys = gen_keys(2, n, d, 200, 0.9, 0.02)
    rng = ora.Rng(5)
    values = np.stack([rng.gaussian(dv) for _ in range(n)]).astype(np.float64)
    q = rng.gaussian(d)
    qc, qs = model.prepare(q)
    hot = model.encode(keys, 1)
    warm = hot.copy()
    warm["flags"] |= ora.FLAG_WARM
    scale = 1.0 / np.sqrt(d)

    def agg(s):
        w = np.exp((np.asarray(s, np.float64) - np.max(s)) * scale)
        return (w / w.sum()) @ values

    def cosine(a, b):
        return float(a @ b / np.sqrt((a @ a) * (b @ b)))

    ot = agg(keys.astype(np.float64) @ q.astype(np.float64))
    ch, cw = cosine(ot, agg(model.score(hot, qc, qs))), cosine(ot, agg(model.score(warm, qc, qs)))
    assert ch > 0.9 and ch + 0.02 >= cw, (ch, cw)


def rht_improves_binary_core_on_outlier_blinded_residuals(make):
    """learned.rs:760-826: a strong common direction blinds the plain sign hash; the Hadamard rotation must lift the
    Spearman correlation of 256 - 2 hamming with the true dot products by at least 0.15."""
    d = 128
    rng = ora.Rng(2026)
    p = np.zeros((128, d), F)
    plain, rot = make(p, d, 42, False), make(p, d, 42, True)
    common = np.zeros(d, F)
    common[[0, 1, 40, 41, 80]] = 10.0
    dirs = []
    for _ in range(3):
        v = rng.gaussian(d)
        dirs.append(v / max(F(np.sqrt(np.sum(v * v, dtype=F))), F(1e-9)))

    def mk():
        e = common.copy()
        for v in dirs:
            e = (e + F(F(2.0) * F(rng.next_gaussian())) * v).astype(F)
        return e

    residuals = np.stack([mk() for _ in range(512)])
    eq = mk()
    s_true = residuals.astype(np.float64) @ eq.astype(np.float64)

    def binary_ranking(m):
        qs = m.prepare(eq)[1]
        return [256.0 - 2.0 * ora.hamming(qs, m.prepare(e)[1]) for e in residuals]

    sp_plain, sp_rht = spearman(binary_ranking(plain), s_true), spearman(binary_ranking(rot), s_true)
    assert sp_rht >= sp_plain + 0.15, (sp_plain, sp_rht)


def rht_preserves_warm_coarse_path(make):
    """learned.rs:835-869: the rotation touches only the sign path; WARM scores are the same with and without it"""
    a = _hot_warm_spearman(make, 0.9, rht=False)[2]
    b = _hot_warm_spearman(make, 0.9, rht=True)[2]
    assert abs(a - b) <= 1e-6, (a, b)


def encode_decode_round_trip_and_key_decode(make):
    """slha-c/src/lib.rs:1034-1191: codec flags, finite decodes, MIX3 latent decode above 2 dB, key decode above latent decode"""
    d = 256
    p, _ = pca_projection(gen_keys(1, 512, d, 64, 0.9, 0.02), d)
    key = gen_keys(2, 1, d, 64, 0.9, 0.02)

    def snr(a, b):
        return 10.0 * np.log10(float(np.sum(a.astype(np.float64) ** 2)) / max(float(np.sum((a.astype(np.float64) - b) ** 2)), 1e-12))

    model = make(p, d, 0xC0FFEE, False)
    for codec, flag in enumerate([0, 0, ora.FLAG_NF4, ora.FLAG_MIXED, ora.FLAG_TQ3, ora.FLAG_MIX3]):
        tile = model.encode(key, codec)
        assert int(tile["flags"][0]) & (ora.FLAG_NF4 | ora.FLAG_MIXED | ora.FLAG_TQ3 | ora.FLAG_MIX3) == flag
        out = model.decode_latent(tile)
        assert np.isfinite(out).all()
        if codec == 5:
            assert snr(key[0], out) > 2.0
    model = make(p, d, 0xB0BA, False)
    tile = model.encode(key, 3)
    assert snr(key[0], model.decode_key(tile)) > snr(key[0], model.decode_latent(tile))


def scenario_scores_match_equation_2_3_and_warm_drops_the_binary_term(make):
    """scirust/tests/slha.rs:48-91"""
    from .helpers import scenario_generate, scenario_projection, scenario_sign_bits, scenario_tile
    model = make(np.zeros((128, 128), F), 128, 3, False)  # (only its scorer is used)
    z = scenario_projection(3)
    q, toks = scenario_generate(4, 1, 0.4)
    tile = scenario_tile(z, toks[0], 0)
    q_sign = scenario_sign_bits(z, q)
    k = ora.dequant(tile)
    coarse = F(0.0)
    for d in range(128):
        coarse = F(coarse + F(q[d] * k[d]))
    manual = coarse + tile["dynamic_lambda"][0] * F(256.0 - 2.0 * ora.hamming(q_sign, tile["residual_bitmap"][0]))
    assert abs(model.score(tile, q, q_sign)[0] - manual) < 1e-4
    z = scenario_projection(2)
    q, toks = scenario_generate(2, 1, 0.5)
    q_sign = scenario_sign_bits(z, q)
    hot = scenario_tile(z, toks[0], 0)
    warm, hot0 = hot.copy(), hot.copy()
    warm["flags"] |= ora.FLAG_WARM
    hot0["dynamic_lambda"] = 0.0
    s_hot, s_warm, s_hot0 = (model.score(t, q, q_sign)[0] for t in (hot, warm, hot0))
    assert abs(s_warm - s_hot0) < 1e-5 and abs(s_hot - s_warm) > 0.0


def sign_lsh_residual_tracks_cosine(make):
    """scirust/tests/slha.rs:93-133; a model of d = 128 with seed s draws the same sign matrix as Projection::new(s)"""
    model = make(np.zeros((128, 128), F), 128, 11, False)
    rng = ora.Rng(99)
    q = rng.gaussian(128)
    q = (q / F(np.sqrt(np.sum(q * q, dtype=F)))).astype(F)
    q_sign = model.prepare(q)[1]
    est, cos = [], []
    for _ in range(400):
        e = rng.gaussian(128)
        align = F(F(F(rng.next_unit()) * F(2.0) - F(1.0)) * F(np.sqrt(F(128.0))))
        e = (e + align * q).astype(F)
        est.append(256.0 - 2.0 * ora.hamming(q_sign, model.prepare(e)[1]))
        cos.append(float(q.astype(np.float64) @ e.astype(np.float64) / np.sqrt(e.astype(np.float64) @ e.astype(np.float64))))
    assert spearman(est, cos) > 0.85


def hot_ranks_at_least_as_well_as_warm(make):
    """scirust/tests/slha.rs:135-161"""
    from .helpers import scenario_generate, scenario_projection, scenario_sign_bits, scenario_tile
    model = make(np.zeros((128, 128), F), 128, 5, False)
    z = scenario_projection(5)
    q, toks = scenario_generate(123, 256, 0.4)
    q_sign = scenario_sign_bits(z, q)
    hot = np.concatenate([scenario_tile(z, t, i) for i, t in enumerate(toks)])
    warm = hot.copy()
    warm["flags"] |= ora.FLAG_WARM
    s_true = [float((kc + e).astype(np.float64) @ q.astype(np.float64)) for kc, e in toks]
    sp_hot, sp_warm = spearman(model.score(hot, q, q_sign), s_true), spearman(model.score(warm, q, q_sign), s_true)
    assert sp_hot > 0.8 and sp_hot + 0.02 >= sp_warm, (sp_hot, sp_warm)


CASES = [
    scenario_scores_match_equation_2_3_and_warm_drops_the_binary_term,
    sign_lsh_residual_tracks_cosine,
    hot_ranks_at_least_as_well_as_warm,
    pca_captures_dominant_subspace_and_hot_beats_warm,
    grouped_int4_does_not_hurt_end_to_end,
    attention_output_is_high_fidelity_and_hot_ge_warm,
    rht_improves_binary_core_on_outlier_blinded_residuals,
    rht_preserves_warm_coarse_path,
    encode_decode_round_trip_and_key_decode,
]
