"""ctypes binding of the CPU oracle (libslha_oracle.so) -- TEST INFRASTRUCTURE ONLY.

May be imported by tests/, by the smoke check and by the benchmark's CPU-baseline
leg.  The shipped package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libslha_oracle.so")

TILE_DTYPE = np.dtype(
    [
        ("latent_kv", np.uint8, 64),
        ("residual_bitmap", np.uint64, 4),
        ("scale", np.float32),
        ("dynamic_lambda", np.float32),
        ("residual_sigma", np.float32),
        ("token_id", np.uint32),
        ("position", np.uint32),
        ("head_id", np.uint16),
        ("flags", np.uint16),
        ("group_scales", np.uint8, 8),
    ]
)
assert TILE_DTYPE.itemsize == 128

FLAG_WARM, FLAG_NF4, FLAG_MIXED, FLAG_TQ3, FLAG_TQ3_NOCORR, FLAG_MIX3 = 1, 2, 4, 8, 16, 32
HOT, WARM, COLD = 0, 1, 2


def build():
    """Compile the oracle with its Makefile (gcc, -ffp-contract=off)."""
    subprocess.check_call(["make", "-s", "-C", _HERE], stdout=subprocess.DEVNULL)


def _load():
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    vp, sz, f32p = C.c_void_p, C.c_size_t, C.c_void_p
    sig = {
        "ora_rng_init": (None, [vp, C.c_uint64]),
        "ora_rng_next_u64": (C.c_uint64, [vp]),
        "ora_rng_next_unit": (C.c_float, [vp]),
        "ora_rng_next_gaussian": (C.c_float, [vp]),
        "ora_rng_fill_gaussian": (None, [vp, f32p, sz]),
        "ora_quantize_latent": (None, [vp, vp, vp]),
        "ora_quantize_latent_grouped": (None, [vp, vp, vp, vp]),
        "ora_quantize_latent_grouped32": (None, [vp, vp, vp, vp]),
        "ora_quantize_latent_nf4": (None, [vp, vp, vp, vp]),
        "ora_quantize_latent_mixed": (None, [vp, vp, vp, vp]),
        "ora_quantize_latent_tq3": (None, [vp, vp, vp, vp]),
        "ora_quantize_latent_mix3": (None, [vp, vp, vp, vp]),
        "ora_nf4_nearest": (C.c_uint8, [C.c_float]),
        "ora_dequant_latent": (None, [vp, vp]),
        "ora_hamming": (C.c_uint32, [vp, vp]),
        "ora_compute_score_scalar": (C.c_float, [vp, vp, vp]),
        "ora_score_tiles": (None, [vp, sz, vp, vp, vp]),
        "ora_validate_tile": (C.c_int, [vp]),
        "ora_next_pow2": (sz, [sz]),
        "ora_fwht_inplace": (None, [vp, sz]),
        "ora_model_from_projection": (vp, [vp, sz, C.c_uint64, C.c_int]),
        "ora_model_set_scale": (None, [vp, vp]),
        "ora_model_set_z": (None, [vp, vp]),
        "ora_model_free": (None, [vp]),
        "ora_model_d": (sz, [vp]),
        "ora_model_d_pad": (sz, [vp]),
        "ora_model_z": (vp, [vp]),
        "ora_model_rht_diag": (vp, [vp]),
        "ora_model_latent": (None, [vp, vp, vp]),
        "ora_model_query_coarse": (None, [vp, vp, vp]),
        "ora_model_reconstruct": (None, [vp, vp, vp]),
        "ora_model_sign_bits": (None, [vp, vp, vp]),
        "ora_model_encode": (C.c_int, [vp, vp, C.c_uint32, C.c_int, C.c_int, vp]),
        "ora_model_encode_batch": (None, [vp, vp, sz, vp, vp, C.c_int, vp]),
        "ora_model_prepare_query": (None, [vp, vp, vp, vp]),
        "ora_model_decode_latent": (None, [vp, vp, vp]),
        "ora_model_decode_key": (None, [vp, vp, vp]),
        "ora_weights_checksum": (C.c_uint32, [vp, vp, sz]),
        "ora_weights_from_bytes": (vp, [vp, sz, vp, sz]),
        "ora_analytic_lambda_c": (C.c_float, []),
        "ora_rms": (C.c_double, [vp, sz]),
        "ora_scenario_sign_bits": (None, [vp, vp, vp]),
        "ora_scenario_build_tile": (None, [vp, vp, vp, C.c_uint32, C.c_int, vp]),
        "ora_topk": (None, [vp, sz, sz, vp, vp]),
        "ora_cache_new": (vp, [sz, C.c_int, C.c_int, C.c_uint32, C.c_uint32]),
        "ora_cache_free": (None, [vp]),
        "ora_cache_insert": (sz, [vp, vp]),
        "ora_cache_len": (sz, [vp]),
        "ora_cache_state": (C.c_int, [vp, sz]),
        "ora_cache_tile": (vp, [vp, sz]),
        "ora_cache_importance": (C.c_float, [vp, sz]),
        "ora_cache_seq": (C.c_uint64, [vp, sz]),
        "ora_cache_live_bytes": (sz, [vp]),
        "ora_cache_counts": (None, [vp, vp, vp, vp]),
        "ora_cache_page_out": (None, [vp, sz]),
        "ora_cache_drop_correction": (C.c_int, [vp, sz]),
        "ora_cache_evict": (C.c_int, [vp, sz]),
        "ora_cache_enforce_budget": (C.c_int, [vp]),
        "ora_cache_score_all": (sz, [vp, vp, vp, vp, vp]),
        "ora_cache_observe_scores": (None, [vp, vp, vp, sz, C.c_float]),
        "ora_cache_journal_len": (sz, [vp]),
        "ora_cache_journal_get": (None, [vp, sz, vp, vp, vp]),
        "ora_cache_nocorr_count": (sz, [vp]),
        "ora_cache_reclaimed_correction_bytes": (sz, [vp]),
        "ora_simd_level": (C.c_int, []),
        "ora_score_sink": (C.c_double, [vp, sz, vp, vp, C.c_int, C.c_int]),
        "ora_compute_score_simd": (C.c_float, [vp, vp, vp, C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Rng:
    """scirust/src/rng.rs"""

    def __init__(self, seed):
        self._s = (C.c_uint64 * 1)()
        lib.ora_rng_init(self._s, seed)

    def next_u64(self):
        return lib.ora_rng_next_u64(self._s)

    def next_unit(self):
        return lib.ora_rng_next_unit(self._s)

    def next_gaussian(self):
        return lib.ora_rng_next_gaussian(self._s)

    def gaussian(self, n):
        out = np.empty(n, np.float32)
        lib.ora_rng_fill_gaussian(self._s, _p(out), n)
        return out


_QUANT = {
    0: "ora_quantize_latent",
    1: "ora_quantize_latent_grouped",
    2: "ora_quantize_latent_nf4",
    3: "ora_quantize_latent_mixed",
    4: "ora_quantize_latent_tq3",
    5: "ora_quantize_latent_mix3",
    6: "ora_quantize_latent_grouped32",
}
CODEC_FLAG = {0: 0, 1: 0, 2: FLAG_NF4, 3: FLAG_MIXED, 4: FLAG_TQ3, 5: FLAG_MIX3, 6: 0}


def quantize(v, codec):
    """Returns (latent[64] u8, scale f32, group_scales[8] u8)."""
    v = _f32(v)
    out = np.zeros(64, np.uint8)
    scale = np.zeros(1, np.float32)
    gs = np.full(8, 255, np.uint8)
    if codec == 0:
        lib.ora_quantize_latent(_p(v), _p(out), _p(scale))
    else:
        getattr(lib, _QUANT[codec])(_p(v), _p(out), _p(scale), _p(gs))
    return out, float(scale[0]), gs


def make_tile(latent, scale, gs, flags=0, lam=0.0, sigma=0.0, residual=(0, 0, 0, 0), pos=0):
    t = np.zeros(1, TILE_DTYPE)
    t["latent_kv"][0] = latent
    t["residual_bitmap"][0] = np.array(residual, np.uint64)
    t["scale"], t["dynamic_lambda"], t["residual_sigma"] = scale, lam, sigma
    t["token_id"] = t["position"] = pos
    t["flags"] = flags
    t["group_scales"][0] = gs
    return t


def dequant(tile):
    out = np.empty(128, np.float32)
    lib.ora_dequant_latent(_p(tile), _p(out))
    return out


def hamming(a, b):
    a = np.ascontiguousarray(a, np.uint64)
    b = np.ascontiguousarray(b, np.uint64)
    return lib.ora_hamming(_p(a), _p(b))


def score_tiles(tiles, q_coarse, q_sign):
    tiles = np.ascontiguousarray(tiles)
    qc, qs = _f32(q_coarse), np.ascontiguousarray(q_sign, np.uint64)
    out = np.empty(len(tiles), np.float32)
    lib.ora_score_tiles(_p(tiles), len(tiles), _p(qc), _p(qs), _p(out))
    return out


def score_simd(tile, q_coarse, q_sign, which):
    qc, qs = _f32(q_coarse), np.ascontiguousarray(q_sign, np.uint64)
    return lib.ora_compute_score_simd(_p(tile), _p(qc), _p(qs), which)


def validate_tile(tile):
    return lib.ora_validate_tile(_p(tile))


def topk(scores, k):
    s = _f32(scores)
    k = min(k, len(s))
    idx = np.empty(k, np.uint32)
    val = np.empty(k, np.float32)
    lib.ora_topk(_p(s), len(s), k, _p(idx), _p(val))
    return idx, val


def fwht(v):
    v = _f32(v).copy()
    lib.ora_fwht_inplace(_p(v), len(v))
    return v


class Model:
    """scirust/src/learned.rs LearnedModel built by try_from_projection_with."""

    def __init__(self, p=None, d=None, seed=0, rht=False, scale=None, z=None, handle=None):
        if handle is not None:
            self.h = handle
        else:
            p = _f32(p).reshape(-1)
            assert p.size == 128 * d
            self.h = lib.ora_model_from_projection(_p(p), d, seed, int(rht))
        self.d = lib.ora_model_d(self.h)
        self.d_pad = lib.ora_model_d_pad(self.h)
        if scale is not None:
            lib.ora_model_set_scale(self.h, _p(_f32(scale)))
        if z is not None:
            lib.ora_model_set_z(self.h, _p(_f32(z).reshape(-1)))

    def __del__(self):
        if getattr(self, "h", None):
            lib.ora_model_free(self.h)
            self.h = None

    @property
    def z(self):
        ptr = C.cast(lib.ora_model_z(self.h), C.POINTER(C.c_float))
        return np.ctypeslib.as_array(ptr, shape=(256, self.d_pad)).copy()

    @property
    def rht_diag(self):
        raw = lib.ora_model_rht_diag(self.h)
        if not raw:
            return None
        ptr = C.cast(raw, C.POINTER(C.c_float))
        return np.ctypeslib.as_array(ptr, shape=(self.d_pad,)).copy()

    def latent(self, key):
        out = np.empty(128, np.float32)
        lib.ora_model_latent(self.h, _p(_f32(key)), _p(out))
        return out

    def reconstruct(self, h):
        out = np.empty(self.d, np.float32)
        lib.ora_model_reconstruct(self.h, _p(_f32(h)), _p(out))
        return out

    def sign_bits(self, v):
        out = np.empty(4, np.uint64)
        lib.ora_model_sign_bits(self.h, _p(_f32(v)), _p(out))
        return out

    def encode(self, key, pos=0, warm=False, codec=1):
        t = np.zeros(1, TILE_DTYPE)
        rc = lib.ora_model_encode(self.h, _p(_f32(key)), pos, int(warm), codec, _p(t))
        assert rc == 0
        return t

    def encode_batch(self, keys, codec, pos=None, head=None):
        keys = _f32(keys).reshape(-1, self.d)
        n = len(keys)
        out = np.zeros(n, TILE_DTYPE)
        pp = None if pos is None else np.ascontiguousarray(pos, np.uint32)
        hh = None if head is None else np.ascontiguousarray(head, np.uint16)
        lib.ora_model_encode_batch(
            self.h, _p(keys), n, None if pp is None else _p(pp), None if hh is None else _p(hh), codec, _p(out)
        )
        return out

    def prepare_query(self, q):
        qc = np.empty(128, np.float32)
        qs = np.empty(4, np.uint64)
        lib.ora_model_prepare_query(self.h, _p(_f32(q)), _p(qc), _p(qs))
        return qc, qs

    def decode_latent(self, tile):
        out = np.empty(self.d, np.float32)
        lib.ora_model_decode_latent(self.h, _p(tile), _p(out))
        return out

    def decode_key(self, tile):
        out = np.empty(self.d, np.float32)
        lib.ora_model_decode_key(self.h, _p(tile), _p(out))
        return out


def weights_from_bytes(data):
    buf = np.frombuffer(bytes(data), np.uint8).copy()
    err = C.create_string_buffer(512)
    h = lib.ora_weights_from_bytes(_p(buf), len(buf), err, 512)
    if not h:
        raise ValueError(err.value.decode())
    return Model(handle=h)


def weights_to_bytes(p, d, seed, rht, version=2):
    """scirust/src/weights.rs:86-150 (writer), used to make parser fixtures."""
    import struct

    hdr = struct.pack("<IIIQB3x", 0x534C4857, version, d, seed, int(rht))
    payload = _f32(p).reshape(-1).tobytes()
    if version == 1:
        return hdr + payload
    h, pl = np.frombuffer(hdr, np.uint8).copy(), np.frombuffer(payload, np.uint8).copy()
    ck = lib.ora_weights_checksum(_p(h), _p(pl), len(pl))
    return hdr + struct.pack("<I", ck) + payload


class Cache:
    """scirust/src/ccos.rs ElasticKvCache (recent_window is an extension)."""

    def __init__(self, budget, page_policy=0, evict_policy=0, sink_window=0, recent_window=0):
        self.h = lib.ora_cache_new(budget, page_policy, evict_policy, sink_window, recent_window)

    def __del__(self):
        if getattr(self, "h", None):
            lib.ora_cache_free(self.h)
            self.h = None

    def insert(self, tile):
        return lib.ora_cache_insert(self.h, _p(np.ascontiguousarray(tile)))

    def __len__(self):
        return lib.ora_cache_len(self.h)

    def state(self, s):
        return lib.ora_cache_state(self.h, s)

    def states(self):
        return np.array([self.state(s) for s in range(len(self))], np.uint8)

    def tile(self, s):
        ptr = lib.ora_cache_tile(self.h, s)
        return np.frombuffer(C.string_at(ptr, 128), TILE_DTYPE).copy()

    def tiles(self):
        n = len(self)
        if n == 0:
            return np.zeros(0, TILE_DTYPE)
        return np.concatenate([self.tile(s) for s in range(n)])

    def importance(self, s):
        return lib.ora_cache_importance(self.h, s)

    def seq(self, s):
        return lib.ora_cache_seq(self.h, s)

    def live_bytes(self):
        return lib.ora_cache_live_bytes(self.h)

    def counts(self):
        a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
        lib.ora_cache_counts(self.h, C.byref(a), C.byref(b), C.byref(c))
        return a.value, b.value, c.value

    def page_out(self, s):
        lib.ora_cache_page_out(self.h, s)

    def drop_correction(self, s):
        return bool(lib.ora_cache_drop_correction(self.h, s))

    def evict(self, s):
        return bool(lib.ora_cache_evict(self.h, s))

    def enforce_budget(self):
        return bool(lib.ora_cache_enforce_budget(self.h))

    def score_all(self, q_coarse, q_sign):
        n = len(self)
        slots = np.empty(max(n, 1), np.uint32)
        sc = np.empty(max(n, 1), np.float32)
        qc, qs = _f32(q_coarse), np.ascontiguousarray(q_sign, np.uint64)
        m = lib.ora_cache_score_all(self.h, _p(qc), _p(qs), _p(slots), _p(sc))
        return slots[:m].copy(), sc[:m].copy()

    def observe_scores(self, slots, scores, temperature):
        s = np.ascontiguousarray(slots, np.uint32)
        v = _f32(scores)
        lib.ora_cache_observe_scores(self.h, _p(s), _p(v), len(s), temperature)

    def journal(self):
        """(seq, slot, tile) of every eviction so far, in order: the records an attached EventLog
        receives (scirust/src/ccos.rs:411-420)."""
        out = []
        for i in range(lib.ora_cache_journal_len(self.h)):
            seq, slot, tile = C.c_uint64(), C.c_uint32(), np.zeros(1, TILE_DTYPE)
            lib.ora_cache_journal_get(self.h, i, C.byref(seq), C.byref(slot), _p(tile))
            out.append((seq.value, slot.value, tile))
        return out

    def nocorr_count(self):
        return lib.ora_cache_nocorr_count(self.h)

    def reclaimed_correction_bytes(self):
        return lib.ora_cache_reclaimed_correction_bytes(self.h)


def score_sink(tiles, q_coarse, q_sign, which=-1, threads=1):
    tiles = np.ascontiguousarray(tiles)
    qc, qs = _f32(q_coarse), np.ascontiguousarray(q_sign, np.uint64)
    return lib.ora_score_sink(_p(tiles), len(tiles), _p(qc), _p(qs), which, threads)


def simd_level():
    return lib.ora_simd_level()


# ---- the reference's own CUDA scoring kernel (optional second checker) --------
# oracle/_ref/libslha_ref_cuda.so is built by `make -C oracle ref` from
# slhav2-vram/kernels/slha_score.cu where the reference tree is mounted; it is a
# built artefact only (never in history) and may be absent.
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libslha_ref_cuda.so")
_ref_cuda = None


def build_ref_cuda(reference_root=None):
    """Compiles the reference CUDA kernel if its source tree is present (reference_root, else the environment
    variable SLHA_REFERENCE_ROOT, else a directory `reference` beside this repository); returns True when the
    library exists."""
    if reference_root is None:
        reference_root = os.environ.get("SLHA_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.exists(os.path.join(reference_root, "slhav2-vram", "kernels", "slha_score.cu")):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REF=" + reference_root], stdout=subprocess.DEVNULL)
    return os.path.exists(_REF_CUDA_SO)


def ref_cuda_library():
    """ctypes handle of the built reference CUDA kernel driver, or None when it was never built."""
    global _ref_cuda
    if _ref_cuda is None and os.path.exists(_REF_CUDA_SO):
        _ref_cuda = C.CDLL(_REF_CUDA_SO)
        _ref_cuda.slha_ref_cuda_score.restype = C.c_int
        _ref_cuda.slha_ref_cuda_score.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        _ref_cuda.slha_ref_cuda_time.restype = C.c_int
        _ref_cuda.slha_ref_cuda_time.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                                 C.c_void_p, C.c_void_p]
    return _ref_cuda


def ref_cuda_scores(tiles, q_coarse, q_sign):
    """scores[nq][n] from the reference's CUDA kernel (needs a GPU and the built library)."""
    r = ref_cuda_library()
    if r is None:
        raise RuntimeError("oracle/_ref/libslha_ref_cuda.so has not been built")
    tiles = np.ascontiguousarray(tiles)
    qc = np.ascontiguousarray(q_coarse, np.float32).reshape(-1, 128)
    qs = np.ascontiguousarray(q_sign, np.uint64).reshape(-1, 4)
    out = np.empty((len(qc), len(tiles)), np.float32)
    rc = r.slha_ref_cuda_score(_p(tiles), len(tiles), _p(qc), _p(qs), len(qc), _p(out))
    if rc:
        raise RuntimeError("reference CUDA kernel failed: cudaError %d" % (rc - 1000))
    return out


def softmax_into(scores, scale):
    """metrics::softmax_into (scirust/src/metrics.rs:338-420): f64 logits score * scale, maximum
    subtracted, f32 weights normalised and then renormalised by their rounded sum; NaN, a
    non-finite scale or an empty / all -inf input give zeros, +inf logits share the mass."""
    s = np.asarray(scores, np.float32)
    out = np.zeros(len(s), np.float32)
    if len(s) == 0 or not np.isfinite(scale) or np.any(np.isnan(s)):
        return out
    logit = s.astype(np.float64) * np.float64(np.float32(scale))
    if np.any(np.isnan(logit)):
        return out
    pinf = np.isposinf(logit)
    if pinf.any():
        out[pinf] = np.float32(1.0 / pinf.sum())
        return out
    mx = logit.max()
    if np.isneginf(mx):
        return out
    e = np.exp(logit - mx)
    out = e.astype(np.float32)
    total = e.sum()
    if not np.isfinite(total) or total <= 0:
        return np.zeros(len(s), np.float32)
    out = (out.astype(np.float64) / total).astype(np.float32)
    rounded = out.astype(np.float64).sum()
    if np.isfinite(rounded) and rounded > 0:
        out = (out.astype(np.float64) / rounded).astype(np.float32)
    return out


def attend_topk(top_index, top_score, scale, values, top_count=None, row_base=None):
    """The reference's decode tail (scirust/examples/benchmark_decode.rs:82-95) over every row's selected
    tiles: softmax_into over the row's valid (index, score) pairs, then aggregate_v (:28-38,
    out[j] += w * row[j] in list order, float32).  values: [rows][d_v] float32."""
    ti = np.asarray(top_index, np.uint32)
    ts = np.asarray(top_score, np.float32)
    nq, k = ti.shape
    v = np.asarray(values, np.float32)
    out = np.zeros((nq, v.shape[1]), np.float32)
    weights = np.zeros((nq, k), np.float32)
    for q in range(nq):
        n = k if top_count is None else min(int(top_count[q]), k)
        valid = np.nonzero(ti[q, :n] != 0xFFFFFFFF)[0]
        w = softmax_into(ts[q, valid], scale)
        weights[q, valid] = w
        base = 0 if row_base is None else int(row_base[q])
        acc = np.zeros(v.shape[1], np.float32)
        for i, wi in zip(valid, w):
            acc = (acc + np.float32(wi) * v[(base + int(ti[q, i])) % (1 << 64)]).astype(np.float32)
        out[q] = acc
    return out, weights


# ---- EventLog (scirust/src/eventlog.rs:9-24): 16-byte header + 144-byte records, little-endian -----------------
EVENTLOG_MAGIC, EVENTLOG_VERSION = 0x534C4C47, 2


def eventlog_checksum(seq, slot, tile_bytes):
    """record_checksum (eventlog.rs:146-169): FNV-1a over seq (8 LE bytes), slot (4 LE bytes), the 128 tile bytes."""
    h = 0x811C9DC5
    for b in int(seq).to_bytes(8, "little") + int(slot).to_bytes(4, "little") + bytes(tile_bytes):
        h = ((h ^ b) * 0x01000193) & 0xFFFFFFFF
    return h


def eventlog_bytes(records, version=EVENTLOG_VERSION):
    """The byte-exact file an EventLog holds after `records` ((seq, slot, tile) in order) were appended."""
    out = bytearray()
    out += EVENTLOG_MAGIC.to_bytes(4, "little") + int(version).to_bytes(4, "little") + (128).to_bytes(4, "little") + (0).to_bytes(4, "little")
    for seq, slot, tile in records:
        tb = np.ascontiguousarray(tile).tobytes()
        assert len(tb) == 128
        chk = eventlog_checksum(seq, slot, tb) if version >= 2 else 0
        out += int(seq).to_bytes(8, "little") + int(slot).to_bytes(4, "little") + chk.to_bytes(4, "little") + tb
    return bytes(out)


def eventlog_parse(data):
    """Strict reader (EventLog::open, eventlog.rs:236-300): header, whole records, version-2 checksums."""
    if len(data) < 16:
        raise ValueError("EventLog: file shorter than header")
    magic, version, tile_size = (int.from_bytes(data[o:o + 4], "little") for o in (0, 4, 8))
    if magic != EVENTLOG_MAGIC:
        raise ValueError("EventLog: bad magic")
    if version not in (1, 2):
        raise ValueError("EventLog: unsupported version")
    if tile_size != 128:
        raise ValueError("EventLog: tile-size mismatch")
    if (len(data) - 16) % 144:
        raise ValueError("EventLog: truncated record")
    recs = []
    for o in range(16, len(data), 144):
        seq = int.from_bytes(data[o:o + 8], "little")
        slot = int.from_bytes(data[o + 8:o + 12], "little")
        chk = int.from_bytes(data[o + 12:o + 16], "little")
        tb = data[o + 16:o + 144]
        if version >= 2 and chk != eventlog_checksum(seq, slot, tb):
            raise ValueError("EventLog: checksum mismatch")
        recs.append((seq, slot, np.frombuffer(tb, TILE_DTYPE).copy()))
    return version, recs
