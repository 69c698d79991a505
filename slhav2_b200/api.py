"""Host-side mirror of the reference's operator surface for the tile hot path,
bound to libslha_b200.so through its C ABI (include/slha_b200.h) with ctypes.

Names follow the reference: `Model` stands for scirust's LearnedModel
(learned.rs), `TilePool` for ccos::ElasticKvCache (ccos.rs), the free functions
for the slha-c entry points (slha-c/src/lib.rs).  Arguments may be numpy arrays
(host memory) or objects with `data_ptr()` such as CUDA torch tensors (device
memory); nothing here computes on the CPU -- without the CUDA library every call
raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libslha_b200.so")

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
SEGMENT_DTYPE = np.dtype(
    [("tile_begin", np.uint64), ("n_tiles", np.uint32), ("query_begin", np.uint32), ("n_queries", np.uint32), ("index_base", np.uint32)]
)
assert TILE_DTYPE.itemsize == 128 and SEGMENT_DTYPE.itemsize == 24

OK = 0
ERR_NULL, ERR_PANIC, ERR_DIMENSION, ERR_CODEC, ERR_NONFINITE = -1, -2, -3, -4, -5
ERR_INVALID_TILE, ERR_INVALID_HANDLE, ERR_IO, ERR_UTF8 = -6, -7, -8, -9
ERR_DEVICE, ERR_CAPACITY = -100, -101
CODEC_INT4_SINGLE, CODEC_INT4_GROUPED, CODEC_NF4, CODEC_MIXED, CODEC_TQ3, CODEC_MIX3, CODEC_INT4_GROUPED32 = range(7)
FLAG_WARM, FLAG_NF4, FLAG_MIXED, FLAG_TQ3, FLAG_TQ3_NOCORR, FLAG_MIX3 = 1, 2, 4, 8, 16, 32
F32, BF16 = 0, 1
HOT, WARM, COLD = 0, 1, 2
PAGE_LOWEST_IMPACT_FIRST, PAGE_OLDEST_FIRST = 0, 1
EVICT_CAUSAL, EVICT_IMPORTANCE = 0, 1

# every symbol include/slha_b200.h declares: (restype, argtypes)
_vp, _sz, _i32, _u32, _u64 = C.c_void_p, C.c_size_t, C.c_int32, C.c_uint32, C.c_uint64
SIGNATURES = {
    "slha_abi_version": (_u32, []),
    "slha_tile_size": (_sz, []),
    "slha_tile_align": (_sz, []),
    "slha_last_error_message": (C.c_char_p, []),
    "slha_clear_error": (None, []),
    "slha_init": (_vp, []),
    "slha_shutdown": (_i32, [_vp]),
    "slha_process_tile": (_i32, [_vp, _vp, _vp, _vp]),
    "slha_prepare_query": (_i32, [_vp, _vp, _sz, _vp, _vp]),
    "slha_score_tile": (_i32, [_vp, _vp, _vp, _vp, _vp]),
    "slha_score_tiles": (_i32, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "slha_audit": (_vp, []),
    "slha_free_string": (None, [_vp]),
    "slha_weights_load": (_vp, [C.c_char_p]),
    "slha_model_dim": (_sz, [_vp]),
    "slha_encode_key": (_i32, [_vp, _vp, _sz, _u32, _i32, _vp]),
    "slha_decode_latent": (_i32, [_vp, _vp, _vp, _sz]),
    "slha_decode_key": (_i32, [_vp, _vp, _vp, _sz]),
    "slha_weights_release": (_i32, [_vp]),
    "slha_weights_free": (None, [_vp]),
    "slha_b200_device_count": (_i32, []),
    "slha_b200_set_device": (_i32, [_i32]),
    "slha_b200_set_stream": (_i32, [_vp]),
    "slha_b200_launch_count": (_u64, []),
    "slha_b200_debug_force_generic_score": (_i32, [_i32]),
    "slha_b200_last_score_stats": (_i32, [_vp]),
    "slha_b200_timing_begin": (_i32, [_u32]),
    "slha_b200_timing_end": (_i32, [_vp, _vp, _u32, _vp]),
    "slha_b200_malloc": (_i32, [_sz, C.POINTER(_vp)]),
    "slha_b200_free": (_i32, [_vp]),
    "slha_b200_memcpy": (_i32, [_vp, _vp, _sz]),
    "slha_b200_synchronize": (_i32, []),
    "slha_b200_model_create": (_vp, [_vp, _sz, _u64, _i32, _vp, _vp]),
    "slha_b200_encode_keys": (_i32, [_vp, _vp, _i32, _sz, _vp, _u32, _vp, _i32, _vp]),
    "slha_b200_prepare_queries": (_i32, [_vp, _vp, _sz, _vp, _vp]),
    "slha_b200_score_tiles": (_i32, [_vp, _sz, _vp, _vp, _sz, _vp]),
    "slha_b200_score_segments": (_i32, [_vp, _vp, _sz, _vp, _vp, _sz, _vp, _sz, _vp, _u32, C.c_float]),
    "slha_b200_score_topk": (_i32, [_vp, _vp, _sz, _vp, _vp, _sz, _u32, _vp, _vp, _vp]),
    "slha_b200_score_topk_noalloc": (_i32, [_vp, _vp, _sz, _vp, _vp, _sz, _u32, _vp, _vp, _vp]),
    "slha_b200_topk_merge": (_i32, [_vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp]),
    "slha_b200_topk_merge_strided": (_i32, [_vp, _vp, _u32, _u64, _u32, _u32, _u32, _vp, _vp]),
    "slha_b200_topk_merge_sorted_strided": (_i32, [_vp, _vp, _u32, _u64, _u32, _u32, _u32, _vp, _vp]),
    "slha_b200_attend_topk": (_i32, [_vp, _vp, _vp, _sz, _u32, C.c_float, _vp, _i32, _sz, _sz, _vp, _vp, _vp]),
    "slha_b200_shard_unique_id": (_i32, [_vp]),
    "slha_b200_shard_init": (_i32, [_vp, _i32, _i32, C.POINTER(_vp)]),
    "slha_b200_shard_destroy": (_i32, [_vp]),
    "slha_b200_shard_score_topk": (_i32, [_vp, _vp, _vp, _sz, _vp, _vp, _sz, _u32, _vp, _vp]),
    "slha_b200_shard_set_timing": (_i32, [_vp, _i32]),
    "slha_b200_shard_last_times": (_i32, [_vp, _vp]),
    "slha_b200_shard_status": (_i32, [_vp, _vp]),
    "slha_b200_shard_set_exchange": (_i32, [_vp, _i32]),
    "slha_b200_pool_create": (_i32, [_vp, C.POINTER(_vp)]),
    "slha_b200_pool_destroy": (_i32, [_vp]),
    "slha_b200_pool_insert_tiles": (_i32, [_vp, _vp, _sz, _vp]),
    "slha_b200_pool_append_keys": (_i32, [_vp, _vp, _vp, _i32, _sz, _vp, _u32, _vp, _i32, _vp]),
    "slha_b200_pool_score_all": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "slha_b200_pool_score_topk": (_i32, [_vp, _vp, _vp, _sz, _u32, _vp, _vp, _vp]),
    "slha_b200_pool_observe_scores": (_i32, [_vp, _vp, _vp, _sz, C.c_float]),
    "slha_b200_pool_observe_query": (_i32, [_vp, _vp, _vp, C.c_float]),
    "slha_b200_pool_page_out": (_i32, [_vp, _u32]),
    "slha_b200_pool_drop_correction": (_i32, [_vp, _u32, _vp]),
    "slha_b200_pool_evict": (_i32, [_vp, _u32, _vp]),
    "slha_b200_pool_attach_event_log": (_i32, [_vp, C.c_char_p, _i32, _i32]),
    "slha_b200_pool_rehydrate": (_i32, [_vp, _u64, _vp]),
    "slha_b200_pool_event_log_stats": (_i32, [_vp, _vp]),
    "slha_b200_pool_enforce_budget": (_i32, [_vp, _vp]),
    "slha_b200_pool_set_budget": (_i32, [_vp, _u64]),
    "slha_b200_pool_stats": (_i32, [_vp, _vp]),
    "slha_b200_pool_read": (_i32, [_vp, _u64, _u64, _vp, _vp, _vp, _vp]),
    "slha_b200_pool_tiles_device": (_vp, [_vp]),
}


class SlhaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("SLHA status %d: %s" % (code, message))
        self.code = code
        self.message = message


_lib = None


def load_library():
    """Loads libslha_b200.so.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m slhav2_b200.build` (needs nvcc); "
                "this package has no CPU implementation" % LIB_PATH
            )
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error():
    return load_library().slha_last_error_message().decode(errors="replace")


def _check(code):
    if code != OK:
        raise SlhaError(code, last_error())


def ptr(a):
    """Address of a numpy array (host) or of anything with data_ptr() (device)."""
    if a is None:
        return None
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    if isinstance(a, int):
        return a
    raise TypeError("expected a numpy array, a device tensor or an address")


def _np(a, dtype):
    return a if hasattr(a, "data_ptr") else np.ascontiguousarray(a, dtype=dtype)


def device_count():
    return load_library().slha_b200_device_count()


def set_device(i):
    _check(load_library().slha_b200_set_device(i))


def set_stream(stream):
    """cudaStream_t address of a stream the caller created (e.g. torch.cuda.Stream().cuda_stream), or
    None / 0 for the library's own non-blocking stream.  0 is NOT the CUDA default stream here: work
    a framework enqueued on its default stream is not ordered before calls made on the library's stream,
    so either synchronize first or pass a real stream (cudaStreamLegacy is the handle 1)."""
    _check(load_library().slha_b200_set_stream(stream))


def launch_count():
    return load_library().slha_b200_launch_count()


def debug_force_generic_score(on):
    """Checking aid: the calling thread's score_topk calls use only the generic CUDA-core kernel."""
    _check(load_library().slha_b200_debug_force_generic_score(1 if on else 0))


def last_score_stats():
    """Counters of this thread's latest tensor-core score_topk call."""
    out = np.zeros(4, np.uint64)
    _check(load_library().slha_b200_last_score_stats(ptr(out)))
    return {"rows": int(out[0]), "rows_handed_to_generic_kernel": int(out[1]), "candidates_appended": int(out[2]), "buffer_slots": int(out[3])}


def timing_begin(max_calls):
    _check(load_library().slha_b200_timing_begin(max_calls))


def timing_end(capacity):
    """(score_kernel_ms[], merge_kernel_ms[]) of the calls recorded since timing_begin."""
    a, b = np.zeros(capacity, np.float32), np.zeros(capacity, np.float32)
    n = C.c_uint32()
    _check(load_library().slha_b200_timing_end(ptr(a), ptr(b), capacity, C.addressof(n)))
    m = min(n.value, capacity)
    return a[:m], b[:m]


def synchronize():
    _check(load_library().slha_b200_synchronize())


class DeviceBuffer:
    """Raw device memory owned through the C ABI (for callers without torch)."""

    def __init__(self, nbytes):
        p = C.c_void_p()
        _check(load_library().slha_b200_malloc(nbytes, C.byref(p)))
        self.address, self.nbytes = p.value, nbytes

    def data_ptr(self):
        return self.address

    def upload(self, host):
        host = np.ascontiguousarray(host)
        assert host.nbytes <= self.nbytes
        _check(load_library().slha_b200_memcpy(self.address, host.ctypes.data, host.nbytes))
        return self

    def download(self, dtype, count):
        out = np.empty(count, dtype)
        _check(load_library().slha_b200_memcpy(out.ctypes.data, self.address, out.nbytes))
        return out

    def view(self, offset, nbytes):
        """A window of this buffer (not owning; valid while the buffer lives)."""
        assert 0 <= offset and offset + nbytes <= self.nbytes
        return _DeviceView(self, offset, nbytes)

    def free(self):
        if self.address:
            load_library().slha_b200_free(self.address)
            self.address = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class _DeviceView:
    def __init__(self, owner, offset, nbytes):
        self.owner, self.address, self.nbytes = owner, owner.address + offset, nbytes

    def data_ptr(self):
        return self.address


def to_device(host):
    host = np.ascontiguousarray(host)
    return DeviceBuffer(max(host.nbytes, 1)).upload(host)


class Model:
    """LearnedModel (scirust/src/learned.rs) resident on the GPU."""

    def __init__(self, handle, d):
        self.handle, self.d = handle, d

    @classmethod
    def from_projection(cls, p, d, seed, rht=False, scale=None, z=None):
        """LearnedModel::try_from_projection_with (learned.rs:204-238)."""
        lib = load_library()
        p = np.ascontiguousarray(p, np.float32).reshape(-1)
        if p.size != 128 * d:
            raise SlhaError(ERR_DIMENSION, "projection must be D_C x d")
        s = None if scale is None else np.ascontiguousarray(scale, np.float32)
        zz = None if z is None else np.ascontiguousarray(z, np.float32)
        h = lib.slha_b200_model_create(ptr(p), d, seed, int(rht), ptr(s), ptr(zz))
        if not h:
            raise SlhaError(ERR_IO, last_error())
        return cls(h, d)

    @classmethod
    def load(cls, path):
        """weights::load through slha_weights_load."""
        lib = load_library()
        h = lib.slha_weights_load(os.fsencode(path))
        if not h:
            raise SlhaError(ERR_IO, last_error())
        return cls(h, lib.slha_model_dim(h))

    def release(self):
        if self.handle:
            _check(load_library().slha_weights_release(self.handle))
            self.handle = None

    # --- single-vector entry points of slha.h ---------------------------------
    def encode_key(self, key, position=0, codec=CODEC_INT4_GROUPED):
        key = np.ascontiguousarray(key, np.float32)
        t = np.zeros(1, TILE_DTYPE)
        _check(load_library().slha_encode_key(self.handle, ptr(key), key.size, position, codec, ptr(t)))
        return t

    def prepare_query(self, q):
        q = np.ascontiguousarray(q, np.float32)
        qc, qs = np.zeros(128, np.float32), np.zeros(4, np.uint64)
        _check(load_library().slha_prepare_query(self.handle, ptr(q), q.size, ptr(qc), ptr(qs)))
        return qc, qs

    def score_tiles(self, tiles, q_coarse, q_sign):
        tiles = np.ascontiguousarray(tiles)
        qc, qs = np.ascontiguousarray(q_coarse, np.float32), np.ascontiguousarray(q_sign, np.uint64)
        out = np.zeros(len(tiles), np.float32)
        _check(load_library().slha_score_tiles(self.handle, ptr(tiles), len(tiles), ptr(qc), ptr(qs), ptr(out)))
        return out

    def decode_latent(self, tile):
        out = np.zeros(self.d, np.float32)
        _check(load_library().slha_decode_latent(self.handle, ptr(np.ascontiguousarray(tile)), ptr(out), self.d))
        return out

    def decode_key(self, tile):
        out = np.zeros(self.d, np.float32)
        _check(load_library().slha_decode_key(self.handle, ptr(np.ascontiguousarray(tile)), ptr(out), self.d))
        return out

    # --- batched entry points ----------------------------------------------------
    def encode_keys(self, keys, codec, n=None, key_dtype=F32, positions=None, position_base=0, head_ids=None, out=None):
        """encode_with over a batch; keys/out may live on the host or on the device."""
        if not hasattr(keys, "data_ptr"):
            keys = np.ascontiguousarray(keys, np.float32 if key_dtype == F32 else np.uint16)
            n = keys.size // self.d if n is None else n
        assert n is not None
        pos = None if positions is None else _np(positions, np.uint32)
        heads = None if head_ids is None else _np(head_ids, np.uint16)
        if out is None:
            out = np.zeros(n, TILE_DTYPE)
        _check(load_library().slha_b200_encode_keys(self.handle, ptr(keys), key_dtype, n, ptr(pos), position_base, ptr(heads), codec, ptr(out)))
        return out

    def prepare_queries(self, q, nq=None, q_coarse_out=None, q_sign_out=None):
        if not hasattr(q, "data_ptr"):
            q = np.ascontiguousarray(q, np.float32)
            nq = q.size // self.d if nq is None else nq
        if q_coarse_out is None:
            q_coarse_out = np.zeros((nq, 128), np.float32)
        if q_sign_out is None:
            q_sign_out = np.zeros((nq, 4), np.uint64)
        _check(load_library().slha_b200_prepare_queries(self.handle, ptr(q), nq, ptr(q_coarse_out), ptr(q_sign_out)))
        return q_coarse_out, q_sign_out


def process_tile(tile, q_coarse, q_sign):
    """slha_process_tile: one tile, one prepared query."""
    qc, qs = np.ascontiguousarray(q_coarse, np.float32), np.ascontiguousarray(q_sign, np.uint64)
    out = np.zeros(1, np.float32)
    _check(load_library().slha_process_tile(ptr(np.ascontiguousarray(tile)), ptr(qc), ptr(qs), ptr(out)))
    return float(out[0])


def score_tiles(tiles, n, q_coarse, q_sign, nq, out=None):
    """compute_score for nq prepared queries over n tiles -> [nq, n] scores."""
    if out is None:
        out = np.zeros((nq, n), np.float32)
    _check(load_library().slha_b200_score_tiles(ptr(tiles), n, ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)), nq, ptr(out)))
    return out


def score_segments(tiles, segments, q_coarse, q_sign, nq, out, row_offsets, row_len, fill=0.0):
    """Dense scores of whole segments in one call (the llama.cpp shim's per-layer scoring step): row q of `out`
    starts at element row_offsets[q]; see slha_b200_score_segments."""
    seg = np.ascontiguousarray(segments, SEGMENT_DTYPE)
    off = _np(row_offsets, np.uint64)
    n_out = out.numel() if hasattr(out, "numel") else (out.size if hasattr(out, "size") else out.nbytes // 4)
    _check(load_library().slha_b200_score_segments(ptr(tiles), ptr(seg), len(seg), ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)),
                                                   nq, ptr(out), n_out, ptr(off), row_len, fill))
    return out


def make_segments(rows):
    """rows: iterable of (tile_begin, n_tiles, query_begin, n_queries, index_base)."""
    seg = np.zeros(len(rows), SEGMENT_DTYPE)
    for i, r in enumerate(rows):
        seg[i] = tuple(r)
    return seg


def score_topk(tiles, segments, q_coarse, q_sign, nq, k, out_index=None, out_score=None, out_count=None):
    """Fused scoring + top-k per query over device-resident tiles."""
    seg = np.ascontiguousarray(segments, SEGMENT_DTYPE)
    if out_index is None:
        out_index = np.zeros((nq, k), np.uint32)
    if out_score is None:
        out_score = np.zeros((nq, k), np.float32)
    if out_count is None:
        out_count = np.zeros(nq, np.uint32)
    _check(
        load_library().slha_b200_score_topk(
            ptr(tiles), ptr(seg), len(seg), ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)), nq, k,
            ptr(out_index), ptr(out_score), ptr(out_count),
        )
    )
    return out_index, out_score, out_count


def score_topk_noalloc(tiles, segments, q_coarse, q_sign, nq, k, out_index, out_score, out_count=None):
    """score_topk for callers that may not allocate: all buffers are device memory
    supplied by the caller, the working memory is a fixed array inside the library
    (k <= 1024, nq <= 256; see include/slha_b200.h)."""
    seg = np.ascontiguousarray(segments, SEGMENT_DTYPE)
    _check(
        load_library().slha_b200_score_topk_noalloc(
            ptr(tiles), ptr(seg), len(seg), ptr(q_coarse), ptr(q_sign), nq, k, ptr(out_index), ptr(out_score), ptr(out_count)
        )
    )


def topk_merge(cand_index, cand_score, n_lists, n_queries, k_in, k_out, out_index=None, out_score=None, list_stride=None,
               lists_sorted=False):
    """Merge per-shard top-k lists laid out [list][query][k_in] (list blocks `list_stride` elements apart);
    lists_sorted: every list is ordered best first, as score_topk writes it (slha_b200_topk_merge_sorted_strided)."""
    if out_index is None:
        out_index = np.zeros((n_queries, k_out), np.uint32)
    if out_score is None:
        out_score = np.zeros((n_queries, k_out), np.float32)
    if list_stride is None:
        list_stride = n_queries * k_in
    fn = load_library().slha_b200_topk_merge_sorted_strided if lists_sorted else load_library().slha_b200_topk_merge_strided
    _check(
        fn(
            ptr(_np(cand_index, np.uint32)), ptr(_np(cand_score, np.float32)), n_lists, list_stride, n_queries, k_in,
            k_out, ptr(out_index), ptr(out_score),
        )
    )
    return out_index, out_score


def attend_topk(top_index, top_score, k, scale, values, d_v, value_dtype=F32, top_count=None, value_row_stride=None,
                value_row_base=None, out=None, weights_out=None):
    """Decode tail: softmax over every row's k winners, then the weighted sum of their value rows
    (values: device memory).  Returns out [nq][d_v] (and fills weights_out [nq][k] when given)."""
    ti, ts = _np(top_index, np.uint32), _np(top_score, np.float32)
    nq = (ti.size if isinstance(ti, np.ndarray) else ti.numel()) // k
    if out is None:
        out = np.zeros((nq, d_v), np.float32)
    base = None if value_row_base is None else _np(value_row_base, np.uint64)
    cnt = None if top_count is None else _np(top_count, np.uint32)
    _check(load_library().slha_b200_attend_topk(ptr(ti), ptr(ts), ptr(cnt), nq, k, scale, ptr(values), value_dtype, d_v,
                                                d_v if value_row_stride is None else value_row_stride, ptr(base), ptr(out),
                                                ptr(weights_out)))
    return out


def shard_unique_id():
    """The 128-byte NCCL unique id rank 0 hands to every rank before Shard(...)."""
    buf = np.zeros(128, np.uint8)
    _check(load_library().slha_b200_shard_unique_id(ptr(buf)))
    return buf


class Shard:
    """One rank's handle of the token-range sharded scorer (slha_b200_shard_*): local fused
    score + top-k, one NCCL all-gather, merge -- all inside the library."""

    def __init__(self, unique_id, rank, world):
        h = _vp()
        uid = None if unique_id is None else np.ascontiguousarray(unique_id, np.uint8)
        _check(load_library().slha_b200_shard_init(ptr(uid), rank, world, C.byref(h)))
        self.handle, self.rank, self.world = h.value, rank, world

    def score_topk(self, tiles, segments, q_coarse, q_sign, nq, k, out_index=None, out_score=None):
        seg = np.ascontiguousarray(segments, SEGMENT_DTYPE)
        if out_index is None:
            out_index = np.zeros((nq, k), np.uint32)
        if out_score is None:
            out_score = np.zeros((nq, k), np.float32)
        _check(load_library().slha_b200_shard_score_topk(self.handle, ptr(tiles), ptr(seg), len(seg), ptr(_np(q_coarse, np.float32)),
                                                         ptr(_np(q_sign, np.uint64)), nq, k, ptr(out_index), ptr(out_score)))
        return out_index, out_score

    def set_timing(self, on=True):
        _check(load_library().slha_b200_shard_set_timing(self.handle, 1 if on else 0))

    def last_times(self):
        """(local score + top-k, all-gather, merge) milliseconds of the latest step."""
        ms = np.zeros(3, np.float32)
        _check(load_library().slha_b200_shard_last_times(self.handle, ptr(ms)))
        return ms

    def set_exchange(self, mode):
        """"peer" (default: peer-memory loads where the GPUs can map each other's memory) or "nccl" (always the all-gather)."""
        _check(load_library().slha_b200_shard_set_exchange(self.handle, {"nccl": 1, "peer": 2}[mode]))

    def status(self):
        """How the ranks' lists meet ("single rank", "nccl all-gather", "peer-memory loads"), whether a wait for a peer ran out, steps so far."""
        out = np.zeros(3, np.uint64)
        _check(load_library().slha_b200_shard_status(self.handle, ptr(out)))
        return {"exchange": ("single rank", "nccl all-gather", "peer-memory loads")[int(out[0])], "wait_ran_out": bool(out[1]), "steps": int(out[2])}

    def destroy(self):
        if self.handle:
            load_library().slha_b200_shard_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def audit():
    lib = load_library()
    p = lib.slha_audit()
    if not p:
        raise SlhaError(ERR_PANIC, last_error())
    try:
        return C.string_at(p).decode()
    finally:
        lib.slha_free_string(p)


class _PoolConfig(C.Structure):
    _fields_ = [
        ("capacity_tiles", C.c_uint64),
        ("budget_bytes", C.c_uint64),
        ("page_policy", C.c_int32),
        ("evict_policy", C.c_int32),
        ("sink_window", C.c_uint32),
        ("recent_window", C.c_uint32),
    ]


class TilePool:
    """ccos::ElasticKvCache (scirust/src/ccos.rs) with its arena in HBM."""

    def __init__(self, capacity_tiles, budget_bytes, page_policy=PAGE_LOWEST_IMPACT_FIRST, evict_policy=EVICT_CAUSAL,
                 sink_window=0, recent_window=0):
        cfg = _PoolConfig(capacity_tiles, budget_bytes, page_policy, evict_policy, sink_window, recent_window)
        h = C.c_void_p()
        _check(load_library().slha_b200_pool_create(C.byref(cfg), C.byref(h)))
        self.handle = h.value

    def destroy(self):
        if self.handle:
            load_library().slha_b200_pool_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def insert(self, tiles):
        """ElasticKvCache::insert for each tile in order; returns their slots."""
        if not hasattr(tiles, "data_ptr"):
            tiles = np.ascontiguousarray(tiles)
        n = len(tiles)
        slots = np.zeros(n, np.uint32)
        _check(load_library().slha_b200_pool_insert_tiles(self.handle, ptr(tiles), n, ptr(slots)))
        return slots

    def append_keys(self, model, keys, codec, n=None, key_dtype=F32, positions=None, position_base=0, head_ids=None,
                    want_slots=True):
        if not hasattr(keys, "data_ptr"):
            keys = np.ascontiguousarray(keys, np.float32 if key_dtype == F32 else np.uint16)
            n = keys.size // model.d if n is None else n
        pos = None if positions is None else _np(positions, np.uint32)
        heads = None if head_ids is None else _np(head_ids, np.uint16)
        slots = np.zeros(n, np.uint32) if want_slots else None
        _check(
            load_library().slha_b200_pool_append_keys(
                self.handle, model.handle, ptr(keys), key_dtype, n, ptr(pos), position_base, ptr(heads), codec, ptr(slots)
            )
        )
        return slots

    def stats(self):
        out = np.zeros(8, np.uint64)
        _check(load_library().slha_b200_pool_stats(self.handle, ptr(out)))
        keys = ("len", "live_bytes", "hot", "warm", "cold", "nocorr", "reclaimed_correction_bytes", "free_len")
        return dict(zip(keys, (int(v) for v in out)))

    def __len__(self):
        return self.stats()["len"]

    def live_bytes(self):
        return self.stats()["live_bytes"]

    def counts(self):
        s = self.stats()
        return s["hot"], s["warm"], s["cold"]

    def score_all(self, q_coarse, q_sign):
        n = len(self)
        slots, scores = np.zeros(max(n, 1), np.uint32), np.zeros(max(n, 1), np.float32)
        m = C.c_uint64()
        _check(
            load_library().slha_b200_pool_score_all(
                self.handle, ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)), ptr(slots), ptr(scores), C.addressof(m)
            )
        )
        return slots[: m.value].copy(), scores[: m.value].copy()

    def score_topk(self, q_coarse, q_sign, nq, k, out_slot=None, out_score=None, out_count=None):
        if out_slot is None:
            out_slot = np.zeros((nq, k), np.uint32)
        if out_score is None:
            out_score = np.zeros((nq, k), np.float32)
        if out_count is None:
            out_count = np.zeros(nq, np.uint32)
        _check(
            load_library().slha_b200_pool_score_topk(
                self.handle, ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)), nq, k, ptr(out_slot),
                ptr(out_score), ptr(out_count),
            )
        )
        return out_slot, out_score, out_count

    def attach_event_log(self, path, mode=0, require_durable=False):
        """attach_event_log / attach_durable_event_log (ccos.rs:155-170); mode 0 create, 1 create_new, 2 open,
        3 open_recover, 4 read-only; path None detaches."""
        _check(load_library().slha_b200_pool_attach_event_log(self.handle, None if path is None else str(path).encode(), mode,
                                                              1 if require_durable else 0))

    def rehydrate(self, seq):
        """ElasticKvCache::rehydrate (ccos.rs:451-466): slot of the re-admitted tile, or None."""
        out = C.c_int64(-1)
        _check(load_library().slha_b200_pool_rehydrate(self.handle, seq, C.addressof(out)))
        return None if out.value < 0 else int(out.value)

    def event_log_stats(self):
        out = np.zeros(3, np.uint64)
        _check(load_library().slha_b200_pool_event_log_stats(self.handle, ptr(out)))
        return {"records": int(out[0]), "log_errors": int(out[1]), "blocked_evictions": int(out[2])}

    def observe_scores(self, slots, scores, temperature):
        s, v = _np(slots, np.uint32), _np(scores, np.float32)
        _check(load_library().slha_b200_pool_observe_scores(self.handle, ptr(s), ptr(v), len(s), temperature))

    def observe_query(self, q_coarse, q_sign, temperature):
        _check(load_library().slha_b200_pool_observe_query(self.handle, ptr(_np(q_coarse, np.float32)), ptr(_np(q_sign, np.uint64)), temperature))

    def page_out(self, slot):
        _check(load_library().slha_b200_pool_page_out(self.handle, slot))

    def drop_correction(self, slot):
        r = C.c_int32()
        _check(load_library().slha_b200_pool_drop_correction(self.handle, slot, C.addressof(r)))
        return bool(r.value)

    def evict(self, slot):
        r = C.c_int32()
        _check(load_library().slha_b200_pool_evict(self.handle, slot, C.addressof(r)))
        return bool(r.value)

    def enforce_budget(self):
        r = C.c_int32()
        _check(load_library().slha_b200_pool_enforce_budget(self.handle, C.addressof(r)))
        return bool(r.value)

    def set_budget(self, budget_bytes):
        _check(load_library().slha_b200_pool_set_budget(self.handle, budget_bytes))

    def read(self, first=0, n=None):
        """(tiles, state, importance, seq) of slots [first, first+n) copied to the host."""
        if n is None:
            n = len(self) - first
        tiles, state = np.zeros(n, TILE_DTYPE), np.zeros(n, np.uint8)
        imp, seq = np.zeros(n, np.float32), np.zeros(n, np.uint64)
        if n:
            _check(load_library().slha_b200_pool_read(self.handle, first, n, ptr(tiles), ptr(state), ptr(imp), ptr(seq)))
        return tiles, state, imp, seq

    def tiles_device(self):
        return load_library().slha_b200_pool_tiles_device(self.handle)
