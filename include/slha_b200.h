/*
 * slha_b200.h -- C ABI of libslha_b200.so, a B200 (sm_100a) implementation of
 * the SLHA v2 KV-cache tile hot path: key -> 128-byte tile encode, eq. 2.3
 * scoring over tiles without decompression, deterministic top-k, and the CCOS
 * elastic tile pool kept resident in HBM.
 *
 * Part 1 re-declares, name for name and argument for argument, the C ABI the
 * reference exports from its `slha-c` crate (slha-c/include/slha.h), so a
 * program linked against `libslha` can be relinked against this library.
 * Part 2 adds batched / device-resident entry points that the reference does
 * not have; each says which reference function(s) it batches.
 *
 * All functions return one of the SLHA_* status codes unless stated otherwise
 * and record a per-thread message retrievable with slha_last_error_message().
 * Outputs are left untouched on failure.  There is no CPU fallback: without a
 * CUDA device every compute entry point fails with SLHA_ERR_DEVICE.
 */
#ifndef SLHA_B200_H
#define SLHA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ *
 * Part 1: the reference ABI (slha-c/include/slha.h, ABI version 1)    *
 * ------------------------------------------------------------------ */

#define SLHA_ABI_VERSION 1u /* slha.h:11 */

#define SLHA_D_C 128u /* latent dims per tile            slha.h:13-17 */
#define SLHA_D_S 256u /* sign-LSH residual bits */
#define SLHA_LATENT_BYTES 64u
#define SLHA_RESIDUAL_WORDS 4u
#define SLHA_N_GROUPS 8u

/* status codes, slha.h:20-29 */
#define SLHA_OK 0
#define SLHA_ERR_NULL (-1)
#define SLHA_ERR_PANIC (-2)
#define SLHA_ERR_DIMENSION (-3)
#define SLHA_ERR_CODEC (-4)
#define SLHA_ERR_NONFINITE (-5)
#define SLHA_ERR_INVALID_TILE (-6)
#define SLHA_ERR_INVALID_HANDLE (-7)
#define SLHA_ERR_IO (-8)
#define SLHA_ERR_UTF8 (-9)
/* additions of this library (not in the reference) */
#define SLHA_ERR_DEVICE (-100)   /* no CUDA device / CUDA runtime error */
#define SLHA_ERR_CAPACITY (-101) /* pool or scratch capacity exceeded */

/* codec ids, slha.h:32-37 */
#define SLHA_CODEC_INT4_SINGLE 0
#define SLHA_CODEC_INT4_GROUPED 1
#define SLHA_CODEC_NF4 2
#define SLHA_CODEC_MIXED 3
#define SLHA_CODEC_TQ3 4
#define SLHA_CODEC_MIX3 5
/* addition: MX INT4 with 32-dim groups on the unchanged tile layout (the
 * same scale byte is written for both 16-dim halves, so every decoder of the
 * reference layout reads it unmodified). */
#define SLHA_B200_CODEC_INT4_GROUPED32 6

/* tile flags, slha.h:40-46 */
#define SLHA_FLAG_HOT 0u
#define SLHA_FLAG_WARM (1u << 0)
#define SLHA_FLAG_NF4 (1u << 1)
#define SLHA_FLAG_MIXED (1u << 2)
#define SLHA_FLAG_TQ3 (1u << 3)
#define SLHA_FLAG_TQ3_NOCORR (1u << 4)
#define SLHA_FLAG_MIX3 (1u << 5)

/* Tile alignment, slha.h:48-57: a host built against a reference library whose
 * slha_tile_align() is 128 defines SLHA_CACHE_LINE_128=1; this library reports 64
 * (slha_tile_align()) and accepts tiles at any address (slha.h:150). */
#if defined(SLHA_CACHE_LINE_128) && SLHA_CACHE_LINE_128
#define SLHA_TILE_ALIGN 128u
#else
#define SLHA_TILE_ALIGN 64u
#endif

/* compile-time checks in C11, C++11 and MSVC (the role of slha.h:66-79) */
#if defined(__cplusplus)
#define SLHA_STATIC_ASSERT(cond, msg) static_assert((cond), msg)
#elif defined(__STDC_VERSION__) && __STDC_VERSION__ >= 201112L
#define SLHA_STATIC_ASSERT(cond, msg) _Static_assert((cond), msg)
#else
#define SLHA_STATIC_ASSERT(cond, msg) typedef char slha_static_assertion_failed[(cond) ? 1 : -1]
#endif

/* The 128-byte tile, slha.h:87-110.  Little-endian, no padding. */
typedef struct
#if defined(__GNUC__) || defined(__clang__)
    __attribute__((aligned(SLHA_TILE_ALIGN)))
#elif defined(_MSC_VER)
    __declspec(align(64))
#endif
{
    uint8_t latent_kv[SLHA_LATENT_BYTES];           /*   0 */
    uint64_t residual_bitmap[SLHA_RESIDUAL_WORDS];  /*  64 */
    float scale;                                    /*  96 */
    float dynamic_lambda;                           /* 100 */
    float residual_sigma;                           /* 104 */
    uint32_t token_id;                              /* 108 */
    uint32_t position;                              /* 112 */
    uint16_t head_id;                               /* 116 */
    uint16_t flags;                                 /* 118 */
    uint8_t group_scales[SLHA_N_GROUPS];            /* 120 */
} SciRustSlhaTile;

/* the layout every exchange of tiles relies on (the checks of slha.h:100-117) */
SLHA_STATIC_ASSERT(sizeof(SciRustSlhaTile) == 128u, "a tile is 128 bytes");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, latent_kv) == 0u, "latent_kv at byte 0");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, residual_bitmap) == 64u, "residual_bitmap at byte 64");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, scale) == 96u, "scale at byte 96");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, dynamic_lambda) == 100u, "dynamic_lambda at byte 100");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, residual_sigma) == 104u, "residual_sigma at byte 104");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, token_id) == 108u, "token_id at byte 108");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, position) == 112u, "position at byte 112");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, head_id) == 116u, "head_id at byte 116");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, flags) == 118u, "flags at byte 118");
SLHA_STATIC_ASSERT(offsetof(SciRustSlhaTile, group_scales) == 120u, "group_scales at byte 120");

typedef struct SlhaContext SlhaContext; /* slha.h:119 */
typedef struct SlhaModel SlhaModel;     /* slha.h:120 */

uint32_t slha_abi_version(void);           /* slha.h:123 */
size_t slha_tile_size(void);               /* slha.h:124 */
size_t slha_tile_align(void);              /* slha.h:125 */
const char* slha_last_error_message(void); /* slha.h:133 */
void slha_clear_error(void);               /* slha.h:134 */
SlhaContext* slha_init(void);              /* slha.h:140 */
int32_t slha_shutdown(SlhaContext* context); /* slha.h:147 */

/* slha.h:153-158.  One tile, one prepared query, host pointers. */
int32_t slha_process_tile(const SciRustSlhaTile* tile, const float* q_coarse,
                          const uint64_t* q_sign, float* score_out);
/* slha.h:167-173.  q (d floats) -> q_coarse (128 floats) + q_sign (4 words). */
int32_t slha_prepare_query(const SlhaModel* model, const float* q, size_t d, float* q_coarse,
                           uint64_t* q_sign);
/* slha.h:182-188 */
int32_t slha_score_tile(const SlhaModel* model, const SciRustSlhaTile* tile,
                        const float* q_coarse, const uint64_t* q_sign, float* score_out);
/* slha.h:197-204.  n_tiles <= 1<<20 (slha-c/src/lib.rs:208). */
int32_t slha_score_tiles(const SlhaModel* model, const SciRustSlhaTile* tiles, size_t n_tiles,
                         const float* q_coarse, const uint64_t* q_sign, float* scores_out);
char* slha_audit(void);               /* slha.h:210 */
void slha_free_string(char* string);  /* slha.h:213 */
SlhaModel* slha_weights_load(const char* path); /* slha.h:219 */
size_t slha_model_dim(const SlhaModel* model);  /* slha.h:225 */
/* slha.h:233-240 */
int32_t slha_encode_key(const SlhaModel* model, const float* key, size_t d, uint32_t position,
                        int32_t codec, SciRustSlhaTile* out_tile);
/* slha.h:248-253 */
int32_t slha_decode_latent(const SlhaModel* model, const SciRustSlhaTile* tile, float* out,
                           size_t d);
/* slha.h:262-267 */
int32_t slha_decode_key(const SlhaModel* model, const SciRustSlhaTile* tile, float* out, size_t d);
int32_t slha_weights_release(SlhaModel* model); /* slha.h:272 */
void slha_weights_free(SlhaModel* model);       /* slha.h:278 */

/* ------------------------------------------------------------------ *
 * Part 2: batched and device-resident entry points                    *
 *                                                                      *
 * Data pointers marked "host or device" are classified at run time;    *
 * host buffers are staged through the library's stream.  Work is       *
 * enqueued on the calling thread's stream.  With the library's own     *
 * stream a call returns after the stream has been drained.  After      *
 * slha_b200_set_stream(s) the caller owns synchronisation: calls whose *
 * outputs are device memory only enqueue work on s and return; calls   *
 * with host outputs still wait for their own copies.                  *
 * ------------------------------------------------------------------ */

/* Number of CUDA devices visible; 0 when there is none. */
int32_t slha_b200_device_count(void);
/* Select the device used by the calling thread's subsequent calls. */
int32_t slha_b200_set_device(int32_t device);
/* Use `cuda_stream` (a cudaStream_t) for the calling thread's subsequent
 * calls; NULL restores the library's own per-device stream, which is
 * non-blocking: it is NOT ordered after work on the CUDA default stream.
 * A caller whose producers run on the default stream passes cudaStreamLegacy
 * or cudaStreamPerThread explicitly, or synchronizes before calling. */
int32_t slha_b200_set_stream(void* cuda_stream);
/* Kernels launched by this library in this process so far. */
uint64_t slha_b200_launch_count(void);
/* Checking aid, no counterpart in the reference: with on != 0 the calling
 * thread's slha_b200_score_topk / slha_b200_pool_score_topk calls use only the
 * generic CUDA-core scoring kernel (every codec) and never the tensor-core
 * kernel, so that a test can require both to give the same answers; the same
 * thread's slha_b200_pool_enforce_budget calls run their phases one by one
 * from the host instead of in the single cooperative launch.  The library
 * reads no environment variable; this call is the only switch. */
int32_t slha_b200_debug_force_generic_score(int32_t on);
/* Counters of the calling thread's latest fused score + top-k call that ran on the
 * tensor-core kernel (no counterpart in the reference; the stats getter planned
 * for operators): out[0] query rows, out[1] rows that were handed to the generic
 * kernel (another codec, a query outside the fp16 split, a full candidate buffer),
 * out[2] candidates the rows' buffers received in all, out[3] slots per buffer.
 * Waits for the stream.  All zero when no such call has run. */
int32_t slha_b200_last_score_stats(uint64_t* out /* 4 values */);
/* Device timing of the fused score + top-k path: after timing_begin, each of
 * the calling thread's next `max_calls` slha_b200_score_topk /
 * slha_b200_pool_score_topk calls records CUDA events on its stream around the
 * scoring kernel (the tensor-core kernel when it runs, else the generic kernel)
 * and around what follows it (the generic kernel's pass over rows the
 * tensor-core kernel handed back, compaction, merge).  timing_end drains the stream,
 * writes per-call milliseconds (host arrays of `capacity` floats, may be NULL)
 * and the number of recorded calls, and stops recording. */
int32_t slha_b200_timing_begin(uint32_t max_calls);
int32_t slha_b200_timing_end(float* score_ms, float* merge_ms, uint32_t capacity, uint32_t* n_out);
/* Raw device memory for callers that have no CUDA runtime of their own. */
int32_t slha_b200_malloc(size_t bytes, void** out);
int32_t slha_b200_free(void* ptr);
int32_t slha_b200_memcpy(void* dst, const void* src, size_t bytes); /* any direction, synchronous */
int32_t slha_b200_synchronize(void);

/*
 * Build a model from an in-memory projection: the library-side equivalent of
 * LearnedModel::try_from_projection_with (scirust/src/learned.rs:204-238),
 * needed because slha_weights_load rejects d <= 128
 * (scirust/src/weights.rs:195-199).  `projection` is 128 x d row-major.
 * `scale` (128 floats, may be NULL = all ones) is the per-component whitening
 * scale s_k of learned.rs:257-273.  `z` (256 x d_pad, may be NULL) overrides
 * the sign-LSH matrix that is otherwise drawn from SplitMix64(seed) exactly as
 * learned.rs:168-170 does.  Returns NULL on error.
 */
SlhaModel* slha_b200_model_create(const float* projection, size_t d, uint64_t seed, int32_t rht,
                                  const float* scale, const float* z);

#define SLHA_B200_F32 0
#define SLHA_B200_BF16 1

/*
 * Encode n keys into n tiles: slha_encode_key (slha.h:233) over a batch.
 * keys: n x d, float32 or bfloat16 (key_dtype), host or device.
 * positions: n uint32 (host or device) or NULL for position_base + i.
 * head_ids: n uint16 (host or device) or NULL for 0 (the reference always
 * writes 0, learned.rs:404).  tiles_out: n tiles, host or device.
 * Tile bytes equal those of the reference's scalar encoder bit for bit.
 */
int32_t slha_b200_encode_keys(const SlhaModel* model, const void* keys, int32_t key_dtype,
                              size_t n, const uint32_t* positions, uint32_t position_base,
                              const uint16_t* head_ids, int32_t codec, SciRustSlhaTile* tiles_out);

/* slha_prepare_query (slha.h:167) over nq queries: q is nq x d float32,
 * q_coarse_out nq x 128 floats, q_sign_out nq x 4 words; host or device. */
int32_t slha_b200_prepare_queries(const SlhaModel* model, const float* q, size_t nq,
                                  float* q_coarse_out, uint64_t* q_sign_out);

/* slha_score_tiles (slha.h:197) for nq prepared queries over n tiles without
 * the 1<<20 cap: scores_out[j*n + i] = compute_score(tile i, query j).
 * All pointers host or device. */
int32_t slha_b200_score_tiles(const SciRustSlhaTile* tiles, size_t n, const float* q_coarse,
                              const uint64_t* q_sign, size_t nq, float* scores_out);

/*
 * A segment is a contiguous run of tiles scored by a contiguous group of
 * queries (one KV head and its GQA query heads; one token shard).  The tiles
 * of a segment are read once for the whole group.
 */
typedef struct {
    uint64_t tile_begin;  /* index of the segment's first tile in `tiles` */
    uint32_t n_tiles;     /* tiles in the segment */
    uint32_t query_begin; /* first query row scored against it */
    uint32_t n_queries;   /* queries in the group */
    uint32_t index_base;  /* added to the in-segment tile index in the results */
} SlhaB200Segment;

/*
 * Fused eq. 2.3 scoring + top-k.  For every query j of every segment, writes
 * the k best (index, score) pairs of that segment to out_index[j*k ..] /
 * out_score[j*k ..], ordered by score descending with ties resolved towards
 * the lower index (the ordering convention of scirust/src/metrics.rs:186-192;
 * the reference itself has no top-k step).  Rows with fewer than k tiles are
 * padded with index 0xFFFFFFFF and score -inf; out_count[j] (may be NULL) is
 * the number of valid entries.  k is 1..4096 (SLHA_ERR_DIMENSION beyond).
 * tiles must be device memory; segments,
 * queries and outputs are host or device.  Outputs in page-locked host memory
 * that the GPU can address (cudaHostAlloc, mapped cudaHostRegister) are written
 * in place by the kernel that produces them, other host outputs through a
 * staging copy; the same holds for the other top-k entry points below.  Full
 * score vectors are never written to memory.  Tiles in device memory are not
 * validated (slha_score_tiles validates, slha-c/src/lib.rs:244-286): every
 * kernel decodes a tile by the precedence of SciRustSlhaTile::dequant_at
 * (scirust/src/attention/slha_v2/tile.rs:141-151: mixed, TQ3, MIX3, NF4, INT4;
 * SLHA_FLAG_TQ3_NOCORR makes a TQ3 / MIX3 decode ignore the correction plane's
 * bytes and means nothing elsewhere), so a tile the validator would refuse still
 * scores as the reference's compute_score scores it.
 */
int32_t slha_b200_score_topk(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments,
                             size_t n_segments, const float* q_coarse, const uint64_t* q_sign,
                             size_t n_queries, uint32_t k, uint32_t* out_index, float* out_score,
                             uint32_t* out_count);

/* The scoring step of the llama.cpp shim (integration/llama.cpp/shim/
 * slha_llama.cpp:1387-1503: one slha_score_tiles call per (token, head) vector,
 * each zero-filling its row first) for a whole layer in ONE call: every query
 * row of a segment against every tile of the segment (a segment = the tile
 * store of one KV head; its query rows = the (token, head) vectors of the GQA
 * group).  Row q is written at scores_out[row_offsets[q] + index_base + i] for
 * tile i of its segment and the rest of the row, up to element row_len, is set
 * to `fill` (the shim: 0.0f for the padded positions [n_written, n_kv)); rows
 * may lie anywhere inside scores_out[0 .. scores_len) (the strides of ggml's
 * [n_kv, n_token, n_head] destination become row offsets).  tiles: device
 * memory; every other pointer host or device.  With a host scores_out the
 * elements no row covers come back as zero; a device scores_out is written
 * only where rows lie.  No counterpart in the reference's C ABI. */
int32_t slha_b200_score_segments(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments, size_t n_segments,
                                 const float* q_coarse, const uint64_t* q_sign, size_t n_queries, float* scores_out,
                                 size_t scores_len, const uint64_t* row_offsets, uint32_t row_len, float fill);

/*
 * slha_b200_score_topk for callers that must not allocate.  It has no
 * counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a decode loop
 * inside a latency budget that cannot absorb an allocation (cudaMalloc takes
 * a device-wide lock and may synchronise), or an inference server whose memory
 * pool owns every byte of HBM so that a stray allocation fails or fragments
 * it.  The promise is about DEVICE memory: the host side of the call still
 * uses ordinary C++ (a small closure per call, error strings on failure).  The regular
 * entry point sizes its work lists and candidate buffers per call shape and
 * obtains them with cudaMalloc; this one keeps them in one fixed array that
 * lives inside the library.
 *
 * Same arguments and results as slha_b200_score_topk, except:
 *  - tiles, q_coarse, q_sign and the three outputs must be device memory,
 *    segments must be host memory (nothing is staged);
 *  - limits of the fixed array (4 MiB + 22 KiB per GPU, held from library load
 *    until the process exits): k <= 1024, n_queries <= 256, and at most 512
 *    (segment, query) pairs over the non-empty segments; work items are sized
 *    so that their candidate lists fit, whatever the segment lengths.  A call
 *    beyond these limits fails with SLHA_ERR_CAPACITY and says which one it
 *    hit; devices 0..15 only;
 *  - the first call on each device resolves the array's device address and
 *    raises the kernels' shared-memory limit; make that first call outside any
 *    stream capture;
 *  - all calls on a device share the array, which keeps what the previous call
 *    left in it; a call overwrites everything it later reads, so back-to-back
 *    calls on one stream are safe, but two calls that overlap on the GPU
 *    (different streams or threads without ordering) race on it.
 * It calls no cudaMalloc / cudaFree and no library routine that allocates
 * device memory.  The segment table and query ranges are copied from ordinary
 * (pageable) host arrays, so each call synchronises briefly with its stream.
 */
int32_t slha_b200_score_topk_noalloc(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments,
                                     size_t n_segments, const float* q_coarse, const uint64_t* q_sign,
                                     size_t n_queries, uint32_t k, uint32_t* out_index,
                                     float* out_score, uint32_t* out_count);

/*
 * Decode tail on the selected tiles: for every query row, softmax over its k
 * (index, score) winners -- logits score * scale, maximum subtracted, as
 * metrics::softmax_into (scirust/src/metrics.rs:338-420) -- and the weighted
 * sum of their value rows, as aggregate_v of the reference's decode proxy
 * (scirust/examples/benchmark_decode.rs:28-38, :82-95; the proxy runs both over
 * the whole context, here they run over the top-k).  Entries with index
 * 0xFFFFFFFF (padding) and entries past top_count[j] weigh nothing.
 *   values            device memory, rows of d_v elements (float32 or
 *                     bfloat16), `value_row_stride` elements apart
 *   value_row_base    per query row (may be NULL = 0): the value row of winner
 *                     i of row j is value_row_base[j] + top_index[j*k + i],
 *                     modulo 2^64 (the base carries the KV head's first row
 *                     minus the segment's index_base)
 *   out               n_queries x d_v floats; weights_out (may be NULL)
 *                     n_queries x k softmax weights.  Host or device.
 * Results agree with the sequential float32 / float64 reference arithmetic to
 * about 1e-6 relative (sums are taken in a different, fixed order).
 */
int32_t slha_b200_attend_topk(const uint32_t* top_index, const float* top_score,
                              const uint32_t* top_count, size_t n_queries, uint32_t k, float scale,
                              const void* values, int32_t value_dtype, size_t d_v,
                              size_t value_row_stride, const uint64_t* value_row_base, float* out,
                              float* weights_out);

/*
 * Token-range sharding over the GPUs of one node, one handle per rank (one
 * process or host thread per GPU).  The reference has no multi-device path;
 * these calls implement the sharding the tile scores' independence allows
 * (ElasticKvCache::score_all, scirust/src/ccos.rs:346-355): every rank scores
 * the tiles in its own HBM and keeps its own top k per query row, ONE
 * ncclAllGather moves every rank's [2][n_queries][k] block (indices, then score
 * bits), and every rank merges the `world` lists with the ordering rule of
 * scirust/src/metrics.rs:186-192, so all ranks hold the same global result.
 *
 * NCCL is bound at run time (libnccl.so.2, the copy already loaded in the
 * process when there is one); a host that never calls these functions needs
 * no NCCL.  Rank 0 obtains the 128-byte unique id and hands it to the other
 * ranks by any transport the host has (a file, a socket, MPI, a torch
 * broadcast).  shard_init is collective: every rank of `world` must call it.
 * With world == 1 no id and no NCCL are needed and a step is plain
 * slha_b200_score_topk.
 */
typedef struct SlhaB200Shard SlhaB200Shard;
int32_t slha_b200_shard_unique_id(void* id_out /* 128 bytes */);
int32_t slha_b200_shard_init(const void* nccl_unique_id, int32_t rank, int32_t world, SlhaB200Shard** out);
int32_t slha_b200_shard_destroy(SlhaB200Shard* shard);
/*
 * One sharded decode step, collective over the ranks: same arguments as
 * slha_b200_score_topk for THIS rank's tiles and segment table (segments in
 * host memory; index_base = the global token position of the rank's first
 * tile), every rank passes the same queries and k.  out_index / out_score
 * ([n_queries][k], host or device) receive the merged global top k on every
 * rank.  The three device steps (local fused score + top-k, all-gather, merge)
 * are enqueued back to back on the calling thread's stream without a host
 * round trip; with a caller-supplied stream and device outputs the call
 * returns once they are enqueued.
 */
int32_t slha_b200_shard_score_topk(SlhaB200Shard* shard, const SciRustSlhaTile* tiles,
                                   const SlhaB200Segment* segments, size_t n_segments,
                                   const float* q_coarse, const uint64_t* q_sign, size_t n_queries,
                                   uint32_t k, uint32_t* out_index, float* out_score);
/* Device timing of the steps of this handle: with on != 0 every step records
 * CUDA events on its stream; last_times waits for the latest step and writes
 * its three durations in milliseconds: local score + top-k, all-gather, merge. */
int32_t slha_b200_shard_set_timing(SlhaB200Shard* shard, int32_t on);
int32_t slha_b200_shard_last_times(SlhaB200Shard* shard, float* ms_out /* 3 floats */);
/* out[0]: how the ranks' lists meet -- 0 one rank, 1 ncclAllGather, 2 peer-memory loads: where the ranks are
 * processes of one node whose GPUs can map each other's memory (CUDA IPC), no all-gather runs; every rank
 * leaves its sorted block in its own memory, raises a flag in every peer's memory, and the merge kernel reads
 * from the owners' blocks the few entries it needs over NVLink.  out[1]: 1 when a wait for a peer's flag ran
 * out (ten seconds; the rows of that step came back empty).  out[2]: steps enqueued on this handle. */
int32_t slha_b200_shard_status(SlhaB200Shard* shard, uint64_t* out /* 3 values */);
/* mode 2 (the default): peer-memory loads where possible, else ncclAllGather; mode 1: ncclAllGather always.
 * Every rank makes the same call, between steps. */
int32_t slha_b200_shard_set_exchange(SlhaB200Shard* shard, int32_t mode);

/*
 * Merge n_lists candidate lists per query (layout [list][query][k_in], as an
 * all-gather of per-shard slha_b200_score_topk outputs produces) into the
 * global top k_out per query with the same ordering rule.  Device pointers.
 */
int32_t slha_b200_topk_merge(const uint32_t* cand_index, const float* cand_score,
                             uint32_t n_lists, uint32_t n_queries, uint32_t k_in, uint32_t k_out,
                             uint32_t* out_index, float* out_score);

/* Same, for lists whose per-list blocks are `list_stride` elements apart (for
 * instance index and score blocks interleaved in one gathered buffer). */
int32_t slha_b200_topk_merge_strided(const uint32_t* cand_index, const float* cand_score,
                                     uint32_t n_lists, uint64_t list_stride, uint32_t n_queries,
                                     uint32_t k_in, uint32_t k_out, uint32_t* out_index,
                                     float* out_score);

/* Same, for lists that are each ordered best first with absent entries (index
 * 0xFFFFFFFF) only at their ends -- what slha_b200_score_topk writes.  The
 * merge then reads the lists' ceil(k_out / n_lists)-th entries first: the
 * smallest of them is reached by at least k_out candidates, so only the keys
 * at or above it are gathered (shards of one context leave little more than
 * k_out of the n_lists * k_in).  Lists that are not ordered give wrong results. */
int32_t slha_b200_topk_merge_sorted_strided(const uint32_t* cand_index, const float* cand_score,
                                            uint32_t n_lists, uint64_t list_stride, uint32_t n_queries,
                                            uint32_t k_in, uint32_t k_out, uint32_t* out_index,
                                            float* out_score);

/* -------- CCOS elastic tile pool (scirust/src/ccos.rs ElasticKvCache) -------- */

typedef struct SlhaB200Pool SlhaB200Pool;

#define SLHA_B200_STATE_HOT 0
#define SLHA_B200_STATE_WARM 1
#define SLHA_B200_STATE_COLD 2
#define SLHA_B200_PAGE_LOWEST_IMPACT_FIRST 0 /* ccos.rs:47-56 PageOutPolicy */
#define SLHA_B200_PAGE_OLDEST_FIRST 1
#define SLHA_B200_EVICT_CAUSAL 0 /* ccos.rs:64-89 EvictionPolicy */
#define SLHA_B200_EVICT_IMPORTANCE 1

typedef struct {
    uint64_t capacity_tiles; /* slots reserved in HBM (128 B tile + 13 B bookkeeping each) */
    uint64_t budget_bytes;   /* logical byte budget of enforce_budget */
    int32_t page_policy;
    int32_t evict_policy;
    uint32_t sink_window;    /* EvictionPolicy::Importance{sink_window}, ccos.rs:76-89 */
    uint32_t recent_window;  /* addition: also pin the newest positions; 0 = reference behaviour */
} SlhaB200PoolConfig;

/* ElasticKvCache::new / with_budget / with_eviction, ccos.rs:132-214 */
int32_t slha_b200_pool_create(const SlhaB200PoolConfig* config, SlhaB200Pool** out);
int32_t slha_b200_pool_destroy(SlhaB200Pool* pool);
/* ElasticKvCache::insert (ccos.rs:217-259) for n ready-made tiles, in order;
 * slots_out (n uint32, host, may be NULL) receives the slot of each. */
int32_t slha_b200_pool_insert_tiles(SlhaB200Pool* pool, const SciRustSlhaTile* tiles, size_t n,
                                    uint32_t* slots_out);
/* encode_with + insert without the tiles leaving HBM. */
int32_t slha_b200_pool_append_keys(SlhaB200Pool* pool, const SlhaModel* model, const void* keys,
                                   int32_t key_dtype, size_t n, const uint32_t* positions,
                                   uint32_t position_base, const uint16_t* head_ids, int32_t codec,
                                   uint32_t* slots_out);
/* ElasticKvCache::score_all (ccos.rs:346-355): (slot, score) of every
 * non-COLD slot in slot order for one query; n_out receives the count.
 * slots_out / scores_out (host or device) must hold pool length entries. */
int32_t slha_b200_pool_score_all(SlhaB200Pool* pool, const float* q_coarse, const uint64_t* q_sign,
                                 uint32_t* slots_out, float* scores_out, uint64_t* n_out);
/* score_all + top-k over the live slots for nq queries; indices are slots. */
int32_t slha_b200_pool_score_topk(SlhaB200Pool* pool, const float* q_coarse,
                                  const uint64_t* q_sign, size_t nq, uint32_t k,
                                  uint32_t* out_slot, float* out_score, uint32_t* out_count);
/* ElasticKvCache::observe_scores (ccos.rs:275-314) */
int32_t slha_b200_pool_observe_scores(SlhaB200Pool* pool, const uint32_t* slots,
                                      const float* scores, size_t n, float temperature);
/* score_all followed by observe_scores, entirely on the device. */
int32_t slha_b200_pool_observe_query(SlhaB200Pool* pool, const float* q_coarse,
                                     const uint64_t* q_sign, float temperature);
int32_t slha_b200_pool_page_out(SlhaB200Pool* pool, uint32_t slot);                      /* ccos.rs:365 */
int32_t slha_b200_pool_drop_correction(SlhaB200Pool* pool, uint32_t slot, int32_t* dropped); /* ccos.rs:386 */
int32_t slha_b200_pool_evict(SlhaB200Pool* pool, uint32_t slot, int32_t* evicted);        /* ccos.rs:404 */
/*
 * COLD persistence: attach the reference's EventLog (scirust/src/eventlog.rs:9-24 -- 16-byte header,
 * 144-byte records of (seq, slot, FNV-1a checksum, tile), byte-identical for identical evictions) as
 * ElasticKvCache::attach_event_log / attach_durable_event_log do (ccos.rs:155-170).  From then on every
 * eviction (slha_b200_pool_evict and the eviction phase of enforce_budget) first brings the doomed
 * tiles to the host and appends their records in eviction order, then flips the slots; with
 * require_durable != 0 each record is fsync'ed and a record that cannot be written keeps its slot live
 * (ccos.rs:404-438).  mode: 0 create / truncate, 1 create only if absent, 2 open an existing log
 * strictly (header, whole records, checksums), 3 open and drop one partial record at the tail,
 * 4 open read-only.  path == NULL detaches.
 */
int32_t slha_b200_pool_attach_event_log(SlhaB200Pool* pool, const char* path, int32_t mode,
                                        int32_t require_durable);
/* ElasticKvCache::rehydrate (ccos.rs:451-466): the most recent record with eviction sequence `seq`
 * re-enters the pool as a fresh admission (WARM if its tile carries the WARM flag, else HOT);
 * slot_out gets its slot, or -1 when no log is attached or no record matches. */
int32_t slha_b200_pool_rehydrate(SlhaB200Pool* pool, uint64_t seq, int64_t* slot_out);
/* out[0] records in the attached log, out[1] log_errors, out[2] blocked_evictions (ccos.rs:173-181) */
int32_t slha_b200_pool_event_log_stats(SlhaB200Pool* pool, uint64_t* out /* 3 values */);
/* ElasticKvCache::enforce_budget (ccos.rs:555-614); within_budget gets its bool. */
int32_t slha_b200_pool_enforce_budget(SlhaB200Pool* pool, int32_t* within_budget);
int32_t slha_b200_pool_set_budget(SlhaB200Pool* pool, uint64_t budget_bytes);
/* len, live_bytes (ccos.rs:484), counts (ccos.rs:510), nocorr_count,
 * reclaimed_correction_bytes (ccos.rs:488-508) in one read-back:
 * out[0..7] = len, live_bytes, hot, warm, cold, nocorr, reclaimed, free_len */
int32_t slha_b200_pool_stats(SlhaB200Pool* pool, uint64_t out[8]);
/* Copy-outs for parity checks: tile(), state(), importance(), seq of ccos.rs:357-363, :262 */
int32_t slha_b200_pool_read(SlhaB200Pool* pool, uint64_t first, uint64_t n,
                            SciRustSlhaTile* tiles_out, uint8_t* state_out,
                            float* importance_out, uint64_t* seq_out);
/* Device address of the pool's tile array (slot-indexed), for zero-copy scoring. */
const SciRustSlhaTile* slha_b200_pool_tiles_device(SlhaB200Pool* pool);

#ifdef __cplusplus
}
#endif
#endif /* SLHA_B200_H */
