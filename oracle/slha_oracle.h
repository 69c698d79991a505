/*
 * CPU oracle for the SLHA v2 tile hot path  --  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's scalar algorithm (Rust crate
 * `scirust`).  It exists so the CUDA path can be checked bit-for-bit (tile
 * bytes, Hamming distances) and within 1e-3 (scores).  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may load it; the shipped
 * library never links or calls anything in this directory.
 *
 * Pinning: the reference's CPU code is Rust and no Rust toolchain exists on the
 * build machine, so the oracle is pinned by the reference's own known-answer
 * tests and fixtures (tests/test_oracle_kats.py, tests/test_oracle_ccos.py) and by
 * the reference's unit, property and end-to-end tests rebuilt from its own
 * seeds on its restated PRNG (tests/test_oracle_reference_properties.py,
 * tests/test_oracle_ccos_reference_suite.py,
 * tests/test_oracle_learned_reference_suite.py).  The reference holds no golden
 * tile bytes: the encode path is pinned at the level of those tests'
 * thresholds, not byte for byte.  Its scoring functions are in addition checked against the reference's real
 * CUDA kernel (slhav2-vram/kernels/slha_score.cu, compiled from the reference
 * tree into oracle/_ref/ by `make ref`) in tests/test_gpu_reference_kernel.py.
 *
 * Every function names the reference file:line it follows.  Build with
 * -ffp-contract=off: the reference never fuses multiply-add and all sums are
 * strictly sequential.
 */
#ifndef SLHA_ORACLE_H
#define SLHA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORA_D_C 128
#define ORA_D_S 256
#define ORA_LATENT_BYTES 64
#define ORA_RESIDUAL_WORDS 4
#define ORA_N_GROUPS 8
#define ORA_GROUP_DIM 16

/* scirust/src/attention/slha_v2/constants.rs:22-48 */
#define ORA_FLAG_WARM 1u
#define ORA_FLAG_NF4 2u
#define ORA_FLAG_MIXED 4u
#define ORA_FLAG_TQ3 8u
#define ORA_FLAG_TQ3_NOCORR 16u
#define ORA_FLAG_MIX3 32u

/* scirust/src/attention/slha_v2/tile.rs:52-77 (repr(C), 128 bytes, no padding) */
typedef struct {
    uint8_t latent_kv[ORA_LATENT_BYTES];
    uint64_t residual_bitmap[ORA_RESIDUAL_WORDS];
    float scale;
    float dynamic_lambda;
    float residual_sigma;
    uint32_t token_id;
    uint32_t position;
    uint16_t head_id;
    uint16_t flags;
    uint8_t group_scales[ORA_N_GROUPS];
} ora_tile;

/* ---- rng.rs ------------------------------------------------------------ */
typedef struct { uint64_t state; } ora_rng;
void ora_rng_init(ora_rng* r, uint64_t seed);
uint64_t ora_rng_next_u64(ora_rng* r);
float ora_rng_next_unit(ora_rng* r);
float ora_rng_next_gaussian(ora_rng* r);
void ora_rng_fill_gaussian(ora_rng* r, float* out, size_t n);

/* ---- codecs (codec directory) ---------------------------------------------- */
void ora_quantize_latent(const float* v, uint8_t* out, float* scale);
void ora_quantize_latent_grouped(const float* v, uint8_t* out, float* global, uint8_t* gs);
/* Layout-compatible extension (not in the reference): absmax over 32 dims,
 * the same scale byte written to both 16-dim groups of the pair. */
void ora_quantize_latent_grouped32(const float* v, uint8_t* out, float* global, uint8_t* gs);
void ora_quantize_latent_nf4(const float* v, uint8_t* out, float* global, uint8_t* gs);
void ora_quantize_latent_mixed(const float* v, uint8_t* out, float* global, uint8_t* gs);
void ora_quantize_latent_tq3(const float* v, uint8_t* out, float* global, uint8_t* gs);
void ora_quantize_latent_mix3(const float* v, uint8_t* out, float* global, uint8_t* gs);
uint8_t ora_nf4_nearest(float t);

/* ---- tile.rs: dequant + scalar score ---------------------------------- */
float ora_dequant_at(const ora_tile* t, int d);
void ora_dequant_latent(const ora_tile* t, float* out);
uint32_t ora_hamming(const uint64_t* a, const uint64_t* b);
float ora_compute_score_scalar(const ora_tile* t, const float* q_coarse, const uint64_t* q_sign);
void ora_score_tiles(const ora_tile* tiles, size_t n, const float* q_coarse,
                     const uint64_t* q_sign, float* out);
/* slha-c/src/lib.rs:244-286; returns 0 ok, -5 non-finite, -6 invalid */
int ora_validate_tile(const ora_tile* t);

/* ---- incoherence.rs ---------------------------------------------------- */
size_t ora_next_pow2(size_t n);
void ora_fwht_inplace(float* v, size_t n);

/* ---- learned.rs --------------------------------------------------------- */
typedef struct ora_model ora_model;
/* codec ids follow slha-c/include/slha.h:32-37; id 6 = grouped32 extension */
ora_model* ora_model_from_projection(const float* p, size_t d, uint64_t seed, int rht);
void ora_model_set_scale(ora_model* m, const float* scale128);
void ora_model_set_z(ora_model* m, const float* z); /* D_S x d_pad, fixture override */
void ora_model_free(ora_model* m);
size_t ora_model_d(const ora_model* m);
size_t ora_model_d_pad(const ora_model* m);
const float* ora_model_z(const ora_model* m);
const float* ora_model_rht_diag(const ora_model* m); /* NULL when no RHT */
void ora_model_latent(const ora_model* m, const float* key, float* h);
void ora_model_query_coarse(const ora_model* m, const float* q, float* out);
void ora_model_reconstruct(const ora_model* m, const float* h, float* r);
void ora_model_sign_bits(const ora_model* m, const float* v, uint64_t* out);
int ora_model_encode(const ora_model* m, const float* key, uint32_t pos, int warm,
                     int codec, ora_tile* out);
void ora_model_encode_batch(const ora_model* m, const float* keys, size_t n,
                            const uint32_t* pos, const uint16_t* head, int codec,
                            ora_tile* out);
void ora_model_prepare_query(const ora_model* m, const float* q, float* q_coarse,
                             uint64_t* q_sign);
void ora_model_decode_latent(const ora_model* m, const ora_tile* t, float* out);
void ora_model_decode_key(const ora_model* m, const ora_tile* t, float* out);

/* weights.rs:68-80 (FNV-1a) and :159-270 (parser).  Returns NULL + message. */
uint32_t ora_weights_checksum(const uint8_t* hdr24, const uint8_t* payload, size_t n);
ora_model* ora_weights_from_bytes(const uint8_t* bytes, size_t len, char* err, size_t errlen);

/* ---- scenario.rs -------------------------------------------------------- */
float ora_analytic_lambda_c(void);
double ora_rms(const float* v, size_t n);
void ora_scenario_sign_bits(const float* z, const float* v, uint64_t* out);
void ora_scenario_build_tile(const float* z, const float* k_coarse, const float* e,
                             uint32_t pos, int warm, ora_tile* out);

/* ---- top-k (ordering of metrics.rs:186-192: score desc by total order,
 *      ties -> lower index) ------------------------------------------------ */
void ora_topk(const float* scores, size_t n, size_t k, uint32_t* idx_out, float* score_out);

/* ---- ccos.rs: ElasticKvCache -------------------------------------------- */
typedef struct ora_cache ora_cache;
enum { ORA_HOT = 0, ORA_WARM = 1, ORA_COLD = 2 };
enum { ORA_PAGE_LOWEST_IMPACT = 0, ORA_PAGE_OLDEST = 1 };
enum { ORA_EVICT_CAUSAL = 0, ORA_EVICT_IMPORTANCE = 1 };
ora_cache* ora_cache_new(size_t budget_bytes, int page_policy, int evict_policy,
                         uint32_t sink_window, uint32_t recent_window);
void ora_cache_free(ora_cache* c);
size_t ora_cache_insert(ora_cache* c, const ora_tile* t);
size_t ora_cache_len(const ora_cache* c);
int ora_cache_state(const ora_cache* c, size_t slot);
const ora_tile* ora_cache_tile(const ora_cache* c, size_t slot);
float ora_cache_importance(const ora_cache* c, size_t slot);
uint64_t ora_cache_seq(const ora_cache* c, size_t slot);
size_t ora_cache_live_bytes(const ora_cache* c);
void ora_cache_counts(const ora_cache* c, size_t* hot, size_t* warm, size_t* cold);
void ora_cache_page_out(ora_cache* c, size_t slot);
int ora_cache_drop_correction(ora_cache* c, size_t slot);
int ora_cache_evict(ora_cache* c, size_t slot);
int ora_cache_enforce_budget(ora_cache* c);
/* score_all: writes (slot, score) for every non-COLD slot; returns the count */
size_t ora_cache_score_all(const ora_cache* c, const float* q_coarse, const uint64_t* q_sign,
                           uint32_t* slots, float* scores);
void ora_cache_observe_scores(ora_cache* c, const uint32_t* slots, const float* scores,
                              size_t n, float temperature);
size_t ora_cache_journal_len(const ora_cache* c);
void ora_cache_journal_get(const ora_cache* c, size_t i, uint64_t* seq, uint32_t* slot, ora_tile* tile);
size_t ora_cache_nocorr_count(const ora_cache* c);
size_t ora_cache_reclaimed_correction_bytes(const ora_cache* c);

/* ---- timed CPU baseline loops (bench only) ------------------------------ */
/* which: 0 scalar, 1 AVX2 restatement, 2 AVX-512 restatement, -1 best available */
int ora_simd_level(void);
double ora_score_sink(const ora_tile* tiles, size_t n, const float* q_coarse,
                      const uint64_t* q_sign, int which, int threads);
float ora_compute_score_simd(const ora_tile* t, const float* q_coarse, const uint64_t* q_sign,
                             int which);

#ifdef __cplusplus
}
#endif
#endif
