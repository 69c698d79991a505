/*
 * CPU oracle (test infrastructure only): the timed CPU baseline.
 *
 * Restates the reference's vectorised `compute_score` for the two codecs the
 * benchmark workloads use (uniform/grouped INT4 and NF4) at the AVX2 and
 * AVX-512 levels, with the same runtime dispatch rule (AVX-512 > AVX2 >
 * scalar, scirust/src/attention/slha_v2/simd.rs:23-84).  Other codecs take the
 * scalar path here.  Rust's std::arch intrinsics map one-to-one onto
 * <immintrin.h>.  The reference binary itself cannot be built (no Rust
 * toolchain), so this is a "port" baseline, not the reference executable.
 * See slha_oracle.h for the rules that govern this directory.
 */
#include "slha_oracle.h"

#include <immintrin.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float NF4_CB[16] = {-1.0f,   -0.7075f, -0.5421f, -0.4165f, -0.3108f, -0.2158f,
                                 -0.1272f, -0.0421f, 0.0421f,  0.1272f,  0.2158f,  0.3108f,
                                 0.4165f,  0.5421f,  0.7075f,  1.0f};

int ora_simd_level(void) {
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx512f")) return 2;
    if (__builtin_cpu_supports("avx2")) return 1;
    return 0;
}

static inline float residual_term(const ora_tile* t, const uint64_t* q_sign) {
    /* tile.rs:261-264; popcount lowers to POPCNT like u64::count_ones */
    uint32_t h = 0;
    for (int w = 0; w < 4; ++w) h += (uint32_t)__builtin_popcountll(q_sign[w] ^ t->residual_bitmap[w]);
    return t->dynamic_lambda * (256.0f - 2.0f * (float)h);
}

/* simd.rs:94-141 (INT4) and :240-293 (NF4): 8-wide, separate mul and add */
__attribute__((target("avx2"))) static float score_avx2(const ora_tile* t, const float* q,
                                                         const uint64_t* q_sign, int nf4) {
    const float inv255 = 1.0f / 255.0f;
    const __m256 eight = _mm256_set1_ps(8.0f);
    const __m256 cb_lo = _mm256_loadu_ps(NF4_CB), cb_hi = _mm256_loadu_ps(NF4_CB + 8);
    const __m256i seven = _mm256_set1_epi32(7);
    const __m128i mask = _mm_set1_epi8(0x0F);
    __m256 acc = _mm256_setzero_ps();
    for (int g = 0; g < 8; ++g) {
        __m256 gs = _mm256_set1_ps(t->scale * ((float)t->group_scales[g] * inv255));
        __m128i packed = _mm_loadl_epi64((const __m128i*)(t->latent_kv + g * 8));
        __m128i lo = _mm_and_si128(packed, mask);
        __m128i hi = _mm_and_si128(_mm_srli_epi16(packed, 4), mask);
        __m128i d16 = _mm_unpacklo_epi8(lo, hi);
        for (int half = 0; half < 2; ++half) {
            __m128i bytes = half ? _mm_srli_si128(d16, 8) : d16;
            __m256i nib = _mm256_cvtepu8_epi32(bytes);
            __m256 level;
            if (nf4) {
                __m256 lo_v = _mm256_permutevar8x32_ps(cb_lo, nib);
                __m256 hi_v = _mm256_permutevar8x32_ps(cb_hi, nib);
                __m256 pick = _mm256_castsi256_ps(_mm256_cmpgt_epi32(nib, seven));
                level = _mm256_blendv_ps(lo_v, hi_v, pick);
            } else {
                level = _mm256_sub_ps(_mm256_cvtepi32_ps(nib), eight);
            }
            __m256 v = _mm256_mul_ps(gs, level);
            __m256 qv = _mm256_loadu_ps(q + g * 16 + half * 8);
            acc = _mm256_add_ps(acc, _mm256_mul_ps(v, qv));
        }
    }
    float tmp[8];
    _mm256_storeu_ps(tmp, acc);
    float coarse = 0.0f;
    for (int i = 0; i < 8; ++i) coarse += tmp[i];
    if (t->flags & ORA_FLAG_WARM) return coarse;
    return coarse + residual_term(t, q_sign);
}

/* simd.rs:465-499 (INT4) and :600-634 (NF4): one 16-wide FMA per group */
__attribute__((target("avx512f,avx512vl,avx512bw"))) static float score_avx512(
    const ora_tile* t, const float* q, const uint64_t* q_sign, int nf4) {
    const float inv255 = 1.0f / 255.0f;
    const __m512 eight = _mm512_set1_ps(8.0f);
    const __m512 cb = _mm512_loadu_ps(NF4_CB);
    const __m128i mask = _mm_set1_epi8(0x0F);
    __m512 acc = _mm512_setzero_ps();
    for (int g = 0; g < 8; ++g) {
        __m512 gs = _mm512_set1_ps(t->scale * ((float)t->group_scales[g] * inv255));
        __m128i packed = _mm_loadl_epi64((const __m128i*)(t->latent_kv + g * 8));
        __m128i lo = _mm_and_si128(packed, mask);
        __m128i hi = _mm_and_si128(_mm_srli_epi16(packed, 4), mask);
        __m128i d16 = _mm_unpacklo_epi8(lo, hi);
        __m512i idx = _mm512_cvtepu8_epi32(d16);
        __m512 level = nf4 ? _mm512_permutexvar_ps(idx, cb) : _mm512_sub_ps(_mm512_cvtepi32_ps(idx), eight);
        __m512 v = _mm512_mul_ps(gs, level);
        acc = _mm512_fmadd_ps(v, _mm512_loadu_ps(q + g * 16), acc);
    }
    float coarse = _mm512_reduce_add_ps(acc);
    if (t->flags & ORA_FLAG_WARM) return coarse;
    return coarse + residual_term(t, q_sign);
}

float ora_compute_score_simd(const ora_tile* t, const float* q, const uint64_t* q_sign, int which) {
    if (which < 0) which = ora_simd_level();
    /* flag precedence of simd.rs:34-44: only plain INT4 / NF4 tiles are vectorised here */
    if (which == 0 || (t->flags & (ORA_FLAG_MIXED | ORA_FLAG_TQ3 | ORA_FLAG_MIX3)))
        return ora_compute_score_scalar(t, q, q_sign);
    int nf4 = (t->flags & ORA_FLAG_NF4) != 0;
    return which == 2 ? score_avx512(t, q, q_sign, nf4) : score_avx2(t, q, q_sign, nf4);
}

/* Loop shape of scirust/examples/bench_vs_fp16.rs:133-147: fixed query, walk a
 * contiguous tile array, accumulate into a sink.  `threads` > 1 splits the
 * array into contiguous ranges, one per thread. */
double ora_score_sink(const ora_tile* tiles, size_t n, const float* q, const uint64_t* q_sign,
                      int which, int threads) {
    if (which < 0) which = ora_simd_level();
    double sink = 0.0;
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads) reduction(+ : sink)
    for (long long i = 0; i < (long long)n; ++i)
        sink += (double)ora_compute_score_simd(&tiles[i], q, q_sign, which);
    return sink;
}
