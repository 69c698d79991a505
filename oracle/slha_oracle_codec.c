/*
 * CPU oracle (test infrastructure only): PRNG, the six latent quantisers,
 * per-codec dequantisation, Hamming distance and the scalar score.
 * See slha_oracle.h for the rules that govern this directory.
 */
#include "slha_oracle.h"

#include <math.h>
#include <string.h>

/* ------------------------------------------------------------------------
 * scirust/src/rng.rs:13-51  SplitMix64 + Box-Muller (cosine branch only)
 * ---------------------------------------------------------------------- */
void ora_rng_init(ora_rng* r, uint64_t seed) { r->state = seed ^ 0x9E3779B97F4A7C15ull; }

uint64_t ora_rng_next_u64(ora_rng* r) {
    r->state += 0x9E3779B97F4A7C15ull;
    uint64_t z = r->state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

float ora_rng_next_unit(ora_rng* r) {
    /* rng.rs:33-36: top 24 bits scaled by 2^-24 */
    return (float)(ora_rng_next_u64(r) >> 40) * (1.0f / (float)(1ull << 24));
}

float ora_rng_next_gaussian(ora_rng* r) {
    /* rng.rs:39-44 */
    float u1 = ora_rng_next_unit(r);
    if (!(u1 > 1.0e-7f)) u1 = 1.0e-7f;
    float u2 = ora_rng_next_unit(r);
    float rad = sqrtf(-2.0f * logf(u1));
    return rad * cosf(2.0f * 3.14159265358979323846f * u2);
}

void ora_rng_fill_gaussian(ora_rng* r, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = ora_rng_next_gaussian(r);
}

/* ------------------------------------------------------------------------
 * Rust numeric-cast semantics used by the quantisers
 * ---------------------------------------------------------------------- */
static int sat_i32(float x) { /* `x as i32`: saturating, NaN -> 0 */
    if (x != x) return 0;
    if (x >= 2147483648.0f) return 2147483647;
    if (x <= -2147483648.0f) return (-2147483647 - 1);
    return (int)x;
}
static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
static float fmax_rs(float a, float b) { /* f32::max: NaN-ignoring */
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}
static uint8_t scale_byte(float step, float global) {
    /* `(step / global * 255.0).round().clamp(1.0, 255.0) as u8`  int4.rs:48-49 */
    float r = roundf(step / global * 255.0f);
    if (r != r) return 0;
    if (r < 1.0f) r = 1.0f;
    if (r > 255.0f) r = 255.0f;
    return (uint8_t)r;
}
static void put_nibble(uint8_t* out, int d, uint8_t nib) {
    /* int4.rs:17-21: even dim -> low nibble, odd dim -> high nibble */
    if ((d & 1) == 0) out[d >> 1] = (uint8_t)((out[d >> 1] & 0xF0) | nib);
    else out[d >> 1] = (uint8_t)((out[d >> 1] & 0x0F) | (nib << 4));
}
static uint8_t int4_nibble(float v, float step) {
    int q = clampi(sat_i32(roundf(v / step)), -8, 7) + 8;
    return (uint8_t)(q & 0x0F);
}

/* codec/int4.rs:9-24 */
void ora_quantize_latent(const float* v, uint8_t* out, float* scale) {
    float max_abs = 0.0f;
    for (int d = 0; d < ORA_D_C; ++d) max_abs = fmax_rs(max_abs, fabsf(v[d]));
    float s = max_abs > 0.0f ? max_abs / 7.0f : 1.0f;
    memset(out, 0, ORA_LATENT_BYTES);
    for (int d = 0; d < ORA_D_C; ++d) put_nibble(out, d, int4_nibble(v[d], s));
    *scale = s;
}

static float pick_global(const float* steps) {
    float g = 0.0f;
    for (int i = 0; i < ORA_N_GROUPS; ++i) g = fmax_rs(g, steps[i]);
    return g > 0.0f ? g : 1.0f;
}

/* codec/int4.rs:34-63 */
void ora_quantize_latent_grouped(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    for (int g = 0; g < ORA_N_GROUPS; ++g) {
        float mx = 0.0f;
        for (int d = g * ORA_GROUP_DIM; d < (g + 1) * ORA_GROUP_DIM; ++d) mx = fmax_rs(mx, fabsf(v[d]));
        step[g] = mx / 7.0f;
    }
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    for (int d = 0; d < ORA_D_C; ++d) {
        float eff = gl * ((float)gs[d / ORA_GROUP_DIM] / 255.0f);
        put_nibble(out, d, int4_nibble(v[d], eff));
    }
    *global = gl;
}

/* Extension, no reference counterpart: MX group of 32 dims on the same tile
 * layout.  The decoder is unchanged because it indexes gs[d/16] (tile.rs:133). */
void ora_quantize_latent_grouped32(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    for (int g = 0; g < ORA_N_GROUPS; g += 2) {
        float mx = 0.0f;
        for (int d = g * ORA_GROUP_DIM; d < (g + 2) * ORA_GROUP_DIM; ++d) mx = fmax_rs(mx, fabsf(v[d]));
        step[g] = step[g + 1] = mx / 7.0f;
    }
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    for (int d = 0; d < ORA_D_C; ++d) {
        float eff = gl * ((float)gs[d / ORA_GROUP_DIM] / 255.0f);
        put_nibble(out, d, int4_nibble(v[d], eff));
    }
    *global = gl;
}

/* constants.rs:138-141 */
static const float NF4[16] = {-1.0f,   -0.7075f, -0.5421f, -0.4165f, -0.3108f, -0.2158f,
                              -0.1272f, -0.0421f, 0.0421f,  0.1272f,  0.2158f,  0.3108f,
                              0.4165f,  0.5421f,  0.7075f,  1.0f};

/* codec/nf4.rs:7-18: first minimum wins (strict <) */
uint8_t ora_nf4_nearest(float t) {
    int best = 0;
    float best_d = INFINITY;
    for (int i = 0; i < 16; ++i) {
        float dd = fabsf(t - NF4[i]);
        if (dd < best_d) { best_d = dd; best = i; }
    }
    return (uint8_t)best;
}

/* codec/nf4.rs:23-57 */
void ora_quantize_latent_nf4(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    for (int g = 0; g < ORA_N_GROUPS; ++g) {
        float mx = 0.0f;
        for (int d = g * ORA_GROUP_DIM; d < (g + 1) * ORA_GROUP_DIM; ++d) mx = fmax_rs(mx, fabsf(v[d]));
        step[g] = mx;
    }
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    for (int d = 0; d < ORA_D_C; ++d) {
        float eff = gl * ((float)gs[d / ORA_GROUP_DIM] / 255.0f);
        float t = 0.0f;
        if (eff > 0.0f) {
            t = v[d] / eff; /* f32::clamp(-1, 1); NaN stays NaN */
            if (t < -1.0f) t = -1.0f;
            if (t > 1.0f) t = 1.0f;
        }
        put_nibble(out, d, ora_nf4_nearest(t));
    }
    *global = gl;
}

static void head_body_steps(const float* v, float body_div, float* step) {
    /* mixed.rs:15-27 / mix3.rs:13-25: 8-bit head step max/127, 7 body groups */
    float hi = 0.0f;
    for (int d = 0; d < 8; ++d) hi = fmax_rs(hi, fabsf(v[d]));
    step[0] = hi / 127.0f;
    for (int g = 0; g < 7; ++g) {
        float mx = 0.0f;
        for (int d = 8 + g * 16; d < 8 + (g + 1) * 16; ++d) mx = fmax_rs(mx, fabsf(v[d]));
        step[1 + g] = mx / body_div;
    }
}

/* codec/mixed.rs:13-57 */
void ora_quantize_latent_mixed(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    head_body_steps(v, 7.0f, step);
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    float eff_hi = gl * ((float)gs[0] / 255.0f);
    for (int d = 0; d < 8; ++d) {
        int q = clampi(sat_i32(roundf(v[d] / eff_hi)), -128, 127) + 128;
        out[d] = (uint8_t)q;
    }
    for (int ld = 0; ld < 112; ++ld) {
        float eff = gl * ((float)gs[1 + ld / 16] / 255.0f);
        uint8_t nib = int4_nibble(v[8 + ld], eff);
        int byte = 8 + (ld >> 1);
        if ((ld & 1) == 0) out[byte] = (uint8_t)((out[byte] & 0xF0) | nib);
        else out[byte] = (uint8_t)((out[byte] & 0x0F) | (nib << 4));
    }
    *global = gl;
}

static void tq3_put(uint8_t* out, int code_off, int corr_off, int ld, float t) {
    /* tq3.rs:31-46: 3-bit little-endian bit stream + 1-bit correction plane */
    int code = clampi(sat_i32(roundf(t + 3.5f)), 0, 7);
    int bit = 3 * ld, byte = code_off + (bit >> 3), shift = bit & 7;
    out[byte] |= (uint8_t)(code << shift);
    if (shift > 5) out[byte + 1] |= (uint8_t)(code >> (8 - shift));
    float level = (float)code - 3.5f;
    if (t - level > 0.0f) out[corr_off + (ld >> 3)] |= (uint8_t)(1u << (ld & 7));
}

/* codec/tq3.rs:10-49 */
void ora_quantize_latent_tq3(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    for (int g = 0; g < ORA_N_GROUPS; ++g) {
        float mx = 0.0f;
        for (int d = g * 16; d < (g + 1) * 16; ++d) mx = fmax_rs(mx, fabsf(v[d]));
        step[g] = mx / 3.5f;
    }
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    for (int d = 0; d < ORA_D_C; ++d) {
        float eff = gl * ((float)gs[d / 16] / 255.0f);
        tq3_put(out, 0, 48, d, v[d] / eff);
    }
    *global = gl;
}

/* codec/mix3.rs:11-62 */
void ora_quantize_latent_mix3(const float* v, uint8_t* out, float* global, uint8_t* gs) {
    float step[ORA_N_GROUPS];
    head_body_steps(v, 3.5f, step);
    float gl = pick_global(step);
    for (int g = 0; g < ORA_N_GROUPS; ++g) gs[g] = scale_byte(step[g], gl);
    memset(out, 0, ORA_LATENT_BYTES);
    float eff_hi = gl * ((float)gs[0] / 255.0f);
    for (int d = 0; d < 8; ++d) {
        int q = clampi(sat_i32(roundf(v[d] / eff_hi)), -128, 127) + 128;
        out[d] = (uint8_t)q;
    }
    for (int ld = 0; ld < 112; ++ld) {
        float eff = gl * ((float)gs[1 + ld / 16] / 255.0f);
        tq3_put(out, 8, 50, ld, v[8 + ld] / eff);
    }
    *global = gl;
}

/* ------------------------------------------------------------------------
 * tile.rs:133-255  per-codec dequantisation (flag precedence
 * MIXED > TQ3 > MIX3 > NF4 > INT4, tile.rs:141-159)
 * ---------------------------------------------------------------------- */
static float group_scale(const ora_tile* t, int d) {
    return t->scale * ((float)t->group_scales[d / ORA_GROUP_DIM] / 255.0f); /* tile.rs:133-135 */
}
static float alt_scale(const ora_tile* t, int g) {
    /* tile.rs:168,175: `scale * gs as f32 / 255.0` parses as (scale*gs)/255 */
    return t->scale * (float)t->group_scales[g] / 255.0f;
}
static int code3(const uint8_t* lat, int off, int end, int ld) {
    int bit = 3 * ld, byte = off + (bit >> 3), shift = bit & 7;
    unsigned lo = lat[byte];
    unsigned hi = (byte + 1 < end) ? ((unsigned)lat[byte + 1] << 8) : 0u;
    return (int)(((lo | hi) >> shift) & 7u);
}

float ora_dequant_at(const ora_tile* t, int d) {
    const uint8_t* lat = t->latent_kv;
    if (t->flags & ORA_FLAG_MIXED) { /* tile.rs:165-181 */
        if (d < 8) return (float)((int)lat[d] - 128) * alt_scale(t, 0);
        if (d < 120) {
            int ld = d - 8;
            uint8_t b = lat[8 + (ld >> 1)];
            int nib = (ld & 1) ? (b >> 4) : (b & 0x0F);
            return (float)(nib - 8) * alt_scale(t, 1 + ld / 16);
        }
        return 0.0f;
    }
    if (t->flags & ORA_FLAG_TQ3) { /* tile.rs:188-209 */
        float level = (float)code3(lat, 0, 48, d) - 3.5f;
        if (!(t->flags & ORA_FLAG_TQ3_NOCORR)) {
            int corr = (lat[48 + (d >> 3)] >> (d & 7)) & 1;
            level += (corr ? 1.0f : -1.0f) * 0.25f;
        }
        return level * group_scale(t, d);
    }
    if (t->flags & ORA_FLAG_MIX3) { /* tile.rs:218-246 */
        if (d < 8) return (float)((int)lat[d] - 128) * alt_scale(t, 0);
        if (d >= 120) return 0.0f;
        int ld = d - 8;
        float level = (float)code3(lat, 8, 50, ld) - 3.5f;
        if (!(t->flags & ORA_FLAG_TQ3_NOCORR)) {
            int corr = (lat[50 + (ld >> 3)] >> (ld & 7)) & 1;
            level += (corr ? 1.0f : -1.0f) * 0.25f;
        }
        return level * alt_scale(t, 1 + ld / 16);
    }
    uint8_t b = lat[d >> 1];
    int nib = (d & 1) ? (b >> 4) : (b & 0x0F);
    float level = (t->flags & ORA_FLAG_NF4) ? NF4[nib] : (float)(nib - 8);
    return level * group_scale(t, d);
}

void ora_dequant_latent(const ora_tile* t, float* out) {
    for (int d = 0; d < ORA_D_C; ++d) out[d] = ora_dequant_at(t, d);
}

/* simd.rs:1253-1259 */
uint32_t ora_hamming(const uint64_t* a, const uint64_t* b) {
    uint32_t h = 0;
    for (int w = 0; w < ORA_RESIDUAL_WORDS; ++w) h += (uint32_t)__builtin_popcountll(a[w] ^ b[w]);
    return h;
}

/* tile.rs:267-281 (eq. 2.3) with residual_term tile.rs:261-264 */
float ora_compute_score_scalar(const ora_tile* t, const float* q_coarse, const uint64_t* q_sign) {
    float k[ORA_D_C];
    ora_dequant_latent(t, k);
    float coarse = 0.0f;
    for (int d = 0; d < ORA_D_C; ++d) coarse += q_coarse[d] * k[d];
    if (t->flags & ORA_FLAG_WARM) return coarse;
    uint32_t ham = ora_hamming(q_sign, t->residual_bitmap);
    return coarse + t->dynamic_lambda * ((float)ORA_D_S - 2.0f * (float)ham);
}

void ora_score_tiles(const ora_tile* tiles, size_t n, const float* q_coarse,
                     const uint64_t* q_sign, float* out) {
    for (size_t i = 0; i < n; ++i) out[i] = ora_compute_score_scalar(&tiles[i], q_coarse, q_sign);
}

/* slha-c/src/lib.rs:244-286 */
int ora_validate_tile(const ora_tile* t) {
    const unsigned known = 1u | 2u | 4u | 8u | 16u | 32u;
    if (t->flags & ~known) return -6;
    unsigned codec = t->flags & (2u | 4u | 8u | 32u);
    if (__builtin_popcount(codec) > 1) return -6;
    if ((t->flags & 16u) && !(t->flags & (8u | 32u))) return -6;
    if (!isfinite(t->scale) || !isfinite(t->dynamic_lambda) || !isfinite(t->residual_sigma)) return -5;
    if (t->scale < 0.0f || t->dynamic_lambda < 0.0f || t->residual_sigma < 0.0f) return -6;
    return 0;
}
