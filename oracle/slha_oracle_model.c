/*
 * CPU oracle (test infrastructure only): the learned-projection model --
 * latent, reconstruct, randomised Hadamard transform, sign-LSH bits, tile
 * assembly, query preparation, `.slhw` parsing and the scenario encoder.
 * See slha_oracle.h for the rules that govern this directory.
 */
#include "slha_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

struct ora_model {
    size_t d, d_pad;
    float* evec;  /* D_C x d, row-major */
    float scale[ORA_D_C];
    float* z;     /* D_S x d_pad */
    float* diag;  /* d_pad, +-1, NULL when no RHT */
};

/* incoherence.rs:29-35 */
size_t ora_next_pow2(size_t n) {
    size_t p = 1;
    while (p < n) p <<= 1;
    return p;
}

/* incoherence.rs:45-70: butterflies h = 1,2,4..., then multiply by 1/sqrt(n) */
void ora_fwht_inplace(float* v, size_t n) {
    for (size_t h = 1; h < n; h <<= 1) {
        for (size_t i = 0; i < n; i += h << 1) {
            for (size_t j = i; j < i + h; ++j) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
        }
    }
    float inv = 1.0f / sqrtf((float)n); /* `.sqrt().recip()` */
    for (size_t i = 0; i < n; ++i) v[i] *= inv;
}

/* learned.rs:204-238 (try_from_projection_with) + incoherence.rs:89-97 */
ora_model* ora_model_from_projection(const float* p, size_t d, uint64_t seed, int rht) {
    ora_model* m = (ora_model*)calloc(1, sizeof(ora_model));
    m->d = d;
    m->d_pad = rht ? ora_next_pow2(d) : d;
    m->evec = (float*)malloc(sizeof(float) * ORA_D_C * d);
    memcpy(m->evec, p, sizeof(float) * ORA_D_C * d);
    for (int k = 0; k < ORA_D_C; ++k) m->scale[k] = 1.0f;
    if (rht) {
        ora_rng r;
        ora_rng_init(&r, seed ^ 0xA2A2A2A2A2A2A2A2ull); /* learned.rs:158-165 */
        m->diag = (float*)malloc(sizeof(float) * m->d_pad);
        for (size_t i = 0; i < m->d_pad; ++i) m->diag[i] = ora_rng_next_unit(&r) < 0.5f ? -1.0f : 1.0f;
    }
    ora_rng r;
    ora_rng_init(&r, seed);
    m->z = (float*)malloc(sizeof(float) * ORA_D_S * m->d_pad);
    ora_rng_fill_gaussian(&r, m->z, (size_t)ORA_D_S * m->d_pad);
    return m;
}

void ora_model_set_scale(ora_model* m, const float* s) { memcpy(m->scale, s, sizeof(m->scale)); }
void ora_model_set_z(ora_model* m, const float* z) {
    memcpy(m->z, z, sizeof(float) * ORA_D_S * m->d_pad);
}
void ora_model_free(ora_model* m) {
    if (!m) return;
    free(m->evec);
    free(m->z);
    free(m->diag);
    free(m);
}
size_t ora_model_d(const ora_model* m) { return m->d; }
size_t ora_model_d_pad(const ora_model* m) { return m->d_pad; }
const float* ora_model_z(const ora_model* m) { return m->z; }
const float* ora_model_rht_diag(const ora_model* m) { return m->diag; }

/* learned.rs:247-254 */
static float evec_dot(const ora_model* m, int k, const float* v) {
    const float* row = m->evec + (size_t)k * m->d;
    float acc = 0.0f;
    for (size_t i = 0; i < m->d; ++i) acc += row[i] * v[i];
    return acc;
}

/* learned.rs:257-263 */
void ora_model_latent(const ora_model* m, const float* key, float* h) {
    for (int k = 0; k < ORA_D_C; ++k) h[k] = evec_dot(m, k, key) / m->scale[k];
}

/* learned.rs:267-273 */
void ora_model_query_coarse(const ora_model* m, const float* q, float* out) {
    for (int k = 0; k < ORA_D_C; ++k) out[k] = evec_dot(m, k, q) * m->scale[k];
}

/* learned.rs:276-286: k outer, i inner, sequential accumulation into r[i] */
void ora_model_reconstruct(const ora_model* m, const float* h, float* r) {
    for (size_t i = 0; i < m->d; ++i) r[i] = 0.0f;
    for (int k = 0; k < ORA_D_C; ++k) {
        float w = h[k] * m->scale[k];
        const float* row = m->evec + (size_t)k * m->d;
        for (size_t i = 0; i < m->d; ++i) r[i] += w * row[i];
    }
}

/* learned.rs:326-347 with incoherence.rs:110-125 */
void ora_model_sign_bits(const ora_model* m, const float* v, uint64_t* out) {
    float* buf = (float*)malloc(sizeof(float) * m->d_pad);
    if (m->diag) {
        memcpy(buf, v, sizeof(float) * m->d);
        for (size_t i = m->d; i < m->d_pad; ++i) buf[i] = 0.0f;
        for (size_t i = 0; i < m->d_pad; ++i) buf[i] *= m->diag[i];
        ora_fwht_inplace(buf, m->d_pad);
    } else {
        memcpy(buf, v, sizeof(float) * m->d);
    }
    for (int w = 0; w < ORA_RESIDUAL_WORDS; ++w) out[w] = 0;
    for (int s = 0; s < ORA_D_S; ++s) {
        const float* row = m->z + (size_t)s * m->d_pad;
        float acc = 0.0f;
        for (size_t i = 0; i < m->d_pad; ++i) acc += row[i] * buf[i];
        if (acc < 0.0f) out[s >> 6] |= 1ull << (s & 63);
    }
    free(buf);
}

float ora_analytic_lambda_c(void) {
    /* scenario.rs:30-32 / learned.rs:394: sqrt(PI / (2 * 256)) in f32 */
    return sqrtf(3.14159265358979323846f / (2.0f * (float)ORA_D_S));
}

/* learned.rs:353-408 (encode_with).  codec 6 = grouped32 extension. */
int ora_model_encode(const ora_model* m, const float* key, uint32_t pos, int warm, int codec,
                     ora_tile* out) {
    float h[ORA_D_C];
    ora_tile t;
    memset(&t, 0, sizeof(t));
    ora_model_latent(m, key, h);
    uint16_t cflag = 0;
    switch (codec) {
        case 0:
            ora_quantize_latent(h, t.latent_kv, &t.scale);
            memset(t.group_scales, 255, ORA_N_GROUPS);
            break;
        case 1: ora_quantize_latent_grouped(h, t.latent_kv, &t.scale, t.group_scales); break;
        case 2: ora_quantize_latent_nf4(h, t.latent_kv, &t.scale, t.group_scales); cflag = ORA_FLAG_NF4; break;
        case 3: ora_quantize_latent_mixed(h, t.latent_kv, &t.scale, t.group_scales); cflag = ORA_FLAG_MIXED; break;
        case 4: ora_quantize_latent_tq3(h, t.latent_kv, &t.scale, t.group_scales); cflag = ORA_FLAG_TQ3; break;
        case 5: ora_quantize_latent_mix3(h, t.latent_kv, &t.scale, t.group_scales); cflag = ORA_FLAG_MIX3; break;
        case 6: ora_quantize_latent_grouped32(h, t.latent_kv, &t.scale, t.group_scales); break;
        default: return -4;
    }
    float* recon = (float*)malloc(sizeof(float) * m->d);
    float* e = (float*)malloc(sizeof(float) * m->d);
    ora_model_reconstruct(m, h, recon);
    for (size_t i = 0; i < m->d; ++i) e[i] = key[i] - recon[i];
    ora_model_sign_bits(m, e, t.residual_bitmap);
    float ss = 0.0f; /* learned.rs:393: f32 sequential sum, / d, sqrt */
    for (size_t i = 0; i < m->d; ++i) ss += e[i] * e[i];
    float sigma = sqrtf(ss / (float)m->d);
    t.residual_sigma = sigma;
    t.dynamic_lambda = sigma * ora_analytic_lambda_c();
    t.token_id = pos;
    t.position = pos;
    t.head_id = 0;
    t.flags = (uint16_t)((warm ? ORA_FLAG_WARM : 0u) | cflag);
    free(recon);
    free(e);
    *out = t;
    return 0;
}

/* Batched form used by the parity tests: per-key position and head id (the
 * head id is written after encoding; the reference always writes 0,
 * learned.rs:404). */
void ora_model_encode_batch(const ora_model* m, const float* keys, size_t n, const uint32_t* pos,
                            const uint16_t* head, int codec, ora_tile* out) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
        ora_model_encode(m, keys + (size_t)i * m->d, pos ? pos[i] : (uint32_t)i, 0, codec, &out[i]);
        if (head) out[i].head_id = head[i];
    }
}

/* slha-c/src/lib.rs:420-463 */
void ora_model_prepare_query(const ora_model* m, const float* q, float* q_coarse, uint64_t* q_sign) {
    ora_model_query_coarse(m, q, q_coarse);
    ora_model_sign_bits(m, q, q_sign);
}

/* slha-c/src/lib.rs:773-823: dequantise, reconstruct */
void ora_model_decode_latent(const ora_model* m, const ora_tile* t, float* out) {
    float k[ORA_D_C];
    ora_dequant_latent(t, k);
    ora_model_reconstruct(m, k, out);
}

/* learned.rs:290-322 (reconstruct_from_tile) */
void ora_model_decode_key(const ora_model* m, const ora_tile* t, float* out) {
    ora_model_decode_latent(m, t, out);
    if (m->diag) return;
    float sc = t->residual_sigma * sqrtf(3.14159265358979323846f / 2.0f) / (float)ORA_D_S;
    for (int s = 0; s < ORA_D_S; ++s) {
        float sign = ((t->residual_bitmap[s >> 6] >> (s & 63)) & 1ull) ? -1.0f : 1.0f;
        const float* row = m->z + (size_t)s * m->d_pad;
        for (size_t i = 0; i < m->d; ++i) out[i] += sign * sc * row[i];
    }
}

/* weights.rs:68-80 */
uint32_t ora_weights_checksum(const uint8_t* hdr24, const uint8_t* payload, size_t n) {
    uint32_t h = 0x811C9DC5u;
    for (size_t i = 0; i < 24; ++i) { h ^= hdr24[i]; h *= 0x01000193u; }
    for (size_t i = 0; i < n; ++i) { h ^= payload[i]; h *= 0x01000193u; }
    return h;
}

static uint32_t rd32(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/* weights.rs:159-270 */
ora_model* ora_weights_from_bytes(const uint8_t* b, size_t len, char* err, size_t errlen) {
#define FAIL(...) do { snprintf(err, errlen, __VA_ARGS__); return NULL; } while (0)
    if (len < 24) FAIL("weights: truncated header");
    if (rd32(b) != 0x534C4857u) FAIL("weights: bad magic (not an SLHW file)");
    uint32_t version = rd32(b + 4);
    size_t header;
    if (version == 1) header = 24;
    else if (version == 2) header = 28;
    else FAIL("weights: unsupported version %u (supported: 1 and 2)", version);
    if (len < header) FAIL("weights: truncated header");
    size_t d = rd32(b + 8);
    if (d <= ORA_D_C) FAIL("weights: invalid dimension %zu (must be greater than D_C=128)", d);
    uint64_t seed = 0;
    for (int i = 0; i < 8; ++i) seed |= (uint64_t)b[12 + i] << (8 * i);
    if (b[20] > 1) FAIL("weights: invalid RHT flag %u (expected 0 or 1)", b[20]);
    int rht = b[20];
    if (b[21] || b[22] || b[23]) FAIL("weights: non-zero reserved header bytes");
    size_t expected = header + (size_t)ORA_D_C * d * 4;
    if (len != expected) FAIL("weights: size mismatch (got %zu, expected %zu)", len, expected);
    if (version == 2) {
        uint32_t stored = rd32(b + 24);
        uint32_t calc = ora_weights_checksum(b, b + 28, len - 28);
        if (stored != calc) FAIL("weights: checksum mismatch (stored %#010x, calculated %#010x)", stored, calc);
    }
    size_t n = (size_t)ORA_D_C * d;
    float* p = (float*)malloc(sizeof(float) * n);
    for (size_t i = 0; i < n; ++i) {
        uint32_t u = rd32(b + header + 4 * i);
        memcpy(&p[i], &u, 4);
        if (!isfinite(p[i])) { free(p); FAIL("weights: non-finite projection value at index %zu", i); }
    }
    ora_model* m = ora_model_from_projection(p, d, seed, rht);
    free(p);
    return m;
#undef FAIL
}

/* metrics.rs:207-225: f64 accumulation */
double ora_rms(const float* v, size_t n) {
    if (n == 0) return 0.0;
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += (double)v[i] * (double)v[i];
    return sqrt(s / (double)n);
}

/* scenario.rs:70-83 */
void ora_scenario_sign_bits(const float* z, const float* v, uint64_t* out) {
    for (int w = 0; w < ORA_RESIDUAL_WORDS; ++w) out[w] = 0;
    for (int s = 0; s < ORA_D_S; ++s) {
        const float* row = z + (size_t)s * ORA_D_C;
        float acc = 0.0f;
        for (int k = 0; k < ORA_D_C; ++k) acc += row[k] * v[k];
        if (acc < 0.0f) out[s >> 6] |= 1ull << (s & 63);
    }
}

/* scenario.rs:95-114 */
void ora_scenario_build_tile(const float* z, const float* k_coarse, const float* e, uint32_t pos,
                             int warm, ora_tile* out) {
    ora_tile t;
    memset(&t, 0, sizeof(t));
    ora_quantize_latent_grouped(k_coarse, t.latent_kv, &t.scale, t.group_scales);
    ora_scenario_sign_bits(z, e, t.residual_bitmap);
    float sigma = (float)ora_rms(e, ORA_D_C);
    t.residual_sigma = sigma;
    t.dynamic_lambda = sigma * ora_analytic_lambda_c();
    t.token_id = pos;
    t.position = pos;
    t.flags = warm ? ORA_FLAG_WARM : 0;
    *out = t;
}
