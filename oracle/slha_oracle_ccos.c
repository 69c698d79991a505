/*
 * CPU oracle (test infrastructure only): deterministic top-k and the CCOS
 * ElasticKvCache state machine (scirust/src/ccos.rs).
 * See slha_oracle.h for the rules that govern this directory.
 */
#include "slha_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* f32::total_cmp as an order-preserving unsigned key */
static uint32_t total_key(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/* ---- top-k ---------------------------------------------------------------
 * Order of scirust/src/metrics.rs:186-192: score descending by total order,
 * ties -> lower index. */
typedef struct { uint32_t key; uint32_t idx; } tk_item;
static int tk_cmp(const void* a, const void* b) {
    const tk_item* x = (const tk_item*)a;
    const tk_item* y = (const tk_item*)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    if (x->idx != y->idx) return x->idx < y->idx ? -1 : 1;
    return 0;
}
void ora_topk(const float* scores, size_t n, size_t k, uint32_t* idx_out, float* score_out) {
    tk_item* it = (tk_item*)malloc(sizeof(tk_item) * (n ? n : 1));
    for (size_t i = 0; i < n; ++i) { it[i].key = total_key(scores[i]); it[i].idx = (uint32_t)i; }
    qsort(it, n, sizeof(tk_item), tk_cmp);
    if (k > n) k = n;
    for (size_t i = 0; i < k; ++i) { idx_out[i] = it[i].idx; score_out[i] = scores[it[i].idx]; }
    free(it);
}

/* ---- ElasticKvCache ------------------------------------------------------ */
struct ora_cache {
    ora_tile* tiles;
    uint8_t* state;
    uint64_t* seq;
    float* importance;
    size_t len, cap;
    size_t* free_list;
    size_t free_len, free_cap;
    size_t budget, live;
    int page_policy, evict_policy;
    uint32_t sink_window;
    uint32_t recent_window; /* extension, 0 = reference behaviour */
    uint64_t next_seq;
    /* what an attached EventLog would receive (ccos.rs:411-420): one (seq, slot, tile) per eviction, in order */
    uint64_t* j_seq;
    uint32_t* j_slot;
    ora_tile* j_tile;
    size_t j_len, j_cap;
};

ora_cache* ora_cache_new(size_t budget, int page_policy, int evict_policy, uint32_t sink_window,
                         uint32_t recent_window) {
    ora_cache* c = (ora_cache*)calloc(1, sizeof(ora_cache));
    c->budget = budget;
    c->page_policy = page_policy;
    c->evict_policy = evict_policy;
    c->sink_window = sink_window;
    c->recent_window = recent_window;
    return c;
}
void ora_cache_free(ora_cache* c) {
    if (!c) return;
    free(c->tiles); free(c->state); free(c->seq); free(c->importance); free(c->free_list);
    free(c->j_seq); free(c->j_slot); free(c->j_tile);
    free(c);
}

static int corr_bytes(const ora_tile* t) { /* tile.rs:118-126 */
    if (t->flags & ORA_FLAG_TQ3) return 16;
    if (t->flags & ORA_FLAG_MIX3) return 14;
    return 0;
}
static size_t slot_live_bytes(const ora_cache* c, size_t s) { /* ccos.rs:468-482 */
    size_t base;
    if (c->state[s] == ORA_HOT) base = 128;
    else if (c->state[s] == ORA_WARM) base = 96;
    else return 0;
    const ora_tile* t = &c->tiles[s];
    return base - ((t->flags & ORA_FLAG_TQ3_NOCORR) ? (size_t)corr_bytes(t) : 0);
}

/* ccos.rs:217-259 */
size_t ora_cache_insert(ora_cache* c, const ora_tile* t) {
    uint8_t st = (t->flags & ORA_FLAG_WARM) ? ORA_WARM : ORA_HOT;
    size_t slot;
    if (c->free_len) {
        slot = c->free_list[--c->free_len]; /* LIFO, ccos.rs:242 */
    } else {
        if (c->len == c->cap) {
            c->cap = c->cap ? c->cap * 2 : 64;
            c->tiles = (ora_tile*)realloc(c->tiles, c->cap * sizeof(ora_tile));
            c->state = (uint8_t*)realloc(c->state, c->cap);
            c->seq = (uint64_t*)realloc(c->seq, c->cap * sizeof(uint64_t));
            c->importance = (float*)realloc(c->importance, c->cap * sizeof(float));
        }
        slot = c->len++;
    }
    c->tiles[slot] = *t;
    c->state[slot] = st;
    c->seq[slot] = c->next_seq++;
    c->importance[slot] = 0.0f;
    c->live += slot_live_bytes(c, slot);
    return slot;
}

size_t ora_cache_len(const ora_cache* c) { return c->len; }
int ora_cache_state(const ora_cache* c, size_t s) { return c->state[s]; }
const ora_tile* ora_cache_tile(const ora_cache* c, size_t s) { return &c->tiles[s]; }
float ora_cache_importance(const ora_cache* c, size_t s) { return c->importance[s]; }
uint64_t ora_cache_seq(const ora_cache* c, size_t s) { return c->seq[s]; }
size_t ora_cache_live_bytes(const ora_cache* c) { return c->live; }
void ora_cache_counts(const ora_cache* c, size_t* hot, size_t* warm, size_t* cold) {
    size_t h = 0, w = 0, k = 0;
    for (size_t s = 0; s < c->len; ++s) {
        if (c->state[s] == ORA_HOT) ++h; else if (c->state[s] == ORA_WARM) ++w; else ++k;
    }
    *hot = h; *warm = w; *cold = k;
}

/* ccos.rs:365-380 */
void ora_cache_page_out(ora_cache* c, size_t s) {
    if (c->state[s] != ORA_HOT) return;
    c->live -= slot_live_bytes(c, s);
    memset(c->tiles[s].residual_bitmap, 0, sizeof(c->tiles[s].residual_bitmap));
    c->tiles[s].dynamic_lambda = 0.0f;
    c->tiles[s].flags |= ORA_FLAG_WARM;
    c->state[s] = ORA_WARM;
    c->live += slot_live_bytes(c, s);
}

/* ccos.rs:386-397 */
int ora_cache_drop_correction(ora_cache* c, size_t s) {
    ora_tile* t = &c->tiles[s];
    int n = corr_bytes(t);
    if (c->state[s] == ORA_COLD || n == 0 || (t->flags & ORA_FLAG_TQ3_NOCORR)) return 0;
    memset(t->latent_kv + ORA_LATENT_BYTES - n, 0, (size_t)n);
    t->flags |= ORA_FLAG_TQ3_NOCORR;
    c->live -= (size_t)n;
    return 1;
}

/* ccos.rs:404-438 with a log that never fails: the record an EventLog would get is journalled */
int ora_cache_evict(ora_cache* c, size_t s) {
    if (s >= c->len || c->state[s] == ORA_COLD) return 0;
    if (c->j_len == c->j_cap) {
        c->j_cap = c->j_cap ? c->j_cap * 2 : 64;
        c->j_seq = (uint64_t*)realloc(c->j_seq, c->j_cap * sizeof(uint64_t));
        c->j_slot = (uint32_t*)realloc(c->j_slot, c->j_cap * sizeof(uint32_t));
        c->j_tile = (ora_tile*)realloc(c->j_tile, c->j_cap * sizeof(ora_tile));
    }
    c->j_seq[c->j_len] = c->seq[s];
    c->j_slot[c->j_len] = (uint32_t)s;
    c->j_tile[c->j_len] = c->tiles[s];
    c->j_len++;
    c->live -= slot_live_bytes(c, s);
    c->state[s] = ORA_COLD;
    if (c->free_len == c->free_cap) {
        c->free_cap = c->free_cap ? c->free_cap * 2 : 64;
        c->free_list = (size_t*)realloc(c->free_list, c->free_cap * sizeof(size_t));
    }
    c->free_list[c->free_len++] = s;
    return 1;
}

/* stable merge sort over slot indices with a context comparator */
typedef int (*slot_cmp)(const ora_cache*, size_t, size_t, uint32_t);
static void msort(const ora_cache* c, size_t* a, size_t* tmp, size_t n, slot_cmp cmp, uint32_t aux) {
    if (n < 2) return;
    size_t h = n / 2;
    msort(c, a, tmp, h, cmp, aux);
    msort(c, a + h, tmp, n - h, cmp, aux);
    size_t i = 0, j = h, k = 0;
    while (i < h && j < n) tmp[k++] = (cmp(c, a[j], a[i], aux) < 0) ? a[j++] : a[i++];
    while (i < h) tmp[k++] = a[i++];
    while (j < n) tmp[k++] = a[j++];
    memcpy(a, tmp, n * sizeof(size_t));
}
static int cmp_sigma(const ora_cache* c, size_t a, size_t b, uint32_t aux) {
    (void)aux;
    uint32_t x = total_key(c->tiles[a].residual_sigma), y = total_key(c->tiles[b].residual_sigma);
    return x < y ? -1 : (x > y ? 1 : 0);
}
static int cmp_seq(const ora_cache* c, size_t a, size_t b, uint32_t aux) {
    (void)aux;
    return c->seq[a] < c->seq[b] ? -1 : (c->seq[a] > c->seq[b] ? 1 : 0);
}
static int is_pinned(const ora_cache* c, size_t s, uint32_t max_pos) {
    /* ccos.rs:592-594: sinks are positions < sink_window.  The recent window
     * (positions within recent_window of the newest live position) is an
     * extension with no reference counterpart; 0 disables it. */
    uint32_t p = c->tiles[s].position;
    if (p < c->sink_window) return 1;
    if (c->recent_window && max_pos - p < c->recent_window) return 1;
    return 0;
}
static int cmp_importance(const ora_cache* c, size_t a, size_t b, uint32_t max_pos) {
    int sa = is_pinned(c, a, max_pos), sb = is_pinned(c, b, max_pos);
    if (sa != sb) return sa < sb ? -1 : 1;
    uint32_t x = total_key(c->importance[a]), y = total_key(c->importance[b]);
    if (x != y) return x < y ? -1 : 1;
    return cmp_seq(c, a, b, 0);
}

/* ccos.rs:526-539 */
static size_t paging_order(const ora_cache* c, int state, size_t* out, size_t* tmp) {
    size_t n = 0;
    for (size_t s = 0; s < c->len; ++s) if (c->state[s] == state) out[n++] = s;
    msort(c, out, tmp, n, c->page_policy == ORA_PAGE_LOWEST_IMPACT ? cmp_sigma : cmp_seq, 0);
    return n;
}

/* ccos.rs:555-614 */
int ora_cache_enforce_budget(ora_cache* c) {
    if (c->live <= c->budget) return 1;
    size_t* ord = (size_t*)malloc(sizeof(size_t) * (c->len + 1));
    size_t* tmp = (size_t*)malloc(sizeof(size_t) * (c->len + 1));
    int ok = 0;
    size_t n = paging_order(c, ORA_HOT, ord, tmp);
    for (size_t i = 0; i < n; ++i) {
        if (c->live <= c->budget) { ok = 1; goto done; }
        ora_cache_drop_correction(c, ord[i]);
    }
    n = paging_order(c, ORA_HOT, ord, tmp);
    for (size_t i = 0; i < n; ++i) {
        if (c->live <= c->budget) { ok = 1; goto done; }
        ora_cache_page_out(c, ord[i]);
    }
    n = paging_order(c, ORA_WARM, ord, tmp);
    for (size_t i = 0; i < n; ++i) {
        if (c->live <= c->budget) { ok = 1; goto done; }
        ora_cache_drop_correction(c, ord[i]);
    }
    n = 0;
    uint32_t max_pos = 0;
    for (size_t s = 0; s < c->len; ++s)
        if (c->state[s] != ORA_COLD) {
            ord[n++] = s;
            if (c->tiles[s].position > max_pos) max_pos = c->tiles[s].position;
        }
    if (c->evict_policy == ORA_EVICT_CAUSAL) msort(c, ord, tmp, n, cmp_seq, 0);
    else msort(c, ord, tmp, n, cmp_importance, max_pos);
    for (size_t i = 0; i < n; ++i) {
        if (c->live <= c->budget) { ok = 1; goto done; }
        ora_cache_evict(c, ord[i]);
    }
    ok = c->live <= c->budget;
done:
    free(ord);
    free(tmp);
    return ok;
}

/* ccos.rs:346-355 */
size_t ora_cache_score_all(const ora_cache* c, const float* q_coarse, const uint64_t* q_sign,
                           uint32_t* slots, float* scores) {
    size_t n = 0;
    for (size_t s = 0; s < c->len; ++s) {
        if (c->state[s] == ORA_COLD) continue;
        slots[n] = (uint32_t)s;
        scores[n] = ora_compute_score_scalar(&c->tiles[s], q_coarse, q_sign);
        ++n;
    }
    return n;
}

/* ccos.rs:275-314 */
void ora_cache_observe_scores(ora_cache* c, const uint32_t* slots, const float* scores, size_t n,
                              float temperature) {
    if (n == 0 || !isfinite(temperature) || temperature <= 0.0f) return;
    size_t m = 0;
    size_t* ls = (size_t*)malloc(sizeof(size_t) * n);
    float* sc = (float*)malloc(sizeof(float) * n);
    for (size_t i = 0; i < n; ++i) {
        if (slots[i] < c->len && c->state[slots[i]] != ORA_COLD) { ls[m] = slots[i]; sc[m] = scores[i]; ++m; }
    }
    int bad = (m == 0);
    for (size_t i = 0; i < m && !bad; ++i) if (!isfinite(sc[i])) bad = 1;
    if (!bad) {
        float mx = -INFINITY;
        for (size_t i = 0; i < m; ++i) if (sc[i] > mx) mx = sc[i];
        float sum = 0.0f;
        for (size_t i = 0; i < m; ++i) { sc[i] = expf((sc[i] - mx) / temperature); sum += sc[i]; }
        if (isfinite(sum) && sum > 0.0f) {
            float inv = 1.0f / sum;
            for (size_t i = 0; i < m; ++i) c->importance[ls[i]] += sc[i] * inv;
        }
    }
    free(ls);
    free(sc);
}

size_t ora_cache_journal_len(const ora_cache* c) { return c->j_len; }
void ora_cache_journal_get(const ora_cache* c, size_t i, uint64_t* seq, uint32_t* slot, ora_tile* tile) {
    *seq = c->j_seq[i];
    *slot = c->j_slot[i];
    *tile = c->j_tile[i];
}

size_t ora_cache_nocorr_count(const ora_cache* c) {
    size_t n = 0;
    for (size_t s = 0; s < c->len; ++s)
        if (c->state[s] != ORA_COLD && (c->tiles[s].flags & ORA_FLAG_TQ3_NOCORR)) ++n;
    return n;
}
size_t ora_cache_reclaimed_correction_bytes(const ora_cache* c) {
    size_t n = 0;
    for (size_t s = 0; s < c->len; ++s)
        if (c->state[s] != ORA_COLD && (c->tiles[s].flags & ORA_FLAG_TQ3_NOCORR)) n += (size_t)corr_bytes(&c->tiles[s]);
    return n;
}
