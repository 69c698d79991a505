// Eq. 2.3 tile scoring and deterministic top-k for sm_100a.
//
// Math restated from scirust/src/attention/slha_v2/tile.rs:133-281
// (per-codec dequantisation, compute_score_scalar): score = sum_d q[d]*k[d]
// (+ lambda * (256 - 2*hamming(q_sign, residual)) unless the tile is WARM).
//
// Mapping: eight lanes share one 128-byte tile.  Every lane copies one 16-byte
// chunk with cp.async (a warp instruction moves four whole tiles, 512
// contiguous bytes), the chunks land XOR-swizzled in a per-warp shared-memory
// ring, and lane s then decodes "unit" s of the tile: the 16 latent dims that
// share scale byte group_scales[s] (8 dims for the 8-bit head of the mixed
// layouts) and residual word s.  Query dims for the unit live in registers.
// Partial sums of eight consecutive iterations are combined with a transposed
// butterfly (7 shuffles per query per 32 tiles) so that lane s ends up owning
// the finished scores of one tile.  Scores either go to memory (full mode) or
// straight into a per-CTA streaming top-k (threshold filter + radix reselect in
// shared memory); full score vectors are never written in top-k mode.
#include <cuda_fp16.h>

#include <cfloat>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace slha {
namespace {

constexpr int ITER = 8;        // 4-tile iterations per warp block
constexpr int BLK_TILES = 32;  // tiles per warp block
constexpr int DEPTH = 2;       // cp.async ring depth (blocks per warp)
constexpr int ITER_BYTES = 512;
constexpr int BLK_BYTES = ITER * ITER_BYTES;

__device__ __forceinline__ uint32_t score_key(float f) {
    // order-preserving map of f32 total order (Rust f32::total_cmp) onto u32
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_score(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
__device__ __forceinline__ uint64_t make_comp(float score, uint32_t idx) {
    // larger is better; ties on score resolve towards the lower index
    return ((uint64_t)score_key(score) << 32) | (uint64_t)(0xFFFFFFFFu - idx);
}

// byte offset inside one iteration's 512-byte stage area: tile t (0..3), tile
// byte `b`.  16-byte chunks of odd tiles are XOR-ed with 4 so that the two tiles
// of a half-warp occupy disjoint banks for 8-byte latent reads.
__device__ __forceinline__ uint32_t stage_off(int t, int b) {
    int c = b >> 4;
    return (uint32_t)((((t << 3) + (c ^ ((t & 1) << 2))) << 4) + (b & 15));
}
__device__ __forceinline__ uint32_t lds32(const unsigned char* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}
__device__ __forceinline__ uint2 lds64(const unsigned char* p) {
    return *reinterpret_cast<const uint2*>(p);
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
    uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// NF4 codebook, scirust/src/attention/slha_v2/constants.rs:138-141
__constant__ float c_nf4[16] = {-1.0f,   -0.7075f, -0.5421f, -0.4165f, -0.3108f, -0.2158f,
                                -0.1272f, -0.0421f, 0.0421f,  0.1272f,  0.2158f,  0.3108f,
                                0.4165f,  0.5421f,  0.7075f,  1.0f};

// 48 code bits of a 16-dim TQ3 unit starting at tile byte `b` (b is even).
__device__ __forceinline__ uint64_t load_codes48(const unsigned char* st, int t, int b) {
    int a0 = b & ~3;
    uint64_t w = (uint64_t)lds32(st + stage_off(t, a0)) | ((uint64_t)lds32(st + stage_off(t, a0 + 4)) << 32);
    return w >> ((b & 3) * 8);
}
__device__ __forceinline__ uint32_t load_u16(const unsigned char* st, int t, int b) {
    return (lds32(st + stage_off(t, b & ~3)) >> ((b & 3) * 8)) & 0xFFFFu;
}

// Partial scores of one tile for lane (t, s): unit s of the latent against the
// G queries, plus this lane's share of the Hamming term (residual word s).
//   qreg : query dims 16s..16s+15 for aligned-unit codecs (INT4, NF4, TQ3)
//   qsm  : all 128 dims per query in shared memory (head+body codecs)
//   lut  : NF4 codebook replicated per bank, lut[nib*32 + lane]
template <int G>
__device__ __forceinline__ void tile_partial(const unsigned char* st, int t, int s, int lane,
                                             const float (&qreg)[G][16], const uint32_t (&qs)[G],
                                             const float* qsm, const float* lut, float (&out)[G]) {
    uint32_t flags = lds32(st + stage_off(t, 116)) >> 16;
    // precedence of dequant_at (tile.rs:141-151) for tiles that carry several codec flags: mixed, then TQ3, then MIX3
    if ((flags & F_TQ3) && !(flags & F_MIXED)) flags &= ~(uint32_t)F_MIX3;
    const float scale = __uint_as_float(lds32(st + stage_off(t, 96)));
    const float lam = (flags & F_WARM) ? 0.0f : __uint_as_float(lds32(st + stage_off(t, 100)));
    const float gsb = (float)((lds32(st + stage_off(t, 120 + (s & 4))) >> ((s & 3) * 8)) & 0xFFu);
    const uint32_t rw = lds32(st + stage_off(t, 64 + 4 * s));
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = 0.0f;
    float eff;
    if (!(flags & (F_MIXED | F_MIX3))) {
        eff = scale * (gsb / 255.0f);  // tile.rs:133-135
        if (flags & F_TQ3) {           // tile.rs:188-209
            const uint64_t codes = load_codes48(st, t, 6 * s);
            const uint32_t corr = load_u16(st, t, 48 + 2 * s);
            const bool nocorr = (flags & F_NOCORR) != 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float level = (float)(int)((codes >> (3 * j)) & 7u);
                level += nocorr ? -3.5f : (((corr >> j) & 1u) ? -3.25f : -3.75f);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = fmaf(level, qreg[g][j], acc[g]);
            }
        } else {
            const uint2 w = lds64(st + stage_off(t, 8 * s));
            const bool nf4 = (flags & F_NF4) != 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t nib = ((j < 8 ? w.x : w.y) >> (4 * (j & 7))) & 15u;
                const float level = nf4 ? lut[nib * 32 + lane] : (float)((int)nib - 8);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = fmaf(level, qreg[g][j], acc[g]);
            }
        }
    } else {
        // head+body layouts (tile.rs:165-181, :218-246): unit 0 = eight signed
        // bytes, units 1..7 = 16 body dims starting at dim 16*s-8, tail dropped.
        eff = scale * gsb / 255.0f;
        if (s == 0) {
            const uint2 w = lds64(st + stage_off(t, 0));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float level = (float)((int)(((j < 4 ? w.x : w.y) >> (8 * (j & 3))) & 0xFFu) - 128);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = fmaf(level, qsm[g * D_C + j], acc[g]);
            }
        } else {
            const float* qb = qsm + 16 * s - 8;
            if (flags & F_MIXED) {
                const uint2 w = lds64(st + stage_off(t, 8 * s));
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float level = (float)((int)(((j < 8 ? w.x : w.y) >> (4 * (j & 7))) & 15u) - 8);
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g] = fmaf(level, qb[g * D_C + j], acc[g]);
                }
            } else {
                const uint64_t codes = load_codes48(st, t, 6 * s + 2);
                const uint32_t corr = load_u16(st, t, 48 + 2 * s);
                const bool nocorr = (flags & F_NOCORR) != 0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float level = (float)(int)((codes >> (3 * j)) & 7u);
                    level += nocorr ? -3.5f : (((corr >> j) & 1u) ? -3.25f : -3.75f);
#pragma unroll
                    for (int g = 0; g < G; ++g) acc[g] = fmaf(level, qb[g * D_C + j], acc[g]);
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
        out[g] = fmaf(acc[g], eff, lam * (float)(32 - 2 * __popc(rw ^ qs[g])));
}

// Combine v[0..7] (one value per iteration) across the 8 lanes of a tile group
// so that lane s keeps the total of iteration s.  7 shuffles.
__device__ __forceinline__ float transpose_reduce8(const float (&v)[ITER], int s) {
    float w[4], x[2];
    const bool h4 = (s & 4) != 0, h2 = (s & 2) != 0, h1 = (s & 1) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = h4 ? v[i] : v[i + 4];
        const float keep = h4 ? v[i + 4] : v[i];
        w[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 4);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = h2 ? w[i] : w[i + 2];
        const float keep = h2 ? w[i + 2] : w[i];
        x[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 2);
    }
    const float send = h1 ? x[0] : x[1];
    const float keep = h1 ? x[1] : x[0];
    return keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
}

// ---- block-wide exact selection of the k largest 64-bit keys ---------------
// hist: 260 ints of shared memory.  On return keys[0..k) hold the winners
// (unordered), *cnt_p == k and *pivot_p is a value such that exactly the
// winners are >= pivot.  All threads of the block must call.
__device__ void block_select_topk(uint64_t* keys, int* cnt_p, uint32_t k, uint64_t* pivot_p,
                                  int* hist) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int cnt = *cnt_p;
    uint64_t prefix = 0;
    uint32_t need = k;
    int shift = 56;
    for (;; shift -= 8) {
        for (int b = tid; b < 256; b += nt) hist[b] = 0;
        __syncthreads();
        for (int i = tid; i < cnt; i += nt) {
            const uint64_t key = keys[i];
            if (shift == 56 || (key >> (shift + 8)) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid < 32) {
            // lane l owns bins 255-8l .. 248-8l (descending)
            int c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * tid - j]; tot += c[j]; }
            int incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (tid >= o) incl += y;
            }
            const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= (int)need);
            if (tid == __ffs(ok) - 1) {
                int run = incl - tot;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (run + c[j] >= (int)need) {
                        hist[256] = 255 - 8 * tid - j;
                        hist[257] = run;
                        hist[258] = c[j];
                        break;
                    }
                    run += c[j];
                }
            }
        }
        __syncthreads();
        const int digit = hist[256], above = hist[257], binc = hist[258];
        __syncthreads();
        need -= (uint32_t)above;
        prefix = (prefix << 8) | (uint64_t)digit;
        if ((uint32_t)binc == need || shift == 0) break;  // whole bin wins / key exhausted
    }
    const uint64_t pivot = prefix << shift;
    if (tid == 0) hist[259] = 0;
    __syncthreads();
    for (int base = 0; base < cnt; base += nt) {
        const int i = base + tid;
        const uint64_t key = i < cnt ? keys[i] : 0;
        const bool keep = i < cnt && key >= pivot;
        __syncthreads();
        if (keep) keys[atomicAdd(&hist[259], 1)] = key;
        __syncthreads();
    }
    if (tid == 0) {
        *cnt_p = hist[259];
        *pivot_p = pivot;
    }
    __syncthreads();
}

// One unit of scoring work: a run of tiles of one segment against <= G queries.
struct WorkItem {
    uint64_t tile_begin;   // first tile (index into the tile array)
    uint32_t n_tiles;
    uint32_t index_base;   // reported index of the first tile
    uint32_t query_begin;  // first query row
    uint32_t n_queries;    // 1..G
    uint32_t list_begin;   // candidate list of query 0 of this item; +1 per query
    uint32_t pad;
};

struct ScoreArgs {
    const unsigned char* tiles;
    const uint8_t* state;  // optional per-tile CCOS state (COLD tiles are skipped)
    const WorkItem* items;
    const WorkItem* stream_items;  // score_stream_kernel: item i as that kernel walks it (interleaved chunks of a stream, or items[i] itself)
    const float* q_coarse;    // [nq][128]
    const uint32_t* q_sign;   // [nq][8]
    // full mode
    float* scores;            // [nq][score_stride]
    uint64_t score_stride;
    const unsigned long long* row_offset;  // optional (full-score mode): row q starts at scores + row_offset[q] instead of q * score_stride
    uint32_t row_len;         // with row_offset: work items marked as the last of their segment fill the row's elements
    float row_fill;           //   [index_base + n_tiles, row_len) with row_fill
    // top-k mode
    uint32_t k, cap;
    uint32_t list_cap;        // slots per candidate list (>= k)
    uint64_t* cand_keys;      // [n_lists][list_cap]
    uint32_t* cand_cnt;       // [n_lists]
    // implicit work decomposition (items == nullptr): every CTA takes
    // `item_tiles` consecutive tiles of one array against the launch's queries
    uint64_t total_tiles;
    uint32_t item_tiles, nq_launch;
    uint32_t n_items;
    const uint32_t* cta_begin;    // tensor-core kernel: item range of every persistent CTA
    unsigned long long* gpivot;   // tensor-core kernel: per query row, shared selection threshold
    unsigned long long* grange;   // per query row: bucket mapping of the shared score histogram (0 = none yet)
    uint32_t* ghist;              // per query row: 256 bucket counts of appended candidates
    uint32_t* gcount;             // per query row: candidates appended to the row's buffer
    uint32_t* gflag;              // per query row: 1 = the generic kernel scores the row's work items
    uint64_t* gbuf;               // per query row: gcap composite keys
    uint32_t gcap;
    uint32_t nf4_table;           // tensor-core kernel: build the NF4 shared-memory table (else NF4 tiles are handed back)
    uint32_t mixed;               // tensor-core kernel: query fragments arranged for mixed 8/4 tiles (other tiles are handed back)
};

template <int G, bool TOPK>
__global__ void __launch_bounds__(256) score_kernel(ScoreArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int t = lane >> 3, s = lane & 7;
    WorkItem it;
    if (a.items) {
        it = a.items[blockIdx.x];
        if (a.gflag) {  // launched behind the tensor-core kernel: only work items one of whose rows it handed back
            uint32_t f = 0;
            for (uint32_t g = 0; g < it.n_queries; ++g) f |= a.gflag[it.query_begin + g];
            if (!f) return;
        }
    } else {
        it.tile_begin = (uint64_t)blockIdx.x * a.item_tiles;
        it.n_tiles = (uint32_t)min((uint64_t)a.item_tiles, a.total_tiles - it.tile_begin);
        it.index_base = (uint32_t)it.tile_begin;
        it.query_begin = 0;
        it.n_queries = a.nq_launch;
        it.list_begin = 0;
    }

    // shared layout: q (G*128 f32) | nf4 lut (16*32 f32) | stage ring | [top-k state]
    float* qsm = reinterpret_cast<float*>(smem);
    float* lut = qsm + G * D_C;
    unsigned char* stage = reinterpret_cast<unsigned char*>(lut + 16 * 32) + (size_t)warp * DEPTH * BLK_BYTES;
    unsigned char* tail = reinterpret_cast<unsigned char*>(lut + 16 * 32) + (size_t)nwarps * DEPTH * BLK_BYTES;
    uint64_t* keys = reinterpret_cast<uint64_t*>(tail);                       // [G][cap]
    uint64_t* pivot = keys + (TOPK ? (size_t)G * a.cap : 0);                  // [G]
    int* cnt = reinterpret_cast<int*>(pivot + G);                             // [G]
    int* hist = cnt + G;                                                      // 260

    for (int i = tid; i < G * D_C; i += blockDim.x) {
        const int g = i / D_C;
        qsm[i] = g < (int)it.n_queries ? a.q_coarse[(size_t)(it.query_begin + g) * D_C + (i % D_C)] : 0.0f;
    }
    for (int i = tid; i < 16 * 32; i += blockDim.x) lut[i] = c_nf4[i >> 5];
    if (TOPK && tid < G) { cnt[tid] = 0; pivot[tid] = 0; }
    __syncthreads();

    float qreg[G][16];
    uint32_t qs[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int j = 0; j < 16; ++j) qreg[g][j] = qsm[g * D_C + 16 * s + j];
        qs[g] = g < (int)it.n_queries ? a.q_sign[(size_t)(it.query_begin + g) * 8 + s] : 0u;
    }

    const unsigned char* tbase = a.tiles + it.tile_begin * TILE_BYTES;
    const uint8_t* sbase = a.state ? a.state + it.tile_begin : nullptr;
    const uint32_t n = it.n_tiles;
    const uint32_t n_blocks = (n + BLK_TILES - 1) / BLK_TILES;
    const uint32_t n_rounds = (n_blocks + nwarps - 1) / nwarps;

    auto issue = [&](uint32_t blk, int slot, uint32_t& st_lane) {
        // st_lane: CCOS state byte of tile blk*32+lane (HOT when there is no state array)
        st_lane = ST_HOT;
        if (blk < n_blocks) {
            const uint32_t my = blk * BLK_TILES + lane;
            if (sbase && my < n) st_lane = sbase[my];
            unsigned char* dst = stage + slot * BLK_BYTES;
#pragma unroll
            for (int i = 0; i < ITER; ++i) {
                const uint32_t ti = blk * BLK_TILES + i * 4 + t;
                const uint32_t stt = __shfl_sync(0xFFFFFFFFu, st_lane, i * 4 + t);
                const bool live = ti < n && stt != ST_COLD;
                const unsigned char* src = tbase + (size_t)(live ? ti : 0) * TILE_BYTES + s * 16;
                cp_async16(dst + i * ITER_BYTES + stage_off(t, s * 16), src, live ? 16 : 0);
            }
        }
        cp_async_commit();
    };

    uint32_t st_cur = ST_HOT, st_next = ST_HOT;
    issue(warp, 0, st_cur);
    for (uint32_t r = 0; r < n_rounds; ++r) {
        const uint32_t blk = r * nwarps + warp;
        issue((r + 1) * nwarps + warp, (r + 1) & 1, st_next);
        cp_async_wait<1>();
        __syncwarp();
        if (blk < n_blocks) {
            const unsigned char* src = stage + (r & 1) * BLK_BYTES;
            float part[G][ITER];
#pragma unroll
            for (int i = 0; i < ITER; ++i) {
                float o[G];
                tile_partial<G>(src + i * ITER_BYTES, t, s, lane, qreg, qs, qsm, lut, o);
#pragma unroll
                for (int g = 0; g < G; ++g) part[g][i] = o[g];
            }
            // lane s now finishes tile blk*32 + 4*s + t
            const uint32_t ti = blk * BLK_TILES + 4 * s + t;
            const uint32_t stt = __shfl_sync(0xFFFFFFFFu, st_cur, 4 * s + t);
            const bool live = ti < n && stt != ST_COLD;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float sc = transpose_reduce8(part[g], s);
                if (g < (int)it.n_queries) {
                    if (TOPK) {
                        if (live) {
                            const uint64_t comp = make_comp(sc, it.index_base + ti);
                            if (comp >= pivot[g]) keys[(size_t)g * a.cap + atomicAdd(&cnt[g], 1)] = comp;
                        }
                    } else if (ti < n) {
                        const size_t row0 = a.row_offset ? (size_t)a.row_offset[it.query_begin + g] : (size_t)(it.query_begin + g) * a.score_stride;
                        a.scores[row0 + it.index_base + ti] = live ? sc : -INFINITY;
                    }
                }
            }
        }
        __syncwarp();
        st_cur = st_next;
        if (TOPK) {
            // keep room for one more round of appends (<= nwarps*32 per query)
            // (snapshot the counters between two barriers so that every thread
            // takes the same decision before anyone appends again)
            __syncthreads();
            int snap[G];
#pragma unroll
            for (int g = 0; g < G; ++g) snap[g] = cnt[g];
            __syncthreads();
#pragma unroll
            for (int g = 0; g < G; ++g)
                if (g < (int)it.n_queries && snap[g] + nwarps * BLK_TILES > (int)a.cap)
                    block_select_topk(keys + (size_t)g * a.cap, &cnt[g], a.k, &pivot[g], hist);
        }
    }
    cp_async_wait<0>();
    if (!TOPK && a.row_offset && it.pad) {
        // the last work item of a segment: the rest of the rows up to row_len
        for (uint32_t g = 0; g < it.n_queries; ++g) {
            float* row = a.scores + a.row_offset[it.query_begin + g];
            for (uint32_t e = it.index_base + it.n_tiles + (uint32_t)tid; e < a.row_len; e += blockDim.x) row[e] = a.row_fill;
        }
    }
    if (TOPK) {
        __syncthreads();
        for (int g = 0; g < (int)it.n_queries; ++g) {
            if (cnt[g] > (int)a.k) block_select_topk(keys + (size_t)g * a.cap, &cnt[g], a.k, &pivot[g], hist);
            const int c = cnt[g];
            uint64_t* dst = a.cand_keys + (size_t)(it.list_begin + g) * a.list_cap;
            for (int i = tid; i < c; i += blockDim.x) dst[i] = keys[(size_t)g * a.cap + i];
            if (tid == 0) a.cand_cnt[it.list_begin + g] = (uint32_t)c;
        }
    }
}

}  // namespace
}  // namespace slha

#include "score_mma.cuh"
#include "score_wide.cuh"
#include "score_merge.cuh"
#include "score_host.cuh"

// ---------------------------------------------------------------------------
// slha_b200_score_topk_noalloc: fused score + top-k whose working memory is a
// fixed array inside this library instead of memory obtained at call time.
// ---------------------------------------------------------------------------
namespace slha {
namespace {

constexpr uint32_t NA_MAX_ITEMS = 512;    // work items per call
constexpr uint32_t NA_MAX_LISTS = 512;    // candidate lists (work item x query) per call
constexpr uint32_t NA_MAX_QUERIES = 256;  // query rows per call
constexpr uint32_t NA_MAX_K = 1024;       // results per query

struct NoAllocScratch {
    WorkItem items[NA_MAX_ITEMS];
    uint32_t q_list_begin[NA_MAX_QUERIES];
    uint32_t q_list_count[NA_MAX_QUERIES];
    uint32_t cand_cnt[NA_MAX_LISTS];
    uint64_t cand_keys[(size_t)NA_MAX_LISTS * NA_MAX_K];
};

// The scratch itself: 4 MiB + 22 KiB of device memory held by every GPU that
// loads this library, until the process exits.  In host code this name is only
// a stand-in for the symbol; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

struct NoAllocDevice {
    bool ready = false;
    NoAllocScratch* scratch = nullptr;  // device address of g_noalloc_scratch on this device
};
NoAllocDevice g_noalloc_dev[16];
std::mutex g_noalloc_mu;

// Once per device, with that device current: resolve the scratch address and
// raise the kernels' dynamic shared-memory limits.
Status noalloc_setup(Ctx* c, NoAllocScratch** out) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocDevice& d = g_noalloc_dev[c->device & 15];
    if (!d.ready) {
        SLHA_CUDA(cudaSetDevice(c->device));
        void* p = nullptr;
        SLHA_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        SLHA_CUDA(cudaFuncSetAttribute(score_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<CompLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        d.scratch = reinterpret_cast<NoAllocScratch*>(p);
        d.ready = true;
    }
    *out = d.scratch;
    return Status();
}

}  // namespace

Status score_topk_noalloc(Ctx* c, const SciRustSlhaTile* tiles, const SlhaB200Segment* segs, size_t n_segs,
                          const float* d_q_coarse, const uint64_t* d_q_sign, size_t nq, uint32_t k,
                          uint32_t* d_out_index, float* d_out_score, uint32_t* d_out_count) {
    if (nq == 0) return Status();
    if (k == 0 || k > NA_MAX_K)
        return Status(SLHA_ERR_CAPACITY, "score_topk_noalloc: k must be in 1.." + std::to_string(NA_MAX_K));
    if (nq > NA_MAX_QUERIES)
        return Status(SLHA_ERR_CAPACITY, "score_topk_noalloc: at most " + std::to_string(NA_MAX_QUERIES) + " query rows per call");
    NoAllocScratch* sc;
    SLHA_TRY(noalloc_setup(c, &sc));

    // work decomposition in fixed-size host arrays (nothing is allocated)
    static thread_local WorkItem items[NA_MAX_ITEMS];
    static thread_local uint32_t q_begin[NA_MAX_QUERIES], q_count[NA_MAX_QUERIES];
    std::memset(q_count, 0, sizeof(uint32_t) * nq);
    std::memset(q_begin, 0, sizeof(uint32_t) * nq);
    const int threads = 128, nwarps = threads / 32;
    const uint32_t round = (uint32_t)nwarps * BLK_TILES;
    uint64_t total = 0;
    for (size_t i = 0; i < n_segs; ++i) total += (uint64_t)segs[i].n_tiles * ((segs[i].n_queries + 3) / 4);
    // Every (segment, group of <= 4 queries) stream is cut into items of equal size.  The item
    // size starts where 128 items would cover the call and grows until the items and their
    // candidate lists (one per item and query) fit the fixed scratch; only a call whose streams
    // alone exceed it (one item each) is refused.
    uint64_t streams = 0, stream_lists = 0;
    for (size_t i = 0; i < n_segs; ++i)
        if (segs[i].n_tiles) {
            streams += (segs[i].n_queries + 3) / 4;
            stream_lists += segs[i].n_queries;
        }
    if (streams > NA_MAX_ITEMS || stream_lists > NA_MAX_LISTS)
        return Status(SLHA_ERR_CAPACITY, "score_topk_noalloc: the segments x query groups alone need more than " +
                                             std::to_string(NA_MAX_ITEMS) + " work items or " + std::to_string(NA_MAX_LISTS) +
                                             " candidate lists, the size of the fixed scratch");
    uint64_t item_tiles = std::max<uint64_t>(4096, (total + 127) / 128);
    item_tiles = (item_tiles + round - 1) / round * round;
    for (;;) {
        uint64_t need_items = 0, need_lists = 0;
        for (size_t i = 0; i < n_segs; ++i) {
            const uint64_t parts = (segs[i].n_tiles + item_tiles - 1) / item_tiles;
            need_items += parts * ((segs[i].n_queries + 3) / 4);
            need_lists += parts * segs[i].n_queries;
        }
        if (need_items <= NA_MAX_ITEMS && need_lists <= NA_MAX_LISTS) break;
        item_tiles = (item_tiles + item_tiles / 4 + round - 1) / round * round;  // (ends: one part per stream fits, checked above)
    }
    uint32_t n_items = 0, n_lists = 0, max_parts = 1;
    for (size_t i = 0; i < n_segs; ++i) {
        const SlhaB200Segment& s = segs[i];
        if ((uint64_t)s.query_begin + s.n_queries > nq)
            return Status(SLHA_ERR_DIMENSION, "segment query range exceeds n_queries");
        const uint32_t parts = (uint32_t)((s.n_tiles + item_tiles - 1) / item_tiles);
        max_parts = std::max(max_parts, parts);
        for (uint32_t q0 = 0; q0 < s.n_queries; q0 += 4) {
            const uint32_t gq = std::min<uint32_t>(4, s.n_queries - q0);
            if (n_items + parts > NA_MAX_ITEMS || n_lists + parts * gq > NA_MAX_LISTS)
                return Status(SLHA_ERR_CAPACITY,
                              "score_topk_noalloc: the call needs more than " + std::to_string(NA_MAX_ITEMS) +
                                  " work items or " + std::to_string(NA_MAX_LISTS) +
                                  " candidate lists (too many segments x query groups for the fixed scratch)");
            for (uint32_t g = 0; g < gq; ++g) {
                const uint32_t Q = s.query_begin + q0 + g;
                if (q_count[Q]) return Status(SLHA_ERR_DIMENSION, "a query row belongs to two segments");
                q_begin[Q] = n_lists + g;
                q_count[Q] = parts | (gq << 24);
            }
            for (uint32_t part = 0; part < parts; ++part) {
                WorkItem& w = items[n_items++];
                w.tile_begin = s.tile_begin + (uint64_t)part * item_tiles;
                w.n_tiles = (uint32_t)std::min<uint64_t>(item_tiles, s.n_tiles - (uint64_t)part * item_tiles);
                w.index_base = s.index_base + (uint32_t)(part * item_tiles);
                w.query_begin = s.query_begin + q0;
                w.n_queries = gq;
                w.list_begin = n_lists + part * gq;
                w.pad = gq;
            }
            n_lists += parts * gq;
        }
    }
    // queries without tiles still need a defined (empty) list range
    for (size_t Q = 0; Q < nq; ++Q)
        if (!q_count[Q]) q_count[Q] = 1u << 24;
    if (n_items)
        SLHA_CUDA(cudaMemcpyAsync(sc->items, items, sizeof(WorkItem) * n_items, cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaMemcpyAsync(sc->q_list_begin, q_begin, 4 * nq, cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaMemcpyAsync(sc->q_list_count, q_count, 4 * nq, cudaMemcpyHostToDevice, c->stream));
    // Every list count is rewritten by the scoring kernel and lists are read only up
    // to their count, so nothing left in the scratch by the previous call is visible.
    const uint32_t cap = std::max<uint32_t>(2 * k, k + 2 * round);
    if (n_items) {
        ScoreArgs a{};
        a.tiles = reinterpret_cast<const unsigned char*>(tiles);
        a.items = sc->items;
        a.q_coarse = d_q_coarse;
        a.q_sign = reinterpret_cast<const uint32_t*>(d_q_sign);
        a.k = k;
        a.cap = cap;
        a.list_cap = k;
        a.cand_keys = sc->cand_keys;
        a.cand_cnt = sc->cand_cnt;
        score_kernel<4, true><<<n_items, threads, score_smem_bytes(4, nwarps, true, cap), c->stream>>>(a);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
    }
    uint32_t kp2 = 2;
    while (kp2 < k) kp2 <<= 1;
    CompLists L{sc->cand_keys, sc->cand_cnt, sc->q_list_begin, sc->q_list_count, k};
    const uint32_t cap_s = merge_cap((uint64_t)max_parts * k, kp2, k);
    topk_merge_kernel<CompLists><<<(uint32_t)nq, merge_threads(cap_s), merge_smem(cap_s, kp2), c->stream>>>(
        L, k, kp2, cap_s, d_out_index, d_out_score, d_out_count);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

}  // namespace slha

#ifdef SLHA_STREAM_PROBE
extern "C" int slha_debug_stream_probe(unsigned long long* out) {  // development build only
    return (int)cudaMemcpyFromSymbol(out, slha::g_stream_probe, sizeof(unsigned long long) * 160 * 8);
}
extern "C" int slha_debug_merge_probe(unsigned long long* out) {  // development build only
    return (int)cudaMemcpyFromSymbol(out, slha::g_merge_probe, sizeof(unsigned long long) * 64 * 12);
}
extern "C" int slha_debug_wide_probe(unsigned long long* out) {  // development build only
    return (int)cudaMemcpyFromSymbol(out, slha::g_wide_probe, sizeof(unsigned long long) * 160 * 24);
}
#endif
