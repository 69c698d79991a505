// Wide scoring: many queries per KV head (16 or more: batched decode, the 64-queries-per-head
// configuration).  Included by score.cu after score_mma.cuh.
//
// With that many queries per tile the coarse term of eq. 2.3 is a real contraction --
// 128 tiles x 128 dims x 64 queries per block -- and it runs on the fifth-generation tensor cores:
//   A (128 tiles x K)  the block's tiles, dequantised to exact fp16 values (n - 8) gs 2^-12 in
//                      shared memory, K-major with the 128-byte swizzle the MMA unit reads,
//   B (128 columns x K) the work item's up to 64 queries, each as an fp16 hi and lo column
//                      (q = hi + lo keeps ~22 bits), resident in shared memory for the whole item,
//   D (128 x 128 fp32)  in tensor memory (TMEM), two accumulators so that the MMAs of one block run
//                      while the previous block's scores are finished,
// issued with tcgen05.mma by one thread, tracked with tcgen05.commit -> mbarrier, read back with
// tcgen05.ld.  K = 128 dims (+16 for TQ3 tiles: level = (n - 8) / 2 + c / 4 with the nibble
// n = 2 code + correction bit, so the score also needs c / 4 sum_g gs_g Q_g, Q_g the query's sum over
// scale group g; those eight products per tile ride along as one more K step).
// Warps: sixteen workers and one MMA warp.  The work around the MMA is latency-bound CUDA-core code
// (dequantisation, 64 Hamming distances per tile), so it is spread over as many warps as the
// register file allows: every worker stages its share of block b + 1 (one tile row quarter each)
// while the MMAs of block b run, then turns its share of block b's accumulators into scores --
// worker w reads TMEM lanes 32 (w & 3) .. + 31 (its 32 tiles) and the 16 queries of column chunk
// w >> 2 -- adds the Hamming term only where the coarse score can reach the row's threshold, filters
// and appends candidates to the rows' buffers (the streaming top-k state of score_stream_kernel).
// Every wait on an mbarrier is bounded; a wait that runs out flags the item's rows for the generic
// kernel and lets the CTA finish (tensor memory is always given back).
// Codecs: INT4 / MX-INT4 launches and TQ3 launches; any other tile hands the item's rows back.
#pragma once

namespace slha {
namespace {

#ifdef SLHA_STREAM_PROBE
#define WPROBE_DECL unsigned long long wp_t = probe_now(), wp_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define WPROBE_LAP(i) do { const unsigned long long n_ = probe_now(); wp_acc[i] += n_ - wp_t; wp_t = n_; } while (0)
#define WPROBE_OUT(base, cnt) do { if ((threadIdx.x & 31) == 0) for (int i_ = 0; i_ < cnt; ++i_) g_wide_probe[blockIdx.x][base + i_] = wp_acc[i_]; } while (0)
__device__ unsigned long long g_wide_probe[160][24];
#else
#define WPROBE_DECL
#define WPROBE_LAP(i)
#define WPROBE_OUT(base, cnt)
#endif
constexpr int WIDE_M = 128;                         // tiles per block
constexpr int WIDE_NQ = 64;                         // query rows per work item
constexpr int WIDE_SLAB = WIDE_M * 128;             // one 64-element K slab of A or B: 128 rows x 128 bytes
constexpr int WIDE_A_BYTES = 3 * WIDE_SLAB;         // K = 64 + 64 + 16 (third slab: first 32 bytes of every row)
constexpr int WIDE_RAW_BYTES = WIDE_M * TILE_BYTES; // the block's tiles as they lie in HBM
constexpr int WIDE_WORKERS = 512;                   // threads of the sixteen worker warps
constexpr int WIDE_THREADS = WIDE_WORKERS + 32;     // + the MMA warp
constexpr uint32_t WIDE_SPIN = 1u << 22;            // polls of one mbarrier wait before it gives up (~0.2 s)

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
// a threshold's score word as a float; words at or below the key of -inf mean "no threshold yet"
__device__ __forceinline__ float wide_thr(uint32_t key) { return key > 0x00800000u ? key_score(key) : -INFINITY; }
__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
// false when the phase did not complete within WIDE_SPIN polls
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < WIDE_SPIN; ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
// Named barrier `id` over `nthreads` threads that also tells every one of them whether any brought `fail`: the
// warps of a role leave their loop together, so that none is left waiting at a later barrier of the role.
__device__ __forceinline__ bool role_any(uint32_t id, uint32_t nthreads, bool fail) {
    uint32_t any;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, %2, %3, q;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(any) : "r"((uint32_t)fail), "r"(id), "r"(nthreads) : "memory");
    return any != 0;
}
// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart (tcgen05 shared-memory matrix descriptor)
__device__ __forceinline__ uint64_t wide_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// instruction descriptor: D fp32, A and B fp16, both K-major, N = 128, M = 128
constexpr uint32_t WIDE_IDESC = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void wide_mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem), "l"(da), "l"(db), "r"(WIDE_IDESC), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void wide_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void wide_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
        "%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Threshold refresh of NR consecutive query rows by one warp (all loads of the NR histograms in flight
// together): the lower edge of the highest bucket whose count from the top reaches k, minus half a
// bucket, is a proven bound (see stream_refresh_threshold).
template <int NR>
__device__ __forceinline__ void wide_refresh_rows(const ScoreArgs& a, uint32_t Q0, int nrows, const float2* rng, uint32_t* pvh, float* thr, int lane) {
    uint32_t c[NR][8];
    unsigned long long seen = 0ull;
    if (lane < nrows) seen = *reinterpret_cast<volatile unsigned long long*>(a.gpivot + Q0 + lane);
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
        for (int j = 0; j < 8; ++j) c[r][j] = 0u;
        if (r < nrows && rng[r].y != 0.0f) {  // (uniform)
            const uint32_t* hq = a.ghist + (size_t)(Q0 + r) * 256 + 248 - 8 * lane;  // buckets 255-8l .. 248-8l (descending)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(c[r][7]), "=r"(c[r][6]), "=r"(c[r][5]), "=r"(c[r][4]) : "l"(hq));
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(c[r][3]), "=r"(c[r][2]), "=r"(c[r][1]), "=r"(c[r][0]) : "l"(hq + 4));
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        if (r >= nrows) break;  // (uniform)
        uint32_t best = (uint32_t)(__shfl_sync(0xFFFFFFFFu, seen, r) >> 32);
        const float2 rr = rng[r];
        if (rr.y != 0.0f) {
            uint32_t tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) tot += c[r][j];
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += y;
            }
            const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= a.k);
            uint32_t ek = 0;
            if (ok != 0u && lane == __ffs(ok) - 1) {
                uint32_t run = incl - tot;
                int b = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (run + c[r][j] >= a.k) { b = 255 - 8 * lane - j; break; }
                    run += c[r][j];
                }
                if (b >= 1) {
                    const uint32_t e = score_key(rr.x + ((float)b - 0.5f) / rr.y);
                    ek = e > 8u ? e - 8u : 0u;
                }
            }
            ek = __reduce_max_sync(0xFFFFFFFFu, ek);
            if (ek > best) {
                best = ek;
                if (lane == 0) atomicMax(a.gpivot + Q0 + r, (unsigned long long)ek << 32);
            }
        }
        if (lane == 0 && best > pvh[r]) {
            pvh[r] = best;
            thr[r] = wide_thr(best);
        }
    }
}

// KINDW 0: INT4 / MX-INT4 tiles, 1: TQ3 tiles, 2: mixed 8/4 tiles (the eight 8-bit head levels b - 128 take the K slots of
// their own eight dims and of the eight dropped tail dims: (b - 128) gs = (b - 128) (16 gh + gl) with the scale byte's two
// nibbles, two exact fp16 products per dim; the 112 INT4 dims follow as in kind 0, shifted by one word).  DENSE: every score is written to its row of a.scores (row q starts at
// a.row_offset[q]) instead of going through the top-k filter: the dense scores of a layer for callers that replace
// attention logits (the llama.cpp shim).
template <int KINDW, bool DENSE>
__global__ void __launch_bounds__(WIDE_THREADS, 1) score_wide_kernel(ScoreArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // shared layout (1024-byte aligned base): B | A[0] | A[1] | raw[0] | raw[1] | sign words | thresholds | mappings | barriers
    const uint32_t base_s = ((uint32_t)__cvta_generic_to_shared(smem_raw) + 1023u) & ~1023u;
    unsigned char* base = smem_raw + (base_s - (uint32_t)__cvta_generic_to_shared(smem_raw));
    const uint32_t B_s = base_s, A_s = base_s + WIDE_A_BYTES, raw_s = A_s + 2 * WIDE_A_BYTES;
    unsigned char* raw = base + 3 * WIDE_A_BYTES;
    unsigned char* tail = raw + 2 * WIDE_RAW_BYTES;
    uint32_t* qs_w = reinterpret_cast<uint32_t*>(tail);            // [64][8]
    uint32_t* pvh = qs_w + 512;                                     // [64] score word of the row's threshold
    float* thr = reinterpret_cast<float*>(pvh + 64);                // [64] the same threshold as a float
    float2* rng = reinterpret_cast<float2*>(thr + 64);              // [64] (smin, inv)
    float2* rmap = rng + 64;                                        // [64] (-smin inv, inv)
    uint64_t* bars = reinterpret_cast<uint64_t*>(rmap + 64);        // full[2], mma_done[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);    // [0] TMEM base, [1] error flag, [2] bail
    float2* colmm = reinterpret_cast<float2*>(bars + 8);            // [4][64] per tile quarter: (min, max) coarse score of a column
    unsigned long long* roff = reinterpret_cast<unsigned long long*>(colmm);  // DENSE: [64] where the item's rows start in a.scores
    const uint32_t bars_s = base_s + 3 * WIDE_A_BYTES + 2 * WIDE_RAW_BYTES + 2048 + 256 + 256 + 512 + 512;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int MMA_WARP = WIDE_WORKERS / 32;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(bars_s + 8 * i, WIDE_WORKERS);  // full: every worker has staged its share
            mbar_init(bars_s + 16 + 8 * i, 1);        // mma_done: one tcgen05.commit
        }
        tmem_slot[1] = 0;
        tmem_slot[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == MMA_WARP) {  // two accumulators of 128 columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(bars_s + 48), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_slot[0];
    uint32_t magic;
    asm volatile("mov.u32 %0, 0x64006400;\n" : "=r"(magic));
    WPROBE_DECL;
    WPROBE_LAP(7);

    uint32_t nblk = 0;  // blocks this CTA has pushed through the two stages so far (all roles count alike)
    const uint32_t item_end = a.cta_begin[blockIdx.x + 1];
    for (uint32_t item_id = a.cta_begin[blockIdx.x]; item_id < item_end; ++item_id) {
        const WorkItem it = a.items[item_id];
        const int nq = (int)it.n_queries;
        __syncthreads();  // the previous item's MMAs and scores are finished: B, thresholds and sign words may change
        if (DENSE && tid < WIDE_NQ) roff[tid] = tid < nq ? a.row_offset[it.query_begin + tid] : 0ull;
        if (!DENSE && tid < WIDE_NQ) {
            const bool have = tid < nq;
            const unsigned long long pv = have ? *reinterpret_cast<volatile unsigned long long*>(a.gpivot + it.query_begin + tid) : ~0ull;
            pvh[tid] = (uint32_t)(pv >> 32);
            thr[tid] = have ? wide_thr((uint32_t)(pv >> 32)) : INFINITY;
            const unsigned long long pr = have ? *reinterpret_cast<volatile unsigned long long*>(a.grange + it.query_begin + tid) : 0ull;
            rng[tid] = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
            rmap[tid] = make_float2(-rng[tid].x * rng[tid].y, rng[tid].y);
        }
        for (int e = tid; e < WIDE_NQ * 8; e += WIDE_THREADS) qs_w[e] = (e >> 3) < nq ? a.q_sign[(size_t)(it.query_begin + (e >> 3)) * 8 + (e & 7)] : 0u;
        // B: column n = 2 q + part (fp16 hi / lo of query q); k slot 8 i + j holds dim 8 i + {0,4,1,5,2,6,3,7}[j], the order in
        // which the workers produce a tile's values; 16-byte chunk i of a row at chunk (i ^ (row & 7)) of its 128-byte line
        bool big = false;
        for (int u = tid; u < 128 * 18; u += WIDE_THREADS) {
            const int n = u / 18, i = u % 18, qi = n >> 1;
            const float* q = a.q_coarse + (size_t)(it.query_begin + (qi < nq ? qi : 0)) * D_C;
            float v[8];
            if (KINDW == 2 && i < 2) {
                // head chunk i: slots 0..3 meet the high-nibble products of dims 4 i .. 4 i + 3, slots 4..7 the low-nibble ones
                const float4 x = *reinterpret_cast<const float4*>(q + 4 * i);
                v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = x.x; v[5] = x.y; v[6] = x.z; v[7] = x.w;
            } else if (i < 16) {
                const int d0 = KINDW == 2 ? 8 * (i - 1) : 8 * i;  // (mixed: latent word i holds dims 8 (i - 1) ..)
                const float4 x = *reinterpret_cast<const float4*>(q + d0), y = *reinterpret_cast<const float4*>(q + d0 + 4);
                v[0] = x.x; v[1] = y.x; v[2] = x.y; v[3] = y.y; v[4] = x.z; v[5] = y.z; v[6] = x.w; v[7] = y.w;
            } else if (i == 16 && KINDW == 1) {
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float s = 0.0f;
                    for (int d = 0; d < 16; ++d) s += q[16 * g + d];
                    v[g] = s;
                }
            } else {
#pragma unroll
                for (int g = 0; g < 8; ++g) v[g] = 0.0f;
            }
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float x0 = qi < nq ? v[2 * j] : 0.0f, x1 = qi < nq ? v[2 * j + 1] : 0.0f;
                big |= fabsf(x0) > 60000.0f || fabsf(x1) > 60000.0f;
                if (n & 1) { x0 = half_residual(x0); x1 = half_residual(x1); }
                w[j] = pack_half2(x0, x1);
            }
            const uint32_t slab = (uint32_t)i >> 3, chunk = (uint32_t)i & 7u;
            sts_v4(B_s + slab * WIDE_SLAB + (uint32_t)n * 128u + ((chunk ^ ((uint32_t)n & 7u)) << 4), w[0], w[1], w[2], w[3]);
        }
        if (big) tmem_slot[2] = 1;  // a query too large for the fp16 split
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // B was written with ordinary stores, the MMA reads it through the async proxy
        const bool need_map = __syncthreads_or(!DENSE && tid < nq && rng[tid].y == 0.0f) != 0;  // a row of the item has no bucket mapping yet
        const bool too_big = tmem_slot[2] != 0;
        const uint32_t n = it.n_tiles;
        WPROBE_LAP(0);  // item set-up
        const uint32_t blocks = too_big ? 0u : (n + WIDE_M - 1) / WIDE_M;

        if (warp == MMA_WARP) {
            // ---- MMA warp: one thread issues the K steps of every block ----
            for (uint32_t b = 0; b < blocks; ++b) {
                const uint32_t g = nblk + b, s = g & 1u, use = g >> 1;
                if (!mbar_wait(bars_s + 8 * s, use & 1u)) { tmem_slot[1] = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const uint32_t as = A_s + s * WIDE_A_BYTES;
#pragma unroll
                    for (int ks = 0; ks < (KINDW == 1 ? 9 : 8); ++ks) {
                        const uint32_t off = (uint32_t)(ks >> 2) * WIDE_SLAB + (uint32_t)(ks & 3) * 32u;
                        wide_mma(tmem + s * 128u, wide_desc(as + off), wide_desc(B_s + off), ks > 0 ? 1u : 0u);
                    }
                    wide_commit(bars_s + 16 + 8 * s);
                }
                __syncwarp();
            }
        } else {
            // ---- workers ----
            // staging share: tile row tid / 4 of the block, latent quarter tid & 3; two 16-byte chunks of the raw copy
            auto stage = [&](uint32_t b) {
                const uint32_t s = (nblk + b) & 1u;
                const uint32_t t0 = b * WIDE_M;
                const unsigned char* src = a.tiles + (it.tile_begin + t0) * TILE_BYTES;
                const uint32_t rs = raw_s + s * WIDE_RAW_BYTES;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint32_t chunk = (uint32_t)i * WIDE_WORKERS + (uint32_t)tid, row = chunk >> 3;
                    const bool in = t0 + row < n;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(rs + chunk * 16u), "l"(in ? src + (size_t)chunk * 16 : a.tiles), "r"(in ? 16 : 0));
                }
                cp_async_commit();
                cp_async_wait<0>();
                asm volatile("bar.sync 3, 512;\n" ::: "memory");  // the workers see each other's copies
                WPROBE_LAP(2);  // copy
                const uint32_t r = (uint32_t)tid >> 2, c = (uint32_t)tid & 3u;
                const uint32_t row_s = rs + r * TILE_BYTES;
                const uint32_t flags = lds_u16<118>(row_s);
                const bool live = t0 + r < n;
                // a codec this launch does not decode: the item's rows go to the generic kernel
                if (live && ((KINDW == 1)   ? !(flags & F_TQ3) || (flags & (F_NF4 | F_MIXED | F_MIX3))
                             : (KINDW == 2) ? !(flags & F_MIXED) || (flags & (F_NF4 | F_TQ3 | F_MIX3))
                                            : (flags & (F_NF4 | F_MIXED | F_TQ3 | F_MIX3)) != 0))
                    tmem_slot[2] = 1;
                uint32_t nib[4];
                if (KINDW == 1) {
                    const uint32_t w0 = lds_u32(row_s + 12u * c), w1 = lds_u32(row_s + 12u * c + 4u), w2 = lds_u32(row_s + 12u * c + 8u);
                    const uint32_t cr = (flags & F_NOCORR) ? 0u : lds_u32(row_s + 48u + 4u * c);  // (the plane's bytes are ignored once flagged as dropped)
                    const uint32_t w[4] = {w0, w1, w2, 0u};
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const int wi = (24 * m) >> 5, sh = (24 * m) & 31;
                        uint32_t x = __funnelshift_r(w[wi], w[wi + 1], sh) & 0xFFFFFFu;  // eight 3-bit codes
                        x = (x & 0xFFFu) | ((x & 0xFFF000u) << 4);
                        x = (x & 0x003F003Fu) | ((x & 0x0FC00FC0u) << 2);
                        x = (x & 0x07070707u) | ((x & 0x38383838u) << 1);
                        uint32_t cb = (cr >> (8 * m)) & 0xFFu;                             // their correction bits
                        cb = (cb | (cb << 12)) & 0x000F000Fu;
                        cb = (cb | (cb << 6)) & 0x03030303u;
                        cb = (cb | (cb << 3)) & 0x11111111u;
                        nib[m] = (x << 1) | cb;
                    }
                } else {
                    const uint4 L = lds_v4<0>(row_s + 16u * c);
                    nib[0] = L.x; nib[1] = L.y; nib[2] = L.z; nib[3] = L.w;
                }
                uint32_t G0, C0, G1, C1;
                int4c_scales(lds_u16<120>(row_s + 2u * c), magic, G0, C0, G1, C1);
                const uint32_t arow = A_s + s * WIDE_A_BYTES + r * 128u;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    uint32_t o[4];
                    if (KINDW == 2 && c == 0 && m < 2) {
                        // four head bytes b -> (b - 128) gh 2^-8 (slots 0..3) and (b - 128) gl 2^-12 (slots 4..7), gh / gl the nibbles
                        // of the head's scale byte: products below 2048, exact in fp16
                        const uint32_t gs0 = lds_u16<120>(row_s) & 0xFFu;
                        uint32_t gh, gl, b01, b23;
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(gh) : "r"(0x64006400u | (gs0 >> 4) * 0x10001u), "r"(0xE400E400u));   // (gh, gh)
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(gl) : "r"(0x64006400u | (gs0 & 15u) * 0x10001u), "r"(0xE400E400u));  // (gl, gl)
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(gh) : "r"(gh), "r"(0x1C001C00u));  // x 2^-8
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(gl) : "r"(gl), "r"(0x0C000C00u));  // x 2^-12
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(b01) : "r"(prmt(nib[m], magic, 0x7150u)), "r"(0xE480E480u));  // bytes 0, 1 minus 128
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(b23) : "r"(prmt(nib[m], magic, 0x7352u)), "r"(0xE480E480u));  // bytes 2, 3
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(o[0]) : "r"(b01), "r"(gh));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(o[1]) : "r"(b23), "r"(gh));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(o[2]) : "r"(b01), "r"(gl));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(o[3]) : "r"(b23), "r"(gl));
                    } else {
                        int4c_word(nib[m], m < 2 ? G0 : G1, m < 2 ? C0 : C1, o);
                    }
                    if (!live) o[0] = o[1] = o[2] = o[3] = 0u;
                    const uint32_t word = 4u * c + (uint32_t)m, slab = word >> 3, chunk = word & 7u;
                    sts_v4(arow + slab * WIDE_SLAB + ((chunk ^ (r & 7u)) << 4), o[0], o[1], o[2], o[3]);
                }
                if (c == 0) {
                    // third slab: the eight scale bytes times c 2^-13 (TQ3: c = 1, or 2 once the correction plane is gone), then zeros
                    uint32_t e[4] = {0u, 0u, 0u, 0u};
                    if (KINDW == 1 && live) {
                        const uint2 gsb = lds_v2<120>(row_s);
                        const uint32_t f = (flags & F_NOCORR) ? 0x0C000C00u : 0x08000800u;  // 2^-12 or 2^-13 as fp16, twice
                        uint32_t t;
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(t) : "r"(prmt(gsb.x, magic, 0x7150u)), "r"(0xE400E400u));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(e[0]) : "r"(t), "r"(f));
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(t) : "r"(prmt(gsb.x, magic, 0x7352u)), "r"(0xE400E400u));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(e[1]) : "r"(t), "r"(f));
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(t) : "r"(prmt(gsb.y, magic, 0x7150u)), "r"(0xE400E400u));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(e[2]) : "r"(t), "r"(f));
                        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(t) : "r"(prmt(gsb.y, magic, 0x7352u)), "r"(0xE400E400u));
                        asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(e[3]) : "r"(t), "r"(f));
                    }
                    sts_v4(arow + 2 * WIDE_SLAB + ((0u ^ (r & 7u)) << 4), e[0], e[1], e[2], e[3]);
                    sts_v4(arow + 2 * WIDE_SLAB + ((1u ^ (r & 7u)) << 4), 0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                mbar_arrive(bars_s + 8 * s);
                WPROBE_LAP(3);  // dequantise
            };
            // scoring share: TMEM lanes (tile rows) 32 qt .. + 31, query columns 16 ch .. + 15
            const int qt = warp & 3, ch = warp >> 2, r = 32 * qt + lane;
            const bool cols = 16 * ch < nq;  // this worker has query columns in this item
            if (blocks) stage(0);
            for (uint32_t b = 0; b < blocks; ++b) {
                const uint32_t g = nblk + b, s = g & 1u, use = g >> 1;
                if (b + 1 < blocks) stage(b + 1);  // (its buffers were released by the barrier that ended block b - 1)
                // (a wait that ran out anywhere ends the item for all workers together: barriers follow)
                if (role_any(1, WIDE_WORKERS, !mbar_wait(bars_s + 16 + 8 * s, use & 1u))) { tmem_slot[1] = 1; break; }
                WPROBE_LAP(1);  // wait for the accumulators
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                {
                const uint32_t t0 = b * WIDE_M + (uint32_t)r;
                const uint32_t row_s = raw_s + s * WIDE_RAW_BYTES + (uint32_t)r * TILE_BYTES;
                const uint2 meta = lds_v2<96>(row_s);
                const uint32_t flags = lds_u16<118>(row_s);
                const bool live = t0 < n;
                const uint4 ra = lds_v4<64>(row_s), rb2 = lds_v4<80>(row_s);
                const float lam = (flags & F_WARM) ? 0.0f : __uint_as_float(meta.y);
                const float su = __uint_as_float(meta.x) * (KINDW == 1 ? 2048.0f / 255.0f : 4096.0f / 255.0f);
                const uint32_t nidx = ~(it.index_base + t0);
                const uint32_t tm = tmem + ((uint32_t)(32 * qt) << 16) + s * 128u + (uint32_t)ch * 32u;
                const uint32_t Q0 = it.query_begin + 16u * (uint32_t)ch;
                auto full_score = [&](float coarse, int q) {
                    const uint32_t* qw = qs_w + 8 * q;
                    const int h = __popc(ra.x ^ qw[0]) + __popc(ra.y ^ qw[1]) + __popc(ra.z ^ qw[2]) + __popc(ra.w ^ qw[3]) +
                                  __popc(rb2.x ^ qw[4]) + __popc(rb2.y ^ qw[5]) + __popc(rb2.z ^ qw[6]) + __popc(rb2.w ^ qw[7]);
                    return fmaf(lam, (float)(256 - 2 * h), coarse);
                };
                if (DENSE) {
                    if (cols) {
                        uint32_t v[32];
                        wide_tmem_ld32(tm, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int q = 16 * ch + j;
                            if (q >= nq || !live) continue;
                            // (the 32 lanes of the warp hold 32 consecutive tiles: one 128-byte store per row)
                            a.scores[roff[q] + it.index_base + t0] = full_score((__uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1])) * su, q);
                        }
                    }
                } else {
                if (b == 0) {
                    // The first block of an item is walked before it is filtered.  (1) Rows without a bucket mapping get one
                    // from the block's coarse scores (any monotone mapping is valid): column minima and maxima per tile
                    // quarter by a butterfly, combined by one thread per row, one load and one compare-and-swap for all rows
                    // at once.  (2) A counting pass puts every score of the block into the rows' histograms without
                    // appending anything, and the thresholds are derived -- all CTAs of the grid count their first blocks at
                    // about the same time, 128 tiles each; otherwise each CTA would append its whole first block.
                    if (need_map) {
                        if (cols) {
                            uint32_t v[32];
                            wide_tmem_ld32(tm, v);
                            float mn[16], mx[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float coarse = (__uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1])) * su;
                                mn[j] = live ? coarse : INFINITY;
                                mx[j] = live ? coarse : -INFINITY;
                            }
#pragma unroll
                            for (int step = 0; step < 4; ++step) {
                                const int half = 8 >> step, off = 16 >> step;
                                const bool up = (lane & off) != 0;
#pragma unroll
                                for (int i = 0; i < half; ++i) {
                                    const float rmn = __shfl_xor_sync(0xFFFFFFFFu, up ? mn[i] : mn[i + half], off);
                                    const float rmx = __shfl_xor_sync(0xFFFFFFFFu, up ? mx[i] : mx[i + half], off);
                                    mn[i] = fminf(up ? mn[i + half] : mn[i], rmn);
                                    mx[i] = fmaxf(up ? mx[i + half] : mx[i], rmx);
                                }
                            }
                            mn[0] = fminf(mn[0], __shfl_xor_sync(0xFFFFFFFFu, mn[0], 1));
                            mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xFFFFFFFFu, mx[0], 1));
                            if (!(lane & 1)) colmm[qt * WIDE_NQ + 16 * ch + (lane >> 1)] = make_float2(mn[0], mx[0]);  // column 16 ch + lane / 2
                        }
                        asm volatile("bar.sync 2, 512;\n" ::: "memory");
                        if (tid < nq && rng[tid].y == 0.0f) {
                            float lo_s = INFINITY, hi_s = -INFINITY;
                            for (int w2 = 0; w2 < 4; ++w2) {
                                lo_s = fminf(lo_s, colmm[w2 * WIDE_NQ + tid].x);
                                hi_s = fmaxf(hi_s, colmm[w2 * WIDE_NQ + tid].y);
                            }
                            const uint32_t Q = it.query_begin + (uint32_t)tid;
                            unsigned long long pr = *reinterpret_cast<volatile unsigned long long*>(a.grange + Q);
                            if (!pr && hi_s > lo_s) {
                                const float span = hi_s - lo_s, lo = lo_s - 1.5f * span, inv = 256.0f / (4.0f * span);
                                if (isfinite(lo) && isfinite(inv) && inv > 0.0f) {
                                    const unsigned long long mine_r = (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(inv) << 32);
                                    const unsigned long long old = atomicCAS(a.grange + Q, 0ull, mine_r);
                                    pr = old ? old : mine_r;
                                }
                            }
                            if (pr) {
                                const float2 rr = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
                                rng[tid] = rr;
                                rmap[tid] = make_float2(-rr.x * rr.y, rr.y);
                            }
                        }
                        asm volatile("bar.sync 2, 512;\n" ::: "memory");
                    }
                    WPROBE_LAP(4);  // bucket mappings
                    if (cols) {
                        uint32_t v[32];
                        wide_tmem_ld32(tm, v);  // (collective: every lane of the warp takes part, live tile or not)
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int q = 16 * ch + j;
                            if (q >= nq || !live) continue;
                            const float sc = full_score((__uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1])) * su, q);
                            const float2 rm = rmap[q];
                            atomicAdd(a.ghist + (size_t)(Q0 + (uint32_t)j) * 256 + min(max(__float2int_rz(fmaf(sc, rm.y, rm.x)), 0), 255), 1u);
                        }
                    }
                    asm volatile("bar.sync 2, 512;\n" ::: "memory");
                    WPROBE_LAP(5);  // counting pass
                    const int rows = min(4, nq - 4 * warp);
                    if (rows > 0) wide_refresh_rows<4>(a, it.query_begin + 4u * (uint32_t)warp, rows, rng + 4 * warp, pvh + 4 * warp, thr + 4 * warp, lane);
                    asm volatile("bar.sync 2, 512;\n" ::: "memory");
                    WPROBE_LAP(6);  // thresholds
                }
                if (cols) {
                    uint32_t v[32];
                    wide_tmem_ld32(tm, v);
                    uint32_t keys[16], bal[16], pm = 0, mine_cnt = 0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int q = 16 * ch + j;
                        bal[j] = 0;
                        keys[j] = 0;
                        if (q >= nq) continue;  // (uniform)
                        const float coarse = (__uint_as_float(v[2 * j]) + __uint_as_float(v[2 * j + 1])) * su;
                        // the residual term lies in [-256 lambda, 256 lambda]
                        bool p = live && fmaf(lam, 257.0f, coarse + fabsf(coarse) * 1e-6f) >= thr[q];
                        if (p) {
                            keys[j] = score_key(full_score(coarse, q));
                            p = keys[j] >= pvh[q];
                        }
                        bal[j] = __ballot_sync(0xFFFFFFFFu, p);
                        if (p) pm |= 1u << j;
                        if (lane == j) mine_cnt = (uint32_t)__popc(bal[j]);
                    }
                    // slots of the sixteen rows' candidates: lane j reserves for row 16 ch + j, one round trip for all
                    uint32_t slot0 = 0;
                    if (mine_cnt) slot0 = atomicAdd(a.gcount + Q0 + (uint32_t)lane, mine_cnt);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (!bal[j]) continue;  // (uniform)
                        const uint32_t base_j = __shfl_sync(0xFFFFFFFFu, slot0, j);
                        if (pm >> j & 1u) {
                            const uint32_t Q = Q0 + (uint32_t)j;
                            const uint32_t at = base_j + (uint32_t)__popc(bal[j] & ((1u << lane) - 1u));
                            if (at < a.gcap) a.gbuf[(size_t)Q * a.gcap + at] = ((uint64_t)keys[j] << 32) | (uint64_t)nidx;
                            else a.gflag[Q] = 1u;  // the row's buffer is full: the generic kernel scores the row
                            if (b != 0) {  // (the first block was counted by its counting pass)
                                const float2 rm = rmap[16 * ch + j];
                                atomicAdd(a.ghist + (size_t)Q * 256 + min(max(__float2int_rz(fmaf(key_score(keys[j]), rm.y, rm.x)), 0), 255), 1u);
                            }
                        }
                    }
                }
                }  // !DENSE
                WPROBE_LAP(1 + 8);  // filter and append (index 9)
                // thresholds again after every second block; worker w looks after rows 4 w .. 4 w + 3
                if (!DENSE && (b & 1u) == 1u && b + 1 < blocks) {
                    const int rows = min(4, nq - 4 * warp);
                    if (rows > 0) wide_refresh_rows<4>(a, it.query_begin + 4u * (uint32_t)warp, rows, rng + 4 * warp, pvh + 4 * warp, thr + 4 * warp, lane);
                    WPROBE_LAP(6);
                }
                }
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                // all workers are done with block b (its raw tiles, its accumulator): the stage may be refilled
                asm volatile("bar.sync 1, 512;\n" ::: "memory");
                WPROBE_LAP(2 + 8);  // end-of-block barrier (index 10)
            }
            if (warp == 0) WPROBE_OUT(0, 12);
        }
        nblk += blocks;
        __syncthreads();
        // rows this CTA could not score (another codec, a query outside the fp16 split, a wait that ran out) go to the generic kernel
        if ((tmem_slot[2] || tmem_slot[1]) && tid < nq) a.gflag[it.query_begin + tid] = 1u;
        if (tmem_slot[1]) break;  // a wait ran out: the barriers' phases are no longer known
        __syncthreads();
        if (tid == 0) tmem_slot[2] = 0;  // (ordered before the next item's writers by the barrier at its start)
    }
    __syncthreads();
    if (tmem_slot[1]) {
        // flag every remaining item of this CTA as well
        for (uint32_t item_id = a.cta_begin[blockIdx.x]; item_id < item_end; ++item_id)
            for (uint32_t q = tid; q < a.items[item_id].n_queries; q += WIDE_THREADS) a.gflag[a.items[item_id].query_begin + q] = 1u;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(256u) : "memory");
}

}  // namespace
}  // namespace slha
