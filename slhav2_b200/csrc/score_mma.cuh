// Tensor-core variant of the fused score + top-k kernel for the nibble codecs
// (uniform / MX INT4 and NF4), the layouts of BASELINE configs 1, 2 and 5.
// Included by score.cu.
//
// With a GQA group of four queries the CUDA-core kernel is bound by instruction
// issue (128 FMAs per tile and query plus the nibble decode), not by HBM.  Here
// the coarse dot product of eq. 2.3 is an m16n8k16 MMA per 16 tiles and
// 16-dim scale group:
//   A (16 tiles x 16 dims)  = the group's nibbles turned into exact fp16 levels
//                             (n - 8 by an fp16 magic-number trick, or the NF4
//                             codebook entry as an fp16 hi + lo pair from a
//                             bank-replicated shared-memory table),
//   B (16 dims x 8 columns) = the four queries, each as an fp16 hi and lo
//                             column (q = hi + lo keeps ~22 bits), so a thread's
//                             two accumulator columns add up to one query,
//   D fp32, started from zero for every group and folded into the running score
//   with the tile's effective group scale (scale * gs[j] / 255) on the CUDA
//   cores, which is what keeps per-group micro-scaling exact.
// The MMA's k index is permuted (identically for A and B) so that the four k
// slots a thread owns are the four nibbles of one 16-bit word of the tile.
// The Hamming term (8 XOR + POPC per tile and query), tile staging (cp.async
// into an XOR-swizzled ring) and the streaming top-k are as in score_kernel.
// Tiles of any other codec make the CTA hand the whole work item back
// (retry flag) to score_kernel, which is launched right after.
#pragma once

namespace slha {
namespace {

constexpr int MMA_SET_TILES = 16;
constexpr int MMA_SET_BYTES = MMA_SET_TILES * TILE_BYTES;  // 2 KiB
constexpr int MMA_DEPTH = 3;                               // cp.async ring slots per warp
constexpr int MMA_NS = 1;                                  // sets per warp between checks of the reselect flag
constexpr int NF4_LUT_BYTES = 256 * 16 * 8;                // [byte][16 lanes] x (hi pair, lo pair)

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {  // (a & b) | c
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Two nibbles of byte `sel` of w -> half2 (n_lo - 8, n_hi - 8), exact.
//   (byte, byte) masked to (n_lo | n_hi << 20) OR-ed into 1024.0h gives
//   (1024 + n_lo, 1024 + 16 n_hi); one fp16 FMA by (1, 1/16) + (-1032, -72).
__device__ __forceinline__ uint32_t int4_pair(uint32_t w, uint32_t sel) {
    const uint32_t v = lop3_and_or(prmt(w, 0u, sel), 0x00F0000Fu, 0x64006400u);
    return hfma2_u32(v, 0x2C003C00u, 0xD480E408u);
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float half_residual(float x) {  // x - fp16(x)
    return x - __half2float(__float2half_rn(x));
}
// shared-memory loads on 32-bit shared-window addresses (keeps the address math 32-bit)
template <int IMM>
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(addr), "n"(IMM));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
template <int IMM>
__device__ __forceinline__ void cp_async16_s(uint32_t dst, const unsigned char* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1+%2], 16, %3;\n" ::"r"(dst), "l"(src), "n"(IMM), "r"(src_bytes));
}
__device__ __forceinline__ int popc8(const uint4& a, const uint4& b, const uint32_t (&q)[8]) {
    return __popc(a.x ^ q[0]) + __popc(a.y ^ q[1]) + __popc(a.z ^ q[2]) + __popc(a.w ^ q[3]) +
           __popc(b.x ^ q[4]) + __popc(b.y ^ q[5]) + __popc(b.z ^ q[6]) + __popc(b.w ^ q[7]);
}

// Per-thread constants of the fragment gather.
struct LaneConst {
    uint32_t cw[4];     // byte offset (in a tile row) of my word of groups 2c, 2c+1: ((c ^ g) << 4) + 4*(t>>1)
    uint32_t c4, c5, c6, c7;  // byte offsets of the residual / metadata chunks
    uint32_t sel0, sel1;      // prmt selectors of my two latent bytes
    uint32_t sh0, sh1;        // right shifts that bring (my byte << 7) to bits 7..14 (NF4 table index)
    uint32_t lut_lane;        // shared address of my replica column of the NF4 table
};

// Coarse sums of one 16-tile set for rows g (acc0) and g+8 (acc1), query t.
// MODE 0: every row uniform INT4, 1: every row NF4, 2: per-row choice.
template <int MODE>
__device__ __forceinline__ void coarse_set(uint32_t r0, uint32_t r1, const LaneConst& L, const uint32_t (&bq)[8][2],
                                           uint32_t f0, uint32_t f1, const uint4& x0, const uint4& x1,
                                           float& acc0, float& acc1) {
    acc0 = 0.0f;
    acc1 = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t ad0 = r0 + L.cw[c], ad1 = r1 + L.cw[c];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            const int j = 2 * c + jj;
            const uint32_t w0 = jj ? lds_u32<8>(ad0) : lds_u32<0>(ad0);
            const uint32_t w1 = jj ? lds_u32<8>(ad1) : lds_u32<0>(ad1);
            uint32_t a0, a1, a2, a3, l0 = 0, l1 = 0, l2 = 0, l3 = 0;
            const bool n0 = MODE == 1 || (MODE == 2 && (f0 & F_NF4));
            const bool n1 = MODE == 1 || (MODE == 2 && (f1 & F_NF4));
            if (MODE != 0 && n0) {
                const uint2 e0 = lds_v2(L.lut_lane + ((__funnelshift_r(w0, w0, L.sh0)) & 0x7F80u));
                const uint2 e1 = lds_v2(L.lut_lane + ((__funnelshift_r(w0, w0, L.sh1)) & 0x7F80u));
                a0 = e0.x; a2 = e1.x; l0 = e0.y; l2 = e1.y;
            } else {
                a0 = int4_pair(w0, L.sel0);
                a2 = int4_pair(w0, L.sel1);
            }
            if (MODE != 0 && n1) {
                const uint2 e0 = lds_v2(L.lut_lane + ((__funnelshift_r(w1, w1, L.sh0)) & 0x7F80u));
                const uint2 e1 = lds_v2(L.lut_lane + ((__funnelshift_r(w1, w1, L.sh1)) & 0x7F80u));
                a1 = e0.x; a3 = e1.x; l1 = e0.y; l3 = e1.y;
            } else {
                a1 = int4_pair(w1, L.sel0);
                a3 = int4_pair(w1, L.sel1);
            }
            float d[4];
            mma_f16_zero(d, a0, a1, a2, a3, bq[j][0], bq[j][1]);
            if (MODE != 0) mma_f16(d, l0, l1, l2, l3, bq[j][0], bq[j][1]);
            // gs[j] as float: byte j of (x.z, x.w) dropped into the mantissa of 2^23
            const uint32_t gw0 = j < 4 ? x0.z : x0.w, gw1 = j < 4 ? x1.z : x1.w;
            const float gs0 = __uint_as_float(prmt(gw0, 0x4B000000u, 0x7440u + (j & 3))) - 8388608.0f;
            const float gs1 = __uint_as_float(prmt(gw1, 0x4B000000u, 0x7440u + (j & 3))) - 8388608.0f;
            acc0 = fmaf(d[0] + d[1], gs0, acc0);
            acc1 = fmaf(d[2] + d[3], gs1, acc1);
        }
    }
}


template <bool TOPK>
__global__ void __launch_bounds__(512) score_mma_kernel(ScoreArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // shared layout: nf4 table | stage ring | [keys | pivot | cnt | ctl | hist]
    const uint32_t lut_bytes = a.nf4_table ? NF4_LUT_BYTES : 0;  // the table is left out when no NF4 tile is expected
    uint2* lut = reinterpret_cast<uint2*>(smem);
    unsigned char* tail = smem + lut_bytes + (size_t)nwarps * MMA_DEPTH * MMA_SET_BYTES;
    uint64_t* keys = reinterpret_cast<uint64_t*>(tail);            // [4][cap]
    uint64_t* pivot = keys + (TOPK ? (size_t)4 * a.cap : 0);       // [4]
    int* cnt = reinterpret_cast<int*>(pivot + 4);                  // [4]
    int* ctl = cnt + 4;   // [0] want: some query's buffer is nearly full  [1] arrived  [2] done warps  [3] bail
    int* bail = ctl + 3;
    int* hist = ctl + 4;  // 260
    const uint32_t smem_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t stage_s = smem_s + lut_bytes + (uint32_t)warp * MMA_DEPTH * MMA_SET_BYTES;

    // NF4 codebook as fp16 hi + lo pairs per byte (two nibbles), 16 bank-aligned replicas
    for (int e = tid; e < (a.nf4_table ? 256 * 16 : 0); e += blockDim.x) {
        const int b = e >> 4;
        const float c0 = c_nf4[b & 15], c1 = c_nf4[b >> 4];
        lut[e] = make_uint2(pack_half2(c0, c1), pack_half2(half_residual(c0), half_residual(c1)));
    }
    LaneConst L;
#pragma unroll
    for (int c = 0; c < 4; ++c) L.cw[c] = (uint32_t)(((c ^ g) << 4) + 4 * (t >> 1));
    L.c4 = (uint32_t)((4 ^ g) << 4);
    L.c5 = (uint32_t)((5 ^ g) << 4);
    L.c6 = (uint32_t)((6 ^ g) << 4);
    L.c7 = (uint32_t)((7 ^ g) << 4);
    L.sel0 = (t & 1) ? 0x4242u : 0x4040u;
    L.sel1 = (t & 1) ? 0x4343u : 0x4141u;
    L.sh0 = (t & 1) ? 9u : 25u;
    L.sh1 = (t & 1) ? 17u : 1u;
    L.lut_lane = smem_s + (uint32_t)(lane & 15) * 8u;
    // cp.async of a set: lane copies 16-byte chunks lane, lane+32, lane+64, lane+96
    uint32_t dst_off[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = (lane >> 3) + 4 * i, c = lane & 7;
        dst_off[i] = (uint32_t)(r * TILE_BYTES + ((c ^ (r & 7)) << 4));
    }
    // appends may continue for up to two sets per warp after the flag is raised
    const uint32_t cap_soft = a.cap - (uint32_t)nwarps * 2 * MMA_SET_TILES;
    const uint32_t resel_min = (a.k + cap_soft) / 2;
    const uint32_t key_row = (uint32_t)t * a.cap;

    const uint32_t item_end = a.cta_begin[blockIdx.x + 1];
    for (uint32_t item_id = a.cta_begin[blockIdx.x]; item_id < item_end; ++item_id) {
        const WorkItem it = a.items[item_id];
        __syncthreads();  // previous item fully retired (and the table is visible)
        if (TOPK && tid < 4) { cnt[tid] = 0; pivot[tid] = 0; }
        if (tid == 0) { ctl[0] = ctl[1] = ctl[2] = ctl[3] = 0; }
        // B fragments: column n = g is query g>>1, part g&1 (hi / lo); k slots
        // {2t, 2t+1, 2t+8, 2t+9} of group j carry dims 16j + 4t + {0,1,2,3}
        uint32_t bq[8][2];
        uint32_t qs[8];
        {
            const int qi = g >> 1;
            const bool have = qi < (int)it.n_queries;
            const float* q = a.q_coarse + (size_t)(it.query_begin + (have ? qi : 0)) * D_C;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(q + 16 * j + 4 * t);
                float v[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (!have) v[i] = 0.0f;
                    if (g & 1) v[i] = half_residual(v[i]);
                }
                bq[j][0] = pack_half2(v[0], v[1]);
                bq[j][1] = pack_half2(v[2], v[3]);
            }
            // sign words of query t (the query whose scores this thread finishes)
#pragma unroll
            for (int w = 0; w < 8; ++w)
                qs[w] = t < (int)it.n_queries ? a.q_sign[(size_t)(it.query_begin + t) * 8 + w] : 0u;
        }
        __syncthreads();

        const unsigned char* tbase = a.tiles + it.tile_begin * TILE_BYTES + lane * 16;
        const uint8_t* sbase = a.state ? a.state + it.tile_begin : nullptr;
        const uint32_t n = it.n_tiles;
        const uint32_t n_sets = (n + MMA_SET_TILES - 1) / MMA_SET_TILES;
        const uint32_t my_sets = (n_sets + nwarps - 1) / nwarps;  // sets this warp walks (the last may be past the end)
        auto set_index = [&](uint32_t q) { return q * nwarps + warp; };
        auto issue = [&](uint32_t q) {
            const uint32_t s = set_index(q);
            if (q < my_sets && s < n_sets) {
                const uint32_t dst = stage_s + (q % MMA_DEPTH) * MMA_SET_BYTES;
                const unsigned char* src = tbase + (size_t)s * MMA_SET_BYTES;
                if ((s + 1) * MMA_SET_TILES <= n) {
                    cp_async16_s<0>(dst + dst_off[0], src, 16);
                    cp_async16_s<512>(dst + dst_off[1], src, 16);
                    cp_async16_s<1024>(dst + dst_off[2], src, 16);
                    cp_async16_s<1536>(dst + dst_off[3], src, 16);
                } else {
                    // ragged last set: rows past the end are zero-filled (source not read)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const bool live = s * MMA_SET_TILES + (lane >> 3) + 4 * i < n;
                        cp_async16_s<0>(dst + dst_off[i], live ? src + 512 * i : tbase, live ? 16 : 0);
                    }
                }
            }
            cp_async_commit();
        };
        // Thresholds are shared between the CTAs that scan the same query's tiles:
        // a CTA's pivot (k of its own elements are >= it) is a proven lower bound of
        // the query's k-th best composite key, so the maximum over CTAs is too.
        auto refresh_pivots = [&]() {
            if (lane < (int)it.n_queries) {
                const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(a.gpivot + it.query_begin + lane);
                if (seen > pivot[lane]) pivot[lane] = seen;
            }
        };
        // All warps meet here when a query's buffer is nearly full (flag ctl[0]).  No
        // barrier is executed in the steady state: every warp polls the flag between
        // sets, finished warps poll it in the drain loop, so everyone arrives.
        auto rendezvous = [&]() {
            __syncwarp();
            if (lane == 0) atomicAdd(&ctl[1], 1);
            for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
                if (*reinterpret_cast<volatile int*>(ctl + 1) >= nwarps) break;
                __nanosleep(40);
            }
            __syncthreads();
#pragma unroll 1
            for (int qq = 0; qq < (int)it.n_queries; ++qq) {
                if (cnt[qq] > (int)resel_min) {
                    block_select_topk(keys + (size_t)qq * a.cap, &cnt[qq], a.k, &pivot[qq], hist);
                    if (tid == 0) atomicMax(a.gpivot + it.query_begin + qq, (unsigned long long)pivot[qq]);
                }
            }
            if (warp == 0) refresh_pivots();
            if (tid == 0) { ctl[0] = 0; ctl[1] = 0; }
            __syncthreads();
        };
#pragma unroll
        for (int i = 0; i < MMA_DEPTH - 1; ++i) issue(i);
        bool gave_up = false;
        for (uint32_t q = 0; q < my_sets; ++q) {
            issue(q + MMA_DEPTH - 1);
            cp_async_wait<MMA_DEPTH - 1>();
            __syncwarp();
            const uint32_t s = set_index(q);
            if (s < n_sets && !gave_up) {
                const uint32_t r0 = stage_s + (q % MMA_DEPTH) * MMA_SET_BYTES + (uint32_t)g * TILE_BYTES;
                const uint32_t r1 = r0 + 8 * TILE_BYTES;
                const uint2 m0 = lds_v2(r0 + L.c6), m1 = lds_v2(r1 + L.c6);  // scale, lambda
                const uint4 x0 = lds_v4(r0 + L.c7), x1 = lds_v4(r1 + L.c7);  // position, head|flags, gs[8]
                const uint32_t f0 = x0.y >> 16, f1 = x1.y >> 16;
                const uint32_t fo = __reduce_or_sync(0xFFFFFFFFu, f0 | f1);
                if ((fo & (F_MIXED | F_TQ3 | F_MIX3)) || ((fo & F_NF4) && !a.nf4_table)) {
                    gave_up = true;  // a codec this kernel does not decode: hand the item back
                    if (lane == 0) bail[0] = 1;
                } else {
                    float acc0, acc1;
                    if (!(fo & F_NF4)) {
                        coarse_set<0>(r0, r1, L, bq, f0, f1, x0, x1, acc0, acc1);
                    } else if (__reduce_and_sync(0xFFFFFFFFu, f0 & f1) & F_NF4) {
                        coarse_set<1>(r0, r1, L, bq, f0, f1, x0, x1, acc0, acc1);
                    } else {
                        coarse_set<2>(r0, r1, L, bq, f0, f1, x0, x1, acc0, acc1);
                    }
                    // Hamming term of query t for both rows
                    const int h0 = popc8(lds_v4(r0 + L.c4), lds_v4(r0 + L.c5), qs);
                    const int h1 = popc8(lds_v4(r1 + L.c4), lds_v4(r1 + L.c5), qs);
                    const float lam0 = (f0 & F_WARM) ? 0.0f : __uint_as_float(m0.y);
                    const float lam1 = (f1 & F_WARM) ? 0.0f : __uint_as_float(m1.y);
                    const float sc0 = fmaf(acc0, __uint_as_float(m0.x) * (1.0f / 255.0f), lam0 * (float)(256 - 2 * h0));
                    const float sc1 = fmaf(acc1, __uint_as_float(m1.x) * (1.0f / 255.0f), lam1 * (float)(256 - 2 * h1));
                    if (t < (int)it.n_queries) {
                        const uint32_t t0 = s * MMA_SET_TILES + g, t1 = t0 + 8;
                        const bool live0 = t0 < n && (!sbase || sbase[t0] != ST_COLD);
                        const bool live1 = t1 < n && (!sbase || sbase[t1] != ST_COLD);
                        if (TOPK) {
                            const uint64_t pv = pivot[t];
                            const uint64_t comp0 = make_comp(sc0, it.index_base + t0);
                            const uint64_t comp1 = make_comp(sc1, it.index_base + t1);
                            if (live0 && comp0 >= pv) {
                                const uint32_t pos = (uint32_t)atomicAdd(&cnt[t], 1);
                                if (pos < a.cap) keys[key_row + pos] = comp0;
                                if (pos >= cap_soft) *reinterpret_cast<volatile int*>(ctl) = 1;
                            }
                            if (live1 && comp1 >= pv) {
                                const uint32_t pos = (uint32_t)atomicAdd(&cnt[t], 1);
                                if (pos < a.cap) keys[key_row + pos] = comp1;
                                if (pos >= cap_soft) *reinterpret_cast<volatile int*>(ctl) = 1;
                            }
                        } else {
                            float* o = a.scores + (size_t)(it.query_begin + t) * a.score_stride + it.index_base;
                            if (t0 < n) o[t0] = live0 ? sc0 : -INFINITY;
                            if (t1 < n) o[t1] = live1 ? sc1 : -INFINITY;
                        }
                    }
                }
            }
            __syncwarp();
            if (TOPK) {
                if (*reinterpret_cast<volatile int*>(ctl)) rendezvous();
                else if (warp == 0 && (q & 31) == 31) refresh_pivots();
            }
        }
        if (TOPK) {
            // drain: warps that ran out of sets keep serving reselect rendezvous until all are done
            __syncwarp();
            if (lane == 0) atomicAdd(&ctl[2], 1);
            for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
                if (*reinterpret_cast<volatile int*>(ctl)) rendezvous();
                else if (*reinterpret_cast<volatile int*>(ctl + 2) >= nwarps) break;
                else __nanosleep(100);
            }
        }
        cp_async_wait<0>();
        __syncthreads();
        if (bail[0]) {
            if (tid == 0) a.retry[item_id] = 1;
            continue;
        }
        if (TOPK) {
#pragma unroll 1
            for (int qq = 0; qq < (int)it.n_queries; ++qq) {
                if (cnt[qq] > (int)a.k) {
                    block_select_topk(keys + (size_t)qq * a.cap, &cnt[qq], a.k, &pivot[qq], hist);
                    if (tid == 0) atomicMax(a.gpivot + it.query_begin + qq, (unsigned long long)pivot[qq]);
                }
                // write the survivors that still clear the query's shared threshold, compacted
                const int c = cnt[qq];
                uint64_t* dst = a.cand_keys + (size_t)(it.list_begin + qq) * a.k;
                const unsigned long long gp = *reinterpret_cast<volatile unsigned long long*>(a.gpivot + it.query_begin + qq);
                if (tid == 0) hist[0] = 0;
                __syncthreads();
                for (int i0 = 0; i0 < c; i0 += blockDim.x) {
                    const int i = i0 + tid;
                    const uint64_t key = i < c ? keys[(size_t)qq * a.cap + i] : 0ull;
                    const bool keep = i < c && key >= gp;
                    const unsigned bal = __ballot_sync(0xFFFFFFFFu, keep);
                    int base = 0;
                    if (lane == 0 && bal) base = atomicAdd(&hist[0], __popc(bal));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    if (keep) dst[base + __popc(bal & ((1u << lane) - 1))] = key;
                }
                __syncthreads();
                if (tid == 0) a.cand_cnt[it.list_begin + qq] = (uint32_t)hist[0];
            }
        }
    }
}

}  // namespace
}  // namespace slha
