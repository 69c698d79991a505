// Tensor-core variant of the fused score + top-k kernel for the nibble codecs
// (uniform / MX INT4 and NF4), the layouts of decode KV caches.
// Included by score.cu.
//
// With a GQA group of four queries the CUDA-core kernel is bound by instruction
// issue (128 FMAs per tile and query plus the nibble decode), not by HBM.  Here
// the coarse dot product of eq. 2.3 is an m16n8k16 MMA per 16 tiles and
// 16-dim scale group:
//   A (16 tiles x 16 dims)  = the group's nibbles turned into exact fp16 levels
//                             (n - 8 by an fp16 magic-number trick, or the NF4
//                             codebook entry as an fp16 hi + lo pair from a
//                             bank-replicated shared-memory table); odd k slots
//                             hold 16x the level, which the trick yields for free,
//   B (16 dims x 8 columns) = the four queries, each as an fp16 hi and lo
//                             column (q = hi + lo keeps ~22 bits), so a thread's
//                             two accumulator columns add up to one query; even k
//                             slots hold 16x the query, so every product is 16x
//                             and the sum is divided by 16 at the end (exact),
//   D fp32, started from zero for every group and folded into the running score
//   with the tile's effective group scale (scale * gs[j] / 255) on the CUDA
//   cores, which is what keeps per-group micro-scaling exact.
// The MMA's k index is permuted (identically for A and B) so that the four k
// slots a thread owns are the four nibbles of one 16-bit word of the tile.
// The Hamming term is 8 XOR + POPC per tile and query.  Tiles are staged by
// cp.async into a per-warp ring whose rows are padded to 144 bytes: every
// shared-memory address of the inner loop is then "row base + immediate" and
// all fragment loads are conflict-free without an XOR swizzle.
// Tiles of any other codec make the CTA hand the whole work item back
// (retry flag) to score_kernel, which is launched right after.
#pragma once

namespace slha {
namespace {

constexpr int MMA_SET_TILES = 16;
constexpr int MMA_SET_BYTES = MMA_SET_TILES * TILE_BYTES;  // 2 KiB of tiles in global memory
constexpr int MMA_ROW = TILE_BYTES + 16;                   // padded row of the staging ring
constexpr int MMA_SET_STRIDE = MMA_SET_TILES * MMA_ROW;    // one staged set
constexpr int MMA_HALF = 8 * MMA_ROW;                      // row g -> row g + 8
#ifndef SLHA_MMA_DEPTH
#define SLHA_MMA_DEPTH 2
#endif
constexpr int MMA_DEPTH = SLHA_MMA_DEPTH;                  // cp.async ring slots per warp
constexpr int NF4_LUT_BYTES = 256 * 16 * 8;                // [byte][16 lanes] x (hi pair, lo pair)
constexpr int SEL_HIST_INTS = 4 * 256 + 48;                // block_select_multi: 4 histograms + state

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
// The four nibbles n0..n3 of a 16-bit word h (n0 lowest) -> half2 (n0 - 8, 16 (n1 - 8))
// and half2 (n2 - 8, 16 (n3 - 8)), exact.  h duplicated into both halves of a word
// has n0 at bit 0 and n1 at bit 20 (after >> 8: n2 and n3); OR-ing those into
// 1024.0h gives (1024 + n0, 1024 + 16 n1), and one fp16 add of (-1032, -1152)
// finishes.  The odd slots carry 16x the level: the B operand carries 16x the query
// in the even slots instead, and the final score is divided by 16 (all exact).
// `magic` is 0x64006400 held in a register the compiler cannot rebuild from an immediate.
__device__ __forceinline__ void int4_quad(uint32_t h, uint32_t magic, uint32_t& lo, uint32_t& hi) {
    const uint32_t t = h * 0x10001u;
    uint32_t v0, v1;
    asm("lop3.b32 %0, %1, 0x00F0000F, %2, 0xEA;\n" : "=r"(v0) : "r"(t), "r"(magic));
    asm("lop3.b32 %0, %1, 0x00F0000F, %2, 0xEA;\n" : "=r"(v1) : "r"(t >> 8), "r"(magic));
    asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(lo) : "r"(v0), "r"(0xE480E408u));
    asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(hi) : "r"(v1), "r"(0xE480E408u));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float half_residual(float x) {  // x - fp16(x)
    return x - __half2float(__float2half_rn(x));
}
// shared-memory loads on 32-bit shared-window addresses plus an immediate
template <int IMM>
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1+%2];\n" : "=h"(v) : "r"(addr), "n"(IMM));
    return (uint32_t)v;
}
template <int IMM>
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(IMM));
    return v;
}
template <int IMM>
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr), "n"(IMM));
    return v;
}
template <int SRC_IMM, int DST_IMM>
__device__ __forceinline__ void cp_async16_s(uint32_t dst, const unsigned char* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0+%1], [%2+%3], 16, %4;\n" ::"r"(dst), "n"(DST_IMM), "l"(src), "n"(SRC_IMM),
                 "r"(src_bytes));
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// TQ3 rows of a staged 16-tile set, rewritten in place as nibble rows: nibble d of the 64 latent
// bytes becomes 2 code_d + correction_d (codes: 3 bits at bit 3d of bytes 0..47; correction bits:
// bit d of bytes 48..63, zero once the correction plane has been dropped).  A lane rewrites half a
// row (64 dims: 24 code bytes and 8 correction bytes in, 32 bytes out); every lane reads before
// any lane writes.
__device__ __forceinline__ void tq3_to_nibbles(uint32_t set_s, int lane) {
    const uint32_t h = (uint32_t)lane & 1u, row = set_s + (uint32_t)(lane >> 1) * MMA_ROW;
    const uint2 c0 = lds_v2<0>(row + 24u * h), c1 = lds_v2<8>(row + 24u * h), c2 = lds_v2<16>(row + 24u * h);
    const uint2 cr = lds_v2<48>(row + 8u * h);
    __syncwarp();
    const uint32_t w[7] = {c0.x, c0.y, c1.x, c1.y, c2.x, c2.y, 0u};
    uint32_t o[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const int wi = (24 * m) >> 5, sh = (24 * m) & 31;
        uint32_t x = __funnelshift_r(w[wi], w[wi + 1], sh) & 0xFFFFFFu;
        x = (x & 0xFFFu) | ((x & 0xFFF000u) << 4);
        x = (x & 0x003F003Fu) | ((x & 0x0FC00FC0u) << 2);
        x = (x & 0x07070707u) | ((x & 0x38383838u) << 1);
        uint32_t c = ((m < 4 ? cr.x : cr.y) >> (8 * (m & 3))) & 0xFFu;
        c = (c | (c << 12)) & 0x000F000Fu;
        c = (c | (c << 6)) & 0x03030303u;
        c = (c | (c << 3)) & 0x11111111u;
        o[m] = (x << 1) | c;
    }
    sts_v4(row + 32u * h, o[0], o[1], o[2], o[3]);
    sts_v4(row + 32u * h + 16u, o[4], o[5], o[6], o[7]);
    __syncwarp();
}
__device__ __forceinline__ int popc8(const uint4& a, const uint4& b, const uint32_t (&q)[8]) {
    return __popc(a.x ^ q[0]) + __popc(a.y ^ q[1]) + __popc(a.z ^ q[2]) + __popc(a.w ^ q[3]) +
           __popc(b.x ^ q[4]) + __popc(b.y ^ q[5]) + __popc(b.z ^ q[6]) + __popc(b.w ^ q[7]);
}

// Coarse sums of one 16-tile set for rows g (acc0) and g+8 (acc1), query t.
// hb = shared address of row g of the set + 2t: halfword t of every 8-byte scale
// group holds the four nibbles this thread feeds to the MMA of that group.
// MODE 0: every row uniform INT4, 1: every row NF4, 2: per-row choice, 3: every row mixed 8/4
// (group 0 holds the eight 8-bit head levels, halfword t = dims 2t and 2t+1, which fill k slots
// 2t and 2t+1 as byte - 128 while slots 2t+8 and 2t+9 stay empty; groups 1..7 are INT4 groups of
// dims 16 J - 8 ..; the B operand is arranged to match when the launch scores mixed tiles).
template <int MODE, int J>
__device__ __forceinline__ void coarse_group(uint32_t hb, uint32_t lut_lane, uint32_t magic, const uint32_t (&bq)[8][2], uint32_t f0,
                                             uint32_t f1, const uint4& x0, const uint4& x1, float& acc0, float& acc1) {
    const uint32_t h0 = lds_u16<8 * J>(hb), h1 = lds_u16<8 * J + MMA_HALF>(hb);
    uint32_t a0, a1, a2, a3, l0 = 0, l1 = 0, l2 = 0, l3 = 0;
    const bool n0 = MODE == 1 || (MODE == 2 && (f0 & F_NF4));
    const bool n1 = MODE == 1 || (MODE == 2 && (f1 & F_NF4));
    (void)n0;
    (void)n1;
    if (MODE == 3 && J == 0) {
        // bytes (b0, b1) -> half2 (1024 + b0, 1024 + b1) - 1152
        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(a0) : "r"(prmt(h0, magic, 0x7150u)), "r"(0xE480E480u));
        asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(a1) : "r"(prmt(h1, magic, 0x7150u)), "r"(0xE480E480u));
        a2 = 0u;
        a3 = 0u;
    } else {
    if (MODE != 0 && n0) {
        // table entry of byte b at lut_lane + 128 b
        const uint2 e0 = lds_v2<0>(lut_lane + ((h0 & 0xFFu) << 7));
        const uint2 e1 = lds_v2<0>(lut_lane + ((h0 >> 8) << 7));
        a0 = e0.x; a2 = e1.x; l0 = e0.y; l2 = e1.y;
    } else {
        int4_quad(h0, magic, a0, a2);
    }
    if (MODE != 0 && n1) {
        const uint2 e0 = lds_v2<0>(lut_lane + ((h1 & 0xFFu) << 7));
        const uint2 e1 = lds_v2<0>(lut_lane + ((h1 >> 8) << 7));
        a1 = e0.x; a3 = e1.x; l1 = e0.y; l3 = e1.y;
    } else {
        int4_quad(h1, magic, a1, a3);
    }
    }
    float d[4];
    mma_f16_zero(d, a0, a1, a2, a3, bq[J][0], bq[J][1]);
    if (MODE == 1 || MODE == 2) mma_f16(d, l0, l1, l2, l3, bq[J][0], bq[J][1]);
    // gs[J] as float: byte J of (x.z, x.w)
    const uint32_t gw0 = J < 4 ? x0.z : x0.w, gw1 = J < 4 ? x1.z : x1.w;
    // (byte -> float on the ALU / FMA pipes: 2^23 + b as a bit pattern, minus 2^23)
    acc0 = fmaf(d[0] + d[1], __uint_as_float(__byte_perm(gw0, 0x4B000000u, 0x7440 + (J & 3))) - 8388608.0f, acc0);
    acc1 = fmaf(d[2] + d[3], __uint_as_float(__byte_perm(gw1, 0x4B000000u, 0x7440 + (J & 3))) - 8388608.0f, acc1);
}

template <int MODE>
__device__ __forceinline__ void coarse_set(uint32_t hb, uint32_t lut_lane, uint32_t magic, const uint32_t (&bq)[8][2], uint32_t f0,
                                           uint32_t f1, const uint4& x0, const uint4& x1, float& acc0, float& acc1) {
    acc0 = 0.0f;
    acc1 = 0.0f;
    coarse_group<MODE, 0>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 1>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 2>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 3>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 4>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 5>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 6>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
    coarse_group<MODE, 7>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
}

// ---- launches that hold only INT4 / MX-INT4 tiles (KIND 3) --------------------------------
// Thread (g, t) of the warp owns the 16 latent bytes 16t..16t+15 of rows g and g+8: dims
// 32t..32t+31, i.e. the two scale groups 2t and 2t+1, fetched with one 16-byte load per row.
// The group scale is folded into the A operand, so the eight MMAs of a set chain on one
// accumulator and nothing is scaled per group afterwards:
//   a nibble n masked in place at bits 4..7 of a 16-bit half is the fp16 value n * 2^-20;
//   fma(n * 2^-20, gs * 2^8, -8 gs * 2^-12) = (n - 8) gs * 2^-12, exact: |(n - 8) gs| <= 2040
//   has 11 significant bits and the result is a normal fp16 number (>= 2^-12).
// k slot pairs (2t, 2t+1) / (2t+8, 2t+9) of MMA 2i take nibbles (0, 4) / (1, 5) of the
// thread's word i, those of MMA 2i+1 nibbles (2, 6) / (3, 7); the B fragments carry the
// queries' dims in the same order.  Sum = 2^-12 sum_d level_d gs_g q_d.
__device__ __forceinline__ void int4c_scales(uint32_t h, uint32_t magic, uint32_t& G0, uint32_t& C0, uint32_t& G1, uint32_t& C1) {
    // h = the two scale bytes (groups 2t, 2t+1) -> half2 (gs * 256) twice and (-gs * 2^-9) twice
    uint32_t b0, b1;
    asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(b0) : "r"(prmt(h, magic, 0x5050u)), "r"(0xE400E400u));
    asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(b1) : "r"(prmt(h, magic, 0x5151u)), "r"(0xE400E400u));
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(G0) : "r"(b0), "r"(0x5C005C00u));
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(C0) : "r"(b0), "r"(0x98009800u));
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(G1) : "r"(b1), "r"(0x5C005C00u));
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(C1) : "r"(b1), "r"(0x98009800u));
}
__device__ __forceinline__ void int4c_word(uint32_t w, uint32_t G, uint32_t C, uint32_t (&o)[4]) {
    o[0] = hfma2_u32((w << 4) & 0x00F000F0u, G, C);  // nibbles 0, 4
    o[1] = hfma2_u32(w & 0x00F000F0u, G, C);         // nibbles 1, 5
    o[2] = hfma2_u32((w >> 4) & 0x00F000F0u, G, C);  // nibbles 2, 6
    o[3] = hfma2_u32((w >> 8) & 0x00F000F0u, G, C);  // nibbles 3, 7
}
// rb = shared address of row g of the staged set; t = lane & 3
__device__ __forceinline__ void coarse_set_int4c(uint32_t rb, uint32_t t, uint32_t magic, const uint32_t (&bq)[8][2], float& acc0, float& acc1) {
    const uint32_t cb = rb + 16u * t, hb = rb + 2u * t;
    const uint4 L0 = lds_v4<0>(cb), L1 = lds_v4<MMA_HALF>(cb);
    const uint32_t h0 = lds_u16<120>(hb), h1 = lds_u16<120 + MMA_HALF>(hb);
    uint32_t G00, C00, G01, C01, G10, C10, G11, C11;
    int4c_scales(h0, magic, G00, C00, G01, C01);
    int4c_scales(h1, magic, G10, C10, G11, C11);
    const uint32_t w0[4] = {L0.x, L0.y, L0.z, L0.w}, w1[4] = {L1.x, L1.y, L1.z, L1.w};
    float d[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t o0[4], o1[4];
        int4c_word(w0[i], i < 2 ? G00 : G01, i < 2 ? C00 : C01, o0);
        int4c_word(w1[i], i < 2 ? G10 : G11, i < 2 ? C10 : C11, o1);
        if (i == 0) mma_f16_zero(d, o0[0], o1[0], o0[1], o1[1], bq[0][0], bq[0][1]);
        else mma_f16(d, o0[0], o1[0], o0[1], o1[1], bq[2 * i][0], bq[2 * i][1]);
        mma_f16(d, o0[2], o1[2], o0[3], o1[3], bq[2 * i + 1][0], bq[2 * i + 1][1]);
    }
    acc0 = d[0] + d[1];
    acc1 = d[2] + d[3];
}

#ifdef SLHA_SCORE_PROFILE
// development aid (never built into the shipped library): per-CTA cycle counts of warp 0
__device__ unsigned long long g_score_prof[148 * 8];
__device__ unsigned long long g_sel_prof[148 * 8];  // calls, passes, refines, ties, cycles: minmax, passes, compaction
#define SEL_ADD(i, v) do { if (threadIdx.x == 0 && nq > 1 && blockIdx.x < 148) atomicAdd(&g_sel_prof[blockIdx.x * 8 + (i)], (unsigned long long)(v)); } while (0)
#define PROF_T(x) const long long x = clock64()
#define PROF_ADD(i, v) do { if (tid == 0) prof[i] += (unsigned long long)(v); } while (0)
#else
#define SEL_ADD(i, v)
#define PROF_T(x)
#define PROF_ADD(i, v)
#endif

// Bucket of a score inside [smin, smin + 256 / inv): monotone in the score.
__device__ __forceinline__ int sel_bucket_f(float sc, float smin, float inv) {
    const int b = (int)((sc - smin) * inv);
    return b < 0 ? 0 : (b > 255 ? 255 : b);
}
__device__ __forceinline__ int sel_bucket(uint32_t h, float smin, float inv) {
    return sel_bucket_f(key_score(h), smin, inv);
}
// Range [lo, hi] (order keys of scores) -> (smin, inv); false when the range cannot
// be bucketed (one single score, or a non-finite bound).
__device__ __forceinline__ bool sel_range(uint32_t lo, uint32_t hi, float& smin, float& inv) {
    smin = key_score(lo);
    const float smax = key_score(hi);
    inv = 256.0f / (smax - smin);
    return hi > lo && isfinite(smin) && isfinite(smax) && isfinite(inv);
}

// Shrinks up to four candidate buffers (keys[q][cap], counts cnt[q]) to between k
// and k + slack entries each and raises pivot[q] accordingly; only buffers with
// more than `trigger` entries are touched.  The four queries share every barrier.
//
// Selection works on the score (high word of the composite key): 256 equal-width
// buckets over [min, max] of the scores at or above the pivot; the bucket in which
// the count from the top reaches k is kept whole if that leaves at most k + slack
// keys, otherwise it becomes the next range.  Scores spread smoothly over such a
// range, so the histogram atomics do not pile up on one address the way the bytes
// of the key do.  Keys below the current pivot are dropped (the pivot is a proven
// lower bound of the query's k-th best key).  The new pivot is the smallest kept
// score.  Queries whose range collapses to one score with too many keys (equal
// scores), or holds a non-finite score, are reported in the returned bit mask
// (uniform over the block) and left for block_select_topk, which also orders by
// index.  hist: SEL_HIST_INTS ints.  All threads of the block must call.
// pivot_only: no selection, the buffers are only purged of keys below the pivot.
__device__ uint32_t block_select_multi(uint64_t* keys, uint32_t cap, int* cnt, int nq, uint32_t k, uint32_t slack,
                                       int trigger, uint64_t* pivot, int* hist, bool pivot_only = false) {
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
    // [q][8]: 0 range lo, 1 range hi, 2 need, 3 active, 4 exact selection wanted, 5 kept, 6 selected, 7 pivotal bucket
    uint32_t* st = reinterpret_cast<uint32_t*>(hist + 1024);
    if (tid < 4) {
        const bool act = tid < nq && cnt[tid] > trigger;
        uint32_t* s = st + 8 * tid;
        s[0] = pivot_only ? (tid < nq ? (uint32_t)(pivot[tid] >> 32) : 0u) : 0xFFFFFFFFu;
        s[1] = 0u;
        s[2] = k;
        s[3] = act && !pivot_only;
        s[4] = 0u;
        s[5] = 0u;
        s[6] = act;
        s[7] = 0u;
        if (act && cnt[tid] > (int)cap) cnt[tid] = (int)cap;
    }
    __syncthreads();
    if (!(st[6] | st[14] | st[22] | st[30])) return 0u;
    SEL_ADD(0, 1);
    PROF_T(ts0);
    // smallest and largest score at or above the pivot
    for (int q = 0; q < nq; ++q) {
        if (!st[8 * q + 3]) continue;
        const uint64_t* kq = keys + (size_t)q * cap;
        const uint32_t floor_h = (uint32_t)(pivot[q] >> 32);
        uint32_t mx = 0u, mn = 0xFFFFFFFFu;
        const int c = cnt[q];
#pragma unroll 4
        for (int i = tid; i < c; i += nt) {
            const uint32_t h = (uint32_t)(kq[i] >> 32);
            if (h >= floor_h) { mx = max(mx, h); mn = min(mn, h); }
        }
        mx = __reduce_max_sync(0xFFFFFFFFu, mx);
        mn = __reduce_min_sync(0xFFFFFFFFu, mn);
        if (lane == 0) { atomicMax(&st[8 * q + 1], mx); atomicMin(&st[8 * q], mn); }
    }
    __syncthreads();
    PROF_T(ts1);
    SEL_ADD(4, ts1 - ts0);
    for (int pass = 0; pass < 12; ++pass) {
        if (!(st[3] | st[11] | st[19] | st[27])) break;
        SEL_ADD(1, 1);
        for (int b = tid; b < 1024; b += nt) hist[b] = 0;
        __syncthreads();
        for (int q = 0; q < nq; ++q) {
            if (!st[8 * q + 3]) continue;
            const uint32_t lo = st[8 * q], hi = st[8 * q + 1];
            float smin, inv;
            if (!sel_range(lo, hi, smin, inv)) continue;  // settled by the scan below
            const uint64_t* kq = keys + (size_t)q * cap;
            // four keys per round: the loads go out together, then the atomics
            const int c = cnt[q];
            for (int i0 = tid; i0 < c; i0 += 4 * nt) {
                uint32_t h[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) h[u] = i0 + u * nt < c ? (uint32_t)(kq[i0 + u * nt] >> 32) : 0u;
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + u * nt < c && h[u] >= lo && h[u] <= hi) atomicAdd(&hist[256 * q + sel_bucket(h[u], smin, inv)], 1);
            }
        }
        __syncthreads();
        bool refine = false;
        if (warp < nq && st[8 * warp + 3]) {
            uint32_t* s = st + 8 * warp;
            const int* hq = hist + 256 * warp;
            const uint32_t lo = s[0], hi = s[1], need = s[2];
            float smin, inv;
            if (!sel_range(lo, hi, smin, inv)) {
                // everything left in the range stays; more than allowed means equal
                // (or non-finite) scores: the exact selection sorts it out
                __syncwarp();
                if (lane == 0) { s[3] = 0u; s[4] = 1u; s[7] = 0u; }
            } else {
                // lane l owns buckets 255-8l .. 248-8l (descending)
                int c[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { c[j] = hq[255 - 8 * lane - j]; tot += c[j]; }
                int incl = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if (lane >= o) incl += y;
                }
                const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= (int)need);
                if (ok == 0u) {
                    // fewer than `need` keys at or above the pivot: all of them stay
                    if (lane == 0) { s[3] = 0u; s[7] = 0u; }
                } else {
                    int bsel = 0, run = 0, binc = 0;
                    if (lane == __ffs(ok) - 1) {
                        run = incl - tot;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (run + c[j] >= (int)need) { bsel = 255 - 8 * lane - j; binc = c[j]; break; }
                            run += c[j];
                        }
                    }
                    const int src = __ffs(ok) - 1;
                    bsel = __shfl_sync(0xFFFFFFFFu, bsel, src);
                    run = __shfl_sync(0xFFFFFFFFu, run, src);
                    binc = __shfl_sync(0xFFFFFFFFu, binc, src);
                    const uint32_t kept = (k - need) + (uint32_t)(run + binc);
                    if (kept <= k + slack) {
                        if (lane == 0) { s[3] = 0u; s[7] = (uint32_t)bsel; }
                    } else {
                        // next range: the scores of the pivotal bucket
                        refine = true;
                        __syncwarp();
                        if (lane == 0) { s[2] = need - (uint32_t)run; s[7] = (uint32_t)bsel; }
                    }
                }
            }
        }
        if (!__syncthreads_or(refine)) continue;
        SEL_ADD(2, 1);
        // smallest and largest score inside the pivotal bucket of the queries still active
        uint32_t nlo[4], nhi[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { nlo[q] = 0xFFFFFFFFu; nhi[q] = 0u; }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (q >= nq || !st[8 * q + 3]) continue;
            const uint32_t lo = st[8 * q], hi = st[8 * q + 1];
            const int bsel = (int)st[8 * q + 7];
            float smin, inv;
            sel_range(lo, hi, smin, inv);
            const uint64_t* kq = keys + (size_t)q * cap;
            for (int i = tid; i < cnt[q]; i += nt) {
                const uint32_t h = (uint32_t)(kq[i] >> 32);
                if (h >= lo && h <= hi && sel_bucket(h, smin, inv) == bsel) { nlo[q] = min(nlo[q], h); nhi[q] = max(nhi[q], h); }
            }
            nlo[q] = __reduce_min_sync(0xFFFFFFFFu, nlo[q]);
            nhi[q] = __reduce_max_sync(0xFFFFFFFFu, nhi[q]);
        }
        __syncthreads();  // every thread has read the old range
        if (tid < 4 && tid < nq && st[8 * tid + 3]) { st[8 * tid] = 0xFFFFFFFFu; st[8 * tid + 1] = 0u; }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (q < nq && st[8 * q + 3] && lane == 0) { atomicMin(&st[8 * q], nlo[q]); atomicMax(&st[8 * q + 1], nhi[q]); }
        __syncthreads();
    }
    PROF_T(ts2);
    SEL_ADD(5, ts2 - ts1);
    // (a range that is still open after the last pass stays whole and goes to the exact selection)
    if (tid < 4) {
        if (st[8 * tid + 3]) { st[8 * tid + 3] = 0u; st[8 * tid + 4] = 1u; st[8 * tid + 7] = 0u; }
        st[8 * tid + 2] = 0xFFFFFFFFu;  // from here on: the smallest score kept
    }
    __syncthreads();
    // compact the selected buffers in place: keys above the last range, and those of
    // the range whose bucket is the pivotal one or higher, stay
    int maxc = 0;
    for (int q = 0; q < nq; ++q)
        if (st[8 * q + 6]) maxc = max(maxc, cnt[q]);
    const int R = (maxc + nt - 1) / nt;
    if (R <= 10) {
        // every warp owns R*32 consecutive slots: it reads them all, the warps' counts are
        // summed once, then it writes its survivors (order preserved, no read-after-write)
        int* wcnt = hist;  // [4][32]
#pragma unroll 1
        for (int q = 0; q < nq; ++q) {
            if (!st[8 * q + 6]) continue;
            const uint32_t rlo = st[8 * q], rhi = st[8 * q + 1];
            int bsel = (int)st[8 * q + 7];
            float smin, inv;
            if (!sel_range(rlo, rhi, smin, inv)) bsel = -1;  // whole range stays
            uint64_t* kq = keys + (size_t)q * cap;
            const int c = cnt[q];
            uint64_t key[10];
            unsigned bal[10];
            int wtot = 0;
            uint32_t km = 0xFFFFFFFFu;
#pragma unroll
            for (int j = 0; j < 10; ++j) {
                bal[j] = 0u;
                key[j] = 0ull;
                if (j < R) {
                    const int i = (warp * R + j) * 32 + lane;
                    const bool in = i < c;
                    key[j] = in ? kq[i] : 0ull;
                    const uint32_t h = (uint32_t)(key[j] >> 32);
                    const bool keep = in && h >= rlo && (h > rhi || bsel < 0 || sel_bucket(h, smin, inv) >= bsel);
                    if (keep) km = min(km, h);
                    bal[j] = __ballot_sync(0xFFFFFFFFu, keep);
                    wtot += __popc(bal[j]);
                }
            }
            km = __reduce_min_sync(0xFFFFFFFFu, km);
            if (lane == 0) {
                wcnt[q * 32 + warp] = wtot;
                if (km != 0xFFFFFFFFu) atomicMin(&st[8 * q + 2], km);
            }
            __syncthreads();
            const int v = lane < (nt >> 5) ? wcnt[q * 32 + lane] : 0;
            int run = __reduce_add_sync(0xFFFFFFFFu, lane < warp ? v : 0);
            const int total = __reduce_add_sync(0xFFFFFFFFu, v);
#pragma unroll
            for (int j = 0; j < 10; ++j) {
                if (j < R) {
                    if (bal[j] >> lane & 1u) kq[run + __popc(bal[j] & ((1u << lane) - 1u))] = key[j];
                    run += __popc(bal[j]);
                }
            }
            if (tid == 0) st[8 * q + 5] = (uint32_t)total;
        }
        __syncthreads();
    } else {
        float smin[4], inv[4];
        uint32_t rlo[4], rhi[4];
        int bsel[4];
        uint32_t kmin[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            kmin[q] = 0xFFFFFFFFu;
            rlo[q] = rhi[q] = 0u;
            bsel[q] = 0;
            smin[q] = inv[q] = 0.0f;
            if (q < nq && st[8 * q + 6]) {
                rlo[q] = st[8 * q];
                rhi[q] = st[8 * q + 1];
                bsel[q] = (int)st[8 * q + 7];
                if (!sel_range(rlo[q], rhi[q], smin[q], inv[q])) bsel[q] = -1;  // whole range stays
            }
        }
        for (int i0 = 0; i0 < maxc; i0 += nt) {
            const int i = i0 + tid;
            uint64_t key[4];
            bool keep[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const bool in = q < nq && st[8 * q + 6] && i < cnt[q];
                key[q] = in ? keys[(size_t)q * cap + i] : 0ull;
                const uint32_t h = (uint32_t)(key[q] >> 32);
                keep[q] = in && h >= rlo[q] && (h > rhi[q] || bsel[q] < 0 || sel_bucket(h, smin[q], inv[q]) >= bsel[q]);
                if (keep[q]) kmin[q] = min(kmin[q], h);
            }
            __syncthreads();  // every read of this round precedes its writes (they land below i0 + nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const unsigned bal = __ballot_sync(0xFFFFFFFFu, keep[q]);
                if (bal) {
                    int base = 0;
                    if (lane == 0) base = (int)atomicAdd(&st[8 * q + 5], (uint32_t)__popc(bal));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    if (keep[q]) keys[(size_t)q * cap + base + __popc(bal & ((1u << lane) - 1u))] = key[q];
                }
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (q >= nq || !st[8 * q + 6]) continue;
            const uint32_t m = __reduce_min_sync(0xFFFFFFFFu, kmin[q]);
            if (lane == 0 && m != 0xFFFFFFFFu) atomicMin(&st[8 * q + 2], m);
        }
        __syncthreads();
    }
    // the new pivot: the smallest score kept, provided k keys were kept (fewer prove nothing)
    if (tid < 4 && st[8 * tid + 6]) {
        cnt[tid] = (int)st[8 * tid + 5];
        const uint64_t np = st[8 * tid + 2] == 0xFFFFFFFFu ? 0ull : (uint64_t)st[8 * tid + 2] << 32;
        if (st[8 * tid + 5] >= k && np > pivot[tid]) pivot[tid] = np;
    }
    uint32_t ties = 0u;
#pragma unroll
    for (int q = 0; q < 4; ++q)
        if (st[8 * q + 6] && st[8 * q + 4] && st[8 * q + 5] > k + slack) ties |= 1u << q;
    __syncthreads();
    PROF_T(ts3);
    SEL_ADD(6, ts3 - ts2);
    SEL_ADD(3, ties != 0u);
    return ties;
}

// State of one work item of score_mma_kernel that its helper functions share.
struct MmaItem {
    uint64_t* keys;    // [4][nwarps][rs] candidate regions
    uint64_t* pivot;   // [4]
    int* cntw;         // [4][32] published region counts
    int* bail;
    float2* rng;       // [4]
    int* hist;         // SEL_HIST_INTS
    uint32_t rs;       // slots per region
    int room;          // rs - MMA_SET_TILES
    uint32_t sel_slack;
    uint32_t query_begin;
    int nq;
};

// Thresholds are shared between the CTAs that scan the same query's tiles: a CTA's
// pivot (k of its own elements are >= it) is a proven lower bound of the query's k-th
// best composite key, so the maximum over CTAs is too.  Lanes 0..nq-1 of one warp.
__device__ __forceinline__ void mma_refresh_pivots(const ScoreArgs& a, const MmaItem& m, int lane) {
    if (lane < m.nq) {
        const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(a.gpivot + m.query_begin + lane);
        if (seen > m.pivot[lane]) m.pivot[lane] = seen;
    }
}

// Shared score histogram of a query: every CTA counts the candidates it appends into
// 256 buckets of global memory (one bucket mapping per query, published by the first
// CTA that finishes a selection).  The counts are of real tiles, so the lower edge of
// the highest bucket whose count from the top reaches k is a proven lower bound of the
// query's k-th best score - for all CTAs at once, and without a block-wide selection.
// A whole warp calls this for query q.
__device__ __forceinline__ void mma_hist_pivot(const ScoreArgs& a, const MmaItem& m, int q, int lane) {
    const float2 r = m.rng[q];
    if (r.y == 0.0f) return;
    const uint32_t* hq = a.ghist + (size_t)(m.query_begin + q) * 256 + 248 - 8 * lane;
    uint32_t c[8];  // buckets 255-8l .. 248-8l (descending)
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(c[7]), "=r"(c[6]), "=r"(c[5]), "=r"(c[4]) : "l"(hq));
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(c[3]), "=r"(c[2]), "=r"(c[1]), "=r"(c[0]) : "l"(hq + 4));
    uint32_t tot = 0;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) tot += c[jj];
    uint32_t incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += y;
    }
    const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= a.k);
    if (ok == 0u || lane != __ffs(ok) - 1) return;
    uint32_t run = incl - tot;
    int b = 0;
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
        if (run + c[jj] >= a.k) { b = 255 - 8 * lane - jj; break; }
        run += c[jj];
    }
    if (b < 1) return;
    // half a bucket and a few ulps below the bucket's edge: every counted key of the
    // buckets b.. is above this bound whatever the rounding of the bucket arithmetic
    const float e = r.x + ((float)b - 0.5f) / fabsf(r.y);
    const uint32_t ek = score_key(e);
    const unsigned long long np = (unsigned long long)(ek > 8u ? ek - 8u : 0u) << 32;
    if (np > m.pivot[q]) {
        m.pivot[q] = np;
        atomicMax(a.gpivot + m.query_begin + q, np);
    }
}

// The calling warp drops the keys of its region of query tq that are below the pivot.
// rc: the caller's count of the region of its own query t (updated when t == tq).
__device__ __forceinline__ void mma_purge(const MmaItem& m, int tq, int warp, int nwarps, int lane, int t, int& rc) {
    const int cn = __shfl_sync(0xFFFFFFFFu, rc, tq);  // lane tq is (g = 0, t = tq)
    const uint64_t pv = m.pivot[tq];
    uint64_t* reg = m.keys + (size_t)(tq * nwarps + warp) * m.rs;
    const uint32_t lt_mask = (1u << lane) - 1u;
    int kept = 0;
    for (int i0 = 0; i0 < cn; i0 += 32) {
        const int i = i0 + lane;
        const uint64_t key = i < cn ? reg[i] : 0ull;
        const bool keep = i < cn && key >= pv;
        const unsigned bal = __ballot_sync(0xFFFFFFFFu, keep);  // all reads of the round are done
        if (keep) reg[kept + __popc(bal & lt_mask)] = key;      // lands at or below its old slot
        kept += __popc(bal);
    }
    __syncwarp();
    if (t == tq) rc = kept;
}

// Selection over segmented candidate buffers.  Query q's candidates live in one
// region per warp: m.keys[(q * nw + w) * rs ..] holds m.cntw[q * 32 + w] keys, appended
// and purged by warp w alone.  For every query in `mask` this raises m.pivot[q] so that
// between k and about k + slack of the query's keys stay at or above it; nothing is
// moved - every warp purges its own regions against the new pivots afterwards.
//
// The first histogram pass uses the query's shared bucket mapping (m.rng; created from
// the smallest and largest score in the buffer and published when the query has none
// yet), so the same counts serve two purposes: they are added to the query's shared
// histogram in global memory when this CTA's buffer has not been counted there yet
// (mapping stored negated in m.rng), and they locate the bucket in which the count from
// the top reaches k.  While that bucket is too full it becomes the next range, with 256
// buckets between its smallest and largest score.  The new pivot is half a bucket below
// the pivotal bucket's lower edge.  Returns the queries that cannot be settled this way
// (equal or non-finite scores).  All threads of the block must call; warp w sweeps
// region w.
__device__ __noinline__ uint32_t block_select_seg(const ScoreArgs& a, const MmaItem& m, uint32_t mask, uint32_t slack) {
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nw = nt >> 5;
    const int nq = m.nq;
    const uint32_t k = a.k;
    int* hist = m.hist;
    // [q][8]: 0 range lo, 1 range hi (score words, inclusive), 2 need, 3 active, 4 failed, 5 nothing to raise,
    //         6 selected, 7 pivotal bucket (0xFFFFFFFF: the keys below the mapping)
    uint32_t* st = reinterpret_cast<uint32_t*>(hist + 1024);
    float* fm = reinterpret_cast<float*>(hist + 1024 + 32);           // [q][2] smin, inv of the current pass
    uint32_t* below = reinterpret_cast<uint32_t*>(hist + 1024 + 40);  // [q] keys below the mapping (first pass)
    uint32_t* flush = below + 4;                                      // [q] first-pass counts go to the shared histogram
    if (tid < 4) {
        const bool act = tid < nq && (mask >> tid & 1u);
        uint32_t* s = st + 8 * tid;
        s[0] = act ? (uint32_t)(m.pivot[tid] >> 32) : 0u;
        s[1] = 0xFFFFFFFFu;
        s[2] = k;
        s[3] = act;
        s[4] = 0u;
        s[5] = 0u;
        s[6] = act;
        s[7] = 0u;
        below[tid] = 0u;
        flush[tid] = 0u;
        reinterpret_cast<uint32_t*>(hist)[tid] = 0xFFFFFFFFu;  // smallest / largest score word for a new mapping
        hist[4 + tid] = 0;
    }
    __syncthreads();
    if (!(st[6] | st[14] | st[22] | st[30])) return 0u;
    // queries without a mapping: smallest and largest score in the buffer
    bool fresh = false;
    for (int q = 0; q < nq; ++q) fresh |= st[8 * q + 3] && m.rng[q].y == 0.0f;
    if (fresh) {
        for (int q = 0; q < nq; ++q) {
            if (!st[8 * q + 3] || m.rng[q].y != 0.0f) continue;
            const uint64_t* kq = m.keys + (size_t)(q * nw + warp) * m.rs;
            const int c = m.cntw[q * 32 + warp];
            uint32_t mx = 0u, mn = 0xFFFFFFFFu;
            for (int i = lane; i < c; i += 32) {
                const uint32_t h = (uint32_t)(kq[i] >> 32);
                mx = max(mx, h);
                mn = min(mn, h);
            }
            mx = __reduce_max_sync(0xFFFFFFFFu, mx);
            mn = __reduce_min_sync(0xFFFFFFFFu, mn);
            if (lane == 0) { atomicMin(reinterpret_cast<uint32_t*>(hist) + q, mn); atomicMax(reinterpret_cast<uint32_t*>(hist) + 4 + q, mx); }
        }
        __syncthreads();
        if (tid < nq && st[8 * tid + 3] && m.rng[tid].y == 0.0f) {
            // from the smallest score to a quarter of the span above the largest; the first CTA to publish wins
            const float lo = key_score(reinterpret_cast<uint32_t*>(hist)[tid]), top = key_score(reinterpret_cast<uint32_t*>(hist)[4 + tid]);
            const float hi = top + 0.25f * (top - lo);
            const float inv = 256.0f / (hi - lo);
            if (isfinite(lo) && isfinite(hi) && isfinite(inv) && inv > 0.0f) {
                const unsigned long long mine_r = (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(inv) << 32);
                const unsigned long long old = atomicCAS(a.grange + m.query_begin + tid, 0ull, mine_r);
                const unsigned long long use = old ? old : mine_r;
                m.rng[tid] = make_float2(__uint_as_float((uint32_t)use), -__uint_as_float((uint32_t)(use >> 32)));
            } else {
                st[8 * tid + 3] = 0u;
                st[8 * tid + 4] = 1u;
            }
        }
        __syncthreads();
    }
    if (tid < nq && st[8 * tid + 3]) {
        const float2 r = m.rng[tid];
        fm[2 * tid] = r.x;
        fm[2 * tid + 1] = fabsf(r.y);
        flush[tid] = r.y < 0.0f;
    }
    for (int pass = 0; pass < 12; ++pass) {
        for (int b = tid; b < 1024; b += nt) hist[b] = 0;
        __syncthreads();
        if (!(st[3] | st[11] | st[19] | st[27])) break;
        for (int q = 0; q < nq; ++q) {
            if (!st[8 * q + 3]) continue;
            const uint32_t lo = st[8 * q], hi = st[8 * q + 1];
            const float smin = fm[2 * q], inv = fm[2 * q + 1];
            const uint64_t* kq = m.keys + (size_t)(q * nw + warp) * m.rs;
            const int c = m.cntw[q * 32 + warp];
            for (int i = lane; i < c; i += 32) {
                const uint32_t h = (uint32_t)(kq[i] >> 32);
                if (h < lo || h > hi) continue;
                const float sc = key_score(h);
                if (sc < smin) atomicAdd(&below[q], 1u);
                else atomicAdd(&hist[256 * q + sel_bucket_f(sc, smin, inv)], 1);
            }
        }
        __syncthreads();
        if (pass == 0) {
            // this CTA's buffer enters the query's shared histogram
            for (int b = tid; b < 1024; b += nt) {
                const int q = b >> 8;
                if (q < nq && flush[q] && hist[b]) atomicAdd(a.ghist + (size_t)(m.query_begin + q) * 256 + (b & 255), (uint32_t)hist[b]);
            }
        }
        bool refine = false;
        if (warp < nq && st[8 * warp + 3]) {
            uint32_t* s = st + 8 * warp;
            const int* hq = hist + 256 * warp;
            const uint32_t need = s[2];
            // lane l owns buckets 255-8l .. 248-8l (descending)
            int c[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { c[j] = hq[255 - 8 * lane - j]; tot += c[j]; }
            int incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += y;
            }
            const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= (int)need);
            const int total = __shfl_sync(0xFFFFFFFFu, incl, 31);
            if (ok == 0u) {
                if ((uint32_t)total + below[warp] < need) {
                    // fewer than `need` keys at or above the pivot: nothing can be proven
                    if (lane == 0) { s[3] = 0u; s[5] = 1u; }
                } else {
                    // the k-th key lies below the mapping: the keys down there are the next range
                    refine = true;
                    __syncwarp();
                    if (lane == 0) { s[2] = need - (uint32_t)total; s[7] = 0xFFFFFFFFu; }
                }
            } else {
                int bsel = 0, run = 0, binc = 0;
                const int src = __ffs(ok) - 1;
                if (lane == src) {
                    run = incl - tot;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (run + c[j] >= (int)need) { bsel = 255 - 8 * lane - j; binc = c[j]; break; }
                        run += c[j];
                    }
                }
                bsel = __shfl_sync(0xFFFFFFFFu, bsel, src);
                run = __shfl_sync(0xFFFFFFFFu, run, src);
                binc = __shfl_sync(0xFFFFFFFFu, binc, src);
                const uint32_t kept = (k - need) + (uint32_t)(run + binc);
                if (kept <= k + slack) {
                    if (lane == 0) { s[3] = 0u; s[7] = (uint32_t)bsel; }
                } else {
                    refine = true;  // next range: the scores of the pivotal bucket
                    __syncwarp();
                    if (lane == 0) { s[2] = need - (uint32_t)run; s[7] = (uint32_t)bsel; }
                }
            }
        }
        if (!__syncthreads_or(refine)) continue;
        // smallest and largest score inside the pivotal bucket of the queries still active
        uint32_t nlo[4], nhi[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) { nlo[q] = 0xFFFFFFFFu; nhi[q] = 0u; }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (q >= nq || !st[8 * q + 3]) continue;
            const uint32_t lo = st[8 * q], hi = st[8 * q + 1];
            const int bsel = (int)st[8 * q + 7];
            const float smin = fm[2 * q], inv = fm[2 * q + 1];
            const uint64_t* kq = m.keys + (size_t)(q * nw + warp) * m.rs;
            const int c = m.cntw[q * 32 + warp];
            for (int i = lane; i < c; i += 32) {
                const uint32_t h = (uint32_t)(kq[i] >> 32);
                if (h < lo || h > hi) continue;
                const float sc = key_score(h);
                const int b = sc < smin ? -1 : sel_bucket_f(sc, smin, inv);
                if (b == bsel) { nlo[q] = min(nlo[q], h); nhi[q] = max(nhi[q], h); }
            }
            nlo[q] = __reduce_min_sync(0xFFFFFFFFu, nlo[q]);
            nhi[q] = __reduce_max_sync(0xFFFFFFFFu, nhi[q]);
        }
        __syncthreads();  // every thread has read the old range
        if (tid < 4 && tid < nq && st[8 * tid + 3]) { st[8 * tid] = 0xFFFFFFFFu; st[8 * tid + 1] = 0u; below[tid] = 0u; }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (q < nq && st[8 * q + 3] && lane == 0) { atomicMin(&st[8 * q], nlo[q]); atomicMax(&st[8 * q + 1], nhi[q]); }
        __syncthreads();
        if (tid < nq && st[8 * tid + 3]) {
            float smin, inv;
            if (sel_range(st[8 * tid], st[8 * tid + 1], smin, inv)) {
                fm[2 * tid] = smin;
                fm[2 * tid + 1] = inv;
            } else {
                st[8 * tid + 3] = 0u;  // one single score, too many keys: equal scores
                st[8 * tid + 4] = 1u;
            }
        }
    }
    if (tid < 4 && st[8 * tid + 6] && st[8 * tid + 3]) { st[8 * tid + 3] = 0u; st[8 * tid + 4] = 1u; }  // still open after the last pass
    __syncthreads();
    // The new pivot is the smallest score of the pivotal bucket: exactly the keys counted
    // above stay.  Warp w reports the minimum of its region, thread q combines them.
    {
        uint32_t* wmin = reinterpret_cast<uint32_t*>(hist);  // [q][32]
#pragma unroll 1
        for (int q = 0; q < nq; ++q) {
            if (!st[8 * q + 6] || st[8 * q + 4] || st[8 * q + 5]) continue;
            const uint32_t lo = st[8 * q], hi = st[8 * q + 1];
            const int bsel = (int)st[8 * q + 7];
            const float smin = fm[2 * q], inv = fm[2 * q + 1];
            const uint64_t* kq = m.keys + (size_t)(q * nw + warp) * m.rs;
            const int c = m.cntw[q * 32 + warp];
            uint32_t mn = 0xFFFFFFFFu;
            for (int i = lane; i < c; i += 32) {
                const uint32_t h = (uint32_t)(kq[i] >> 32);
                if (h < lo || h > hi) continue;
                const float sc = key_score(h);
                const int b = sc < smin ? -1 : sel_bucket_f(sc, smin, inv);
                if (b == bsel) mn = min(mn, h);
            }
            mn = __reduce_min_sync(0xFFFFFFFFu, mn);
            if (lane == 0) wmin[q * 32 + warp] = mn;
        }
        __syncthreads();
        if (tid < nq && st[8 * tid + 6] && !st[8 * tid + 4] && !st[8 * tid + 5]) {
            uint32_t mn = 0xFFFFFFFFu;
            for (int w = 0; w < nw; ++w) mn = min(mn, wmin[tid * 32 + w]);
            const uint64_t np = (uint64_t)mn << 32;
            if (mn != 0xFFFFFFFFu && np > m.pivot[tid]) m.pivot[tid] = np;
        }
        if (tid < 4 && st[8 * tid + 6] && flush[tid]) m.rng[tid].y = fabsf(m.rng[tid].y);  // the buffer is counted: appends count themselves from now on
    }
    __syncthreads();
    const uint32_t failed = (st[4] ? 1u : 0u) | (st[12] ? 2u : 0u) | (st[20] ? 4u : 0u) | (st[28] ? 8u : 0u);
    __syncthreads();
    return failed;
}

// Evens out the region counts of query q: warps holding more than the average hand
// their surplus keys (the tail of their region) to warps holding less, through a
// 512-key staging area in m.hist.  Any key may live in any region, so this only makes
// room; it is needed when the best candidates cluster in the sets of a few warps.
// All threads of the block; region counts published.  Returns the caller's count.
__device__ __noinline__ int mma_rebalance(const MmaItem& m, int q, int rc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5, t = lane & 3;
    const int c = lane < nw ? m.cntw[q * 32 + lane] : 0;
    const int total = __reduce_add_sync(0xFFFFFFFFu, c);
    const int target = (total + nw - 1) / nw;
    const int sur = lane < nw ? max(0, c - target) : 0, def = lane < nw ? max(0, target - c) : 0;
    int s_in = sur, d_in = def;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, s_in, o), z = __shfl_up_sync(0xFFFFFFFFu, d_in, o);
        if (lane >= o) { s_in += y; d_in += z; }
    }
    const int moved = __shfl_sync(0xFFFFFFFFu, s_in, 31);
    const int c_me = __shfl_sync(0xFFFFFFFFu, c, warp);
    const int sur_me = __shfl_sync(0xFFFFFFFFu, sur, warp), s_me = __shfl_sync(0xFFFFFFFFu, s_in - sur, warp);
    const int def_me = __shfl_sync(0xFFFFFFFFu, def, warp), d_me = __shfl_sync(0xFFFFFFFFu, d_in - def, warp);
    uint64_t* reg = m.keys + (size_t)(q * nw + warp) * m.rs;
    uint64_t* staging = reinterpret_cast<uint64_t*>(m.hist);  // 512 keys
    for (int c0 = 0; c0 < moved; c0 += 512) {
        {
            const int lo = max(s_me, c0), hi = min(s_me + sur_me, c0 + 512);
            for (int j = lo + lane; j < hi; j += 32) staging[j - c0] = reg[target + (j - s_me)];
        }
        __syncthreads();
        {
            const int lo = max(d_me, c0), hi = min(d_me + def_me, min(moved, c0 + 512));
            for (int j = lo + lane; j < hi; j += 32) reg[c_me + (j - d_me)] = staging[j - c0];
        }
        __syncthreads();
    }
    const int now = sur_me > 0 ? target : c_me + max(0, min(def_me, moved - d_me));
    if (lane == 0) m.cntw[q * 32 + warp] = now;
    __syncthreads();
    return t == q ? now : rc;
}

// Block-wide step, entered by all threads after a barrier: refresh the thresholds
// (shared histogram, other CTAs), let every warp purge its regions, and run a selection
// only for queries that still lack room (final: whose candidates still exceed the list
// size).  Sets *bail when a query cannot be settled.  Returns the caller's region count.
__device__ __noinline__ int mma_settle(const ScoreArgs& a, const MmaItem& m, int rc, bool final) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5, t = lane & 3;
    const int nq = m.nq;
    PROF_T(s0);
    SEL_ADD(0, 1);
    // a bucket mapping another CTA has published meanwhile: known from now on, but this
    // CTA's buffer is not in the shared histogram yet (negated inv, see block_select_seg)
    if (tid < nq && m.rng[tid].y == 0.0f) {
        const unsigned long long pr = *reinterpret_cast<volatile unsigned long long*>(a.grange + m.query_begin + tid);
        if (pr) m.rng[tid] = make_float2(__uint_as_float((uint32_t)pr), -__uint_as_float((uint32_t)(pr >> 32)));
    }
    if (lane < 4) m.cntw[lane * 32 + warp] = rc;  // lane l < 4 is (g = 0, t = l)
    __syncthreads();
    if (warp < nq) mma_hist_pivot(a, m, warp, lane);
    if (warp == nwarps - 1) mma_refresh_pivots(a, m, lane);
    __syncthreads();
    PROF_T(s1);
    SEL_ADD(1, s1 - s0);
    const bool any_pivot = (m.pivot[0] | m.pivot[1] | m.pivot[2] | m.pivot[3]) != 0ull;
#pragma unroll 1
    for (int attempt = 0; attempt < 4; ++attempt) {
        PROF_T(s2);
        if (attempt > 0 || any_pivot) {
#pragma unroll 1
            for (int tq = 0; tq < nq; ++tq) mma_purge(m, tq, warp, nwarps, lane, t, rc);
            if (lane < 4) m.cntw[lane * 32 + warp] = rc;
            __syncthreads();
        }
        PROF_T(s3);
        SEL_ADD(2, s3 - s2);
        SEL_ADD(7, 1);
        uint32_t over = 0u, even = 0u;  // queries lacking room; of those, the ones a redistribution settles
#pragma unroll 1
        for (int q = 0; q < nq; ++q) {
            const int v = lane < nwarps ? m.cntw[q * 32 + lane] : 0;
            const int tot = __reduce_add_sync(0xFFFFFFFFu, v), mx = __reduce_max_sync(0xFFFFFFFFu, v);
            if (final ? tot > (int)a.list_cap : mx > m.room - 2 * MMA_SET_TILES) {
                over |= 1u << q;
                // few enough keys in all (a selection ran, or would drop nothing): only their spread is the problem
                if (!final && tot <= nwarps * (m.room - 4 * MMA_SET_TILES) && (attempt > 0 || tot <= (int)(a.k + m.sel_slack))) even |= 1u << q;
            }
        }
        if (!over) break;
        uint32_t failed = attempt == 3 ? over : 0u;
        if (!failed && (over & ~even)) failed = block_select_seg(a, m, over & ~even, final ? a.list_cap - a.k : m.sel_slack);
        PROF_T(s4);
        SEL_ADD(3, s4 - s3);
        if (failed) {
            SEL_ADD(attempt == 3 ? 5 : 6, 1);
            // equal scores: the generic kernel takes the item
            if (tid == 0) *m.bail = 1;
            break;
        }
#pragma unroll 1
        for (int q = 0; q < nq; ++q)
            if (even >> q & 1u) rc = mma_rebalance(m, q, rc);
    }
    if (tid < nq) atomicMax(a.gpivot + m.query_begin + tid, (unsigned long long)m.pivot[tid]);
    __syncthreads();
    return rc;
}

// KIND 0: nibble codecs (INT4, MX-INT4, NF4); 1: the launch scores mixed 8/4 tiles; 2: TQ3 tiles,
// rewritten in shared memory as nibble rows (2 code + correction bit) before the INT4 path scores
// them.  Separate instantiations, so that the nibble-codec kernel is exactly the code it was.
// EARLY: many CTAs share every query (one long segment cut over the whole grid).  After one set
// of every warp the query's shared histogram already holds far more than k candidates, so four
// warps per CTA fetch a first threshold after their 2nd..5th set instead of waiting for their
// regions to fill, which they would all do at the same moment.
template <bool TOPK, int KIND = 0, bool EARLY = false>
__global__ void __launch_bounds__(512, 1) score_mma_kernel(ScoreArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // shared layout: nf4 table | stage ring | [keys | pivot | cntw | outpos | ctl | rng | hist]
    const uint32_t lut_bytes = a.nf4_table ? NF4_LUT_BYTES : 0;  // the table is left out when no NF4 tile is expected
    uint2* lut = reinterpret_cast<uint2*>(smem);
    unsigned char* tail = smem + lut_bytes + (size_t)nwarps * MMA_DEPTH * MMA_SET_STRIDE;
    // Candidates of query q kept by warp w: keys[(q * nwarps + w) * rs ..], rs = cap / nwarps.
    // A warp appends to and purges its own regions without any block-wide step.
    uint64_t* keys = reinterpret_cast<uint64_t*>(tail);            // [4][nwarps][rs]
    uint64_t* pivot = keys + (TOPK ? (size_t)4 * a.cap : 0);       // [4]
    int* cntw = reinterpret_cast<int*>(pivot + 4);                 // [4][32] region counts, published for block-wide steps
    int* outpos = cntw + 128;                                      // [4] write position in the item's candidate lists
    int* ctl = outpos + 4;  // [0] want: a warp cannot make room alone  [1] arrived  [2] done warps  [3] bail
    int* bail = ctl + 3;
    float2* rng = reinterpret_cast<float2*>(ctl + 4);  // [4] (smin, inv) of the query's shared score histogram; inv 0 = none yet
    int* hist = ctl + 12;  // SEL_HIST_INTS
    const uint32_t smem_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t stage_s = smem_s + lut_bytes + (uint32_t)warp * MMA_DEPTH * MMA_SET_STRIDE;

    // NF4 codebook as fp16 hi + lo pairs per byte (two nibbles), 16 bank-aligned replicas
    for (int e = tid; e < (a.nf4_table ? 256 * 16 : 0); e += blockDim.x) {
        const int b = e >> 4;
        const float c0 = c_nf4[b & 15], c1 = 16.0f * c_nf4[b >> 4];  // odd slots carry 16x (see int4_quad)
        lut[e] = make_uint2(pack_half2(c0, c1), pack_half2(half_residual(c0), half_residual(c1)));
    }
    const uint32_t lut_lane = smem_s + (uint32_t)(lane & 15) * 8u;
    uint32_t magic;  // 1024.0h twice, opaque so that it stays in one register
    asm volatile("mov.u32 %0, 0x64006400;\n" : "=r"(magic));
    // cp.async of a set: lane copies the 16-byte chunks lane, lane+32, lane+64, lane+96,
    // i.e. chunk (lane & 7) of rows (lane >> 3) + {0, 4, 8, 12}
    const uint32_t dst_lane = (uint32_t)((lane >> 3) * MMA_ROW + (lane & 7) * 16);
    const uint32_t row_lane = (uint32_t)g * MMA_ROW;
    const uint32_t rs = a.cap / (uint32_t)nwarps;          // slots per region
    const int room = (int)rs - MMA_SET_TILES;              // a set adds at most 16 keys to a region
    const uint32_t sel_slack = (a.cap - (uint32_t)nwarps * MMA_SET_TILES - a.k) / 4;
    uint64_t* my_reg = keys + (size_t)(t * nwarps + warp) * rs;  // region of query t of this warp
    const uint32_t lt_mask = (1u << lane) - 1u, t_mask = 0x11111111u << t;

#ifdef SLHA_SCORE_PROFILE
    unsigned long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#endif
    const uint32_t item_end = a.cta_begin[blockIdx.x + 1];
    for (uint32_t item_id = a.cta_begin[blockIdx.x]; item_id < item_end; ++item_id) {
        const WorkItem it = a.items[item_id];
        const int nq = (int)it.n_queries;
        PROF_T(t_item);
        __syncthreads();  // previous item fully retired (and the table is visible)
        if (TOPK && tid < 4) {
            // start from the threshold other CTAs have already proven for the query, and
            // from the query's shared histogram range if one has been published
            const bool have = tid < nq;
            outpos[tid] = 0;
            pivot[tid] = have ? *reinterpret_cast<volatile unsigned long long*>(a.gpivot + it.query_begin + tid) : 0ull;
            const unsigned long long pr = have ? *reinterpret_cast<volatile unsigned long long*>(a.grange + it.query_begin + tid) : 0ull;
            rng[tid] = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
        }
        if (tid == 0) { ctl[0] = ctl[1] = ctl[2] = ctl[3] = 0; }
        // B fragments: column n = g is query g>>1, part g&1 (hi / lo); k slots
        // {2t, 2t+1, 2t+8, 2t+9} of group j carry dims 16j + 4t + {0,1,2,3}
        uint32_t bq[8][2];
        uint32_t qs[8];
        uint32_t bE = 0;
        bool big = false;
        {
            const int qi = g >> 1;
            const bool have = qi < nq;
            const float* q = a.q_coarse + (size_t)(it.query_begin + (have ? qi : 0)) * D_C;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (KIND == 3) {
                    // MMA j takes nibbles (o, o + 4 | o + 1, o + 5), o = 2 (j & 1), of the thread's word j >> 1
                    const float* qd = q + 32 * t + 8 * (j >> 1) + 2 * (j & 1);
                    float v[4] = {qd[0], qd[4], qd[1], qd[5]};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (!have) v[i] = 0.0f;
                        big |= fabsf(v[i]) > 60000.0f;
                        if (g & 1) v[i] = half_residual(v[i]);
                    }
                    bq[j][0] = pack_half2(v[0], v[1]);
                    bq[j][1] = pack_half2(v[2], v[3]);
                    continue;
                }
                // mixed 8/4 tiles: group 0 = dims 2t, 2t+1 (8-bit levels, plain in both slots, so
                // both carry 16x the query), groups 1..7 = INT4 groups of dims 16 j - 8 ..
                const int dim0 = !(KIND == 1) ? 16 * j + 4 * t : (j == 0 ? 0 : 16 * j - 8 + 4 * t);
                float4 x = *reinterpret_cast<const float4*>(q + dim0);
                if (KIND == 1 && j == 0) {
                    const float2 y = *reinterpret_cast<const float2*>(q + 2 * t);
                    x = make_float4(y.x, 16.0f * y.y, 0.0f, 0.0f);
                }
                float v[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (!have) v[i] = 0.0f;
                    big |= fabsf(v[i]) > (KIND == 1 && j == 0 && i == 1 ? 64000.0f : 4000.0f);  // 16 v must stay inside fp16
                    if (!(i & 1)) v[i] *= 16.0f;             // even slots carry 16x the query (see int4_quad)
                    if (g & 1) v[i] = half_residual(v[i]);
                }
                bq[j][0] = pack_half2(v[0], v[1]);
                bq[j][1] = pack_half2(v[2], v[3]);
            }
            if (KIND == 2) {
                // B fragment of the group sums: k slots 2t and 2t+1 = groups 2t and 2t+1 of query g>>1
                float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    s0 += q[32 * t + i];
                    s1 += q[32 * t + 16 + i];
                }
                if (!have) s0 = s1 = 0.0f;
                big |= fabsf(s0) > 60000.0f || fabsf(s1) > 60000.0f;
                if (g & 1) { s0 = half_residual(s0); s1 = half_residual(s1); }
                bE = pack_half2(s0, s1);
            }
            // sign words of query t (the query whose scores this thread finishes)
#pragma unroll
            for (int w = 0; w < 8; ++w)
                qs[w] = t < nq ? a.q_sign[(size_t)(it.query_begin + t) * 8 + w] : 0u;
        }
        // a query too large for the fp16 split: the generic kernel takes the item
        const bool too_big = __syncthreads_or(big) != 0;
        if (too_big && tid == 0) bail[0] = 1;

        const uint8_t* sbase = a.state ? a.state + it.tile_begin : nullptr;
        const uint32_t n = it.n_tiles;
        const uint32_t n_sets = too_big ? 0u : (n + MMA_SET_TILES - 1) / MMA_SET_TILES;
        const uint32_t n_full = n / MMA_SET_TILES;
        const bool mine = t < nq;
        uint32_t* gh = a.ghist + (size_t)(it.query_begin + (mine ? t : 0)) * 256;  // my query's shared histogram
        int rc = 0;  // keys in my_reg (the eight lanes of query t hold the same value)
        MmaItem m;
        m.keys = keys; m.pivot = pivot; m.cntw = cntw; m.bail = bail; m.rng = rng; m.hist = hist;
        m.rs = rs; m.room = room; m.sel_slack = sel_slack; m.query_begin = it.query_begin; m.nq = nq;
        // Sets are dealt to the warps round by round; the warp that takes a given slot of a
        // round rotates from round to round, so that a periodic arrangement of the tiles
        // cannot send all the best candidates to the same warp.
        const uint32_t rounds = (n_sets + (uint32_t)nwarps - 1) / (uint32_t)nwarps;
        auto set_of = [&](uint32_t j) { return j * (uint32_t)nwarps + (((uint32_t)warp + j + (j >> 4)) & (uint32_t)(nwarps - 1)); };
        const unsigned char* tbase = a.tiles + it.tile_begin * TILE_BYTES + lane * 16;
        // prefetch state: next round to fetch and its ring slot
        uint32_t j_next = 0, slot_next = 0;
        auto issue = [&]() {
            const uint32_t s_next = set_of(j_next);
            if (j_next < rounds && s_next < n_sets) {
                const uint32_t dst = stage_s + slot_next + dst_lane;
                const unsigned char* src = tbase + (size_t)s_next * MMA_SET_BYTES;
                if (s_next < n_full) {
                    cp_async16_s<0, 0>(dst, src, 16);
                    cp_async16_s<512, 4 * MMA_ROW>(dst, src, 16);
                    cp_async16_s<1024, 8 * MMA_ROW>(dst, src, 16);
                    cp_async16_s<1536, 12 * MMA_ROW>(dst, src, 16);
                } else {
                    // ragged last set: rows past the end are zero-filled (source not read)
                    const uint32_t r = s_next * MMA_SET_TILES + (uint32_t)(lane >> 3);
                    cp_async16_s<0, 0>(dst, r < n ? src : a.tiles, r < n ? 16 : 0);
                    cp_async16_s<0, 4 * MMA_ROW>(dst, r + 4 < n ? src + 512 : a.tiles, r + 4 < n ? 16 : 0);
                    cp_async16_s<0, 8 * MMA_ROW>(dst, r + 8 < n ? src + 1024 : a.tiles, r + 8 < n ? 16 : 0);
                    cp_async16_s<0, 12 * MMA_ROW>(dst, r + 12 < n ? src + 1536 : a.tiles, r + 12 < n ? 16 : 0);
                }
            }
            cp_async_commit();
            ++j_next;
            slot_next = slot_next == (MMA_DEPTH - 1) * MMA_SET_STRIDE ? 0u : slot_next + MMA_SET_STRIDE;
        };
        // All warps meet here when some warp cannot make room in a region alone (flag
        // ctl[0]).  No barrier is executed in the steady state: every warp polls the flag
        // between sets, finished warps poll it in the drain loop, so everyone arrives.
        auto rendezvous = [&]() {
            PROF_T(t_rv0);
            __syncwarp();
            if (lane == 0) atomicAdd(&ctl[1], 1);
            bool met = false;
            for (uint32_t spin = 0; spin < (1u << 24) && !met; ++spin) {
                met = *reinterpret_cast<volatile int*>(ctl + 1) >= nwarps;
                if (!met) __nanosleep(40);
            }
            if (!met && lane == 0) bail[0] = 1;  // the wait ran out: the generic kernel takes the item
            __syncthreads();
            PROF_T(t_rv1);
            rc = mma_settle(a, m, rc, false);
            if (tid == 0) { ctl[0] = 0; ctl[1] = 0; }
            __syncthreads();
            PROF_T(t_rv2);
            PROF_ADD(2, t_rv1 - t_rv0);
            PROF_ADD(3, t_rv2 - t_rv1);
            PROF_ADD(4, 1);
        };
#pragma unroll
        for (int i = 0; i < MMA_DEPTH - 1; ++i) issue();
        PROF_T(t_loop0);
        PROF_ADD(0, t_loop0 - t_item);
        uint32_t slot = 0, polls = 0;
        for (uint32_t j = 0; j < rounds; ++j) {
            issue();
            cp_async_wait<MMA_DEPTH - 1>();
            __syncwarp();
            const uint32_t s = set_of(j);
            const uint32_t rb = stage_s + slot + row_lane;
            slot = slot == (MMA_DEPTH - 1) * MMA_SET_STRIDE ? 0u : slot + MMA_SET_STRIDE;
            if (s >= n_sets) continue;  // the last round may be partial
            const uint2 m0 = lds_v2<96>(rb), m1 = lds_v2<96 + MMA_HALF>(rb);    // scale, lambda
            const uint4 x0 = lds_v4<112>(rb), x1 = lds_v4<112 + MMA_HALF>(rb);  // position, head|flags, gs[8]
            const uint32_t f0 = x0.y >> 16, f1 = x1.y >> 16;
            const uint32_t fo = __reduce_or_sync(0xFFFFFFFFu, f0 | f1);
            // a launch arranged for mixed 8/4 tiles takes nothing else (rows past the end of a ragged
            // last set are zero-filled and their scores dropped, so they count as mixed)
            const uint32_t row0 = s * MMA_SET_TILES + (uint32_t)g;
            const bool all_mixed = KIND == 1 && (__reduce_and_sync(0xFFFFFFFFu, (row0 < n ? f0 : F_MIXED) & (row0 + 8 < n ? f1 : F_MIXED)) & F_MIXED);
            const bool all_tq3 = KIND == 2 && (__reduce_and_sync(0xFFFFFFFFu, (row0 < n ? f0 : F_TQ3) & (row0 + 8 < n ? f1 : F_TQ3)) & F_TQ3);
            if ((fo & F_MIX3) || ((fo & F_TQ3) && !all_tq3) || (KIND == 2 && !all_tq3) ||
                ((fo & F_MIXED) && !all_mixed) || (KIND == 1 && !all_mixed) || ((fo & F_NF4) && (KIND == 3 || !a.nf4_table))) {
                if (lane == 0) bail[0] = 1;  // a codec this kernel does not decode: hand the item back
                break;
            }
            float acc0, acc1;
            const uint32_t hb = rb + 2u * (uint32_t)t;
            if (KIND == 3) {
                coarse_set_int4c(rb, (uint32_t)t, magic, bq, acc0, acc1);
            } else if (KIND == 2) {  // (all_tq3 holds here)
                tq3_to_nibbles(rb - row_lane, lane);
                coarse_set<0>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
                // level = (2 nibble - 15) / 4, or (2 nibble - 14) / 4 without the correction plane:
                // beside the nibble sums X the score needs 8 c sum_g gs_g Q_g (c = 1 or 2, Q_g = the
                // query's sum over group g), one more MMA with the scale bytes as the A operand
                const uint32_t sel = (t & 1) ? 0x7352u : 0x7150u;
                uint32_t ga0, ga1;
                asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(ga0) : "r"(prmt(t < 2 ? x0.z : x0.w, magic, sel)), "r"(0xE400E400u));
                asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(ga1) : "r"(prmt(t < 2 ? x1.z : x1.w, magic, sel)), "r"(0xE400E400u));
                float e[4];
                mma_f16_zero(e, ga0, ga1, 0u, 0u, bE, 0u);
                acc0 = fmaf((f0 & F_NOCORR) ? 16.0f : 8.0f, e[0] + e[1], acc0);
                acc1 = fmaf((f1 & F_NOCORR) ? 16.0f : 8.0f, e[2] + e[3], acc1);
            } else if (KIND == 1) {  // (all_mixed holds here)
                coarse_set<3>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
            } else if (!(fo & F_NF4)) {
                coarse_set<0>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
            } else if (__reduce_and_sync(0xFFFFFFFFu, f0 & f1) & F_NF4) {
                coarse_set<1>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
            } else {
                coarse_set<2>(hb, lut_lane, magic, bq, f0, f1, x0, x1, acc0, acc1);
            }
            // Hamming term of query t for both rows
            const int h0 = popc8(lds_v4<64>(rb), lds_v4<80>(rb), qs);
            const int h1 = popc8(lds_v4<64 + MMA_HALF>(rb), lds_v4<80 + MMA_HALF>(rb), qs);
            const float lam0 = (f0 & F_WARM) ? 0.0f : __uint_as_float(m0.y);
            const float lam1 = (f1 & F_WARM) ? 0.0f : __uint_as_float(m1.y);
            // 1 / (255 x 16 [x 2]); KIND 3: the sums carry 2^-12
            constexpr float unit = KIND == 3 ? 4096.0f / 255.0f : (KIND == 2 ? 1.0f / 8160.0f : 1.0f / 4080.0f);
            // 256 - 2 h without an integer conversion: (2^23 + h) as a bit pattern, times -2, plus 2^24 + 256 (exact)
            const float x0f = fmaf(__uint_as_float(0x4B000000u | (uint32_t)h0), -2.0f, 16777472.0f);
            const float x1f = fmaf(__uint_as_float(0x4B000000u | (uint32_t)h1), -2.0f, 16777472.0f);
            const float sc0 = fmaf(acc0, __uint_as_float(m0.x) * unit, lam0 * x0f);
            const float sc1 = fmaf(acc1, __uint_as_float(m1.x) * unit, lam1 * x1f);
            const uint32_t t0 = s * MMA_SET_TILES + (uint32_t)g, t1 = t0 + 8;
            bool live0 = mine && t0 < n, live1 = mine && t1 < n;
            if (sbase) {
                live0 = live0 && sbase[t0] != ST_COLD;
                live1 = live1 && sbase[t1] != ST_COLD;
            }
            if (TOPK && j == 0) {
                // First set of the warp: a query without a bucket mapping gets one from the 16
                // scores this warp has just computed for it - their range widened by 1.5 spans
                // on both sides.  Any monotone mapping is valid; this one only has to put the
                // final threshold somewhere inside its 256 buckets.  The first CTA to publish wins.
                float mn = fminf(live0 ? sc0 : INFINITY, live1 ? sc1 : INFINITY), mx = fmaxf(live0 ? sc0 : -INFINITY, live1 ? sc1 : -INFINITY);
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                }
                if (g == 0 && mine && rng[t].y == 0.0f) {
                    unsigned long long pr = *reinterpret_cast<volatile unsigned long long*>(a.grange + it.query_begin + t);
                    if (!pr && mx > mn) {
                        const float span = mx - mn, lo = mn - 1.5f * span, inv = 256.0f / (4.0f * span);
                        if (isfinite(lo) && isfinite(inv) && inv > 0.0f) {
                            const unsigned long long mine_r = (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(inv) << 32);
                            const unsigned long long old = atomicCAS(a.grange + it.query_begin + t, 0ull, mine_r);
                            pr = old ? old : mine_r;
                        }
                    }
                    if (pr) rng[t] = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
                }
                __syncwarp();
            }
            if (TOPK) {
                // filter on the score word alone (a superset of the composite comparison: a key that
                // only ties with the threshold's score is dropped again by the next purge)
                const uint32_t pvh = reinterpret_cast<const volatile uint32_t*>(pivot)[2 * t + 1];
                const uint32_t k0 = score_key(sc0), k1 = score_key(sc1);
                const bool p0 = live0 && k0 >= pvh, p1 = live1 && k1 >= pvh;
                if (__any_sync(0xFFFFFFFFu, p0 || p1)) {
                    const uint64_t comp0 = ((uint64_t)k0 << 32) | (uint64_t)(0xFFFFFFFFu - (it.index_base + t0));
                    const uint64_t comp1 = ((uint64_t)k1 << 32) | (uint64_t)(0xFFFFFFFFu - (it.index_base + t1));
                    // the lanes of query t append to the warp's region of that query: slots by ballot, no atomics
                    const unsigned b0 = __ballot_sync(0xFFFFFFFFu, p0) & t_mask, b1 = __ballot_sync(0xFFFFFFFFu, p1) & t_mask;
                    const int n0 = __popc(b0);
                    const float2 r = rng[t];
                    if (p0) {
                        my_reg[rc + __popc(b0 & lt_mask)] = comp0;
                        if (r.y > 0.0f && sc0 >= r.x) atomicAdd(gh + sel_bucket_f(sc0, r.x, r.y), 1u);
                    }
                    if (p1) {
                        my_reg[rc + n0 + __popc(b1 & lt_mask)] = comp1;
                        if (r.y > 0.0f && sc1 >= r.x) atomicAdd(gh + sel_bucket_f(sc1, r.x, r.y), 1u);
                    }
                    rc += n0 + __popc(b1);
                    if (__any_sync(0xFFFFFFFFu, rc > room)) {
                        // a region may not take another set: drop what the current thresholds allow,
                        // and ask for a block-wide step if that does not make room
#pragma unroll 1
                        for (int tq = 0; tq < nq; ++tq) {
                            mma_hist_pivot(a, m, tq, lane);
                            __syncwarp();
                            mma_purge(m, tq, warp, nwarps, lane, t, rc);
                        }
                        if (__any_sync(0xFFFFFFFFu, rc > room - 2 * MMA_SET_TILES) && lane == 0) *reinterpret_cast<volatile int*>(ctl) = 1;
                    }
                }
            } else if (mine) {
                float* o = a.scores + (size_t)(it.query_begin + t) * a.score_stride + it.index_base;
                if (t0 < n) o[t0] = live0 ? sc0 : -INFINITY;
                if (t1 < n) o[t1] = live1 ? sc1 : -INFINITY;
            }
            __syncwarp();
            if (TOPK) {
                if (*reinterpret_cast<volatile int*>(ctl)) {
                    rendezvous();
                    if (bail[0]) break;
                } else if ((++polls & 63u) == (uint32_t)(warp >> 2) * 16u + 8u || (EARLY && polls == 2u + (uint32_t)(warp >> 2))) {
                    // in turn, a warp raises the threshold of query (warp & 3)
                    if ((warp & 3) < nq) mma_hist_pivot(a, m, warp & 3, lane);
                    if ((warp & 3) == 0) mma_refresh_pivots(a, m, lane);
                    __syncwarp();
                }
            }
        }
        PROF_T(t_loop1);
        PROF_ADD(1, t_loop1 - t_loop0);
        if (TOPK) {
            // drain: warps that ran out of sets keep serving block-wide steps until all are done
            __syncwarp();
            if (lane == 0) atomicAdd(&ctl[2], 1);
            bool done = false;
            for (uint32_t spin = 0; spin < (1u << 24) && !done; ++spin) {
                if (*reinterpret_cast<volatile int*>(ctl)) rendezvous();
                else if (*reinterpret_cast<volatile int*>(ctl + 2) >= nwarps) done = true;
                else __nanosleep(100);
            }
            if (!done && lane == 0) bail[0] = 1;  // the wait ran out: the generic kernel takes the item
        }
        cp_async_wait<0>();
        __syncthreads();
        PROF_T(t_drain1);
        PROF_ADD(5, t_drain1 - t_loop1);
        if (TOPK && !bail[0]) rc = mma_settle(a, m, rc, true);  // at most list_cap candidates per query remain
        if (bail[0]) {
            if (tid == 0) a.retry[item_id] = 1;
            continue;
        }
        if (TOPK) {
            // every warp copies its regions behind each other into the item's candidate lists
#pragma unroll 1
            for (int tq = 0; tq < nq; ++tq) {
                const int cn = __shfl_sync(0xFFFFFFFFu, rc, tq);
                int base = 0;
                if (lane == 0 && cn) base = atomicAdd(&outpos[tq], cn);
                base = __shfl_sync(0xFFFFFFFFu, base, 0);
                const uint64_t* reg = keys + (size_t)(tq * nwarps + warp) * rs;
                uint64_t* dst = a.cand_keys + (size_t)(it.list_begin + tq) * a.list_cap;
                for (int i = lane; i < cn; i += 32)
                    if (base + i < (int)a.list_cap) dst[base + i] = reg[i];
            }
            __syncthreads();
            if (tid < nq) a.cand_cnt[it.list_begin + tid] = (uint32_t)min(outpos[tid], (int)a.list_cap);
        }
        PROF_T(t_end);
        PROF_ADD(6, t_end - t_drain1);
        PROF_ADD(7, 1);
    }
#ifdef SLHA_SCORE_PROFILE
    if (tid == 0)
        for (int i = 0; i < 8; ++i) g_score_prof[blockIdx.x * 8 + i] = prof[i];
#endif
}

}  // namespace
}  // namespace slha
