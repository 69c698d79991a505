// Tensor-core kernel of the fused score + top-k path (score_stream_kernel) and the selection
// routine the merge kernel shares with it.  Included by score.cu.
//
// With a GQA group of four queries the CUDA-core kernel is bound by instruction issue (128 FMAs
// per tile and query plus the nibble decode), not by HBM.  Here the coarse dot product of eq. 2.3
// runs as m16n8k16 MMAs over sets of 16 tiles:
//   A (16 tiles x 16 k slots) = exact fp16 levels made from the tiles' nibbles in registers,
//   B (16 k slots x 8 columns) = the four queries, each as an fp16 hi and lo column
//                                (q = hi + lo keeps ~22 bits), so a thread's two accumulator
//                                columns add up to one query; fragments live in shared memory,
//   D fp32.
// Two arrangements of A exist.  Per scale group (NF4, mixed 8/4, TQ3 and INT4 tiles met in such
// launches): one MMA per 16-dim group, levels n - 8 by an fp16 magic-number trick or NF4 codebook
// entries as hi + lo pairs from a bank-replicated shared-memory table, D started from zero per
// group and folded into the score with the tile's effective group scale on the CUDA cores; the
// MMA's k index is permuted so that the four k slots a thread owns are the four nibbles of one
// 16-bit word, odd slots carry 16x the level and B's even slots 16x the query (all exact).
// Contiguous (launches of INT4 / MX-INT4 tiles only): a thread owns 16 latent bytes of a row, the
// group scale is folded into A exactly, and the eight MMAs of a set chain on two accumulators.
// The Hamming term is 8 XOR + POPC per tile and query.  Tiles are staged by cp.async into a per-warp
// ring whose rows are padded to 144 bytes: every shared-memory address of the inner loop is "row
// base + immediate".  Candidates go to per-row buffers in global memory (see score_stream_kernel).
// A tile of another codec than the launch decodes hands its query rows to score_kernel.
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
constexpr uint32_t MMA_CHUNK = 16;  // slots a warp reserves at a time in a row's candidate buffer (larger chunks measured no faster)
#ifndef SLHA_STREAM_THREADS
#define SLHA_STREAM_THREADS 768  // 24 warps at 80 registers: the streaming kernel hides its latencies with warps
#endif
constexpr int MMA_DEPTH = SLHA_MMA_DEPTH;                  // cp.async ring slots per warp
constexpr int MMA_BQ_BYTES = 9 * 32 * 8;                   // B fragments of a work item: [9][32 lanes] x 8 bytes
constexpr int NF4_LUT_BYTES = 256 * 16 * 8;                // [byte][16 lanes] x (hi pair, lo pair)
constexpr int SEL_HIST_INTS = 4 * 256 + 48;                // block_select_multi: 4 histograms + state

#ifdef SLHA_STREAM_PROBE
// development build only: per-CTA timeline of score_stream_kernel (nanoseconds of %globaltimer)
__device__ unsigned long long g_stream_probe[160][8];
__device__ __forceinline__ unsigned long long probe_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
#define PROBE_SET(i) do { if (threadIdx.x == 0) g_stream_probe[blockIdx.x][i] = probe_now(); } while (0)
#define PROBE_MAX(i) do { if ((threadIdx.x & 31) == 0) atomicMax(&g_stream_probe[blockIdx.x][i], probe_now()); } while (0)
#define PROBE_MIN(i) do { if ((threadIdx.x & 31) == 0) atomicMin(&g_stream_probe[blockIdx.x][i], probe_now()); } while (0)
#else
#define PROBE_SET(i)
#define PROBE_MAX(i)
#define PROBE_MIN(i)
#endif
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
// the same with an L2 eviction policy: tiles are read once, so their lines are the first to go and the rows'
// candidate buffers and histograms, which the merge reads next, stay in the L2
template <int SRC_IMM, int DST_IMM>
__device__ __forceinline__ void cp_async16_sp(uint32_t dst, const unsigned char* src, int src_bytes, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0+%1], [%2+%3], 16, %4, %5;\n" ::"r"(dst), "n"(DST_IMM), "l"(src),
                 "n"(SRC_IMM), "r"(src_bytes), "l"(policy));
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// TQ3 rows of a staged 16-tile set, rewritten in place as nibble rows: nibble d of the 64 latent
// bytes becomes 2 code_d + correction_d (codes: 3 bits at bit 3d of bytes 0..47; correction bits:
// bit d of bytes 48..63, taken as zero for a tile flagged as without its correction plane).  A lane rewrites half a
// row (64 dims: 24 code bytes and 8 correction bytes in, 32 bytes out); every lane reads before
// any lane writes.
__device__ __forceinline__ void tq3_to_nibbles(uint32_t set_s, int lane) {
    const uint32_t h = (uint32_t)lane & 1u, row = set_s + (uint32_t)(lane >> 1) * MMA_ROW;
    const uint2 c0 = lds_v2<0>(row + 24u * h), c1 = lds_v2<8>(row + 24u * h), c2 = lds_v2<16>(row + 24u * h);
    uint2 cr = lds_v2<48>(row + 8u * h);
    // a tile flagged as without its correction plane is decoded from the codes alone, whatever the plane's bytes hold
    if (lds_u16<118>(row) & F_NOCORR) cr.x = cr.y = 0u;
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
__device__ __forceinline__ void coarse_group(uint32_t hb, uint32_t lut_lane, uint32_t magic, uint32_t bqa, uint32_t f0,
                                             uint32_t f1, const uint4& x0, const uint4& x1, float& acc0, float& acc1) {
    const uint2 bq = lds_v2<256 * J>(bqa);  // this lane's B fragment of group J
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
    mma_f16_zero(d, a0, a1, a2, a3, bq.x, bq.y);
    if (MODE == 1 || MODE == 2) mma_f16(d, l0, l1, l2, l3, bq.x, bq.y);
    // gs[J] as float: byte J of (x.z, x.w)
    const uint32_t gw0 = J < 4 ? x0.z : x0.w, gw1 = J < 4 ? x1.z : x1.w;
    // (byte -> float on the ALU / FMA pipes: 2^23 + b as a bit pattern, minus 2^23)
    acc0 = fmaf(d[0] + d[1], __uint_as_float(__byte_perm(gw0, 0x4B000000u, 0x7440 + (J & 3))) - 8388608.0f, acc0);
    acc1 = fmaf(d[2] + d[3], __uint_as_float(__byte_perm(gw1, 0x4B000000u, 0x7440 + (J & 3))) - 8388608.0f, acc1);
}

template <int MODE>
__device__ __forceinline__ void coarse_set(uint32_t hb, uint32_t lut_lane, uint32_t magic, uint32_t bq, uint32_t f0,
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
__device__ __forceinline__ void coarse_set_int4c(uint32_t rb, uint32_t t, uint32_t magic, uint32_t bqa, float& acc0, float& acc1) {
    const uint32_t cb = rb + 16u * t, hb = rb + 2u * t;
    const uint4 L0 = lds_v4<0>(cb), L1 = lds_v4<MMA_HALF>(cb);
    const uint32_t h0 = lds_u16<120>(hb), h1 = lds_u16<120 + MMA_HALF>(hb);
    uint32_t G00, C00, G01, C01, G10, C10, G11, C11;
    int4c_scales(h0, magic, G00, C00, G01, C01);
    int4c_scales(h1, magic, G10, C10, G11, C11);
    const uint32_t w0[4] = {L0.x, L0.y, L0.z, L0.w}, w1[4] = {L1.x, L1.y, L1.z, L1.w};
    // two accumulator chains (even / odd MMAs) halve the dependent MMA latency of a set
    float d[4], e[4];
    const uint2 b0 = lds_v2<0>(bqa), b1 = lds_v2<256>(bqa), b2 = lds_v2<512>(bqa), b3 = lds_v2<768>(bqa);
    const uint2 b4 = lds_v2<1024>(bqa), b5 = lds_v2<1280>(bqa), b6 = lds_v2<1536>(bqa), b7 = lds_v2<1792>(bqa);
    const uint2 bq[8] = {b0, b1, b2, b3, b4, b5, b6, b7};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t o0[4], o1[4];
        int4c_word(w0[i], i < 2 ? G00 : G01, i < 2 ? C00 : C01, o0);
        int4c_word(w1[i], i < 2 ? G10 : G11, i < 2 ? C10 : C11, o1);
        if (i == 0) {
            mma_f16_zero(d, o0[0], o1[0], o0[1], o1[1], bq[0].x, bq[0].y);
            mma_f16_zero(e, o0[2], o1[2], o0[3], o1[3], bq[1].x, bq[1].y);
        } else {
            mma_f16(d, o0[0], o1[0], o0[1], o1[1], bq[2 * i].x, bq[2 * i].y);
            mma_f16(e, o0[2], o1[2], o0[3], o1[3], bq[2 * i + 1].x, bq[2 * i + 1].y);
        }
    }
    acc0 = (d[0] + e[0]) + (d[1] + e[1]);
    acc1 = (d[2] + e[2]) + (d[3] + e[3]);
}

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
    for (int pass = 0; pass < 12; ++pass) {
        if (!(st[3] | st[11] | st[19] | st[27])) break;
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
    return ties;
}


// ---- streaming top-k state shared by all CTAs -----------------------------------------------
// Per query row, in global memory (L2-resident), zeroed by one memset per call:
//   gpivot  best proven lower bound of the row's k-th best composite key (score word in the high half)
//   grange  bucket mapping (smin, inv) of the row's score histogram, 0 = none yet
//   gcount  candidates appended to the row's buffer so far
//   gflag   1 = the generic kernel scores the row's work items instead (a tile of another codec,
//           a query outside the fp16 split, or a full candidate buffer)
//   ghist   256 bucket counts of the appended candidates
// and one candidate buffer of gcap composite keys per row.  A CTA keeps no candidates of its own:
// a tile whose score reaches the row's threshold is appended to the row's buffer (one atomic per
// warp, query and set), counted in the row's histogram, and the threshold is re-derived from that
// histogram from time to time - the counts are of real tiles, so the lower edge of the highest
// bucket whose count from the top reaches k is a proven lower bound of the k-th best score, for
// all CTAs at once.  Nothing in the hot loop waits for another warp or CTA.

// A whole warp: raise the threshold of query row Q (shared word *pvh) from the row's histogram
// and from what other CTAs have proven.
__device__ __forceinline__ void stream_refresh_threshold(const ScoreArgs& a, uint32_t Q, float2 r, uint32_t* pvh, int lane) {
    const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(a.gpivot + Q);
    uint32_t best = (uint32_t)(seen >> 32);
    if (r.y != 0.0f) {
        const uint32_t* hq = a.ghist + (size_t)Q * 256 + 248 - 8 * lane;
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
        uint32_t ek = 0;
        if (ok != 0u && lane == __ffs(ok) - 1) {
            uint32_t run = incl - tot;
            int b = 0;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                if (run + c[jj] >= a.k) { b = 255 - 8 * lane - jj; break; }
                run += c[jj];
            }
            if (b >= 1) {
                // half a bucket and a few ulps below the bucket's edge: every counted key of the
                // buckets b.. is above this bound whatever the rounding of the bucket arithmetic
                const uint32_t e = score_key(r.x + ((float)b - 0.5f) / r.y);
                ek = e > 8u ? e - 8u : 0u;
            }
        }
        ek = __reduce_max_sync(0xFFFFFFFFu, ek);
        if (ek > best) {
            best = ek;
            if (lane == 0) atomicMax(a.gpivot + Q, (unsigned long long)ek << 32);
        }
    }
    if (lane == 0 && best > *reinterpret_cast<volatile uint32_t*>(pvh)) atomicMax(pvh, best);
}

// KIND 0: nibble codecs (INT4, MX-INT4, NF4 through the shared-memory table); 1: the launch scores
// mixed 8/4 tiles; 2: TQ3 tiles, rewritten in shared memory as nibble rows (2 code + correction
// bit) before the INT4 path scores them; 3: INT4 / MX-INT4 tiles only (scale folded into A).
// Separate instantiations.  A tile of another codec than the launch was arranged for flags the
// work item's query rows, which the generic kernel then scores.
// IL: the work items are interleaved shares of whole streams (see the planner); the plain instantiation keeps the
// set arithmetic of contiguous ranges out of its loop.  DENSE: every score is written to a.scores (row q at
// q * a.score_stride, tile i of the item at index_base + i; -inf for COLD slots) and nothing is filtered or appended:
// full score vectors (slha_score_tiles, score_all, the softmax of observe_scores) at the streaming kernel's speed.
template <int KIND, int NT, bool IL, bool DENSE = false>
__global__ void __launch_bounds__(NT, 1) score_stream_kernel(ScoreArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // shared layout: nf4 table | stage ring | B fragments | query sign words | thresholds | bucket mappings | flag
    const uint32_t lut_bytes = a.nf4_table ? NF4_LUT_BYTES : 0;  // the table is left out when no NF4 tile is expected
    uint2* lut = reinterpret_cast<uint2*>(smem);
#ifdef SLHA_STREAM_PROBE
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) g_stream_probe[blockIdx.x][i] = i == 6 ? ~0ull : 0ull;
        g_stream_probe[blockIdx.x][0] = probe_now();
    }
    __syncthreads();
#endif
    unsigned char* tail = smem + lut_bytes + (size_t)nwarps * MMA_DEPTH * MMA_SET_STRIDE;
    uint2* bq_w = reinterpret_cast<uint2*>(tail);                        // [9][32]
    uint32_t* qs_w = reinterpret_cast<uint32_t*>(tail + MMA_BQ_BYTES);   // [4][8]
    uint32_t* pvh = qs_w + 32;                                           // [4] score word of the row's threshold
    float2* rng = reinterpret_cast<float2*>(pvh + 4);                    // [4] (smin, inv), inv 0 = none yet
    float2* rmap = rng + 4;                                              // [4] (-smin * inv, inv): the same mapping as the hot path uses it
    int* bail = reinterpret_cast<int*>(rmap + 4);                        // [1]
    const uint32_t smem_s = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t stage_s = smem_s + lut_bytes + (uint32_t)warp * MMA_DEPTH * MMA_SET_STRIDE;
    const uint32_t bqa = smem_s + lut_bytes + (uint32_t)nwarps * MMA_DEPTH * MMA_SET_STRIDE + (uint32_t)lane * 8u;
    const uint32_t qsa = bqa - (uint32_t)lane * 8u + MMA_BQ_BYTES + (uint32_t)t * 32u;

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
    const uint32_t lt_mask = (1u << lane) - 1u, t_mask = 0x11111111u << t;
    uint64_t stream_policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(stream_policy));

    const uint32_t item_end = a.cta_begin[blockIdx.x + 1];
    for (uint32_t item_id = a.cta_begin[blockIdx.x]; item_id < item_end; ++item_id) {
        const WorkItem it = a.stream_items[item_id];
        const int nq = (int)it.n_queries;
        // interleaved: this CTA is number il_c of the il_n CTAs that share the stream [tile_begin, + n_tiles); round r of
        // the stream's static deal belongs to CTA r mod il_n.  Otherwise the item is this CTA's own range.
        constexpr bool il = IL;
        const uint32_t il_n = il ? ((it.pad >> 8) & 0x7FFFFFu) : 1u, il_c = il ? it.list_begin : 0u;
        __syncthreads();  // previous item fully retired (and the table is visible)
        // The first sets are fetched before anything else of the item is prepared: the copy runs while the query
        // fragments are built.
        const uint8_t* sbase = a.state ? a.state + it.tile_begin : nullptr;
        const uint32_t n = it.n_tiles;
        uint32_t n_sets = (n + MMA_SET_TILES - 1) / MMA_SET_TILES;
        const uint32_t n_full = n / MMA_SET_TILES;
        const bool mine = t < nq;
        const uint32_t Qt = it.query_begin + (mine ? (uint32_t)t : 0u);  // the row whose scores this thread finishes
        uint64_t* const dst = a.gbuf + (size_t)Qt * a.gcap;                // the row's candidate buffer
        uint32_t* const hrow = a.ghist + (size_t)Qt * 256;                 // and its histogram
        // sets are dealt to the warps round by round: warp w takes set j * nwarps + w of round j
        const unsigned char* tbase = a.tiles + it.tile_begin * TILE_BYTES + lane * 16;
        // This CTA's rounds of the deal, r = il_c, il_c + il_n, ..; an interleaved CTA walks them starting from a place of its
        // own and wraps around (CTA c of C starts c / C of the way through), so that at any moment the CTAs of a stream are
        // spread over the whole stream -- the first thresholds then come from a sample of all positions even when one
        // end of the stream holds nothing to score (the oldest slots of a pool are mostly COLD).
        const uint32_t all_rounds = (n_sets + (uint32_t)nwarps - 1) / (uint32_t)nwarps;
        const uint32_t my_rounds = all_rounds > il_c ? (all_rounds - il_c + il_n - 1) / il_n : 0u;  // (the same for all warps of the CTA)
        const uint32_t first_round = il ? (uint32_t)(((uint64_t)il_c * my_rounds) / il_n) : 0u;
        auto set_of = [&](uint32_t i) {  // the set this warp takes in its i-th iteration
            if (!il) return i * (uint32_t)nwarps + (uint32_t)warp;
            uint32_t j = i + first_round;
            if (j >= my_rounds) j -= my_rounds;
            return (j * il_n + il_c) * (uint32_t)nwarps + (uint32_t)warp;
        };
        uint32_t iss_no = 0, slot_next = 0;
        auto issue = [&]() {
            const uint32_t s_next = iss_no < my_rounds ? set_of(iss_no) : 0xFFFFFFFFu;
            ++iss_no;
            if (s_next < n_sets) {
                const uint32_t dst = stage_s + slot_next + dst_lane;
                const unsigned char* src = tbase + (size_t)s_next * MMA_SET_BYTES;
                if (s_next < n_full) {
                    cp_async16_sp<0, 0>(dst, src, 16, stream_policy);
                    cp_async16_sp<512, 4 * MMA_ROW>(dst, src, 16, stream_policy);
                    cp_async16_sp<1024, 8 * MMA_ROW>(dst, src, 16, stream_policy);
                    cp_async16_sp<1536, 12 * MMA_ROW>(dst, src, 16, stream_policy);
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
            slot_next = slot_next == (MMA_DEPTH - 1) * MMA_SET_STRIDE ? 0u : slot_next + MMA_SET_STRIDE;
        };
#pragma unroll
        for (int i = 0; i < MMA_DEPTH - 1; ++i) issue();
        bool row_warm = true;
        if (!DENSE && tid < 4) {
            // start from the threshold other CTAs have already proven for the row, and from the
            // row's bucket mapping if one has been published
            const bool have = tid < nq;
            const unsigned long long pv = have ? *reinterpret_cast<volatile unsigned long long*>(a.gpivot + it.query_begin + tid) : 0ull;
            pvh[tid] = (uint32_t)(pv >> 32);
            row_warm = !have || (uint32_t)(pv >> 32) != 0u;
            const unsigned long long pr = have ? *reinterpret_cast<volatile unsigned long long*>(a.grange + it.query_begin + tid) : 0ull;
            rng[tid] = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
            rmap[tid] = make_float2(-rng[tid].x * rng[tid].y, rng[tid].y);
        }
        if (tid == 0) bail[0] = 0;
        if (warp == 1 % nwarps) {
            // sign words of the item's (up to four) queries
            const int qi = lane >> 3;
            qs_w[lane] = qi < nq ? a.q_sign[(size_t)(it.query_begin + qi) * 8 + (lane & 7)] : 0u;
        }
        bool big = false;
        if (warp == 0) {
            // B fragments: column n = g is query g>>1, part g&1 (fp16 hi / lo of the query)
            const int qi = g >> 1;
            const bool have = qi < nq;
            const float* q = a.q_coarse + (size_t)(it.query_begin + (have ? qi : 0)) * D_C;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float v[4];
                if (KIND == 3) {
                    // MMA j takes nibbles (o, o + 4 | o + 1, o + 5), o = 2 (j & 1), of the thread's word j >> 1
                    const float* qd = q + 32 * t + 8 * (j >> 1) + 2 * (j & 1);
                    v[0] = qd[0]; v[1] = qd[4]; v[2] = qd[1]; v[3] = qd[5];
                } else {
                    // k slots {2t, 2t+1, 2t+8, 2t+9} of group j carry dims 16j + 4t + {0,1,2,3}; mixed 8/4 tiles:
                    // group 0 = dims 2t, 2t+1 (8-bit levels, plain in both slots, so both carry 16x the
                    // query), groups 1..7 = INT4 groups of dims 16 j - 8 ..
                    const int dim0 = !(KIND == 1) ? 16 * j + 4 * t : (j == 0 ? 0 : 16 * j - 8 + 4 * t);
                    float4 x = *reinterpret_cast<const float4*>(q + dim0);
                    if (KIND == 1 && j == 0) {
                        const float2 y = *reinterpret_cast<const float2*>(q + 2 * t);
                        x = make_float4(y.x, 16.0f * y.y, 0.0f, 0.0f);
                    }
                    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (!have) v[i] = 0.0f;
                    if (KIND == 3) {
                        big |= fabsf(v[i]) > 60000.0f;
                    } else {
                        big |= fabsf(v[i]) > (KIND == 1 && j == 0 && i == 1 ? 64000.0f : 4000.0f);  // 16 v must stay inside fp16
                        if (!(i & 1)) v[i] *= 16.0f;  // even slots carry 16x the query (see int4_quad)
                    }
                    if (g & 1) v[i] = half_residual(v[i]);
                }
                bq_w[j * 32 + lane] = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
            }
            uint32_t bE = 0;
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
            bq_w[8 * 32 + lane] = make_uint2(bE, 0u);
            if (__any_sync(0xFFFFFFFFu, big) && lane == 0) bail[0] = 1;  // a query too large for the fp16 split
        }
        // The barrier after the first round (below) pays when the round can supply k candidates to a row -- 16 per warp
        // of every CTA that works on the row -- and the rows do not already have thresholds (a CTA that starts its
        // second item on rows other CTAs have been scoring for a while).
        const bool all_warm = __syncthreads_and(row_warm) != 0;
        const bool first_round_barrier = !DENSE && !all_warm && (uint64_t)a.k <= 16ull * (uint64_t)nwarps * (uint64_t)max((it.pad >> 8) & 0x7FFFFFu, 1u);
        PROBE_SET(1);
        const bool too_big = bail[0] != 0;
        if (too_big) n_sets = 0;  // (the sets already on their way are waited for at the item's end and never read)

        uint32_t slot = 0, polls = 0;
        uint32_t cur = 0, end = 0;  // this warp's chunk of the buffer of row Qt (the same in the eight lanes of a query)
        bool dead = false;          // this warp met a tile it cannot decode
        const uint32_t rounds = too_big ? 0u : my_rounds;
        for (uint32_t round = 0; round < rounds; ++round) {
            const uint32_t s = set_of(round);
            if (round == 1 && first_round_barrier) {
                // Every warp of the CTA (and, started together, of the grid) has appended its first set
                // unfiltered, so the rows' histograms hold 16 candidates per warp: first thresholds now,
                // before the second sets are filtered.  (All warps pass here: `rounds` is the same for all.)
                PROBE_MAX(2);
                __syncthreads();
                if (warp < nq) stream_refresh_threshold(a, it.query_begin + (uint32_t)warp, rng[warp], pvh + warp, lane);
                __syncthreads();
                PROBE_SET(3);
            }
            // (the ring advances in every iteration, also when this warp has no set in this round -- the short last round of
            // the stream can come anywhere in a rotated walk -- so that fetches and reads stay in step)
            issue();
            cp_async_wait<MMA_DEPTH - 1>();
            __syncwarp();
            const uint32_t rb = stage_s + slot + row_lane;
            slot = slot == (MMA_DEPTH - 1) * MMA_SET_STRIDE ? 0u : slot + MMA_SET_STRIDE;
            if (dead || s >= n_sets) continue;
            const uint2 m0 = lds_v2<96>(rb), m1 = lds_v2<96 + MMA_HALF>(rb);    // scale, lambda
            const uint4 x0 = lds_v4<112>(rb), x1 = lds_v4<112 + MMA_HALF>(rb);  // position, head|flags, gs[8]
            const uint32_t f0 = x0.y >> 16, f1 = x1.y >> 16;
            const uint32_t fo = __reduce_or_sync(0xFFFFFFFFu, f0 | f1);
            const bool ragged = s >= n_full;
            const uint32_t t0 = s * MMA_SET_TILES + (uint32_t)g, t1 = t0 + 8;
            // a launch arranged for mixed 8/4 (TQ3) tiles takes nothing else (rows past the end of a ragged
            // last set are zero-filled and their scores dropped, so they count as such tiles)
            const bool all_mixed = KIND == 1 && (__reduce_and_sync(0xFFFFFFFFu, (t0 < n ? f0 : F_MIXED) & (t1 < n ? f1 : F_MIXED)) & F_MIXED);
            const bool all_tq3 = KIND == 2 && (__reduce_and_sync(0xFFFFFFFFu, (t0 < n ? f0 : F_TQ3) & (t1 < n ? f1 : F_TQ3)) & F_TQ3);
            if ((fo & F_MIX3) || ((fo & F_TQ3) && !all_tq3) || (KIND == 2 && !all_tq3) ||
                ((fo & F_MIXED) && !all_mixed) || (KIND == 1 && !all_mixed) || ((fo & F_NF4) && (KIND == 3 || !a.nf4_table))) {
                if (lane == 0) bail[0] = 1;  // a codec this launch does not decode: the generic kernel takes the rows
                dead = true;
                continue;
            }
            float acc0, acc1;
            const uint32_t hb = rb + 2u * (uint32_t)t;
            if (KIND == 3) {
                coarse_set_int4c(rb, (uint32_t)t, magic, bqa, acc0, acc1);
            } else if (KIND == 2) {  // (all_tq3 holds here)
                tq3_to_nibbles(rb - row_lane, lane);
                coarse_set<0>(hb, lut_lane, magic, bqa, f0, f1, x0, x1, acc0, acc1);
                // level = (2 nibble - 15) / 4, or (2 nibble - 14) / 4 without the correction plane:
                // beside the nibble sums X the score needs 8 c sum_g gs_g Q_g (c = 1 or 2, Q_g = the
                // query's sum over group g), one more MMA with the scale bytes as the A operand
                const uint32_t sel = (t & 1) ? 0x7352u : 0x7150u;
                uint32_t ga0, ga1;
                asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(ga0) : "r"(prmt(t < 2 ? x0.z : x0.w, magic, sel)), "r"(0xE400E400u));
                asm("add.rn.f16x2 %0, %1, %2;\n" : "=r"(ga1) : "r"(prmt(t < 2 ? x1.z : x1.w, magic, sel)), "r"(0xE400E400u));
                float e[4];
                mma_f16_zero(e, ga0, ga1, 0u, 0u, lds_v2<256 * 8>(bqa).x, 0u);
                acc0 = fmaf((f0 & F_NOCORR) ? 16.0f : 8.0f, e[0] + e[1], acc0);
                acc1 = fmaf((f1 & F_NOCORR) ? 16.0f : 8.0f, e[2] + e[3], acc1);
            } else if (KIND == 1) {  // (all_mixed holds here)
                coarse_set<3>(hb, lut_lane, magic, bqa, f0, f1, x0, x1, acc0, acc1);
            } else if (!(fo & F_NF4)) {
                coarse_set<0>(hb, lut_lane, magic, bqa, f0, f1, x0, x1, acc0, acc1);
            } else if (__reduce_and_sync(0xFFFFFFFFu, f0 & f1) & F_NF4) {
                coarse_set<1>(hb, lut_lane, magic, bqa, f0, f1, x0, x1, acc0, acc1);
            } else {
                coarse_set<2>(hb, lut_lane, magic, bqa, f0, f1, x0, x1, acc0, acc1);
            }
            const float lam0 = (f0 & F_WARM) ? 0.0f : __uint_as_float(m0.y);
            const float lam1 = (f1 & F_WARM) ? 0.0f : __uint_as_float(m1.y);
            // 1 / (255 x 16 [x 2]); KIND 3: the sums carry 2^-12
            constexpr float unit = KIND == 3 ? 4096.0f / 255.0f : (KIND == 2 ? 1.0f / 8160.0f : 1.0f / 4080.0f);
            const float c0 = acc0 * (__uint_as_float(m0.x) * unit), c1 = acc1 * (__uint_as_float(m1.x) * unit);
            const uint32_t pv = reinterpret_cast<const volatile uint32_t*>(pvh)[t];
            // The residual term lies in [-256 lambda, 256 lambda]: a set none of whose tiles can reach its
            // row's threshold even with the largest term needs no Hamming distances (and appends nothing).
            // (257 and the relative slack cover the rounding of the bound itself.)  Only the INT4 launches
            // test for it: with a few CTAs per row and k / n of a few percent (the NF4 decode caches) nearly
            // every set holds a candidate and the test costs more than it saves.
            const bool need = DENSE || KIND != 3 || round == 0 ||
                              __any_sync(0xFFFFFFFFu, (mine && score_key(fmaf(lam0, 257.0f, c0 + fabsf(c0) * 1e-6f)) >= pv) ||
                                                          (mine && score_key(fmaf(lam1, 257.0f, c1 + fabsf(c1) * 1e-6f)) >= pv));
            if (need) {
            // Hamming term of query t for both rows
            int h0, h1;
            {
                const uint4 qa = lds_v4<0>(qsa), qb = lds_v4<16>(qsa);
                const uint32_t qs[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                h0 = popc8(lds_v4<64>(rb), lds_v4<80>(rb), qs);
                h1 = popc8(lds_v4<64 + MMA_HALF>(rb), lds_v4<80 + MMA_HALF>(rb), qs);
            }
            // 256 - 2 h without an integer conversion: (2^23 + h) as a bit pattern, times -2, plus 2^24 + 256 (exact)
            const float x0f = fmaf(__uint_as_float(0x4B000000u | (uint32_t)h0), -2.0f, 16777472.0f);
            const float x1f = fmaf(__uint_as_float(0x4B000000u | (uint32_t)h1), -2.0f, 16777472.0f);
            const float sc0 = fmaf(lam0, x0f, c0);
            const float sc1 = fmaf(lam1, x1f, c1);
            bool live0 = mine && (!ragged || t0 < n), live1 = mine && (!ragged || t1 < n);
            if (sbase) {
                live0 = live0 && sbase[t0] != ST_COLD;
                live1 = live1 && sbase[t1] != ST_COLD;
            }
            if (DENSE) {
                if (mine) {  // (eight lanes of a query hold eight consecutive tiles: 32-byte runs per row)
                    float* row = a.scores + (size_t)Qt * a.score_stride + it.index_base;
                    if (t0 < n) row[t0] = live0 ? sc0 : -INFINITY;
                    if (t1 < n) row[t1] = live1 ? sc1 : -INFINITY;
                }
                __syncwarp();
                continue;
            }
            if (round == 0) {
                // First set of the warp: a row without a bucket mapping gets one from the 16 scores
                // this warp has just computed for it - their range widened by 1.5 spans on both sides.
                // Any monotone mapping is valid; this one only has to put the final threshold somewhere
                // inside its 256 buckets.  The first CTA to publish wins.
                float mn = fminf(live0 ? sc0 : INFINITY, live1 ? sc1 : INFINITY), mx = fmaxf(live0 ? sc0 : -INFINITY, live1 ? sc1 : -INFINITY);
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
                    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                }
                if (g == 0 && mine && rng[t].y == 0.0f) {
                    unsigned long long pr = *reinterpret_cast<volatile unsigned long long*>(a.grange + Qt);
                    if (!pr && mx > mn) {
                        const float span = mx - mn, lo = mn - 1.5f * span, inv = 256.0f / (4.0f * span);
                        if (isfinite(lo) && isfinite(inv) && inv > 0.0f) {
                            const unsigned long long mine_r = (unsigned long long)__float_as_uint(lo) | ((unsigned long long)__float_as_uint(inv) << 32);
                            const unsigned long long old = atomicCAS(a.grange + Qt, 0ull, mine_r);
                            pr = old ? old : mine_r;
                        }
                    }
                    if (pr) {
                        rng[t] = make_float2(__uint_as_float((uint32_t)pr), __uint_as_float((uint32_t)(pr >> 32)));
                        rmap[t] = make_float2(-rng[t].x * rng[t].y, rng[t].y);
                    }
                }
                __syncwarp();
            }
            // filter on the score word alone (a superset of the composite comparison: the merge drops
            // keys below the final threshold)
            const uint32_t k0 = score_key(sc0), k1 = score_key(sc1);
            const bool p0 = live0 && k0 >= pv, p1 = live1 && k1 >= pv;
            if (__any_sync(0xFFFFFFFFu, p0 || p1)) {
                // The eight lanes of query t append to the row's buffer, slots by ballot.  The warp owns a
                // chunk of 16 slots per row, [cur, end), reserved with one atomic; a set brings at most 16
                // candidates per row, so a fresh chunk always fits them.  The unused rest of a chunk is
                // zeroed (an absent key) before the next one is taken and at the end of the work item.
                const unsigned b0 = __ballot_sync(0xFFFFFFFFu, p0) & t_mask, b1 = __ballot_sync(0xFFFFFFFFu, p1) & t_mask;
                const uint32_t n0 = (uint32_t)__popc(b0), nn = n0 + (uint32_t)__popc(b1);
                if (cur + nn > end) {  // (the same in the eight lanes of a query, which are the lanes of t_mask)
                    for (uint32_t z = cur + (uint32_t)g; z < end; z += 8u) dst[z] = 0ull;
                    uint32_t base = 0;
                    if (g == 0) {
                        base = atomicAdd(a.gcount + Qt, MMA_CHUNK);
                        if (base + MMA_CHUNK > a.gcap) {
                            // the row's buffer is full: the generic kernel scores the row; this warp's further
                            // candidates of the row land in the buffer's last chunk, which nobody reads then
                            a.gflag[Qt] = 1u;
                            base = a.gcap - MMA_CHUNK;
                        }
                    }
                    cur = __shfl_sync(t_mask, base, t);  // lane t is (g = 0, t)
                    end = cur + MMA_CHUNK;
                }
                // bucket of the row's histogram: (int)(score * inv - smin * inv), clamped; scores below the
                // mapping (and all scores while the row has no mapping) count in bucket 0, which never decides
                const float2 r = rmap[t];
                if (p0) {
                    dst[cur + (uint32_t)__popc(b0 & lt_mask)] = ((uint64_t)k0 << 32) | (uint64_t)(~(it.index_base + t0));
                    atomicAdd(hrow + min(max(__float2int_rz(fmaf(sc0, r.y, r.x)), 0), 255), 1u);
                }
                if (p1) {
                    dst[cur + n0 + (uint32_t)__popc(b1 & lt_mask)] = ((uint64_t)k1 << 32) | (uint64_t)(~(it.index_base + t1));
                    atomicAdd(hrow + min(max(__float2int_rz(fmaf(sc1, r.y, r.x)), 0), 255), 1u);
                }
                cur += nn;
            }
            }  // need
            __syncwarp();
            // In turn, a warp raises the threshold of query (warp & 3): after its 3rd and 7th set (the first
            // thresholds come from the barrier after the first round), then every 16 sets, the warps of a
            // query staggered.  A stale threshold costs appends (each one a store, a
            // histogram count and, downstream, merge work), a refresh costs one 1 KB read of the row's
            // histogram by one warp.
            ++polls;
            if ((polls & 15u) == (uint32_t)((warp >> 2) & 3) * 4u + 3u || polls == 3u || polls == 7u) {
                const int q = warp & 3;
                if (q < nq) stream_refresh_threshold(a, it.query_begin + (uint32_t)q, rng[q], pvh + q, lane);
                __syncwarp();
            }
        }
        cp_async_wait<0>();
        PROBE_MAX(4);
        PROBE_MIN(6);
        if (!DENSE && mine) {  // the unused rest of the warp's last chunk holds absent keys
            for (uint32_t z = cur + (uint32_t)g; z < end; z += 8u) dst[z] = 0ull;
        }
        __syncthreads();
        // rows this CTA could not score on the tensor cores go to the generic kernel as a whole
        if (bail[0] && tid < nq) a.gflag[it.query_begin + tid] = 1u;
        PROBE_SET(5);
    }
}

}  // namespace
}  // namespace slha
