// Key -> tile encode, query preparation and tile decode for sm_100a.
//
// Restates LearnedModel::{latent, reconstruct, sign_bits, encode_with,
// query_coarse} (scirust/src/learned.rs:247-408), the six quantisers
// (scirust/src/attention/slha_v2/codec/*.rs) and the randomised Hadamard
// transform (scirust/src/incoherence.rs:45-125).
//
// Bit-exactness contract: every decision the reference takes on a float
// (round-half-away, `acc < 0.0`, `t - level > 0.0`, first-minimum NF4 search)
// sits on a float32 sum that the reference accumulates strictly left to right
// with a separate multiply and add.  This kernel keeps that order: each thread
// owns whole output rows and walks the contraction index sequentially with
// __fmul_rn / __fadd_rn (never contracted into FMA), divisions are __fdiv_rn and
// square roots __fsqrt_rn.  Parallelism comes from rows x keys, not from
// splitting a sum, so the tile bytes equal the scalar reference's bit for bit.
#include "common.cuh"

namespace slha {
namespace {

constexpr int ENC_THREADS = 256;

struct EncodeArgs {
    const void* keys;        // [n][d] f32 or bf16
    int key_dtype;
    uint64_t n;
    uint32_t d, d_pad, log2_pad;
    const float* p;          // [128][d]
    const float* pt;         // [d][128]
    const float* scale;      // [128]
    const float* zt;         // [d_pad][256]
    const float* diag;       // [d_pad] or null
    float fwht_inv;          // 1/sqrt(d_pad), rounded as the reference rounds it
    float lambda_c;          // sqrt(pi/512) in f32
    const uint32_t* positions;
    uint32_t position_base;
    const uint16_t* heads;
    int codec;
    unsigned char* tiles;    // output tiles (encode)
    const uint32_t* slots;   // optional scatter: tile i goes to tiles[slots[i]]
    float* q_coarse;         // [n][128]  (query mode)
    uint64_t* q_sign;        // [n][4]    (query mode)
    int kb;                  // keys per CTA pass (power of two, <= 16)
};

__device__ __forceinline__ float rnd_half_away(float x) { return roundf(x); }
__device__ __forceinline__ int sat_i32(float x) {
    // Rust `x as i32`: NaN -> 0, saturating
    if (x != x) return 0;
    if (x >= 2147483648.0f) return 2147483647;
    if (x <= -2147483648.0f) return (-2147483647 - 1);
    return (int)x;
}
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return min(max(v, lo), hi); }
__device__ __forceinline__ uint32_t scale_byte(float step, float global) {
    // `(step / global * 255.0).round().clamp(1.0, 255.0) as u8`  (int4.rs:48-49)
    float r = rnd_half_away(__fmul_rn(__fdiv_rn(step, global), 255.0f));
    if (r != r) return 0;
    return (uint32_t)fminf(fmaxf(r, 1.0f), 255.0f);
}
__device__ __forceinline__ uint32_t int4_nibble(float v, float step) {
    return (uint32_t)(clampi(sat_i32(rnd_half_away(__fdiv_rn(v, step))), -8, 7) + 8) & 15u;
}
__device__ __forceinline__ uint32_t nf4_nearest(float t) {
    // nf4.rs:7-18: linear scan, first minimum wins
    const float cb[16] = {-1.0f,   -0.7075f, -0.5421f, -0.4165f, -0.3108f, -0.2158f,
                          -0.1272f, -0.0421f, 0.0421f,  0.1272f,  0.2158f,  0.3108f,
                          0.4165f,  0.5421f,  0.7075f,  1.0f};
    uint32_t best = 0;
    float best_d = INFINITY;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float dd = fabsf(__fsub_rn(t, cb[i]));
        if (dd < best_d) { best_d = dd; best = i; }
    }
    return best;
}
__device__ __forceinline__ float quad_max(float v) {  // max over the 4 lanes sharing lane>>2
    v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Quantise one 128-float latent held as 4 consecutive dims per lane into the
// 64 latent bytes + scale + 8 scale bytes of a tile in shared memory.
// One warp per key.  `tile` points at 128 zeroed bytes.
__device__ void quantize_warp(const float* h, int codec, unsigned char* tile, int lane) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = h[4 * lane + j];
    uint32_t* tw = reinterpret_cast<uint32_t*>(tile);
    const float amax4 = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    float global;
    uint32_t gsb;  // this lane's scale byte
    const bool headbody = codec == SLHA_CODEC_MIXED || codec == SLHA_CODEC_MIX3;
    int unit;      // scale-byte index of this lane's dims
    if (codec == SLHA_CODEC_INT4_SINGLE) {  // int4.rs:9-24
        const float mx = warp_max(amax4);
        global = mx > 0.0f ? __fdiv_rn(mx, 7.0f) : 1.0f;
        gsb = 255;
        unit = lane >> 2;
    } else if (!headbody) {
        // grouped codecs: step = absmax / {7, 1, 3.5}; int4.rs:34-63, nf4.rs:23-57, tq3.rs:10-49
        float mx = quad_max(amax4);
        if (codec == SLHA_B200_CODEC_INT4_GROUPED32) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
        const float div = codec == SLHA_CODEC_NF4 ? 1.0f : (codec == SLHA_CODEC_TQ3 ? 3.5f : 7.0f);
        const float step = codec == SLHA_CODEC_NF4 ? mx : __fdiv_rn(mx, div);
        const float g = warp_max(step);
        global = g > 0.0f ? g : 1.0f;
        gsb = scale_byte(step, global);
        unit = lane >> 2;
    } else {
        // head (dims 0..7 = lanes 0,1) + 7 body groups of 16 dims starting at dim 8
        // (mixed.rs:15-33, mix3.rs:13-31): body group of dim D is (D-8)/16, i.e.
        // unit u >= 1 spans lanes 4u-2 .. 4u+1; lanes 30,31 hold the dropped tail.
        const int d0 = 4 * lane;
        unit = lane < 2 ? 0 : (d0 < 120 ? 1 + (d0 - 8) / 16 : 8);
        const int first = lane < 2 ? 0 : (unit < 8 ? 4 * unit - 2 : lane);
        const int span = lane < 2 ? 2 : (unit < 8 ? 4 : 1);
        float mx = 0.0f;
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const float o = __shfl_sync(0xFFFFFFFFu, amax4, min(first + l, 31));
            if (l < span) mx = fmaxf(mx, o);
        }
        const float step = lane < 2 ? __fdiv_rn(mx, 127.0f)
                                    : __fdiv_rn(mx, codec == SLHA_CODEC_MIXED ? 7.0f : 3.5f);
        const float g = warp_max(unit < 8 ? step : 0.0f);
        global = g > 0.0f ? g : 1.0f;
        gsb = unit < 8 ? scale_byte(step, global) : 0;
    }
    // publish scale bytes: the first lane of every unit writes its byte
    if (codec == SLHA_CODEC_INT4_SINGLE) {
        if (lane < 8) tile[120 + lane] = 255;
    } else if (!headbody) {
        if ((lane & 3) == 0) tile[120 + unit] = (unsigned char)gsb;
    } else {
        if (lane == 0 || (lane >= 2 && lane < 30 && ((lane - 2) & 3) == 0)) tile[120 + unit] = (unsigned char)gsb;
    }
    if (lane == 0) *reinterpret_cast<float*>(tile + 96) = global;
    const float eff = __fmul_rn(global, __fdiv_rn((float)gsb, 255.0f));

    if (codec == SLHA_CODEC_INT4_SINGLE || codec == SLHA_CODEC_INT4_GROUPED ||
        codec == SLHA_B200_CODEC_INT4_GROUPED32 || codec == SLHA_CODEC_NF4) {
        uint32_t nib[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (codec == SLHA_CODEC_INT4_SINGLE) {
                nib[j] = int4_nibble(v[j], global);
            } else if (codec == SLHA_CODEC_NF4) {
                float tt = 0.0f;
                if (eff > 0.0f) tt = fminf(fmaxf(__fdiv_rn(v[j], eff), -1.0f), 1.0f);
                nib[j] = nf4_nearest(tt);
            } else {
                nib[j] = int4_nibble(v[j], eff);
            }
        }
        reinterpret_cast<uint16_t*>(tile)[lane] =
            (uint16_t)(nib[0] | (nib[1] << 4) | (nib[2] << 8) | (nib[3] << 12));
    } else if (codec == SLHA_CODEC_TQ3) {
        uint32_t codes = 0, corr = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float tt = __fdiv_rn(v[j], eff);
            const int code = clampi(sat_i32(rnd_half_away(__fadd_rn(tt, 3.5f))), 0, 7);
            codes |= (uint32_t)code << (3 * j);
            if (__fsub_rn(tt, __fsub_rn((float)code, 3.5f)) > 0.0f) corr |= 1u << j;
        }
        const int bit = 12 * lane;  // 4 dims x 3 bits
        atomicOr(&tw[bit >> 5], codes << (bit & 31));
        if ((bit & 31) > 20) atomicOr(&tw[(bit >> 5) + 1], codes >> (32 - (bit & 31)));
        atomicOr(&tw[12 + (lane >> 3)], corr << (4 * (lane & 7)));
    } else {
        // head+body
        const int d0 = 4 * lane;
        if (lane < 2) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int q = clampi(sat_i32(rnd_half_away(__fdiv_rn(v[j], eff))), -128, 127) + 128;
                w |= (uint32_t)q << (8 * j);
            }
            tw[lane] = w;
        } else if (d0 < 120) {
            const int ld0 = d0 - 8;
            if (codec == SLHA_CODEC_MIXED) {
                uint32_t nibs = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) nibs |= int4_nibble(v[j], eff) << (4 * j);
                reinterpret_cast<uint16_t*>(tile)[4 + (ld0 >> 2)] = (uint16_t)nibs;
            } else {
                uint32_t codes = 0, corr = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float tt = __fdiv_rn(v[j], eff);
                    const int code = clampi(sat_i32(rnd_half_away(__fadd_rn(tt, 3.5f))), 0, 7);
                    codes |= (uint32_t)code << (3 * j);
                    if (__fsub_rn(tt, __fsub_rn((float)code, 3.5f)) > 0.0f) corr |= 1u << j;
                }
                const int bit = 64 + 3 * ld0;  // code plane starts at byte 8
                atomicOr(&tw[bit >> 5], codes << (bit & 31));
                if ((bit & 31) > 20) atomicOr(&tw[(bit >> 5) + 1], codes >> (32 - (bit & 31)));
                const int cbit = 400 + ld0;    // correction plane starts at byte 50
                atomicOr(&tw[cbit >> 5], corr << (cbit & 31));
            }
        }
    }
}

// acc[j] += x * v[j] for NK keys whose values lie consecutively (16-byte aligned when NK % 4 == 0),
// each as a separate multiply and add (the reference never fuses them).
template <int NK>
__device__ __forceinline__ void axpy_keys(float (&acc)[NK], float x, const float* v) {
    if (NK % 4 == 0) {
#pragma unroll
        for (int j4 = 0; j4 < NK / 4; ++j4) {
            const float4 b4 = reinterpret_cast<const float4*>(v)[j4];
            acc[4 * j4 + 0] = __fadd_rn(acc[4 * j4 + 0], __fmul_rn(x, b4.x));
            acc[4 * j4 + 1] = __fadd_rn(acc[4 * j4 + 1], __fmul_rn(x, b4.y));
            acc[4 * j4 + 2] = __fadd_rn(acc[4 * j4 + 2], __fmul_rn(x, b4.z));
            acc[4 * j4 + 3] = __fadd_rn(acc[4 * j4 + 3], __fmul_rn(x, b4.w));
        }
    } else {
#pragma unroll
        for (int j = 0; j < NK; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(x, v[j]));
    }
}

// NK consecutive floats (16-byte aligned when NK % 4 == 0) to / from registers
template <int NK>
__device__ __forceinline__ void store_keys(float* dst, const float (&v)[NK]) {
    if (NK % 4 == 0) {
#pragma unroll
        for (int j4 = 0; j4 < NK / 4; ++j4)
            reinterpret_cast<float4*>(dst)[j4] = make_float4(v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < NK; ++j) dst[j] = v[j];
    }
}
template <int NK>
__device__ __forceinline__ void load_keys(float (&v)[NK], const float* src) {
    if (NK % 4 == 0) {
#pragma unroll
        for (int j4 = 0; j4 < NK / 4; ++j4) {
            const float4 x = reinterpret_cast<const float4*>(src)[j4];
            v[4 * j4] = x.x; v[4 * j4 + 1] = x.y; v[4 * j4 + 2] = x.z; v[4 * j4 + 3] = x.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < NK; ++j) v[j] = src[j];
    }
}

// Packed pairs of float32 (Blackwell f32x2): one instruction multiplies two independent float32
// pairs, each product rounded to nearest exactly like the scalar multiply, so the two products of
// a key pair cost one issue slot.  The additions stay scalar: the assembler contracts a packed
// multiply followed by a packed add into a packed fused multiply-add even when both carry an
// explicit rounding mode and contraction is switched off (checked on sm_100a, CUDA 12.9), and a
// fused multiply-add rounds once where the reference rounds twice.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void mul2(uint64_t a, uint64_t b, float& lo, float& hi) {
    uint64_t m;
    asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(m) : "l"(a), "l"(b));
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(m));
}

// acc[r][j] += m[r] * v[j] for an R x K register tile: R output rows (or columns) times K keys.
// Each output still sums its products in contraction order, one multiply and one add at a time.
template <int R, int K>
__device__ __forceinline__ void outer_keys(float (&acc)[R][K], const float4& m4, const float* v) {
    static_assert(R == 4 && K % 4 == 0, "the matrix operand is one 16-byte load");
    uint64_t kv[K / 2];
#pragma unroll
    for (int j4 = 0; j4 < K / 4; ++j4) {
        const float4 x = reinterpret_cast<const float4*>(v)[j4];
        kv[2 * j4] = pack2(x.x, x.y);
        kv[2 * j4 + 1] = pack2(x.z, x.w);
    }
    const uint64_t m[4] = {pack2(m4.x, m4.x), pack2(m4.y, m4.y), pack2(m4.z, m4.z), pack2(m4.w, m4.w)};
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < K / 2; ++j) {
            float p0, p1;
            mul2(m[r], kv[j], p0, p1);
            acc[r][2 * j] = __fadd_rn(acc[r][2 * j], p0);
            acc[r][2 * j + 1] = __fadd_rn(acc[r][2 * j + 1], p1);
        }
}
template <int R, int K>
__device__ __forceinline__ void zero_tile(float (&acc)[R][K]) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < K; ++j) acc[r][j] = 0.0f;
}

// KB keys per CTA pass (compile time: 32 unless the model dimension leaves no room).  Every
// contraction is walked sequentially by the thread that owns the output element, for all the keys
// the thread holds at once: one matrix element and KB/8 (latent, residual: half the keys per thread)
// or KB/4 (sign bits) vector loads feed KB or 2 KB multiply-adds.
constexpr int enc_row_stride(int kb) { return kb >= 8 ? kb + 4 : kb; }

template <bool QUERY, int KB>
// (three CTAs of 32 keys share an SM at head dimension 128: 80 registers, 74 KB of shared memory each)
__global__ void __launch_bounds__(ENC_THREADS, KB == 32 ? 3 : 1) encode_kernel(EncodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int PER = KB >= 2 ? KB / 2 : 1;  // keys per thread where two threads share an output row
    const uint32_t d = a.d, dp = a.d_pad;
    // shared: tiles [KB][128 B] | h [KB][128] | keyT [d][KS] | bufT [d_pad][KS] | wsT [128][KS]
    // (keys and the sign-LSH input are stored transposed so that one thread
    // reads the KB values of a contraction index with 16-byte loads).  Rows are KS = KB + 4
    // floats apart: a warp whose lanes walk the rows then spreads its 16-byte accesses over
    // all banks, while lanes that walk the keys of one row stay on consecutive banks.
    constexpr int KS = enc_row_stride(KB);
    unsigned char* tl = smem;
    float* hs = reinterpret_cast<float*>(tl + (size_t)KB * TILE_BYTES);
    float* keyT = hs + (size_t)KB * D_C;
    float* buf = keyT + (((size_t)d * KS + 3) & ~size_t(3));
    float* wsT = buf + (size_t)dp * KS;  // h_k * s_k of every key, transposed like keyT

    for (uint64_t base = (uint64_t)blockIdx.x * KB; base < a.n; base += (uint64_t)gridDim.x * KB) {
        const int nk = (int)min((uint64_t)KB, a.n - base);
        __syncthreads();
        // ---- load keys (transposed: keyT[i][j]); absent keys are zero ------
        const bool f32 = a.key_dtype == SLHA_B200_F32;
        const uint32_t epc = f32 ? 4u : 8u;  // elements per 16-byte chunk
        if (KB >= 8 && d % epc == 0 && (reinterpret_cast<uintptr_t>(a.keys) & 15) == 0) {
            // 16-byte chunks; the lanes of a warp take the same chunk of consecutive keys, so
            // that their transposed stores fall on consecutive banks.  Both loads of a thread
            // are in flight before the first store.
            const uint32_t cpk = d / epc, total = cpk * (uint32_t)KB;
            const uint4* src = reinterpret_cast<const uint4*>(a.keys) + base * cpk;
            for (uint32_t c0 = tid; c0 < total; c0 += 2 * ENC_THREADS) {
                uint4 v[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t c = c0 + u * ENC_THREADS, j = c % KB, ic = c / KB;
                    v[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (c < total && (int)j < nk) v[u] = __ldg(src + (size_t)j * cpk + ic);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const uint32_t c = c0 + u * ENC_THREADS, j = c % KB, ic = c / KB;
                    if (c >= total) continue;
                    float* dst = keyT + (size_t)(ic * epc) * KS + j;
                    const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (f32) {
                            dst[(size_t)q * KS] = __uint_as_float(w[q]);
                        } else {  // bf16 -> f32 widening is exact
                            dst[(size_t)(2 * q) * KS] = __uint_as_float(w[q] << 16);
                            dst[(size_t)(2 * q + 1) * KS] = __uint_as_float(w[q] & 0xFFFF0000u);
                        }
                    }
                }
            }
        } else {
            for (uint32_t e = tid; e < d * (uint32_t)KB; e += ENC_THREADS) {
                const int j = e / d;
                const uint32_t i = e % d;
                float x = 0.0f;
                if (j < nk) {
                    const uint64_t o = (base + j) * d + i;
                    x = f32 ? reinterpret_cast<const float*>(a.keys)[o]
                            : __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(a.keys)[o] << 16);
                }
                keyT[(size_t)i * KS + j] = x;
            }
        }
        for (int e = tid; e < KB * 32; e += ENC_THREADS) reinterpret_cast<uint32_t*>(tl)[e] = 0;
        __syncthreads();

        // With 32 keys per pass every thread holds a 4 x 4 (latent, residual) or 4 x 8 (sign bits)
        // tile of outputs: four matrix elements (one 16-byte load) and four or eight key values
        // (one or two 16-byte broadcast loads) feed 16 or 32 multiply-adds, a third of the
        // register fills per multiply-add of a one-row tile.
        const bool tiled = KB == 32 && d % 4 == 0 &&
                           ((reinterpret_cast<uintptr_t>(a.pt) | reinterpret_cast<uintptr_t>(a.p) |
                             reinterpret_cast<uintptr_t>(a.zt) | reinterpret_cast<uintptr_t>(a.scale)) & 15) == 0;
        // ---- latent / q_coarse: rows 4 lane .. +3, keys 4 warp .. +3 ------------
        if (KB == 32 && tiled) {
            float acc[4][4];
            zero_tile<4, 4>(acc);
            const float4* mp = reinterpret_cast<const float4*>(a.pt) + lane;
#pragma unroll 16
            for (uint32_t i = 0; i < d; ++i)
                outer_keys<4, 4>(acc, __ldg(mp + (size_t)i * (D_C / 4)), keyT + (size_t)i * KS + 4 * warp);
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(a.scale) + lane);
            const float sk[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float hv[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    hv[r] = QUERY ? __fmul_rn(acc[r][j], sk[r]) : __fdiv_rn(acc[r][j], sk[r]);
                    acc[r][j] = __fmul_rn(hv[r], sk[r]);  // w[k][j] = h_j[k] * s_k, the factor of P[k][:] in the reconstruction
                }
                store_keys<4>(hs + (size_t)(4 * warp + j) * D_C + 4 * lane, hv);
            }
            if (!QUERY) {
#pragma unroll
                for (int r = 0; r < 4; ++r) store_keys<4>(wsT + (size_t)(4 * lane + r) * KS + 4 * warp, acc[r]);
            }
        } else {
            // row k = tid & 127, keys of half (tid >> 7)
            const int k = tid & 127, half = tid >> 7;
            const int j0 = (KB >= 2) ? half * PER : 0;
            if (KB >= 2 || half == 0) {
                float acc[PER];
#pragma unroll
                for (int j = 0; j < PER; ++j) acc[j] = 0.0f;
#pragma unroll 8
                for (uint32_t i = 0; i < d; ++i)
                    axpy_keys<PER>(acc, a.pt[(size_t)i * D_C + k], keyT + (size_t)i * KS + j0);
                const float sk = a.scale[k];
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const float hv = QUERY ? __fmul_rn(acc[j], sk) : __fdiv_rn(acc[j], sk);
                    hs[(size_t)(j0 + j) * D_C + k] = hv;
                    // w[k][j] = h_j[k] * s_k, the factor the reconstruction multiplies P[k][:] by
                    acc[j] = __fmul_rn(hv, sk);
                }
                if (!QUERY) store_keys<PER>(wsT + (size_t)k * KS + j0, acc);
            }
        }
        __syncthreads();

        if (QUERY) {
            for (int e = tid; e < nk * D_C; e += ENC_THREADS)
                a.q_coarse[(base + e / D_C) * D_C + (e % D_C)] = hs[e];
            // sign-LSH input is the raw query
            for (uint32_t e = tid; e < dp * (uint32_t)KS; e += ENC_THREADS)
                buf[e] = (e / KS) < d ? keyT[e] : 0.0f;
        } else {
            // ---- quantise: one warp per key ---------------------------------
            for (int j = warp; j < KB; j += ENC_THREADS / 32)
                quantize_warp(hs + (size_t)j * D_C, a.codec, tl + (size_t)j * TILE_BYTES, lane);
            // (no barrier: the residual phase reads the keys and the reconstruction factors, which
            //  the barrier after the latent phase already covers, and does not touch the tiles)
            // ---- residual e = key - sum_k (h_k*s_k) * P[k][:]  (k outer, sequential): a thread owns
            //      column i for half of the keys ---------------------------------------------------
            constexpr int HALVES = KB >= 2 ? 2 : 1;
            // tiled: columns 4 ig .. +3 for keys 4 kg .. +3
            for (uint32_t wi = tid; KB == 32 && tiled && wi < (d / 4) * 8; wi += ENC_THREADS) {
                const uint32_t ig = wi % (d / 4), kg = wi / (d / 4);
                float acc[4][4];
                zero_tile<4, 4>(acc);
                const float4* mp = reinterpret_cast<const float4*>(a.p) + ig;
                const float* wr = wsT + 4 * kg;
#pragma unroll 16
                for (int k = 0; k < D_C; ++k)
                    outer_keys<4, 4>(acc, __ldg(mp + (size_t)k * (d / 4)), wr + (size_t)k * KS);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float kv[4];
                    load_keys<4>(kv, keyT + (size_t)(4 * ig + r) * KS + 4 * kg);
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[r][j] = __fsub_rn(kv[j], acc[r][j]);
                    store_keys<4>(buf + (size_t)(4 * ig + r) * KS + 4 * kg, acc[r]);
                }
            }
            for (uint32_t wi = tid; !(KB == 32 && tiled) && wi < HALVES * d; wi += ENC_THREADS) {
                const uint32_t i = wi % d, half = wi / d;
                float acc[PER];
#pragma unroll
                for (int j = 0; j < PER; ++j) acc[j] = 0.0f;
                const float* wr = wsT + half * PER;
#pragma unroll 8
                for (int k = 0; k < D_C; ++k) axpy_keys<PER>(acc, a.p[(size_t)k * d + i], wr + (size_t)k * KS);
                float kv[PER];
                load_keys<PER>(kv, keyT + (size_t)i * KS + half * PER);
#pragma unroll
                for (int j = 0; j < PER; ++j) acc[j] = __fsub_rn(kv[j], acc[j]);
                store_keys<PER>(buf + (size_t)i * KS + half * PER, acc);
            }
            for (uint32_t e = d * KS + tid; e < dp * KS; e += ENC_THREADS) buf[e] = 0.0f;  // padding rows
        }
        __syncthreads();

        // ---- sigma_E (f32, sequential over i) and tile metadata ---------------
        if (!QUERY && tid < nk) {
            const int j = tid;
            float ss = 0.0f;
            for (uint32_t i = 0; i < d; ++i) {
                const float x = buf[(size_t)i * KS + j];
                ss = __fadd_rn(ss, __fmul_rn(x, x));
            }
            const float sigma = __fsqrt_rn(__fdiv_rn(ss, (float)d));
            unsigned char* tile = tl + (size_t)j * TILE_BYTES;
            const uint32_t pos = a.positions ? a.positions[base + j] : a.position_base + (uint32_t)(base + j);
            *reinterpret_cast<float*>(tile + 100) = __fmul_rn(sigma, a.lambda_c);
            *reinterpret_cast<float*>(tile + 104) = sigma;
            *reinterpret_cast<uint32_t*>(tile + 108) = pos;
            *reinterpret_cast<uint32_t*>(tile + 112) = pos;
            const uint32_t head = a.heads ? a.heads[base + j] : 0u;
            uint32_t cflag = 0;
            if (a.codec == SLHA_CODEC_NF4) cflag = F_NF4;
            else if (a.codec == SLHA_CODEC_MIXED) cflag = F_MIXED;
            else if (a.codec == SLHA_CODEC_TQ3) cflag = F_TQ3;
            else if (a.codec == SLHA_CODEC_MIX3) cflag = F_MIX3;
            *reinterpret_cast<uint32_t*>(tile + 116) = head | (cflag << 16);
        }
        __syncthreads();

        // ---- optional randomised Hadamard transform of buf ------------------
        if (a.diag) {
            for (uint32_t e = tid; e < dp * (uint32_t)KS; e += ENC_THREADS)
                buf[e] = __fmul_rn(buf[e], a.diag[e / KS]);
            __syncthreads();
            for (uint32_t h = 1; h < dp; h <<= 1) {
                for (uint32_t e = tid; e < (dp / 2) * (uint32_t)KB; e += ENC_THREADS) {
                    const uint32_t j = e % KB, pr = e / KB;
                    const uint32_t lo = ((pr / h) * 2 * h) + (pr % h);
                    float* col = buf + j;
                    const float x = col[(size_t)lo * KS], y = col[(size_t)(lo + h) * KS];
                    col[(size_t)lo * KS] = __fadd_rn(x, y);
                    col[(size_t)(lo + h) * KS] = __fsub_rn(x, y);
                }
                __syncthreads();
            }
            for (uint32_t e = tid; e < dp * (uint32_t)KS; e += ENC_THREADS)
                buf[e] = __fmul_rn(buf[e], a.fwht_inv);
            __syncthreads();
        }

        // ---- sign-LSH, tiled: hyperplanes 4 rg .. +3 for keys 8 kg .. +7 -------
        if (KB == 32 && tiled) {
            const int rg = tid & 63, kg = tid >> 6;
            float acc[4][8];
            zero_tile<4, 8>(acc);
            const float4* mp = reinterpret_cast<const float4*>(a.zt) + rg;
#pragma unroll 16
            for (uint32_t i = 0; i < dp; ++i)
                outer_keys<4, 8>(acc, __ldg(mp + (size_t)i * (D_S / 4)), buf + (size_t)i * KS + 8 * kg);
            // bit s of a key = (acc < 0); this thread holds bits 4 rg .. +3, eight lanes fill a 32-bit word
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t v = (acc[0][j] < 0.0f ? 1u : 0u) | (acc[1][j] < 0.0f ? 2u : 0u) |
                             (acc[2][j] < 0.0f ? 4u : 0u) | (acc[3][j] < 0.0f ? 8u : 0u);
                v <<= 4 * (lane & 7);
                v |= __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                v |= __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                v |= __shfl_xor_sync(0xFFFFFFFFu, v, 4);
                const int key = 8 * kg + j, word = (rg >> 3);
                if ((lane & 7) == 0 && key < nk) {
                    if (QUERY)
                        reinterpret_cast<uint32_t*>(a.q_sign)[(base + key) * 8 + word] = v;
                    else
                        reinterpret_cast<uint32_t*>(tl + (size_t)key * TILE_BYTES + 64)[word] = v;
                }
            }
        } else {
            // thread s owns hyperplane s for all KB keys
            const int s = tid;  // ENC_THREADS == D_S
            float acc[KB];
#pragma unroll
            for (int j = 0; j < KB; ++j) acc[j] = 0.0f;
#pragma unroll 8
            for (uint32_t i = 0; i < dp; ++i) axpy_keys<KB>(acc, a.zt[(size_t)i * D_S + s], buf + (size_t)i * KS);
#pragma unroll
            for (int j = 0; j < KB; ++j) {
                const unsigned b = __ballot_sync(0xFFFFFFFFu, acc[j] < 0.0f);
                if (lane == 0 && j < nk) {
                    if (QUERY)
                        reinterpret_cast<uint32_t*>(a.q_sign)[(base + j) * 8 + warp] = b;
                    else
                        reinterpret_cast<uint32_t*>(tl + (size_t)j * TILE_BYTES + 64)[warp] = b;
                }
            }
        }
        __syncthreads();

        // ---- write tiles: 8 x 16 B per tile ------------------------------------
        if (!QUERY) {
            for (int e = tid; e < nk * 8; e += ENC_THREADS) {
                const int j = e >> 3, c = e & 7;
                const uint64_t dst = a.slots ? a.slots[base + j] : base + j;
                reinterpret_cast<uint4*>(a.tiles + dst * TILE_BYTES)[c] =
                    reinterpret_cast<const uint4*>(tl + (size_t)j * TILE_BYTES)[c];
            }
        }
    }
}

// reconstruct (learned.rs:276-286) from the dequantised latent of one tile, and
// optionally the sign-sketch estimate of reconstruct_from_tile (learned.rs:290-322)
__global__ void decode_kernel(const unsigned char* tile, const float* p, const float* scale,
                              const float* z, uint32_t d, uint32_t d_pad, int with_residual,
                              float* out) {
    __shared__ float k[D_C];
    __shared__ float sgn[D_S];
    const uint32_t flags = *reinterpret_cast<const uint16_t*>(tile + 118);
    const float sc = *reinterpret_cast<const float*>(tile + 96);
    for (int dd = threadIdx.x; dd < D_C; dd += blockDim.x) {
        // tile.rs:133-255
        float v;
        auto alt = [&](int g) { return __fdiv_rn(__fmul_rn(sc, (float)tile[120 + g]), 255.0f); };
        auto grp = [&](int dim) { return __fmul_rn(sc, __fdiv_rn((float)tile[120 + dim / 16], 255.0f)); };
        auto code3 = [&](int off, int end, int ld) {
            const int bit = 3 * ld, byte = off + (bit >> 3), sh = bit & 7;
            const uint32_t lo = tile[byte], hi = (byte + 1 < end) ? ((uint32_t)tile[byte + 1] << 8) : 0u;
            return (int)(((lo | hi) >> sh) & 7u);
        };
        if (flags & F_MIXED) {
            if (dd < 8) v = __fmul_rn((float)((int)tile[dd] - 128), alt(0));
            else if (dd < 120) {
                const int ld = dd - 8;
                const uint32_t b = tile[8 + (ld >> 1)];
                v = __fmul_rn((float)((int)((ld & 1) ? (b >> 4) : (b & 15)) - 8), alt(1 + ld / 16));
            } else v = 0.0f;
        } else if (flags & F_TQ3) {
            float level = (float)code3(0, 48, dd) - 3.5f;
            if (!(flags & F_NOCORR)) level += ((tile[48 + (dd >> 3)] >> (dd & 7)) & 1) ? 0.25f : -0.25f;
            v = __fmul_rn(level, grp(dd));
        } else if (flags & F_MIX3) {
            if (dd < 8) v = __fmul_rn((float)((int)tile[dd] - 128), alt(0));
            else if (dd >= 120) v = 0.0f;
            else {
                const int ld = dd - 8;
                float level = (float)code3(8, 50, ld) - 3.5f;
                if (!(flags & F_NOCORR)) level += ((tile[50 + (ld >> 3)] >> (ld & 7)) & 1) ? 0.25f : -0.25f;
                v = __fmul_rn(level, alt(1 + ld / 16));
            }
        } else {
            const uint32_t b = tile[dd >> 1];
            const uint32_t nib = (dd & 1) ? (b >> 4) : (b & 15);
            const float cb[16] = {-1.0f,   -0.7075f, -0.5421f, -0.4165f, -0.3108f, -0.2158f,
                                  -0.1272f, -0.0421f, 0.0421f,  0.1272f,  0.2158f,  0.3108f,
                                  0.4165f,  0.5421f,  0.7075f,  1.0f};
            const float level = (flags & F_NF4) ? cb[nib] : (float)((int)nib - 8);
            v = __fmul_rn(level, grp(dd));
        }
        k[dd] = v;
    }
    const float sigma = *reinterpret_cast<const float*>(tile + 104);
    const float rs = __fdiv_rn(__fmul_rn(sigma, __fsqrt_rn(__fdiv_rn(3.14159265358979323846f, 2.0f))), (float)D_S);
    for (int s = threadIdx.x; s < D_S; s += blockDim.x) {
        const uint64_t w = reinterpret_cast<const uint64_t*>(tile + 64)[s >> 6];
        sgn[s] = ((w >> (s & 63)) & 1ull) ? -1.0f : 1.0f;
    }
    __syncthreads();
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < d; i += gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int kk = 0; kk < D_C; ++kk)
            acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(k[kk], scale[kk]), p[(size_t)kk * d + i]));
        if (with_residual)
            for (int s = 0; s < D_S; ++s)
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sgn[s], rs), z[(size_t)s * d_pad + i]));
        out[i] = acc;
    }
}

size_t encode_smem(uint32_t d, uint32_t dp, int kb) {
    const size_t ks = (size_t)enc_row_stride(kb);
    return (((d * ks + 3) & ~size_t(3)) + (size_t)kb * D_C + ks * dp + ks * D_C) * 4 + (size_t)kb * TILE_BYTES;
}

Status fill_args(const Model* m, EncodeArgs& a, int* kb_out) {
    a.d = (uint32_t)m->d;
    a.d_pad = (uint32_t)m->d_pad;
    a.p = m->d_p;
    a.pt = m->d_pt;
    a.scale = m->d_scale;
    a.zt = m->d_zt;
    a.diag = m->d_diag;
    a.fwht_inv = 1.0f / sqrtf((float)m->d_pad);
    a.lambda_c = sqrtf(3.14159265358979323846f / (2.0f * (float)D_S));
    // 32 keys per CTA pass when two CTAs still share an SM (their registers allow no more), else fewer
    int kb = 32;
    while (kb > 1 && encode_smem(a.d, a.d_pad, kb) > (kb == 32 ? 100 : 200) * 1024) kb >>= 1;
    if (encode_smem(a.d, a.d_pad, kb) > 200 * 1024)
        return Status(SLHA_ERR_DIMENSION, "model dimension too large for the encode kernel");
    *kb_out = kb;
    a.kb = kb;
    return Status();
}

template <bool QUERY, int KB>
Status run_encode_kb(Ctx* c, EncodeArgs& a) {
    const size_t smem = encode_smem(a.d, a.d_pad, KB);
    static thread_local bool configured[16] = {false};  // the attribute is per device
    if (!configured[c->device & 15]) {
        SLHA_CUDA(cudaFuncSetAttribute(encode_kernel<QUERY, KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured[c->device & 15] = true;
    }
    const uint64_t groups = (a.n + KB - 1) / KB;
    // far more CTAs than fit at once (444 are resident at head dimension 128): the hardware hands
    // out a CTA whenever one finishes, which balances the tail and keeps the CTAs sharing an SM in
    // different phases, so that the arithmetic of one covers the loads, quantisation and barriers
    // of the others.  One resident wave measured 182 M keys/s, 8 CTAs per SM 191, one CTA per pass 199.
    const uint32_t grid = (uint32_t)std::min<uint64_t>(groups, 148ull * 64);
    encode_kernel<QUERY, KB><<<grid, ENC_THREADS, smem, c->stream>>>(a);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

template <bool QUERY>
Status run_encode(Ctx* c, EncodeArgs& a) {
    switch (a.kb) {
        case 32: return run_encode_kb<QUERY, 32>(c, a);
        case 16: return run_encode_kb<QUERY, 16>(c, a);
        case 8: return run_encode_kb<QUERY, 8>(c, a);
        case 4: return run_encode_kb<QUERY, 4>(c, a);
        case 2: return run_encode_kb<QUERY, 2>(c, a);
        default: return run_encode_kb<QUERY, 1>(c, a);
    }
}

}  // namespace

Status launch_encode(Ctx* c, const Model* m, const void* d_keys, int key_dtype, size_t n,
                     const uint32_t* d_positions, uint32_t position_base, const uint16_t* d_heads,
                     int codec, SciRustSlhaTile* d_tiles, const uint32_t* d_slots) {
    if (n == 0) return Status();
    EncodeArgs a{};
    int kb;
    SLHA_TRY(fill_args(m, a, &kb));
    a.keys = d_keys;
    a.key_dtype = key_dtype;
    a.n = n;
    a.positions = d_positions;
    a.position_base = position_base;
    a.heads = d_heads;
    a.codec = codec;
    a.tiles = reinterpret_cast<unsigned char*>(d_tiles);
    a.slots = d_slots;
    return run_encode<false>(c, a);
}

Status launch_prepare_queries(Ctx* c, const Model* m, const float* d_q, size_t nq,
                              float* d_q_coarse, uint64_t* d_q_sign) {
    if (nq == 0) return Status();
    EncodeArgs a{};
    int kb;
    SLHA_TRY(fill_args(m, a, &kb));
    a.keys = d_q;
    a.key_dtype = SLHA_B200_F32;
    a.n = nq;
    a.q_coarse = d_q_coarse;
    a.q_sign = d_q_sign;
    return run_encode<true>(c, a);
}

Status launch_decode(Ctx* c, const Model* m, const SciRustSlhaTile* d_tile, float* d_out,
                     bool with_residual) {
    const uint32_t d = (uint32_t)m->d;
    decode_kernel<<<(d + 127) / 128, 128, 0, c->stream>>>(
        reinterpret_cast<const unsigned char*>(d_tile), m->d_p, m->d_scale, m->d_z, d,
        (uint32_t)m->d_pad, with_residual && !m->rht, d_out);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

}  // namespace slha
