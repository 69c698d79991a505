// Decode tail on the selected tiles: softmax over the k winners of every query row, then the
// weighted sum of their value rows -- the two steps that follow scoring in the reference's decode
// proxy (scirust/examples/benchmark_decode.rs:82-95: metrics::softmax_into, scirust/src/metrics.rs:338-420,
// then aggregate_v, benchmark_decode.rs:28-38), applied to the top-k instead of the whole context.
// The k (index, score) pairs stay in HBM; what crosses PCIe afterwards is one d_v-vector per query
// row instead of k pairs.
//
// One query row is shared by SPLIT CTAs, each taking a contiguous run of the winners; every CTA
// recomputes the row's maximum and normaliser (k scores, a few KB) so that no CTA waits for another,
// writes its partial sum, and a second small kernel adds the partial sums in a fixed order.
#include <cuda_bf16.h>

#include <cfloat>

#include "runtime.cuh"

namespace slha {
namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_SPLIT = 8;

__device__ __forceinline__ float load_value(const float* p) { return *p; }
__device__ __forceinline__ float load_value(const __nv_bfloat16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
    for (int o = 16; o; o >>= 1) {
        const float y = __shfl_xor_sync(0xFFFFFFFFu, v, o);
        v = is_max ? fmaxf(v, y) : v + y;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = is_max ? fmaxf(r, sh[w]) : r + sh[w];
    return r;
}

// weights_out (optional): [nq][k] softmax weights (0 for absent entries)
template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) attend_partial_kernel(const uint32_t* top_index, const float* top_score,
                                                                     const uint32_t* top_count, uint32_t k, float scale,
                                                                     const T* values, size_t d_v, size_t row_stride,
                                                                     const uint64_t* row_base, float* partial, float* weights_out) {
    extern __shared__ float sm[];  // [k] weights | [8] reduction
    float* w = sm;
    float* red = sm + k;
    const uint32_t Q = blockIdx.y, part = blockIdx.x, tid = threadIdx.x;
    const uint32_t n = top_count ? min(top_count[Q], k) : k;
    const float* sc = top_score + (size_t)Q * k;
    const uint32_t* ix = top_index + (size_t)Q * k;
    // softmax_into: logits = score * scale, maximum subtracted, normalised (absent entries weigh nothing)
    float mx = -INFINITY;
    for (uint32_t i = tid; i < n; i += blockDim.x)
        if (ix[i] != 0xFFFFFFFFu) mx = fmaxf(mx, sc[i] * scale);
    mx = block_reduce(mx, red, true);
    float sum = 0.0f;
    for (uint32_t i = tid; i < k; i += blockDim.x) {
        float e = 0.0f;
        if (i < n && ix[i] != 0xFFFFFFFFu && mx > -INFINITY) e = expf(sc[i] * scale - mx);
        w[i] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    const float inv = (sum > 0.0f && isfinite(sum)) ? 1.0f / sum : 0.0f;
    __syncthreads();
    if (weights_out && part == 0)
        for (uint32_t i = tid; i < k; i += blockDim.x) weights_out[(size_t)Q * k + i] = w[i] * inv;
    // this CTA's run of winners; threads cover the value row's columns, row groups take alternate winners
    const uint32_t per = (n + ATT_SPLIT - 1) / ATT_SPLIT;
    const uint32_t lo = min(n, part * per), hi = min(n, lo + per);
    const uint64_t base = row_base ? row_base[Q] : 0ull;
    const uint32_t cols = d_v < (size_t)blockDim.x ? (uint32_t)d_v : blockDim.x;
    const uint32_t groups = blockDim.x / cols, grp = tid / cols, col0 = tid % cols;
    float* out = partial + ((size_t)Q * ATT_SPLIT + part) * d_v;
    for (uint32_t c = col0; c < d_v; c += cols) {
        float acc = 0.0f;
        if (grp < groups) {
            uint32_t i = lo + grp;
            for (; i + 3 * groups < hi; i += 4 * groups) {  // four value rows in flight
                const uint32_t i0 = ix[i], i1 = ix[i + groups], i2 = ix[i + 2 * groups], i3 = ix[i + 3 * groups];
                const float v0 = i0 != 0xFFFFFFFFu ? load_value(values + (base + i0) * row_stride + c) : 0.0f;
                const float v1 = i1 != 0xFFFFFFFFu ? load_value(values + (base + i1) * row_stride + c) : 0.0f;
                const float v2 = i2 != 0xFFFFFFFFu ? load_value(values + (base + i2) * row_stride + c) : 0.0f;
                const float v3 = i3 != 0xFFFFFFFFu ? load_value(values + (base + i3) * row_stride + c) : 0.0f;
                acc = fmaf(w[i], v0, acc);
                acc = fmaf(w[i + groups], v1, acc);
                acc = fmaf(w[i + 2 * groups], v2, acc);
                acc = fmaf(w[i + 3 * groups], v3, acc);
            }
            for (; i < hi; i += groups) {
                const uint32_t i0 = ix[i];
                if (i0 != 0xFFFFFFFFu) acc = fmaf(w[i], load_value(values + (base + i0) * row_stride + c), acc);
            }
        }
        // the row groups' sums are added in a fixed order through shared memory
        float* slot = sm + k + 8;  // [blockDim.x]
        __syncthreads();
        slot[tid] = acc;
        __syncthreads();
        if (grp == 0) {
            float total = 0.0f;
            for (uint32_t g2 = 0; g2 < groups; ++g2) total += slot[g2 * cols + col0];
            out[c] = total * inv;
        }
    }
}

__global__ void attend_reduce_kernel(const float* partial, size_t d_v, float* out) {
    const uint32_t Q = blockIdx.x;
    for (size_t c = threadIdx.x; c < d_v; c += blockDim.x) {
        float s = 0.0f;
        for (int p = 0; p < ATT_SPLIT; ++p) s += partial[((size_t)Q * ATT_SPLIT + p) * d_v + c];
        out[(size_t)Q * d_v + c] = s;
    }
}

}  // namespace

Status launch_attend_topk(Ctx* c, const uint32_t* d_index, const float* d_score, const uint32_t* d_count, size_t nq, uint32_t k,
                          float scale, const void* d_values, int value_dtype, size_t d_v, size_t row_stride,
                          const uint64_t* d_row_base, float* d_out, float* d_weights) {
    if (nq == 0 || d_v == 0) return Status();
    if (k == 0 || k > 8192) return Status(SLHA_ERR_DIMENSION, "attend_topk: k must be in 1..8192");
    if (!isfinite(scale)) return Status(SLHA_ERR_NONFINITE, "attend_topk: scale is not finite");
    void* partial = nullptr;
    SLHA_TRY(ctx_device_scratch(c, nq * ATT_SPLIT * d_v * sizeof(float), &partial));
    const size_t smem = ((size_t)k + 8 + ATT_THREADS) * sizeof(float);
    const dim3 grid(ATT_SPLIT, (uint32_t)nq);
    if (value_dtype == SLHA_B200_BF16)
        attend_partial_kernel<__nv_bfloat16><<<grid, ATT_THREADS, smem, c->stream>>>(
            d_index, d_score, d_count, k, scale, (const __nv_bfloat16*)d_values, d_v, row_stride, d_row_base, (float*)partial, d_weights);
    else
        attend_partial_kernel<float><<<grid, ATT_THREADS, smem, c->stream>>>(d_index, d_score, d_count, k, scale, (const float*)d_values,
                                                                               d_v, row_stride, d_row_base, (float*)partial, d_weights);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    attend_reduce_kernel<<<(uint32_t)nq, 128, 0, c->stream>>>((const float*)partial, d_v, d_out);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

}  // namespace slha
