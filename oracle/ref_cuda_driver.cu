// TEST INFRASTRUCTURE ONLY: host driver around the reference's own CUDA scoring
// kernel (slhav2-vram/kernels/slha_score.cu:128-199, one thread per tile).
// The kernel source is NOT copied here: this file includes it from the reference
// tree at build time (macro SLHA_REF_KERNEL), so the library exists only where
// the reference is mounted; the built oracle/_ref/libslha_ref_cuda.so travels to
// the GPU machine.  Launch geometry follows the reference's own tests
// (slhav2-vram/tests/cuda.rs:542-543): 256-thread blocks, one launch per query.
// Used by the GPU tests to check the CPU restatement and the library against the
// reference's real device code, and by bench.py as an extra timing for context.
#include <cuda_runtime.h>

#include SLHA_REF_KERNEL

namespace {
int fail(cudaError_t e) { return e == cudaSuccess ? 0 : 1000 + (int)e; }
}  // namespace

// Host buffers in, host scores out: scores[q][n] for nq queries.  0 on success.
extern "C" int slha_ref_cuda_score(const unsigned char* tiles, int n_tiles, const float* q_coarse,
                                   const unsigned long long* q_sign, int nq, float* scores_out) {
    unsigned char* d_tiles = nullptr;
    float *d_q = nullptr, *d_out = nullptr;
    unsigned long long* d_s = nullptr;
    cudaError_t e;
    if ((e = cudaMalloc(&d_tiles, (size_t)n_tiles * 128)) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&d_q, (size_t)nq * 128 * 4)) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&d_s, (size_t)nq * 32)) != cudaSuccess) return fail(e);
    if ((e = cudaMalloc(&d_out, (size_t)nq * n_tiles * 4)) != cudaSuccess) return fail(e);
    cudaMemcpy(d_tiles, tiles, (size_t)n_tiles * 128, cudaMemcpyHostToDevice);
    cudaMemcpy(d_q, q_coarse, (size_t)nq * 128 * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_s, q_sign, (size_t)nq * 32, cudaMemcpyHostToDevice);
    for (int q = 0; q < nq; ++q)
        slha_score_kernel<<<(n_tiles + 255) / 256, 256>>>(d_q + (size_t)q * 128, d_s + (size_t)q * 4, d_tiles,
                                                          d_out + (size_t)q * n_tiles, n_tiles);
    e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(scores_out, d_out, (size_t)nq * n_tiles * 4, cudaMemcpyDeviceToHost);
    cudaFree(d_tiles);
    cudaFree(d_q);
    cudaFree(d_s);
    cudaFree(d_out);
    return fail(e);
}

// Device buffers (tiles, prepared queries, a scores buffer of nq * n_tiles floats), `reps` timed
// passes of nq launches each on the given stream; returns the mean milliseconds per pass in *ms_out.
extern "C" int slha_ref_cuda_time(const unsigned char* d_tiles, int n_tiles, const float* d_q_coarse,
                                  const unsigned long long* d_q_sign, int nq, float* d_scores, int reps, void* stream,
                                  float* ms_out) {
    cudaStream_t s = (cudaStream_t)stream;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    for (int r = 0; r < reps + 1; ++r) {
        if (r == 1) cudaEventRecord(a, s);
        for (int q = 0; q < nq; ++q)
            slha_score_kernel<<<(n_tiles + 255) / 256, 256, 0, s>>>(d_q_coarse + (size_t)q * 128, d_q_sign + (size_t)q * 4,
                                                                   d_tiles, d_scores + (size_t)q * n_tiles, n_tiles);
    }
    cudaEventRecord(b, s);
    cudaError_t e = cudaEventSynchronize(b);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    *ms_out = ms / (float)reps;
    return fail(e);
}
