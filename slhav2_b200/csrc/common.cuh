// Shared declarations of libslha_b200: tile layout constants, error channel,
// per-thread execution context (device, stream, scratch arena) and the launch
// counter.  Host-side C++17 + CUDA runtime; no PyTorch types anywhere.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/slha_b200.h"

namespace slha {

constexpr int D_C = 128;
constexpr int D_S = 256;
constexpr int TILE_BYTES = 128;
constexpr uint16_t F_WARM = 1, F_NF4 = 2, F_MIXED = 4, F_TQ3 = 8, F_NOCORR = 16, F_MIX3 = 32;
constexpr uint8_t ST_HOT = 0, ST_WARM = 1, ST_COLD = 2;

// ---- error channel (thread-local message + status), capi.cu -------------
struct Status {
    int32_t code;
    std::string msg;
    Status() : code(SLHA_OK) {}
    Status(int32_t c, std::string m) : code(c), msg(std::move(m)) {}
    bool ok() const { return code == SLHA_OK; }
};
Status cuda_status(cudaError_t e, const char* what);

#define SLHA_CUDA(expr)                                              \
    do {                                                             \
        cudaError_t _e = (expr);                                     \
        if (_e != cudaSuccess) return ::slha::cuda_status(_e, #expr); \
    } while (0)
#define SLHA_TRY(expr)               \
    do {                             \
        ::slha::Status _s = (expr);  \
        if (!_s.ok()) return _s;     \
    } while (0)

// ---- execution context ----------------------------------------------------
// One per (thread, device).  `stream` is the caller's stream when one was set
// with slha_b200_set_stream, else a library-owned non-blocking stream.
struct Ctx {
    int device = 0;
    cudaStream_t stream = nullptr;      // stream used by the current call
    cudaStream_t lib_stream = nullptr;  // the library's own non-blocking stream
    bool own_stream = false;            // stream == lib_stream
};
Status get_ctx(Ctx** out);  // fails with SLHA_ERR_DEVICE when there is no GPU
Status ctx_device_scratch(Ctx* c, size_t bytes, void** out);
Status ctx_host_scratch(Ctx* c, size_t bytes, void** out);
void count_launch(int n = 1);
uint64_t launch_count();
void tls_set_device(int dev);
void tls_set_stream(void* s);

// A bump allocator over the context scratch: all temporaries of one call.
struct Scratch {
    Ctx* c;
    char* base = nullptr;
    size_t cap = 0, off = 0;
    Status reserve(size_t bytes) {
        SLHA_TRY(ctx_device_scratch(c, bytes, (void**)&base));
        cap = bytes;
        off = 0;
        return Status();
    }
    template <typename T>
    T* take(size_t n) {
        off = (off + 255) & ~size_t(255);
        T* p = reinterpret_cast<T*>(base + off);
        off += n * sizeof(T);
        return p;
    }
};
inline size_t pad256(size_t b) { return (b + 255) & ~size_t(255); }

// Is `p` device-accessible memory?  (Unregistered host memory reports false.)
bool is_device_ptr(const void* p);

// ---- model ---------------------------------------------------------------
struct Model {
    size_t d = 0, d_pad = 0;
    bool rht = false;
    int device = 0;
    float* d_p = nullptr;      // 128 x d   projection rows
    float* d_pt = nullptr;     // d x 128   transposed copy (coalesced column access)
    float* d_scale = nullptr;  // 128
    float* d_z = nullptr;      // 256 x d_pad
    float* d_zt = nullptr;     // d_pad x 256 transposed copy
    float* d_diag = nullptr;   // d_pad (+-1) or null
};

// ---- kernels' host launchers (score.cu / encode.cu / pool.cu) -------------
struct ScorePlan;  // cached work decomposition of one slha_b200_score_topk call shape

Status launch_score_segments(Ctx* c, const SciRustSlhaTile* tiles, const SlhaB200Segment* segs, size_t n_segs, const float* d_q_coarse,
                             const uint64_t* d_q_sign, size_t nq, float* d_scores, const unsigned long long* d_row_offsets,
                             uint32_t row_len, float fill);
Status launch_score_full(Ctx* c, const SciRustSlhaTile* tiles, const uint8_t* state, size_t n,
                         const float* q_coarse, const uint64_t* q_sign, size_t nq, float* scores, int codec_hint = -1);
// d_status must hold ~0ull on entry; receives min over bad tiles of (index << 8 | code) with
// code 5 = non-finite metadata, 6 = invalid tile
Status launch_validate_tiles(Ctx* c, const SciRustSlhaTile* tiles, size_t n, unsigned long long* d_status);
Status score_topk_device(Ctx* c, const SciRustSlhaTile* tiles, const uint8_t* state,
                         const SlhaB200Segment* h_segments, size_t n_segments,
                         const float* d_q_coarse, const uint64_t* d_q_sign, size_t n_queries,
                         uint32_t k, uint32_t* d_out_index, float* d_out_score,
                         uint32_t* d_out_count, bool prefer_generic = false,
                         int codec_hint = -1);  // codec_hint: -1 look at the tiles, 0 no NF4 tiles, 1 NF4 tiles
Status score_topk_noalloc(Ctx* c, const SciRustSlhaTile* tiles, const SlhaB200Segment* h_segments, size_t n_segments,
                          const float* d_q_coarse, const uint64_t* d_q_sign, size_t n_queries, uint32_t k,
                          uint32_t* d_out_index, float* d_out_score, uint32_t* d_out_count);
void debug_force_generic_score(bool on);  // calling thread only
bool debug_general_paths();                // the calling thread's switch (also: host-driven enforce_budget phases)
Status last_score_stats(Ctx* c, uint64_t* out4);
bool timing_active();  // the calling thread records kernel events (slha_b200_timing_begin)
Status timing_begin(uint32_t max_calls);
Status timing_end(Ctx* c, float* score_ms, float* merge_ms, uint32_t capacity, uint32_t* n_out);
Status launch_topk_merge_pairs(Ctx* c, const uint32_t* cand_index, const float* cand_score,
                               uint32_t n_lists, uint64_t list_stride, uint32_t n_queries, uint32_t k_in,
                               uint32_t k_out, uint32_t* out_index, float* out_score, bool lists_sorted = false);

Status launch_topk_merge_peers(Ctx* c, const uint32_t* const* d_bases, uint32_t n_lists, uint32_t n_queries, uint32_t k, const uint32_t* d_ready,
                               uint32_t* d_step, uint32_t* d_done, uint32_t* d_status, uint32_t* out_index, float* out_score);

// ---- token-range sharding over NCCL (shard.cu) ----------------------------------
struct Shard;
Status shard_unique_id(void* id128);
Status shard_init(Ctx* c, const void* id128, int rank, int world, Shard** out);
Status shard_destroy(Shard* s);
void shard_info(const Shard* s, int* rank, int* world);
Status shard_set_timing(Shard* s, bool on);
Status shard_last_times(Ctx* c, Shard* s, float* ms3);
Status shard_status(Ctx* c, Shard* s, uint64_t* out3);
Status shard_set_exchange(Shard* s, int mode);
Status shard_step_device(Ctx* c, Shard* s, const SciRustSlhaTile* tiles, const SlhaB200Segment* h_segs, size_t n_segs,
                         const float* d_qc, const uint64_t* d_qs, size_t nq, uint32_t k, uint32_t* d_out_index,
                         float* d_out_score);

// decode tail over the selected tiles (attend.cu)
Status launch_attend_topk(Ctx* c, const uint32_t* d_index, const float* d_score, const uint32_t* d_count, size_t nq, uint32_t k,
                          float scale, const void* d_values, int value_dtype, size_t d_v, size_t row_stride,
                          const uint64_t* d_row_base, float* d_out, float* d_weights);

Status launch_encode(Ctx* c, const Model* m, const void* d_keys, int key_dtype, size_t n,
                     const uint32_t* d_positions, uint32_t position_base, const uint16_t* d_heads,
                     int codec, SciRustSlhaTile* d_tiles, const uint32_t* d_slots);
Status launch_prepare_queries(Ctx* c, const Model* m, const float* d_q, size_t nq,
                              float* d_q_coarse, uint64_t* d_q_sign);
Status launch_decode(Ctx* c, const Model* m, const SciRustSlhaTile* d_tile, float* d_out,
                     bool with_residual);

}  // namespace slha
