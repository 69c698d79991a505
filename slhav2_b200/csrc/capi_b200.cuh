// Part 2 of the C ABI: batched and device-resident entry points.
// Included at the end of capi.cu.
#pragma once

namespace {

Status check_codec(int32_t codec) {
    if (codec < 0 || codec > SLHA_B200_CODEC_INT4_GROUPED32)
        return Status(SLHA_ERR_CODEC, "unknown codec id " + std::to_string(codec) + "; expected an integer from 0 to 6");
    return Status();
}
size_t key_elem_bytes(int32_t dt) { return dt == SLHA_B200_BF16 ? 2 : 4; }

Status pool_check(SlhaB200Pool* pool, Ctx* c, Pool** out) {
    if (!pool) return Status(SLHA_ERR_NULL, "pool handle is NULL");
    Pool* pl = reinterpret_cast<Pool*>(pool);
    if (pl->device != c->device) return Status(SLHA_ERR_DEVICE, "pool lives on another device than the calling thread's");
    *out = pl;
    return Status();
}

}  // namespace

extern "C" {

int32_t slha_b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
int32_t slha_b200_set_device(int32_t device) {
    return ffi([&]() -> Status {
        if (device < 0 || device >= slha_b200_device_count() || device >= 16)
            return Status(SLHA_ERR_DEVICE, "invalid device index " + std::to_string(device));
        tls_set_device(device);
        return Status();
    });
}
int32_t slha_b200_set_stream(void* cuda_stream) {
    g_last_error[0] = 0;
    tls_set_stream(cuda_stream);
    return SLHA_OK;
}
uint64_t slha_b200_launch_count(void) { return launch_count(); }
int32_t slha_b200_debug_force_generic_score(int32_t on) {
    g_last_error[0] = 0;
    debug_force_generic_score(on != 0);
    return SLHA_OK;
}
int32_t slha_b200_last_score_stats(uint64_t* out) {
    return ffi([&]() -> Status {
        if (!out) return Status(SLHA_ERR_NULL, "slha_b200_last_score_stats received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return last_score_stats(c, out);
    });
}
int32_t slha_b200_timing_begin(uint32_t max_calls) {
    return ffi([&]() -> Status {
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return timing_begin(max_calls);
    });
}
int32_t slha_b200_timing_end(float* score_ms, float* merge_ms, uint32_t capacity, uint32_t* n_out) {
    return ffi([&]() -> Status {
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return timing_end(c, score_ms, merge_ms, capacity, n_out);
    });
}

int32_t slha_b200_malloc(size_t bytes, void** out) {
    return ffi([&]() -> Status {
        if (!out) return Status(SLHA_ERR_NULL, "slha_b200_malloc received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaMalloc(out, std::max<size_t>(bytes, 1)));
        return Status();
    });
}
int32_t slha_b200_free(void* ptr) {
    return ffi([&]() -> Status {
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaFree(ptr));
        return Status();
    });
}
int32_t slha_b200_memcpy(void* dst, const void* src, size_t bytes) {
    return ffi([&]() -> Status {
        if (bytes && (!dst || !src)) return Status(SLHA_ERR_NULL, "slha_b200_memcpy received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}
int32_t slha_b200_synchronize(void) {
    return ffi([&]() -> Status {
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}

SlhaModel* slha_b200_model_create(const float* projection, size_t d, uint64_t seed, int32_t rht,
                                  const float* scale, const float* z) {
    SlhaModel* handle = nullptr;
    ffi([&]() -> Status {
        if (!projection) return Status(SLHA_ERR_NULL, "projection is NULL");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        std::shared_ptr<Model> m;
        SLHA_TRY(model_build(cs.c, projection, d, seed, rht != 0, scale, z, &m));
        handle = model_register(std::move(m));
        return Status();
    });
    return handle;
}

int32_t slha_b200_encode_keys(const SlhaModel* model, const void* keys, int32_t key_dtype, size_t n,
                              const uint32_t* positions, uint32_t position_base, const uint16_t* head_ids,
                              int32_t codec, SciRustSlhaTile* tiles_out) {
    return ffi([&]() -> Status {
        if (n == 0) return Status();
        if (!keys || !tiles_out) return Status(SLHA_ERR_NULL, "slha_b200_encode_keys received a NULL data pointer");
        if (key_dtype != SLHA_B200_F32 && key_dtype != SLHA_B200_BF16)
            return Status(SLHA_ERR_DIMENSION, "key_dtype must be SLHA_B200_F32 or SLHA_B200_BF16");
        SLHA_TRY(check_codec(codec));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        std::shared_ptr<Model> m;
        SLHA_TRY(model_on_device(model, c, &m));
        const void* dk;
        const uint32_t* dpos;
        const uint16_t* dhead;
        SLHA_TRY(stage_in(c, keys, n * m->d * key_elem_bytes(key_dtype), &dk));
        SLHA_TRY(stage_in_t(c, positions, n, &dpos));
        SLHA_TRY(stage_in_t(c, head_ids, n, &dhead));
        std::vector<StagedOut> outs(1);
        SLHA_TRY(stage_out(c, tiles_out, n * sizeof(SciRustSlhaTile), &outs[0]));
        SLHA_TRY(launch_encode(c, m.get(), dk, key_dtype, n, dpos, position_base, dhead, codec,
                               (SciRustSlhaTile*)outs[0].dev, nullptr));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_prepare_queries(const SlhaModel* model, const float* q, size_t nq, float* q_coarse_out,
                                  uint64_t* q_sign_out) {
    return ffi([&]() -> Status {
        if (nq == 0) return Status();
        if (!q || !q_coarse_out || !q_sign_out)
            return Status(SLHA_ERR_NULL, "slha_b200_prepare_queries received a NULL data pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        std::shared_ptr<Model> m;
        SLHA_TRY(model_on_device(model, c, &m));
        const float* dq;
        SLHA_TRY(stage_in_t(c, q, nq * m->d, &dq));
        std::vector<StagedOut> outs(2);
        SLHA_TRY(stage_out(c, q_coarse_out, nq * D_C * 4, &outs[0]));
        SLHA_TRY(stage_out(c, q_sign_out, nq * 32, &outs[1]));
        SLHA_TRY(launch_prepare_queries(c, m.get(), dq, nq, (float*)outs[0].dev, (uint64_t*)outs[1].dev));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_score_tiles(const SciRustSlhaTile* tiles, size_t n, const float* q_coarse,
                              const uint64_t* q_sign, size_t nq, float* scores_out) {
    return ffi([&]() -> Status {
        if (n == 0 || nq == 0) return Status();
        if (!tiles || !q_coarse || !q_sign || !scores_out)
            return Status(SLHA_ERR_NULL, "slha_b200_score_tiles received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const SciRustSlhaTile* dt;
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in(c, tiles, n * sizeof(SciRustSlhaTile), (const void**)&dt));
        SLHA_TRY(stage_in_t(c, q_coarse, nq * D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, nq * 4, &ds));
        std::vector<StagedOut> outs(1);
        SLHA_TRY(stage_out(c, scores_out, n * nq * 4, &outs[0]));
        SLHA_TRY(launch_score_full(c, dt, nullptr, n, dq, ds, nq, (float*)outs[0].dev));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_score_segments(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments, size_t n_segments,
                                 const float* q_coarse, const uint64_t* q_sign, size_t n_queries, float* scores_out,
                                 size_t scores_len, const uint64_t* row_offsets, uint32_t row_len, float fill) {
    return ffi([&]() -> Status {
        if (n_queries == 0 || n_segments == 0) return Status();
        if (!tiles || !segments || !q_coarse || !q_sign || !scores_out || !row_offsets)
            return Status(SLHA_ERR_NULL, "slha_b200_score_segments received a NULL pointer");
        if (!is_device_ptr(tiles)) return Status(SLHA_ERR_DEVICE, "slha_b200_score_segments: tiles must be device memory");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        std::vector<SlhaB200Segment> hseg(n_segments);
        std::vector<uint64_t> hoff(n_queries);
        if (is_device_ptr(segments)) { SLHA_CUDA(cudaMemcpyAsync(hseg.data(), segments, n_segments * sizeof(SlhaB200Segment), cudaMemcpyDeviceToHost, c->stream)); SLHA_CUDA(cudaStreamSynchronize(c->stream)); }  // (after the caller's work on this stream)
        else std::memcpy(hseg.data(), segments, n_segments * sizeof(SlhaB200Segment));
        if (is_device_ptr(row_offsets)) { SLHA_CUDA(cudaMemcpyAsync(hoff.data(), row_offsets, n_queries * 8, cudaMemcpyDeviceToHost, c->stream)); SLHA_CUDA(cudaStreamSynchronize(c->stream)); }  // (after the caller's work on this stream)
        else std::memcpy(hoff.data(), row_offsets, n_queries * 8);
        for (size_t q = 0; q < n_queries; ++q)
            if (hoff[q] > scores_len || (uint64_t)row_len > scores_len - hoff[q])
                return Status(SLHA_ERR_DIMENSION, "slha_b200_score_segments: a row reaches beyond scores_len");
        const float* dq;
        const uint64_t* ds;
        const uint64_t* doff;
        SLHA_TRY(stage_in_t(c, q_coarse, n_queries * D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, n_queries * 4, &ds));
        SLHA_TRY(stage_in_t(c, row_offsets, n_queries, &doff));
        std::vector<StagedOut> outs(1);
        SLHA_TRY(stage_out(c, scores_out, scores_len * 4, &outs[0]));
        // a host destination comes back whole: what no row covers is zero
        if (outs[0].is_host) SLHA_CUDA(cudaMemsetAsync(outs[0].dev, 0, scores_len * 4, c->stream));
        SLHA_TRY(launch_score_segments(c, tiles, hseg.data(), n_segments, dq, ds, n_queries, (float*)outs[0].dev,
                                       reinterpret_cast<const unsigned long long*>(doff), row_len, fill));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_score_topk(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments, size_t n_segments,
                             const float* q_coarse, const uint64_t* q_sign, size_t n_queries, uint32_t k,
                             uint32_t* out_index, float* out_score, uint32_t* out_count) {
    return ffi([&]() -> Status {
        if (n_queries == 0) return Status();
        if (!tiles || !segments || !q_coarse || !q_sign || !out_index || !out_score)
            return Status(SLHA_ERR_NULL, "slha_b200_score_topk received a NULL pointer");
        if (!is_device_ptr(tiles)) return Status(SLHA_ERR_DEVICE, "slha_b200_score_topk: tiles must be device memory");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        std::vector<SlhaB200Segment> hseg(n_segments);
        if (is_device_ptr(segments))
            { SLHA_CUDA(cudaMemcpyAsync(hseg.data(), segments, n_segments * sizeof(SlhaB200Segment), cudaMemcpyDeviceToHost, c->stream)); SLHA_CUDA(cudaStreamSynchronize(c->stream)); }  // (after the caller's work on this stream)
        else
            std::memcpy(hseg.data(), segments, n_segments * sizeof(SlhaB200Segment));
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in_t(c, q_coarse, n_queries * D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, n_queries * 4, &ds));
        std::vector<StagedOut> outs(3);
        SLHA_TRY(stage_out(c, out_index, n_queries * k * 4, &outs[0], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_score, n_queries * k * 4, &outs[1], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_count, n_queries * 4, &outs[2], /*in_place_if_pinned=*/true));
        SLHA_TRY(score_topk_device(c, tiles, nullptr, hseg.data(), n_segments, dq, ds, n_queries, k,
                                   (uint32_t*)outs[0].dev, (float*)outs[1].dev, (uint32_t*)outs[2].dev));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_score_topk_noalloc(const SciRustSlhaTile* tiles, const SlhaB200Segment* segments, size_t n_segments,
                                     const float* q_coarse, const uint64_t* q_sign, size_t n_queries, uint32_t k,
                                     uint32_t* out_index, float* out_score, uint32_t* out_count) {
    // Deliberately no CallScope / staging here: those may grow (allocate) the
    // per-thread scratch arena.  Every data pointer except `segments` must
    // already be device memory; the only working memory is the library's fixed
    // device array (see score.cu).
    return ffi([&]() -> Status {
        if (n_queries == 0) return Status();
        if (!tiles || !segments || !q_coarse || !q_sign || !out_index || !out_score)
            return Status(SLHA_ERR_NULL, "slha_b200_score_topk_noalloc received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        if (!is_device_ptr(tiles) || !is_device_ptr(q_coarse) || !is_device_ptr(q_sign) || !is_device_ptr(out_index) ||
            !is_device_ptr(out_score) || (out_count && !is_device_ptr(out_count)))
            return Status(SLHA_ERR_DEVICE, "slha_b200_score_topk_noalloc: tiles, queries and outputs must be device memory");
        if (is_device_ptr(segments))
            return Status(SLHA_ERR_DEVICE, "slha_b200_score_topk_noalloc: segments must be host memory");
        SLHA_TRY(score_topk_noalloc(c, tiles, segments, n_segments, q_coarse, q_sign, n_queries, k, out_index, out_score,
                                    out_count));
        if (sync_by_default(c)) SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}

static int32_t topk_merge_any(const uint32_t* cand_index, const float* cand_score, uint32_t n_lists, uint64_t list_stride,
                              uint32_t n_queries, uint32_t k_in, uint32_t k_out, uint32_t* out_index, float* out_score,
                              bool lists_sorted) {
    return ffi([&]() -> Status {
        if (!cand_index || !cand_score || !out_index || !out_score)
            return Status(SLHA_ERR_NULL, "slha_b200_topk_merge received a NULL pointer");
        if (list_stride < (uint64_t)n_queries * k_in)
            return Status(SLHA_ERR_DIMENSION, "list_stride is smaller than n_queries * k_in");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const size_t nc = n_lists ? (size_t)(n_lists - 1) * list_stride + (size_t)n_queries * k_in : 0;
        const uint32_t* di;
        const float* dsc;
        SLHA_TRY(stage_in_t(c, cand_index, nc, &di));
        SLHA_TRY(stage_in_t(c, cand_score, nc, &dsc));
        std::vector<StagedOut> outs(2);
        SLHA_TRY(stage_out(c, out_index, (size_t)n_queries * k_out * 4, &outs[0], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_score, (size_t)n_queries * k_out * 4, &outs[1], /*in_place_if_pinned=*/true));
        SLHA_TRY(launch_topk_merge_pairs(c, di, dsc, n_lists, list_stride, n_queries, k_in, k_out,
                                         (uint32_t*)outs[0].dev, (float*)outs[1].dev, lists_sorted));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}
int32_t slha_b200_topk_merge_strided(const uint32_t* cand_index, const float* cand_score, uint32_t n_lists,
                                     uint64_t list_stride, uint32_t n_queries, uint32_t k_in, uint32_t k_out,
                                     uint32_t* out_index, float* out_score) {
    return topk_merge_any(cand_index, cand_score, n_lists, list_stride, n_queries, k_in, k_out, out_index, out_score, false);
}
int32_t slha_b200_topk_merge_sorted_strided(const uint32_t* cand_index, const float* cand_score, uint32_t n_lists,
                                            uint64_t list_stride, uint32_t n_queries, uint32_t k_in, uint32_t k_out,
                                            uint32_t* out_index, float* out_score) {
    return topk_merge_any(cand_index, cand_score, n_lists, list_stride, n_queries, k_in, k_out, out_index, out_score, true);
}
int32_t slha_b200_topk_merge(const uint32_t* cand_index, const float* cand_score, uint32_t n_lists,
                             uint32_t n_queries, uint32_t k_in, uint32_t k_out, uint32_t* out_index,
                             float* out_score) {
    return slha_b200_topk_merge_strided(cand_index, cand_score, n_lists, (uint64_t)n_queries * k_in, n_queries, k_in,
                                        k_out, out_index, out_score);
}

int32_t slha_b200_attend_topk(const uint32_t* top_index, const float* top_score, const uint32_t* top_count, size_t n_queries,
                              uint32_t k, float scale, const void* values, int32_t value_dtype, size_t d_v,
                              size_t value_row_stride, const uint64_t* value_row_base, float* out, float* weights_out) {
    return ffi([&]() -> Status {
        if (n_queries == 0) return Status();
        if (!top_index || !top_score || !values || !out)
            return Status(SLHA_ERR_NULL, "slha_b200_attend_topk received a NULL pointer");
        if (value_dtype != SLHA_B200_F32 && value_dtype != SLHA_B200_BF16)
            return Status(SLHA_ERR_DIMENSION, "slha_b200_attend_topk: value_dtype must be SLHA_B200_F32 or SLHA_B200_BF16");
        if (!is_device_ptr(values)) return Status(SLHA_ERR_DEVICE, "slha_b200_attend_topk: values must be device memory");
        if (value_row_stride < d_v) return Status(SLHA_ERR_DIMENSION, "slha_b200_attend_topk: value_row_stride is smaller than d_v");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const uint32_t *di, *dc;
        const float* dsc;
        const uint64_t* db;
        SLHA_TRY(stage_in_t(c, top_index, n_queries * k, &di));
        SLHA_TRY(stage_in_t(c, top_score, n_queries * k, &dsc));
        SLHA_TRY(stage_in_t(c, top_count, n_queries, &dc));
        SLHA_TRY(stage_in_t(c, value_row_base, n_queries, &db));
        std::vector<StagedOut> outs(2);
        SLHA_TRY(stage_out(c, out, n_queries * d_v * 4, &outs[0]));
        SLHA_TRY(stage_out(c, weights_out, n_queries * (size_t)k * 4, &outs[1]));
        SLHA_TRY(launch_attend_topk(c, di, dsc, dc, n_queries, k, scale, values, value_dtype, d_v, value_row_stride, db,
                                    (float*)outs[0].dev, (float*)outs[1].dev));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

// ------------------------------------------------------------------ shards
int32_t slha_b200_shard_unique_id(void* id_out) {
    return ffi([&]() -> Status {
        if (!id_out) return Status(SLHA_ERR_NULL, "slha_b200_shard_unique_id received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return shard_unique_id(id_out);
    });
}
int32_t slha_b200_shard_init(const void* nccl_unique_id, int32_t rank, int32_t world, SlhaB200Shard** out) {
    return ffi([&]() -> Status {
        if (!out) return Status(SLHA_ERR_NULL, "slha_b200_shard_init received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        Shard* s;
        SLHA_TRY(shard_init(c, nccl_unique_id, rank, world, &s));
        *out = reinterpret_cast<SlhaB200Shard*>(s);
        return Status();
    });
}
int32_t slha_b200_shard_destroy(SlhaB200Shard* shard) {
    return ffi([&]() -> Status {
        if (!shard) return Status();
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return shard_destroy(reinterpret_cast<Shard*>(shard));
    });
}
int32_t slha_b200_shard_score_topk(SlhaB200Shard* shard, const SciRustSlhaTile* tiles, const SlhaB200Segment* segments,
                                   size_t n_segments, const float* q_coarse, const uint64_t* q_sign, size_t n_queries,
                                   uint32_t k, uint32_t* out_index, float* out_score) {
    return ffi([&]() -> Status {
        if (!shard) return Status(SLHA_ERR_NULL, "shard handle is NULL");
        if (n_queries == 0) return Status();
        if (!tiles || !segments || !q_coarse || !q_sign || !out_index || !out_score)
            return Status(SLHA_ERR_NULL, "slha_b200_shard_score_topk received a NULL pointer");
        if (!is_device_ptr(tiles)) return Status(SLHA_ERR_DEVICE, "slha_b200_shard_score_topk: tiles must be device memory");
        if (is_device_ptr(segments)) return Status(SLHA_ERR_DEVICE, "slha_b200_shard_score_topk: segments must be host memory");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in_t(c, q_coarse, n_queries * D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, n_queries * 4, &ds));
        std::vector<StagedOut> outs(2);
        SLHA_TRY(stage_out(c, out_index, n_queries * k * 4, &outs[0], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_score, n_queries * k * 4, &outs[1], /*in_place_if_pinned=*/true));
        SLHA_TRY(shard_step_device(c, reinterpret_cast<Shard*>(shard), tiles, segments, n_segments, dq, ds, n_queries, k,
                                   (uint32_t*)outs[0].dev, (float*)outs[1].dev));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}
int32_t slha_b200_shard_set_timing(SlhaB200Shard* shard, int32_t on) {
    return ffi([&]() -> Status {
        if (!shard) return Status(SLHA_ERR_NULL, "shard handle is NULL");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return shard_set_timing(reinterpret_cast<Shard*>(shard), on != 0);
    });
}
int32_t slha_b200_shard_set_exchange(SlhaB200Shard* shard, int32_t mode) {
    return ffi([&]() -> Status {
        if (!shard) return Status(SLHA_ERR_NULL, "slha_b200_shard_set_exchange received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return shard_set_exchange(reinterpret_cast<Shard*>(shard), mode);
    });
}
int32_t slha_b200_shard_status(SlhaB200Shard* shard, uint64_t* out) {
    return ffi([&]() -> Status {
        if (!shard || !out) return Status(SLHA_ERR_NULL, "slha_b200_shard_status received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return shard_status(c, reinterpret_cast<Shard*>(shard), out);
    });
}
int32_t slha_b200_shard_last_times(SlhaB200Shard* shard, float* ms_out) {
    return ffi([&]() -> Status {
        if (!shard || !ms_out) return Status(SLHA_ERR_NULL, "slha_b200_shard_last_times received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        return shard_last_times(c, reinterpret_cast<Shard*>(shard), ms_out);
    });
}

// ------------------------------------------------------------------ pool
int32_t slha_b200_pool_create(const SlhaB200PoolConfig* config, SlhaB200Pool** out) {
    return ffi([&]() -> Status {
        if (!config || !out) return Status(SLHA_ERR_NULL, "slha_b200_pool_create received a NULL pointer");
        if (config->capacity_tiles == 0 || config->capacity_tiles > 0xFFFFFFF0ull)
            return Status(SLHA_ERR_DIMENSION, "capacity_tiles must be in 1..2^32-16");
        if (config->page_policy < 0 || config->page_policy > 1 || config->evict_policy < 0 || config->evict_policy > 1)
            return Status(SLHA_ERR_DIMENSION, "unknown paging or eviction policy");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_create(cs.c, *config, &pl));
        *out = reinterpret_cast<SlhaB200Pool*>(pl);
        return Status();
    });
}
int32_t slha_b200_pool_destroy(SlhaB200Pool* pool) {
    return ffi([&]() -> Status {
        if (!pool) return Status();
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        pool_destroy(reinterpret_cast<Pool*>(pool));
        return Status();
    });
}

int32_t slha_b200_pool_insert_tiles(SlhaB200Pool* pool, const SciRustSlhaTile* tiles, size_t n, uint32_t* slots_out) {
    return ffi([&]() -> Status {
        if (n == 0) return Status();
        if (!tiles) return Status(SLHA_ERR_NULL, "slha_b200_pool_insert_tiles received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        const unsigned char* dt;
        SLHA_TRY(stage_in(c, tiles, n * sizeof(SciRustSlhaTile), (const void**)&dt));
        std::vector<StagedOut> outs(1);
        uint32_t* dslots;
        if (slots_out) {
            SLHA_TRY(stage_out(c, slots_out, n * 4, &outs[0]));
            dslots = (uint32_t*)outs[0].dev;
        } else {
            SLHA_TRY(ctx_device_scratch(c, n * 4, (void**)&dslots));
        }
        SLHA_TRY(pool_reserve(c, pl, dt, n, dslots));
        SLHA_TRY(pool_scatter(c, pl, dt, dslots, n));
        pl->codec_mask |= 0x80000000u;
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_pool_append_keys(SlhaB200Pool* pool, const SlhaModel* model, const void* keys, int32_t key_dtype,
                                   size_t n, const uint32_t* positions, uint32_t position_base,
                                   const uint16_t* head_ids, int32_t codec, uint32_t* slots_out) {
    return ffi([&]() -> Status {
        if (n == 0) return Status();
        if (!keys) return Status(SLHA_ERR_NULL, "slha_b200_pool_append_keys received a NULL pointer");
        if (key_dtype != SLHA_B200_F32 && key_dtype != SLHA_B200_BF16)
            return Status(SLHA_ERR_DIMENSION, "key_dtype must be SLHA_B200_F32 or SLHA_B200_BF16");
        SLHA_TRY(check_codec(codec));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        std::shared_ptr<Model> m;
        SLHA_TRY(model_on_device(model, c, &m));
        const void* dk;
        const uint32_t* dpos;
        const uint16_t* dhead;
        SLHA_TRY(stage_in(c, keys, n * m->d * key_elem_bytes(key_dtype), &dk));
        SLHA_TRY(stage_in_t(c, positions, n, &dpos));
        SLHA_TRY(stage_in_t(c, head_ids, n, &dhead));
        std::vector<StagedOut> outs(1);
        uint32_t* dslots;
        if (slots_out) {
            SLHA_TRY(stage_out(c, slots_out, n * 4, &outs[0]));
            dslots = (uint32_t*)outs[0].dev;
        } else {
            SLHA_TRY(ctx_device_scratch(c, n * 4, (void**)&dslots));
        }
        // freshly encoded tiles are HOT with their correction plane: 128 live bytes each
        SLHA_TRY(pool_reserve(c, pl, nullptr, n, dslots));
        SLHA_TRY(launch_encode(c, m.get(), dk, key_dtype, n, dpos, position_base, dhead, codec,
                               reinterpret_cast<SciRustSlhaTile*>(pl->dev.tiles), dslots));
        pl->codec_mask |= 1u << codec;
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

// What a pool's record of appended codecs says to the scorers: -1 unknown (look at the first tile), -2 only codecs the
// tensor-core kernels do not decode, else bit 0 = NF4 tiles expected, bit 1 = mixed 8/4 only, bit 2 = TQ3 only.
static int pool_codec_hint(const Pool* pl) {
    const uint32_t cm = pl->codec_mask;
    if ((cm & 0x80000000u) || !cm) return -1;
    const bool mixed_only = cm == (1u << SLHA_CODEC_MIXED), tq3_only = cm == (1u << SLHA_CODEC_TQ3);
    const uint32_t nibble = (1u << SLHA_CODEC_INT4_SINGLE) | (1u << SLHA_CODEC_INT4_GROUPED) | (1u << SLHA_CODEC_NF4) | (1u << 6);
    if (!(cm & nibble) && !mixed_only && !tq3_only) return -2;
    return (int)(((cm >> SLHA_CODEC_NF4) & 1u) | (mixed_only ? 2u : 0u) | (tq3_only ? 4u : 0u));
}

int32_t slha_b200_pool_score_all(SlhaB200Pool* pool, const float* q_coarse, const uint64_t* q_sign,
                                 uint32_t* slots_out, float* scores_out, uint64_t* n_out) {
    return ffi([&]() -> Status {
        if (!q_coarse || !q_sign || !slots_out || !scores_out || !n_out)
            return Status(SLHA_ERR_NULL, "slha_b200_pool_score_all received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        const uint64_t len = pl->h_cnt.len;
        if (len == 0) {
            *n_out = 0;
            return Status();
        }
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in_t(c, q_coarse, D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, 4, &ds));
        float* all;
        unsigned long long* dn;
        SLHA_TRY(ctx_device_scratch(c, len * 4, (void**)&all));
        SLHA_TRY(ctx_device_scratch(c, 8, (void**)&dn));
        std::vector<StagedOut> outs(2);
        SLHA_TRY(stage_out(c, slots_out, len * 4, &outs[0]));
        SLHA_TRY(stage_out(c, scores_out, len * 4, &outs[1]));
        SLHA_TRY(launch_score_full(c, reinterpret_cast<const SciRustSlhaTile*>(pl->dev.tiles), pl->dev.state, len, dq,
                                   ds, 1, all, pool_codec_hint(pl)));
        SLHA_TRY(pool_compact_live(c, pl, all, (uint32_t*)outs[0].dev, (float*)outs[1].dev, dn));
        unsigned long long hn = 0;
        SLHA_CUDA(cudaMemcpyAsync(&hn, dn, 8, cudaMemcpyDeviceToHost, c->stream));
        SLHA_TRY(finish_outputs(c, outs, true));
        *n_out = hn;
        return Status();
    });
}

int32_t slha_b200_pool_score_topk(SlhaB200Pool* pool, const float* q_coarse, const uint64_t* q_sign, size_t nq,
                                  uint32_t k, uint32_t* out_slot, float* out_score, uint32_t* out_count) {
    return ffi([&]() -> Status {
        if (nq == 0) return Status();
        if (!q_coarse || !q_sign || !out_slot || !out_score)
            return Status(SLHA_ERR_NULL, "slha_b200_pool_score_topk received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in_t(c, q_coarse, nq * D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, nq * 4, &ds));
        std::vector<StagedOut> outs(3);
        SLHA_TRY(stage_out(c, out_slot, nq * k * 4, &outs[0], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_score, nq * k * 4, &outs[1], /*in_place_if_pinned=*/true));
        SLHA_TRY(stage_out(c, out_count, nq * 4, &outs[2], /*in_place_if_pinned=*/true));
        SlhaB200Segment seg{0, (uint32_t)pl->h_cnt.len, 0, (uint32_t)nq, 0};
        const uint32_t cm = pl->codec_mask;
        const bool known = !(cm & 0x80000000u);
        const bool mixed_only = known && cm == (1u << SLHA_CODEC_MIXED);
        const bool tq3_only = known && cm == (1u << SLHA_CODEC_TQ3);
        const uint32_t nibble = (1u << SLHA_CODEC_INT4_SINGLE) | (1u << SLHA_CODEC_INT4_GROUPED) | (1u << SLHA_CODEC_NF4) | (1u << 6);
        SLHA_TRY(score_topk_device(c, reinterpret_cast<const SciRustSlhaTile*>(pl->dev.tiles), pl->dev.state, &seg, 1,
                                   dq, ds, nq, k, (uint32_t*)outs[0].dev, (float*)outs[1].dev,
                                   (uint32_t*)outs[2].dev, /*prefer_generic=*/known && cm && !(cm & nibble) && !mixed_only && !tq3_only,
                                   known ? (int)(((cm >> SLHA_CODEC_NF4) & 1u) | (mixed_only ? 2u : 0u) | (tq3_only ? 4u : 0u)) : -1));
        return finish_outputs(c, outs, sync_by_default(c));
    });
}

int32_t slha_b200_pool_observe_scores(SlhaB200Pool* pool, const uint32_t* slots, const float* scores, size_t n,
                                      float temperature) {
    return ffi([&]() -> Status {
        if (n == 0) return Status();
        if (!slots || !scores) return Status(SLHA_ERR_NULL, "slha_b200_pool_observe_scores received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        const uint32_t* dsl;
        const float* dsc;
        SLHA_TRY(stage_in_t(c, slots, n, &dsl));
        SLHA_TRY(stage_in_t(c, scores, n, &dsc));
        SLHA_TRY(pool_observe(c, pl, dsl, dsc, n, temperature));
        if (sync_by_default(c)) SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}

int32_t slha_b200_pool_observe_query(SlhaB200Pool* pool, const float* q_coarse, const uint64_t* q_sign,
                                     float temperature) {
    return ffi([&]() -> Status {
        if (!q_coarse || !q_sign) return Status(SLHA_ERR_NULL, "slha_b200_pool_observe_query received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        const uint64_t len = pl->h_cnt.len;
        if (len == 0) return Status();
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in_t(c, q_coarse, D_C, &dq));
        SLHA_TRY(stage_in_t(c, q_sign, 4, &ds));
        float* all;
        SLHA_TRY(ctx_device_scratch(c, len * 4, (void**)&all));
        SLHA_TRY(launch_score_full(c, reinterpret_cast<const SciRustSlhaTile*>(pl->dev.tiles), pl->dev.state, len, dq,
                                   ds, 1, all, pool_codec_hint(pl)));
        SLHA_TRY(pool_observe(c, pl, nullptr, all, len, temperature));
        if (sync_by_default(c)) SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}

static int32_t pool_single(SlhaB200Pool* pool, int op, uint32_t slot, int32_t* result) {
    return ffi([&]() -> Status {
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_check(pool, cs.c, &pl));
        if (slot >= pl->h_cnt.len) return Status(SLHA_ERR_DIMENSION, "slot index out of range");
        int32_t r = 0;
        SLHA_TRY(pool_single_op(cs.c, pl, op, slot, &r));
        if (result) *result = r;
        return Status();
    });
}
int32_t slha_b200_pool_page_out(SlhaB200Pool* pool, uint32_t slot) { return pool_single(pool, 0, slot, nullptr); }
int32_t slha_b200_pool_drop_correction(SlhaB200Pool* pool, uint32_t slot, int32_t* dropped) {
    return pool_single(pool, 1, slot, dropped);
}
int32_t slha_b200_pool_evict(SlhaB200Pool* pool, uint32_t slot, int32_t* evicted) {
    return pool_single(pool, 2, slot, evicted);
}

int32_t slha_b200_pool_attach_event_log(SlhaB200Pool* pool, const char* path, int32_t mode, int32_t require_durable) {
    return ffi([&]() -> Status {
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        if (pl->log) eventlog_close(pl->log);
        pl->log = nullptr;
        pl->require_durable = require_durable != 0;
        if (!path) return Status();  // detach (with require_durable set: every eviction is refused, ccos.rs:429-432)
        return eventlog_open(path, mode, &pl->log);
    });
}
int32_t slha_b200_pool_rehydrate(SlhaB200Pool* pool, uint64_t seq, int64_t* slot_out) {
    return ffi([&]() -> Status {
        if (!slot_out) return Status(SLHA_ERR_NULL, "slha_b200_pool_rehydrate received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_check(pool, cs.c, &pl));
        return pool_rehydrate(cs.c, pl, seq, slot_out);
    });
}
int32_t slha_b200_pool_event_log_stats(SlhaB200Pool* pool, uint64_t* out) {
    return ffi([&]() -> Status {
        if (!out) return Status(SLHA_ERR_NULL, "slha_b200_pool_event_log_stats received a NULL pointer");
        Ctx* c;
        SLHA_TRY(get_ctx(&c));
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        out[0] = pl->log ? eventlog_records(pl->log) : 0;
        out[1] = pl->log_errors;
        out[2] = pl->blocked_evictions;
        return Status();
    });
}
int32_t slha_b200_pool_enforce_budget(SlhaB200Pool* pool, int32_t* within_budget) {
    return ffi([&]() -> Status {
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_check(pool, cs.c, &pl));
        int32_t w = 0;
        SLHA_TRY(pool_enforce_budget(cs.c, pl, &w));
        if (within_budget) *within_budget = w;
        return Status();
    });
}
int32_t slha_b200_pool_set_budget(SlhaB200Pool* pool, uint64_t budget_bytes) {
    return ffi([&]() -> Status {
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_check(pool, cs.c, &pl));
        pl->cfg.budget_bytes = budget_bytes;
        pl->h_cnt.budget = budget_bytes;
        SLHA_CUDA(cudaMemcpyAsync(&pl->dev.cnt->budget, &pl->h_cnt.budget, 8, cudaMemcpyHostToDevice, cs.c->stream));
        SLHA_CUDA(cudaStreamSynchronize(cs.c->stream));
        return Status();
    });
}
int32_t slha_b200_pool_stats(SlhaB200Pool* pool, uint64_t out[8]) {
    return ffi([&]() -> Status {
        if (!out) return Status(SLHA_ERR_NULL, "slha_b200_pool_stats received a NULL pointer");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Pool* pl;
        SLHA_TRY(pool_check(pool, cs.c, &pl));
        return pool_stats(cs.c, pl, out);
    });
}
int32_t slha_b200_pool_read(SlhaB200Pool* pool, uint64_t first, uint64_t n, SciRustSlhaTile* tiles_out,
                            uint8_t* state_out, float* importance_out, uint64_t* seq_out) {
    return ffi([&]() -> Status {
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        Pool* pl;
        SLHA_TRY(pool_check(pool, c, &pl));
        if (first + n > pl->h_cnt.len) return Status(SLHA_ERR_DIMENSION, "slot range exceeds the pool length");
        if (tiles_out)
            SLHA_CUDA(cudaMemcpyAsync(tiles_out, pl->dev.tiles + first * TILE_BYTES, n * TILE_BYTES, cudaMemcpyDefault, c->stream));
        if (state_out) SLHA_CUDA(cudaMemcpyAsync(state_out, pl->dev.state + first, n, cudaMemcpyDefault, c->stream));
        if (importance_out)
            SLHA_CUDA(cudaMemcpyAsync(importance_out, pl->dev.importance + first, n * 4, cudaMemcpyDefault, c->stream));
        if (seq_out) SLHA_CUDA(cudaMemcpyAsync(seq_out, pl->dev.seq + first, n * 8, cudaMemcpyDefault, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    });
}
const SciRustSlhaTile* slha_b200_pool_tiles_device(SlhaB200Pool* pool) {
    return pool ? reinterpret_cast<const SciRustSlhaTile*>(reinterpret_cast<Pool*>(pool)->dev.tiles) : nullptr;
}

}  // extern "C"
