// extern "C" surface of libslha_b200.so (declared in include/slha_b200.h).
// Part 1 mirrors the reference's slha-c crate entry point for entry point
// (slha-c/src/lib.rs:288-950): same argument checks in the same order, same
// status codes, outputs untouched on failure.  Part 2 is the batched / device
// resident surface.  Every entry point converts C++ exceptions into
// SLHA_ERR_PANIC, as the reference converts Rust panics (lib.rs:91-105).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>

#include "pool.cuh"
#include "runtime.cuh"

using namespace slha;

namespace {

constexpr size_t LAST_ERROR_CAPACITY = 512;  // lib.rs:35
thread_local char g_last_error[LAST_ERROR_CAPACITY] = {0};

void set_last_error(const std::string& m) {
    const size_t n = std::min(m.size(), LAST_ERROR_CAPACITY - 1);
    std::memcpy(g_last_error, m.data(), n);
    g_last_error[n] = 0;
}

int32_t ffi(const std::function<Status()>& f) {
    g_last_error[0] = 0;
    try {
        Status s = f();
        if (!s.ok()) set_last_error(s.msg);
        return s.code;
    } catch (const std::exception& e) {
        set_last_error(std::string("exception caught at the SLHA C ABI boundary: ") + e.what());
        return SLHA_ERR_PANIC;
    } catch (...) {
        set_last_error("exception caught at the SLHA C ABI boundary");
        return SLHA_ERR_PANIC;
    }
}

Status finite_check(const float* v, size_t n, const char* name) {  // lib.rs:233-242
    for (size_t i = 0; i < n; ++i)
        if (!std::isfinite(v[i]))
            return Status(SLHA_ERR_NONFINITE, std::string(name) + "[" + std::to_string(i) + "] is not finite");
    return Status();
}

SlhaContext* context_singleton() {
    static uint64_t ctx_storage[1] = {SLHA_ABI_VERSION};
    return reinterpret_cast<SlhaContext*>(ctx_storage);
}

Status model_on_device(const SlhaModel* h, Ctx* c, std::shared_ptr<Model>* out) {
    Status st;
    auto m = model_lookup(h, &st);
    if (!m) return st;
    if (m->device != c->device) return Status(SLHA_ERR_DEVICE, "model lives on another device than the calling thread's");
    *out = std::move(m);
    return Status();
}

// score one host tile with one host query (slha_process_tile / slha_score_tile)
Status score_one(const SciRustSlhaTile* tile, const float* q_coarse, const uint64_t* q_sign, float* score_out) {
    SciRustSlhaTile t;
    std::memcpy(&t, tile, sizeof t);  // unaligned input accepted
    float qc[D_C];
    uint64_t qs[4];
    std::memcpy(qc, q_coarse, sizeof qc);
    std::memcpy(qs, q_sign, sizeof qs);
    SLHA_TRY(validate_tile_host(t));
    SLHA_TRY(finite_check(qc, D_C, "q_coarse"));
    CallScope cs;
    if (!cs.ok()) return cs.st;
    Ctx* c = cs.c;
    const SciRustSlhaTile* dt;
    const float* dq;
    const uint64_t* ds;
    SLHA_TRY(stage_in_t(c, &t, 1, &dt));
    SLHA_TRY(stage_in_t(c, qc, D_C, &dq));
    SLHA_TRY(stage_in_t(c, qs, 4, &ds));
    float* dsc;
    SLHA_TRY(ctx_device_scratch(c, 4, (void**)&dsc));
    SLHA_TRY(launch_score_full(c, dt, nullptr, 1, dq, ds, 1, dsc));
    float sc;
    SLHA_CUDA(cudaMemcpyAsync(&sc, dsc, 4, cudaMemcpyDeviceToHost, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    if (!std::isfinite(sc)) return Status(SLHA_ERR_NONFINITE, "tile scoring produced a non-finite result");
    std::memcpy(score_out, &sc, 4);
    return Status();
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ part 1
uint32_t slha_abi_version(void) { return SLHA_ABI_VERSION; }
size_t slha_tile_size(void) { return sizeof(SciRustSlhaTile); }
size_t slha_tile_align(void) { return alignof(SciRustSlhaTile); }
const char* slha_last_error_message(void) { return g_last_error; }
void slha_clear_error(void) { g_last_error[0] = 0; }

SlhaContext* slha_init(void) {
    g_last_error[0] = 0;
    return context_singleton();
}

int32_t slha_shutdown(SlhaContext* context) {
    g_last_error[0] = 0;
    if (context == nullptr) return SLHA_OK;
    if (context != context_singleton()) {
        set_last_error("context handle was not returned by slha_init");
        return SLHA_ERR_INVALID_HANDLE;
    }
    return SLHA_OK;
}

int32_t slha_process_tile(const SciRustSlhaTile* tile, const float* q_coarse, const uint64_t* q_sign,
                          float* score_out) {
    return ffi([&]() -> Status {
        if (!tile || !q_coarse || !q_sign || !score_out)
            return Status(SLHA_ERR_NULL, "slha_process_tile received a NULL pointer");
        return score_one(tile, q_coarse, q_sign, score_out);
    });
}

int32_t slha_score_tile(const SlhaModel* model, const SciRustSlhaTile* tile, const float* q_coarse,
                        const uint64_t* q_sign, float* score_out) {
    return ffi([&]() -> Status {
        if (!tile || !q_coarse || !q_sign || !score_out)
            return Status(SLHA_ERR_NULL, "slha_score_tile received a NULL pointer");
        Status st;
        if (!model_lookup(model, &st)) return st;
        return score_one(tile, q_coarse, q_sign, score_out);
    });
}

int32_t slha_prepare_query(const SlhaModel* model, const float* q, size_t d, float* q_coarse, uint64_t* q_sign) {
    return ffi([&]() -> Status {
        if (!q || !q_coarse || !q_sign) return Status(SLHA_ERR_NULL, "slha_prepare_query received a NULL data pointer");
        Status st;
        auto m = model_lookup(model, &st);
        if (!m) return st;
        if (d != m->d)
            return Status(SLHA_ERR_DIMENSION, "query dimension mismatch: received " + std::to_string(d) +
                                                  ", expected " + std::to_string(m->d));
        std::vector<float> qh(d);
        std::memcpy(qh.data(), q, d * 4);
        SLHA_TRY(finite_check(qh.data(), d, "q"));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const float* dq;
        SLHA_TRY(stage_in_t(c, qh.data(), d, &dq));
        float* dqc;
        uint64_t* dqs;
        SLHA_TRY(ctx_device_scratch(c, D_C * 4, (void**)&dqc));
        SLHA_TRY(ctx_device_scratch(c, 32, (void**)&dqs));
        SLHA_TRY(launch_prepare_queries(c, m.get(), dq, 1, dqc, dqs));
        float qc[D_C];
        uint64_t qs[4];
        SLHA_CUDA(cudaMemcpyAsync(qc, dqc, sizeof qc, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaMemcpyAsync(qs, dqs, sizeof qs, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        SLHA_TRY(finite_check(qc, D_C, "q_coarse"));
        std::memcpy(q_coarse, qc, sizeof qc);
        std::memcpy(q_sign, qs, sizeof qs);
        return Status();
    });
}

int32_t slha_score_tiles(const SlhaModel* model, const SciRustSlhaTile* tiles, size_t n_tiles,
                         const float* q_coarse, const uint64_t* q_sign, float* scores_out) {
    return ffi([&]() -> Status {
        if (!tiles || !q_coarse || !q_sign || !scores_out)
            return Status(SLHA_ERR_NULL, "slha_score_tiles received a NULL pointer");
        Status st;
        if (!model_lookup(model, &st)) return st;
        if (n_tiles > ((size_t)1 << 20))  // lib.rs:208, :545-550
            return Status(SLHA_ERR_DIMENSION, "n_tiles=" + std::to_string(n_tiles) + " exceeds the safety bound 1048576");
        if (n_tiles == 0) return Status();
        float qc[D_C];
        uint64_t qs[4];
        std::memcpy(qc, q_coarse, sizeof qc);
        std::memcpy(qs, q_sign, sizeof qs);
        SLHA_TRY(finite_check(qc, D_C, "q_coarse"));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const SciRustSlhaTile* dt;
        const float* dq;
        const uint64_t* ds;
        SLHA_TRY(stage_in(c, tiles, n_tiles * sizeof(SciRustSlhaTile), (const void**)&dt));
        SLHA_TRY(stage_in_t(c, qc, D_C, &dq));
        SLHA_TRY(stage_in_t(c, qs, 4, &ds));
        float* dsc;
        unsigned long long* dstat;
        SLHA_TRY(ctx_device_scratch(c, n_tiles * 4, (void**)&dsc));
        SLHA_TRY(ctx_device_scratch(c, 8, (void**)&dstat));
        SLHA_CUDA(cudaMemsetAsync(dstat, 0xFF, 8, c->stream));
        SLHA_TRY(launch_validate_tiles(c, dt, n_tiles, dstat));
        SLHA_TRY(launch_score_full(c, dt, nullptr, n_tiles, dq, ds, 1, dsc));
        std::vector<float> sc(n_tiles);
        unsigned long long stat;
        SLHA_CUDA(cudaMemcpyAsync(&stat, dstat, 8, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaMemcpyAsync(sc.data(), dsc, n_tiles * 4, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        // the reference validates and scores tile by tile and stops at the first
        // failure of either kind (lib.rs:563-581): report whichever comes first
        size_t first_bad = stat == ~0ull ? n_tiles : (size_t)(stat >> 8);
        for (size_t i = 0; i < first_bad; ++i)
            if (!std::isfinite(sc[i]))
                return Status(SLHA_ERR_NONFINITE, "tile " + std::to_string(i) + " scoring produced a non-finite result");
        if (first_bad < n_tiles) {
            SciRustSlhaTile t;
            SLHA_CUDA(cudaMemcpy(&t, dt + first_bad, sizeof t, cudaMemcpyDeviceToHost));
            Status v = validate_tile_host(t);
            return v.ok() ? Status(SLHA_ERR_INVALID_TILE, "tile failed validation") : v;
        }
        std::memcpy(scores_out, sc.data(), n_tiles * 4);
        return Status();
    });
}

char* slha_audit(void) {
    g_last_error[0] = 0;
    try {
        // self-audit: layout, device, and the reference's INT4 known answers
        // (slhav2-vram/tests/cpu.rs:53-115) through the CUDA scoring path
        std::string j = "{\"abi_version\":" + std::to_string(SLHA_ABI_VERSION) +
                        ",\"tile_size\":" + std::to_string(sizeof(SciRustSlhaTile)) +
                        ",\"tile_align\":" + std::to_string(alignof(SciRustSlhaTile)) + ",\"backend\":\"cuda-sm_100a\"";
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess) { cudaGetLastError(); ndev = 0; }
        j += ",\"devices\":" + std::to_string(ndev);
        bool kat_ok = false;
        if (ndev > 0) {
            kat_ok = true;
            const unsigned char fill[3] = {0x88, 0x00, 0xFF};
            const float want[3] = {0.0f, -1024.0f, 896.0f};
            float qc[D_C];
            for (float& v : qc) v = 1.0f;
            uint64_t qs[4] = {0, 0, 0, 0};
            for (int i = 0; i < 3; ++i) {
                SciRustSlhaTile t;
                std::memset(&t, 0, sizeof t);
                std::memset(t.latent_kv, fill[i], 64);
                t.scale = 1.0f;
                std::memset(t.group_scales, 255, 8);
                float s = NAN;
                if (slha_process_tile(&t, qc, qs, &s) != SLHA_OK || std::fabs(s - want[i]) > 1e-4f) kat_ok = false;
            }
        }
        j += std::string(",\"int4_known_answers\":") + (kat_ok ? "true" : "false") + "}";
        char* out = (char*)std::malloc(j.size() + 1);
        if (!out) { set_last_error("out of memory"); return nullptr; }
        std::memcpy(out, j.c_str(), j.size() + 1);
        return out;
    } catch (...) {
        set_last_error("exception caught while running the SLHA self-audit");
        return nullptr;
    }
}

void slha_free_string(char* string) { std::free(string); }

SlhaModel* slha_weights_load(const char* path) {
    SlhaModel* handle = nullptr;
    ffi([&]() -> Status {
        if (!path) return Status(SLHA_ERR_NULL, "weights path is NULL");
        CallScope cs;
        if (!cs.ok()) return cs.st;
        std::shared_ptr<Model> m;
        SLHA_TRY(model_load_slhw(cs.c, path, &m));
        handle = model_register(std::move(m));
        return Status();
    });
    return handle;
}

size_t slha_model_dim(const SlhaModel* model) {
    size_t d = 0;
    ffi([&]() -> Status {
        Status st;
        auto m = model_lookup(model, &st);
        if (!m) return st;
        d = m->d;
        return Status();
    });
    return d;
}

int32_t slha_encode_key(const SlhaModel* model, const float* key, size_t d, uint32_t position, int32_t codec,
                        SciRustSlhaTile* out_tile) {
    return ffi([&]() -> Status {
        if (!key || !out_tile) return Status(SLHA_ERR_NULL, "slha_encode_key received a NULL data pointer");
        Status st;
        auto m = model_lookup(model, &st);
        if (!m) return st;
        if (d != m->d)
            return Status(SLHA_ERR_DIMENSION, "key dimension mismatch: received " + std::to_string(d) +
                                                  ", expected " + std::to_string(m->d));
        if (codec < 0 || codec > 5)
            return Status(SLHA_ERR_CODEC, "unknown codec id " + std::to_string(codec) + "; expected an integer from 0 to 5");
        std::vector<float> kh(d);
        std::memcpy(kh.data(), key, d * 4);
        SLHA_TRY(finite_check(kh.data(), d, "key"));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const float* dk;
        SLHA_TRY(stage_in_t(c, kh.data(), d, &dk));
        SciRustSlhaTile* dt;
        SLHA_TRY(ctx_device_scratch(c, sizeof(SciRustSlhaTile), (void**)&dt));
        SLHA_TRY(launch_encode(c, m.get(), dk, SLHA_B200_F32, 1, nullptr, position, nullptr, codec, dt, nullptr));
        SciRustSlhaTile t;
        SLHA_CUDA(cudaMemcpyAsync(&t, dt, sizeof t, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        SLHA_TRY(validate_tile_host(t));
        std::memcpy(out_tile, &t, sizeof t);
        return Status();
    });
}

static int32_t decode_common(const SlhaModel* model, const SciRustSlhaTile* tile, float* out, size_t d,
                             bool with_residual, const char* who) {
    return ffi([&]() -> Status {
        if (!tile || !out) return Status(SLHA_ERR_NULL, std::string(who) + " received a NULL data pointer");
        Status st;
        auto m = model_lookup(model, &st);
        if (!m) return st;
        if (d != m->d)
            return Status(SLHA_ERR_DIMENSION, "output dimension mismatch: received " + std::to_string(d) +
                                                  ", expected " + std::to_string(m->d));
        SciRustSlhaTile t;
        std::memcpy(&t, tile, sizeof t);
        SLHA_TRY(validate_tile_host(t));
        CallScope cs;
        if (!cs.ok()) return cs.st;
        Ctx* c = cs.c;
        const SciRustSlhaTile* dt;
        SLHA_TRY(stage_in_t(c, &t, 1, &dt));
        float* dout;
        SLHA_TRY(ctx_device_scratch(c, d * 4, (void**)&dout));
        SLHA_TRY(launch_decode(c, m.get(), dt, dout, with_residual));
        std::vector<float> r(d);
        SLHA_CUDA(cudaMemcpyAsync(r.data(), dout, d * 4, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        SLHA_TRY(finite_check(r.data(), d, "reconstruction"));
        std::memcpy(out, r.data(), d * 4);
        return Status();
    });
}
int32_t slha_decode_latent(const SlhaModel* model, const SciRustSlhaTile* tile, float* out, size_t d) {
    return decode_common(model, tile, out, d, false, "slha_decode_latent");
}
int32_t slha_decode_key(const SlhaModel* model, const SciRustSlhaTile* tile, float* out, size_t d) {
    return decode_common(model, tile, out, d, true, "slha_decode_key");
}

int32_t slha_weights_release(SlhaModel* model) {
    if (model == nullptr) {
        g_last_error[0] = 0;
        return SLHA_OK;
    }
    return ffi([&]() -> Status {
        if (reinterpret_cast<uintptr_t>(model) % alignof(uint64_t) != 0)
            return Status(SLHA_ERR_INVALID_HANDLE, "model handle is misaligned");
        if (!model_unregister(model)) return Status(SLHA_ERR_INVALID_HANDLE, "model handle is not a live SLHA handle");
        return Status();
    });
}
void slha_weights_free(SlhaModel* model) { (void)slha_weights_release(model); }

}  // extern "C"

#include "capi_b200.cuh"
