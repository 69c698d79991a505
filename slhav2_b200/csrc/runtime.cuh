// Host runtime shared by the C ABI: per-call scratch arena, host<->device
// staging of "host or device" arguments, the model registry.
#pragma once

#include <memory>
#include <vector>

#include "common.cuh"

namespace slha {

// Resets the calling thread's scratch arena when constructed; the C ABI creates
// one per entry point so that staging buffers live exactly as long as the call.
// On a caller-supplied stream the call may return with its kernels still queued: the
// destructor then records an event, and the next scope on a different stream waits for it.
struct CallScope {
    Ctx* c = nullptr;
    Status st;
    CallScope();
    ~CallScope();
    CallScope(const CallScope&) = delete;
    CallScope& operator=(const CallScope&) = delete;
    bool ok() const { return st.ok(); }
};

// Bring a host-or-device input of `bytes` bytes to the device (no copy when it
// already is device memory).
Status stage_in(Ctx* c, const void* p, size_t bytes, const void** dev);
template <typename T>
Status stage_in_t(Ctx* c, const T* p, size_t count, const T** dev) {
    return stage_in(c, p, count * sizeof(T), reinterpret_cast<const void**>(dev));
}

// A host-or-device output: kernels write to `dev`; finish() copies to the
// caller's host buffer (if it was one) after the stream has been drained.
struct StagedOut {
    void* dev = nullptr;
    void* user = nullptr;
    size_t bytes = 0;
    bool is_host = false;
};
Status stage_out(Ctx* c, void* user, size_t bytes, StagedOut* out, bool in_place_if_pinned = false);
// Copies every host-bound output back and synchronises the stream when any
// copy was needed or `force_sync` is set.
Status finish_outputs(Ctx* c, std::vector<StagedOut>& outs, bool force_sync);
// True when the call must not return before the stream is drained (library
// stream) and false when the caller supplied a stream and owns synchronisation.
bool sync_by_default(const Ctx* c);

// ---- models ------------------------------------------------------------------
std::shared_ptr<Model> model_lookup(const SlhaModel* handle, Status* st);
SlhaModel* model_register(std::shared_ptr<Model> m);
bool model_unregister(SlhaModel* handle);
// LearnedModel::try_from_projection_with (scirust/src/learned.rs:204-238)
Status model_build(Ctx* c, const float* p, size_t d, uint64_t seed, bool rht, const float* scale,
                   const float* z, std::shared_ptr<Model>* out);
// weights::load / from_bytes (scirust/src/weights.rs:159-311)
Status model_load_slhw(Ctx* c, const char* path, std::shared_ptr<Model>* out);

// slha-c/src/lib.rs:244-286 on the host (single tiles of the legacy entry points)
Status validate_tile_host(const SciRustSlhaTile& t);

}  // namespace slha
