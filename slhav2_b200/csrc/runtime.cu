// Host runtime of libslha_b200: execution context, scratch arena, staging,
// model construction (.slhw parsing, sign-LSH matrix generation) and registry.
#include "runtime.cuh"

#include <sys/stat.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>

namespace slha {

Status cuda_status(cudaError_t e, const char* what) {
    return Status(SLHA_ERR_DEVICE, std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what);
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

// ---- per-thread context ------------------------------------------------------
namespace {
struct Block {
    char* p = nullptr;
    size_t cap = 0, off = 0;
};
struct ThreadState {
    int device = 0;
    bool device_chosen = false;
    cudaStream_t user_stream = nullptr;
    bool has_user_stream = false;
    Ctx ctx[16];
    bool ctx_init[16] = {false};
    std::vector<Block> blocks[16];
    std::vector<std::pair<void*, size_t>> hblocks[16];
    // Arena reuse across streams: a call on a caller-supplied stream may return while its
    // kernels still read the arena; the event marks the end of that work, and a later call on
    // ANOTHER stream waits for it before it reuses the arena (same stream: stream order suffices).
    cudaEvent_t arena_done[16] = {nullptr};
    cudaStream_t arena_stream[16] = {nullptr};
    bool arena_pending[16] = {false};
};
thread_local ThreadState tls;
}  // namespace

void tls_set_device(int dev) {
    tls.device = dev;
    tls.device_chosen = true;
}
void tls_set_stream(void* s) {
    tls.user_stream = (cudaStream_t)s;
    tls.has_user_stream = s != nullptr;
}

Status get_ctx(Ctx** out) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return Status(SLHA_ERR_DEVICE, "no CUDA device is available (this library has no CPU fallback)");
    }
    int dev = tls.device;
    if (dev < 0 || dev >= n || dev >= 16) return Status(SLHA_ERR_DEVICE, "invalid device index");
    SLHA_CUDA(cudaSetDevice(dev));
    Ctx& c = tls.ctx[dev];
    if (!tls.ctx_init[dev]) {
        c.device = dev;
        SLHA_CUDA(cudaStreamCreateWithFlags(&c.lib_stream, cudaStreamNonBlocking));
        tls.ctx_init[dev] = true;
    }
    c.stream = tls.has_user_stream ? tls.user_stream : c.lib_stream;
    c.own_stream = !tls.has_user_stream;
    *out = &c;
    return Status();
}
bool sync_by_default(const Ctx* c) { return c->own_stream; }

Status ctx_device_scratch(Ctx* c, size_t bytes, void** out) {
    bytes = pad256(std::max<size_t>(bytes, 256));
    auto& blocks = tls.blocks[c->device];
    for (Block& b : blocks) {
        if (b.cap - b.off >= bytes) {
            *out = b.p + b.off;
            b.off += bytes;
            return Status();
        }
    }
    Block nb;
    nb.cap = std::max<size_t>(bytes, blocks.empty() ? (size_t)8 << 20 : blocks.back().cap * 2);
    SLHA_CUDA(cudaMalloc((void**)&nb.p, nb.cap));
    nb.off = bytes;
    *out = nb.p;
    blocks.push_back(nb);
    return Status();
}
Status ctx_host_scratch(Ctx* c, size_t bytes, void** out) {
    void* p = nullptr;
    SLHA_CUDA(cudaMallocHost(&p, std::max<size_t>(bytes, 256)));
    tls.hblocks[c->device].push_back({p, bytes});
    *out = p;
    return Status();
}

CallScope::CallScope() {
    st = get_ctx(&c);
    if (!st.ok()) return;
    auto& blocks = tls.blocks[c->device];
    if (tls.arena_pending[c->device] && tls.arena_stream[c->device] != c->stream) {
        cudaStreamWaitEvent(c->stream, tls.arena_done[c->device], 0);
        tls.arena_pending[c->device] = false;
    }
    // the previous call has returned, so its staging memory may be reused; when
    // the arena had to chain blocks, replace them by one block of the total size
    if (blocks.size() > 1) {
        size_t total = 0;
        cudaStreamSynchronize(c->stream);
        for (Block& b : blocks) { total += b.cap; cudaFree(b.p); }
        blocks.clear();
        Block nb;
        nb.cap = total;
        if (cudaMalloc((void**)&nb.p, nb.cap) == cudaSuccess) blocks.push_back(nb);
        else cudaGetLastError();
    }
    for (Block& b : blocks) b.off = 0;
    for (auto& hb : tls.hblocks[c->device]) cudaFreeHost(hb.first);
    tls.hblocks[c->device].clear();
}

CallScope::~CallScope() {
    if (!c || c->own_stream) return;  // library stream: the call drained it before returning
    bool used = false;
    for (const Block& b : tls.blocks[c->device]) used |= b.off != 0;
    if (!used) return;
    cudaEvent_t& ev = tls.arena_done[c->device];
    if (!ev && cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        cudaStreamSynchronize(c->stream);  // no event to be had: drain instead
        return;
    }
    cudaEventRecord(ev, c->stream);
    tls.arena_stream[c->device] = c->stream;
    tls.arena_pending[c->device] = true;
}

bool is_device_ptr(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

Status stage_in(Ctx* c, const void* p, size_t bytes, const void** dev) {
    if (p == nullptr || bytes == 0 || is_device_ptr(p)) {
        *dev = p;
        return Status();
    }
    void* d;
    SLHA_TRY(ctx_device_scratch(c, bytes, &d));
    SLHA_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, c->stream));
    *dev = d;
    return Status();
}

Status stage_out(Ctx* c, void* user, size_t bytes, StagedOut* out, bool in_place_if_pinned) {
    out->user = user;
    out->bytes = bytes;
    if (user == nullptr || bytes == 0 || is_device_ptr(user)) {
        out->dev = user;
        out->is_host = false;
        return Status();
    }
    // Page-locked host memory the GPU can address (cudaHostAlloc, cudaHostRegister with mapping) is written in place by the
    // kernels: the results cross the bus while the kernel that produces them runs, instead of in a copy queued behind it.
    // Only for outputs that the call's kernels write once and never read (the caller says so).
    cudaPointerAttributes a;
    if (in_place_if_pinned && cudaPointerGetAttributes(&a, user) == cudaSuccess && a.type == cudaMemoryTypeHost && a.devicePointer != nullptr) {
        out->dev = a.devicePointer;
        out->is_host = false;
        return Status();
    }
    cudaGetLastError();
    out->is_host = true;
    return ctx_device_scratch(c, bytes, &out->dev);
}

Status finish_outputs(Ctx* c, std::vector<StagedOut>& outs, bool force_sync) {
    bool any = false;
    for (StagedOut& o : outs)
        if (o.is_host && o.bytes) {
            SLHA_CUDA(cudaMemcpyAsync(o.user, o.dev, o.bytes, cudaMemcpyDeviceToHost, c->stream));
            any = true;
        }
    if (any || force_sync) SLHA_CUDA(cudaStreamSynchronize(c->stream));
    return Status();
}

// ---- model registry ------------------------------------------------------------
// Handles are addresses of small heap tokens.  A released token is kept forever
// in a retired list so that its address can never become a live handle again
// (same guarantee as slha-c/src/lib.rs:124-205).
namespace {
struct Token { uint64_t opaque; };
struct Registry {
    std::shared_mutex mu;
    std::unordered_map<const void*, std::pair<std::unique_ptr<Token>, std::shared_ptr<Model>>> live;
    std::vector<std::unique_ptr<Token>> retired;
};
Registry& registry() {
    static Registry* r = new Registry();
    return *r;
}
}  // namespace

std::shared_ptr<Model> model_lookup(const SlhaModel* handle, Status* st) {
    if (handle == nullptr) {
        *st = Status(SLHA_ERR_NULL, "model handle is NULL");
        return nullptr;
    }
    if (reinterpret_cast<uintptr_t>(handle) % alignof(uint64_t) != 0) {
        *st = Status(SLHA_ERR_INVALID_HANDLE, "model handle is misaligned");
        return nullptr;
    }
    Registry& r = registry();
    std::shared_lock<std::shared_mutex> lk(r.mu);
    auto it = r.live.find(handle);
    if (it == r.live.end()) {
        *st = Status(SLHA_ERR_INVALID_HANDLE, "model handle is not a live SLHA handle");
        return nullptr;
    }
    return it->second.second;
}
SlhaModel* model_register(std::shared_ptr<Model> m) {
    Registry& r = registry();
    auto tok = std::make_unique<Token>();
    const void* key = tok.get();
    std::unique_lock<std::shared_mutex> lk(r.mu);
    r.live.emplace(key, std::make_pair(std::move(tok), std::move(m)));
    return reinterpret_cast<SlhaModel*>(const_cast<void*>(key));
}
bool model_unregister(SlhaModel* handle) {
    Registry& r = registry();
    std::unique_lock<std::shared_mutex> lk(r.mu);
    auto it = r.live.find(handle);
    if (it == r.live.end()) return false;
    r.retired.push_back(std::move(it->second.first));
    r.live.erase(it);
    return true;
}

// ---- model construction -----------------------------------------------------------
namespace {
// SplitMix64 + Box-Muller, scirust/src/rng.rs:13-51.  The matrix is generated on
// the host with libm logf/cosf (what Rust's f32::ln / f32::cos call) and uploaded.
struct Rng {
    uint64_t state;
    explicit Rng(uint64_t seed) : state(seed ^ 0x9E3779B97F4A7C15ull) {}
    uint64_t next_u64() {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float next_unit() { return (float)(next_u64() >> 40) * (1.0f / (float)(1ull << 24)); }
    float next_gaussian() {
        float u1 = next_unit();
        if (!(u1 > 1.0e-7f)) u1 = 1.0e-7f;
        const float u2 = next_unit();
        const float r = sqrtf(-2.0f * logf(u1));
        return r * cosf(2.0f * 3.14159265358979323846f * u2);
    }
};
void free_model(Model* m) {
    cudaFree(m->d_p);
    cudaFree(m->d_pt);
    cudaFree(m->d_scale);
    cudaFree(m->d_z);
    cudaFree(m->d_zt);
    cudaFree(m->d_diag);
    delete m;
}
Status upload(float** dst, const std::vector<float>& src, cudaStream_t s) {
    SLHA_CUDA(cudaMalloc((void**)dst, std::max<size_t>(src.size() * 4, 256)));
    SLHA_CUDA(cudaMemcpyAsync(*dst, src.data(), src.size() * 4, cudaMemcpyHostToDevice, s));
    return Status();
}
}  // namespace

Status model_build(Ctx* c, const float* p, size_t d, uint64_t seed, bool rht, const float* scale,
                   const float* z, std::shared_ptr<Model>* out) {
    if (d == 0 || d > (1u << 20)) return Status(SLHA_ERR_DIMENSION, "projection must be D_C x d with 0 < d <= 2^20");
    for (size_t i = 0; i < (size_t)D_C * d; ++i)
        if (!std::isfinite(p[i])) return Status(SLHA_ERR_NONFINITE, "projection contains a non-finite value");
    std::shared_ptr<Model> m(new Model(), free_model);
    m->d = d;
    m->rht = rht;
    m->device = c->device;
    size_t dp = d;
    if (rht) {  // incoherence.rs:29-35 next_pow2
        dp = 1;
        while (dp < d) dp <<= 1;
    }
    m->d_pad = dp;
    std::vector<float> P(p, p + (size_t)D_C * d), Pt((size_t)D_C * d), S(D_C, 1.0f);
    for (size_t k = 0; k < (size_t)D_C; ++k)
        for (size_t i = 0; i < d; ++i) Pt[i * D_C + k] = P[k * d + i];
    if (scale) {
        for (int k = 0; k < D_C; ++k) {
            if (!std::isfinite(scale[k]) || scale[k] <= 0.0f)
                return Status(SLHA_ERR_NONFINITE, "whitening scale must be finite and positive");
            S[k] = scale[k];
        }
    }
    std::vector<float> Z((size_t)D_S * dp), Zt((size_t)D_S * dp), diag;
    if (rht) {  // learned.rs:158-165 + incoherence.rs:89-97
        Rng r(seed ^ 0xA2A2A2A2A2A2A2A2ull);
        diag.resize(dp);
        for (size_t i = 0; i < dp; ++i) diag[i] = r.next_unit() < 0.5f ? -1.0f : 1.0f;
    }
    if (z) {
        std::memcpy(Z.data(), z, Z.size() * 4);
    } else {  // learned.rs:168-170
        Rng r(seed);
        for (float& v : Z) v = r.next_gaussian();
    }
    for (size_t s = 0; s < (size_t)D_S; ++s)
        for (size_t i = 0; i < dp; ++i) Zt[i * D_S + s] = Z[s * dp + i];
    SLHA_TRY(upload(&m->d_p, P, c->stream));
    SLHA_TRY(upload(&m->d_pt, Pt, c->stream));
    SLHA_TRY(upload(&m->d_scale, S, c->stream));
    SLHA_TRY(upload(&m->d_z, Z, c->stream));
    SLHA_TRY(upload(&m->d_zt, Zt, c->stream));
    if (rht) SLHA_TRY(upload(&m->d_diag, diag, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    *out = std::move(m);
    return Status();
}

Status model_load_slhw(Ctx* c, const char* path, std::shared_ptr<Model>* out) {
    // weights.rs:284-311: regular file, <= 256 MiB
    struct stat sb;
    if (stat(path, &sb) != 0) return Status(SLHA_ERR_IO, std::string("weights: cannot stat ") + path);
    if (!S_ISREG(sb.st_mode)) return Status(SLHA_ERR_IO, std::string("weights: ") + path + " is not a regular file");
    if ((uint64_t)sb.st_size > 256ull * 1024 * 1024) return Status(SLHA_ERR_IO, "weights: file above the 256 MiB safety cap");
    FILE* f = std::fopen(path, "rb");
    if (!f) return Status(SLHA_ERR_IO, std::string("weights: cannot read ") + path);
    std::vector<unsigned char> b((size_t)sb.st_size);
    const size_t got = b.empty() ? 0 : std::fread(b.data(), 1, b.size(), f);
    std::fclose(f);
    if (got != b.size()) return Status(SLHA_ERR_IO, std::string("weights: short read on ") + path);
    // weights.rs:159-270
    auto u32_at = [&](size_t o) {
        return (uint32_t)b[o] | ((uint32_t)b[o + 1] << 8) | ((uint32_t)b[o + 2] << 16) | ((uint32_t)b[o + 3] << 24);
    };
    if (b.size() < 24) return Status(SLHA_ERR_IO, "weights: truncated header");
    if (u32_at(0) != 0x534C4857u) return Status(SLHA_ERR_IO, "weights: bad magic (not an SLHW file)");
    const uint32_t version = u32_at(4);
    size_t header;
    if (version == 1) header = 24;
    else if (version == 2) header = 28;
    else return Status(SLHA_ERR_IO, "weights: unsupported version " + std::to_string(version) + " (supported: 1 and 2)");
    if (b.size() < header) return Status(SLHA_ERR_IO, "weights: truncated header");
    const size_t d = u32_at(8);
    if (d <= (size_t)D_C)
        return Status(SLHA_ERR_IO, "weights: invalid dimension " + std::to_string(d) + " (must be greater than D_C=128)");
    uint64_t seed = 0;
    for (int i = 0; i < 8; ++i) seed |= (uint64_t)b[12 + i] << (8 * i);
    if (b[20] > 1) return Status(SLHA_ERR_IO, "weights: invalid RHT flag " + std::to_string(b[20]) + " (expected 0 or 1)");
    if (b[21] || b[22] || b[23]) return Status(SLHA_ERR_IO, "weights: non-zero reserved header bytes");
    const size_t expected = header + (size_t)D_C * d * 4;
    if (b.size() != expected)
        return Status(SLHA_ERR_IO, "weights: size mismatch (got " + std::to_string(b.size()) + ", expected " + std::to_string(expected) + ")");
    if (version == 2) {  // FNV-1a over the 24-byte header and the payload, weights.rs:68-80
        uint32_t h = 0x811C9DC5u;
        for (size_t i = 0; i < 24; ++i) { h ^= b[i]; h *= 0x01000193u; }
        for (size_t i = 28; i < b.size(); ++i) { h ^= b[i]; h *= 0x01000193u; }
        if (h != u32_at(24)) return Status(SLHA_ERR_IO, "weights: checksum mismatch");
    }
    std::vector<float> p((size_t)D_C * d);
    std::memcpy(p.data(), b.data() + header, p.size() * 4);
    for (size_t i = 0; i < p.size(); ++i)
        if (!std::isfinite(p[i]))
            return Status(SLHA_ERR_IO, "weights: non-finite projection value at index " + std::to_string(i));
    return model_build(c, p.data(), d, seed, b[20] == 1, nullptr, nullptr, out);
}

Status validate_tile_host(const SciRustSlhaTile& t) {
    const uint16_t known = F_WARM | F_NF4 | F_MIXED | F_TQ3 | F_NOCORR | F_MIX3;
    if (t.flags & ~known) {
        char buf[64];
        std::snprintf(buf, sizeof buf, "tile contains unknown flag bits: 0x%04x", t.flags);
        return Status(SLHA_ERR_INVALID_TILE, buf);
    }
    if (__builtin_popcount(t.flags & (F_NF4 | F_MIXED | F_TQ3 | F_MIX3)) > 1)
        return Status(SLHA_ERR_INVALID_TILE, "tile selects more than one latent codec");
    if ((t.flags & F_NOCORR) && !(t.flags & (F_TQ3 | F_MIX3)))
        return Status(SLHA_ERR_INVALID_TILE, "correction-drop flag requires the TQ3 or MIX3 codec");
    if (!std::isfinite(t.scale) || !std::isfinite(t.dynamic_lambda) || !std::isfinite(t.residual_sigma))
        return Status(SLHA_ERR_NONFINITE, "tile metadata contains a non-finite float");
    if (t.scale < 0.0f || t.dynamic_lambda < 0.0f || t.residual_sigma < 0.0f)
        return Status(SLHA_ERR_INVALID_TILE, "tile scale, dynamic lambda, and residual sigma must be non-negative");
    return Status();
}

}  // namespace slha
