// Token-range sharding behind the C ABI: one handle per rank (one process or thread per GPU).
//
// A step is: fused score + top-k over the rank's own tiles (resident in its own HBM), ONE
// ncclAllGather of the rank's [2][nq][k] candidate block (indices, then score bits), and the
// merge kernel over the `world` gathered lists -- three enqueues on one stream, no host round
// trip between them.  The reference has no multi-device path; what this relies on is that
// tile scores are independent (ElasticKvCache::score_all, scirust/src/ccos.rs:346-355) and
// that top-k is a max-reduction with the ordering of scirust/src/metrics.rs:186-192.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already loaded in the process
// when there is one), so the library itself links only the CUDA runtime and a host that never
// shards needs no NCCL.  No peer-memory loads and no multicast copies are used anywhere: remote
// candidates arrive only through the all-gather into this rank's own buffer.
#include <dlfcn.h>

#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "runtime.cuh"

namespace slha {
namespace {

struct NcclId { char internal[128]; };
using ncclComm_t = void*;
using PFN_GetUniqueId = int (*)(NcclId*);
using PFN_CommInitRank = int (*)(ncclComm_t*, int, NcclId, int);
using PFN_AllGather = int (*)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t);
using PFN_CommDestroy = int (*)(ncclComm_t);
using PFN_GetErrorString = const char* (*)(int);
using PFN_GetVersion = int (*)(int*);
constexpr int NCCL_INT32 = 2;  // ncclInt32 in nccl.h's ncclDataType_t

struct NcclApi {
    void* handle = nullptr;
    PFN_GetUniqueId get_unique_id = nullptr;
    PFN_CommInitRank comm_init_rank = nullptr;
    PFN_AllGather all_gather = nullptr;
    PFN_CommDestroy comm_destroy = nullptr;
    PFN_GetErrorString get_error_string = nullptr;
    PFN_GetVersion get_version = nullptr;
    std::string error;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) {
        const char* e = dlerror();
        g_nccl.error = std::string("NCCL is not available: ") + (e ? e : "dlopen(libnccl.so.2) failed");
        return;
    }
    g_nccl.get_unique_id = (PFN_GetUniqueId)dlsym(g_nccl.handle, "ncclGetUniqueId");
    g_nccl.comm_init_rank = (PFN_CommInitRank)dlsym(g_nccl.handle, "ncclCommInitRank");
    g_nccl.all_gather = (PFN_AllGather)dlsym(g_nccl.handle, "ncclAllGather");
    g_nccl.comm_destroy = (PFN_CommDestroy)dlsym(g_nccl.handle, "ncclCommDestroy");
    g_nccl.get_error_string = (PFN_GetErrorString)dlsym(g_nccl.handle, "ncclGetErrorString");
    g_nccl.get_version = (PFN_GetVersion)dlsym(g_nccl.handle, "ncclGetVersion");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.all_gather || !g_nccl.comm_destroy)
        g_nccl.error = "NCCL is not available: libnccl.so.2 lacks an expected symbol";
}
Status nccl_api(NcclApi** out) {
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.error.empty()) return Status(SLHA_ERR_DEVICE, g_nccl.error);
    *out = &g_nccl;
    return Status();
}
Status nccl_status(NcclApi* api, int rc, const char* what) {
    if (rc == 0) return Status();
    return Status(SLHA_ERR_DEVICE, std::string(what) + " failed: " + (api->get_error_string ? api->get_error_string(rc) : "NCCL error") +
                                       " (" + std::to_string(rc) + ")");
}

struct Buf {
    void* p = nullptr;
    size_t cap = 0;
    Status ensure(size_t need) {
        if (need <= cap) return Status();
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        void* q = nullptr;
        SLHA_CUDA(cudaMalloc(&q, need));
        p = q;
        cap = need;
        return Status();
    }
    ~Buf() { cudaFree(p); }
};

}  // namespace

struct Shard {
    int rank = 0, world = 1, device = 0;
    ncclComm_t comm = nullptr;
    Buf cand, gathered;  // [2][nq][k] and [world][2][nq][k] int32
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // step begin, after local top-k, after all-gather, after merge
    bool timed = false, have_times = false;
    // A decode loop repeats the same step (same buffers, same segment table) thousands of times, and with a
    // shard of a few hundred MB the host needs longer to enqueue the step's memset, kernels and all-gather
    // than the GPU needs to run them.  The second identical call is therefore captured into a CUDA graph,
    // and every further one is a single graph launch.
    std::vector<unsigned char> seen_key, graph_key;
    cudaGraphExec_t graph_exec = nullptr;
    int graph_launches = 0;     // kernels of one step (for the launch counter)
    bool graphs_off = false;    // capture failed once on this handle (e.g. a stream that cannot capture)
};

Status shard_unique_id(void* id128) {
    NcclApi* api;
    SLHA_TRY(nccl_api(&api));
    NcclId id;
    SLHA_TRY(nccl_status(api, api->get_unique_id(&id), "ncclGetUniqueId"));
    std::memcpy(id128, &id, sizeof(id));
    return Status();
}

Status shard_init(Ctx* c, const void* id128, int rank, int world, Shard** out) {
    if (world < 1 || rank < 0 || rank >= world) return Status(SLHA_ERR_DIMENSION, "shard_init: need 0 <= rank < world");
    auto s = std::make_unique<Shard>();
    s->rank = rank;
    s->world = world;
    s->device = c->device;
    if (world > 1) {
        if (!id128) return Status(SLHA_ERR_NULL, "shard_init: world > 1 needs the 128-byte NCCL unique id of rank 0");
        NcclApi* api;
        SLHA_TRY(nccl_api(&api));
        NcclId id;
        std::memcpy(&id, id128, sizeof(id));
        SLHA_TRY(nccl_status(api, api->comm_init_rank(&s->comm, world, id, rank), "ncclCommInitRank"));
    }
    *out = s.release();
    return Status();
}

Status shard_destroy(Shard* s) {
    if (!s) return Status();
    cudaSetDevice(s->device);
    if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
    for (cudaEvent_t e : s->ev)
        if (e) cudaEventDestroy(e);
    if (s->comm) g_nccl.comm_destroy(s->comm);
    delete s;
    return Status();
}

void shard_info(const Shard* s, int* rank, int* world) {
    *rank = s->rank;
    *world = s->world;
}

Status shard_set_timing(Shard* s, bool on) {
    if (on)
        for (cudaEvent_t& e : s->ev)
            if (!e) SLHA_CUDA(cudaEventCreate(&e));
    s->timed = on;
    s->have_times = false;
    return Status();
}

Status shard_last_times(Ctx* c, Shard* s, float* ms3) {
    if (!s->timed || !s->have_times) return Status(SLHA_ERR_DIMENSION, "shard timing: no timed step has run (enable it first)");
    SLHA_CUDA(cudaEventSynchronize(s->ev[3]));
    for (int i = 0; i < 3; ++i) SLHA_CUDA(cudaEventElapsedTime(&ms3[i], s->ev[i], s->ev[i + 1]));
    (void)c;
    return Status();
}

namespace {
// The device part of one step, enqueued on c->stream.
Status shard_enqueue(Ctx* c, Shard* s, const SciRustSlhaTile* tiles, const SlhaB200Segment* h_segs, size_t n_segs,
                     const float* d_qc, const uint64_t* d_qs, size_t nq, uint32_t k, uint32_t* d_out_index,
                     float* d_out_score) {
    const size_t block = 2 * nq * (size_t)k;  // int32 elements of one rank's candidate block
    if (s->timed) SLHA_CUDA(cudaEventRecord(s->ev[0], c->stream));
    if (s->world == 1) {
        SLHA_TRY(score_topk_device(c, tiles, nullptr, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score, nullptr));
        if (s->timed) {
            for (int i = 1; i < 4; ++i) SLHA_CUDA(cudaEventRecord(s->ev[i], c->stream));
            s->have_times = true;
        }
        return Status();
    }
    uint32_t* ci = (uint32_t*)s->cand.p;
    float* csc = reinterpret_cast<float*>(ci + nq * (size_t)k);
    SLHA_TRY(score_topk_device(c, tiles, nullptr, h_segs, n_segs, d_qc, d_qs, nq, k, ci, csc, nullptr));
    if (s->timed) SLHA_CUDA(cudaEventRecord(s->ev[1], c->stream));
    SLHA_TRY(nccl_status(&g_nccl, g_nccl.all_gather(s->cand.p, s->gathered.p, block, NCCL_INT32, s->comm, c->stream), "ncclAllGather"));
    count_launch();
    if (s->timed) SLHA_CUDA(cudaEventRecord(s->ev[2], c->stream));
    const uint32_t* gi = (const uint32_t*)s->gathered.p;
    const float* gsc = reinterpret_cast<const float*>(gi + nq * (size_t)k);
    SLHA_TRY(launch_topk_merge_pairs(c, gi, gsc, (uint32_t)s->world, block, (uint32_t)nq, k, k, d_out_index, d_out_score, /*lists_sorted=*/true));
    if (s->timed) {
        SLHA_CUDA(cudaEventRecord(s->ev[3], c->stream));
        s->have_times = true;
    }
    return Status();
}
}  // namespace

// One step.  d_q_* are device pointers; d_out_* are device pointers of [nq][k] results (merged over
// all ranks).  Everything is enqueued on c->stream.
Status shard_step_device(Ctx* c, Shard* s, const SciRustSlhaTile* tiles, const SlhaB200Segment* h_segs, size_t n_segs,
                         const float* d_qc, const uint64_t* d_qs, size_t nq, uint32_t k, uint32_t* d_out_index,
                         float* d_out_score) {
    if (s->device != c->device) return Status(SLHA_ERR_DEVICE, "shard handle lives on another device than the calling thread's");
    if (s->world > 1) {
        const size_t block = 2 * nq * (size_t)k;
        const void *p0 = s->cand.p, *p1 = s->gathered.p;
        SLHA_TRY(s->cand.ensure(block * 4));
        SLHA_TRY(s->gathered.ensure(block * 4 * (size_t)s->world));
        if (p0 != s->cand.p || p1 != s->gathered.p) s->graph_key.clear();  // (a captured step names the old buffers)
    }
    if (s->timed || s->graphs_off || timing_active()) return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
    // the call's identity: every pointer and size the enqueued work depends on
    std::vector<unsigned char> key(sizeof(SlhaB200Segment) * n_segs + 8 * 8);
    const uint64_t head[8] = {(uint64_t)(uintptr_t)tiles, (uint64_t)(uintptr_t)d_qc, (uint64_t)(uintptr_t)d_qs,
                              (uint64_t)(uintptr_t)d_out_index, (uint64_t)(uintptr_t)d_out_score, (uint64_t)nq, (uint64_t)k,
                              (uint64_t)(uintptr_t)c->stream};
    std::memcpy(key.data(), head, sizeof(head));
    std::memcpy(key.data() + sizeof(head), h_segs, sizeof(SlhaB200Segment) * n_segs);
    if (s->graph_exec && key == s->graph_key) {
        SLHA_CUDA(cudaGraphLaunch(s->graph_exec, c->stream));
        count_launch(s->graph_launches);
        return Status();
    }
    if (key != s->seen_key) {  // first call of this shape: plain (it also sizes the plan's buffers, which a capture may not)
        s->seen_key = key;
        return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
    }
    // second identical call: capture it
    if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        cudaGetLastError();
        s->graphs_off = true;
        return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
    }
    const uint64_t before = launch_count();
    Status st = shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
    const int launches = (int)(launch_count() - before);
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    cudaGraphExec_t exec = nullptr;
    if (st.ok() && e == cudaSuccess && graph && cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
        if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
        s->graph_exec = exec;
        s->graph_key = key;
        s->graph_launches = launches;
        cudaGraphDestroy(graph);
        SLHA_CUDA(cudaGraphLaunch(s->graph_exec, c->stream));
        return Status();
    }
    // the capture did not work out (nothing of it ran): enqueue the step the plain way from now on
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    s->graphs_off = true;
    return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
}

}  // namespace slha
