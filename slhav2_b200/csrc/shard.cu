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
// shards needs no NCCL.
//
// Where the ranks are processes of one node whose GPUs can map each other's memory (CUDA IPC over
// NVLink), the all-gather is not run at all: every rank leaves its sorted top-k block where it
// wrote it, raises a flag in every peer's memory, and the merge kernel reads from the owners'
// buffers exactly the entries it needs -- the samples that bound the k-th best and the few
// leading entries of every list above that bound, a few tens of KB per query row instead of the
// world x k entries an all-gather moves -- with plain peer loads (no multicast copies anywhere).
// Candidate blocks are double-buffered by step parity; a rank can only overwrite a block two steps
// after it published it, by which time every peer has finished the merge that read it (each merge
// waits for all ranks' flags of its step).  Waits are bounded (ten seconds, then an empty row and a
// status word the host can read).  NCCL carries the one-time exchange of the IPC handles and
// remains the exchange when the mapping is not possible.
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
    // peer-memory exchange (see the head of this file): own block = control words | candidate block, parity 0 | parity 1
    void* own_block = nullptr;
    size_t block_bytes = 0;                 // one candidate block (padded)
    std::vector<void*> peer_block;          // every rank's block as mapped into this process (own: own_block)
    void* d_tables = nullptr;               // device: bases[2][world], peer_flags[world]
    bool peers_ok = false, peers_tried = false;
    bool peers_wanted = true;               // slha_b200_shard_set_exchange: false = always the NCCL all-gather
    uint64_t step_no = 0;                   // steps enqueued so far (parity of the candidate block in use)
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // step begin, after local top-k, after all-gather, after merge
    bool timed = false, have_times = false;
    // A decode loop repeats the same step (same buffers, same segment table) thousands of times, and with a
    // shard of a few hundred MB the host needs longer to enqueue the step's memset, kernels and all-gather
    // than the GPU needs to run them.  The second identical call is therefore captured into a CUDA graph,
    // and every further one is a single graph launch.
    std::vector<unsigned char> seen_key[2], graph_key[2];  // (per parity of the step: the peer exchange alternates buffers)
    cudaGraphExec_t graph_exec[2] = {nullptr, nullptr};
    int graph_launches = 0;     // kernels of one step (for the launch counter)
    bool graphs_off = false;    // capture failed once on this handle (e.g. a stream that cannot capture)
};

namespace {
constexpr size_t PEER_CTRL_BYTES = 512;  // flags[64] u32 | step u32 @256 | done u32 @260 | status u32 @264

void peers_release(Shard* s) {
    for (int r = 0; r < (int)s->peer_block.size(); ++r)
        if (r != s->rank && s->peer_block[r]) cudaIpcCloseMemHandle(s->peer_block[r]);
    s->peer_block.clear();
    if (s->own_block) cudaFree(s->own_block);
    if (s->d_tables) cudaFree(s->d_tables);
    s->own_block = nullptr;
    s->d_tables = nullptr;
    s->peers_ok = false;
    cudaGetLastError();
}

// every rank tells every peer "my block of step *step is complete" (flags[rank] in the peer's control words)
__global__ void shard_signal_kernel(uint32_t* const* peer_flags, int world, int rank, const uint32_t* step) {
    __threadfence_system();
    if ((int)threadIdx.x < world) {
        const uint32_t v = *reinterpret_cast<const volatile uint32_t*>(step);
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(peer_flags[threadIdx.x] + rank), "r"(v) : "memory");
    }
}

// Collective over the communicator: (re)allocates this rank's block for candidate blocks of `block_bytes`, exchanges the IPC
// handles through one NCCL all-gather and maps the peers' blocks.  Leaves peers_ok false (on every rank alike) when any rank
// could not map a peer; the step then keeps the NCCL all-gather.
Status peers_setup(Ctx* c, Shard* s, size_t block_bytes) {
    peers_release(s);
    s->peers_tried = true;
    s->graph_key[0].clear();
    s->graph_key[1].clear();
    if (s->world > 64) return Status();
    const int W = s->world;
    s->block_bytes = pad256(block_bytes);
    const size_t total = PEER_CTRL_BYTES + 2 * s->block_bytes;
    struct Msg { cudaIpcMemHandle_t h; int32_t ok; int32_t pad[15]; };  // 128 bytes
    static_assert(sizeof(Msg) == 128, "IPC handle message");
    Msg mine{};
    bool ok = cudaMalloc(&s->own_block, total) == cudaSuccess;
    if (ok) ok = cudaMemsetAsync(s->own_block, 0, PEER_CTRL_BYTES, c->stream) == cudaSuccess;
    const uint32_t one = 1;
    if (ok) ok = cudaMemcpyAsync((char*)s->own_block + 256, &one, 4, cudaMemcpyHostToDevice, c->stream) == cudaSuccess;  // step 1
    if (ok) ok = cudaIpcGetMemHandle(&mine.h, s->own_block) == cudaSuccess;
    mine.ok = ok ? 1 : 0;
    cudaGetLastError();
    // all-gather of the messages (device staging: NCCL moves device memory)
    Msg* d_msgs = nullptr;
    SLHA_CUDA(cudaMalloc((void**)&d_msgs, sizeof(Msg) * (size_t)(W + 1)));
    std::vector<Msg> all((size_t)W);
    Status st;
    auto exchange = [&]() -> Status {
        SLHA_CUDA(cudaMemcpyAsync(d_msgs + W, &mine, sizeof(Msg), cudaMemcpyHostToDevice, c->stream));
        SLHA_TRY(nccl_status(&g_nccl, g_nccl.all_gather(d_msgs + W, d_msgs, sizeof(Msg) / 4, NCCL_INT32, s->comm, c->stream), "ncclAllGather"));
        SLHA_CUDA(cudaMemcpyAsync(all.data(), d_msgs, sizeof(Msg) * (size_t)W, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        return Status();
    };
    st = exchange();
    if (!st.ok()) {
        cudaFree(d_msgs);
        return st;
    }
    for (const Msg& m : all) ok = ok && m.ok == 1;
    s->peer_block.assign((size_t)W, nullptr);
    for (int r = 0; r < W && ok; ++r) {
        if (r == s->rank) {
            s->peer_block[r] = s->own_block;
            continue;
        }
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = false;
            break;
        }
        s->peer_block[r] = p;
    }
    // second round: did every rank map every peer?
    mine.ok = ok ? 1 : 0;
    st = exchange();
    cudaFree(d_msgs);
    if (!st.ok()) return st;
    for (const Msg& m : all) ok = ok && m.ok == 1;
    if (!ok) {
        peers_release(s);
        s->peers_tried = true;
        return Status();
    }
    // device tables: bases[parity][rank], peer_flags[rank]
    std::vector<void*> tab((size_t)3 * W);
    for (int r = 0; r < W; ++r) {
        tab[r] = (char*)s->peer_block[r] + PEER_CTRL_BYTES;
        tab[W + r] = (char*)s->peer_block[r] + PEER_CTRL_BYTES + s->block_bytes;
        tab[2 * W + r] = s->peer_block[r];
    }
    SLHA_CUDA(cudaMalloc(&s->d_tables, tab.size() * sizeof(void*)));
    SLHA_CUDA(cudaMemcpyAsync(s->d_tables, tab.data(), tab.size() * sizeof(void*), cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    s->peers_ok = true;
    s->step_no = 0;
    return Status();
}
}  // namespace

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
    for (cudaGraphExec_t g : s->graph_exec)
        if (g) cudaGraphExecDestroy(g);
    for (cudaEvent_t e : s->ev)
        if (e) cudaEventDestroy(e);
    peers_release(s);
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

// mode 1: the NCCL all-gather always; 2: peer-memory loads where the GPUs can map each other's memory (the default).
// Every rank must make the same choice, between steps.
Status shard_set_exchange(Shard* s, int mode) {
    if (mode != 1 && mode != 2) return Status(SLHA_ERR_DIMENSION, "shard exchange mode must be 1 (NCCL all-gather) or 2 (peer memory)");
    s->peers_wanted = mode == 2;
    if (!s->peers_wanted) peers_release(s);
    s->peers_tried = false;
    s->graph_key[0].clear();
    s->graph_key[1].clear();
    return Status();
}

// out[0]: how the ranks' lists meet (0 one rank, 1 NCCL all-gather, 2 peer-memory loads by the merge kernel),
// out[1]: 1 when a wait for a peer's flag ran out since the handle was made, out[2]: steps enqueued so far
Status shard_status(Ctx* c, Shard* s, uint64_t* out3) {
    out3[0] = s->world == 1 ? 0 : (s->peers_ok ? 2 : 1);
    out3[1] = 0;
    out3[2] = s->step_no;
    if (s->peers_ok) {
        uint32_t st = 0;
        SLHA_CUDA(cudaMemcpyAsync(&st, (char*)s->own_block + 264, 4, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        out3[1] = st;
    }
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
    if (s->peers_ok) {
        const int W = s->world;
        const int parity = (int)(s->step_no & 1);
        uint32_t* ci = reinterpret_cast<uint32_t*>((char*)s->own_block + PEER_CTRL_BYTES + (size_t)parity * s->block_bytes);
        float* csc = reinterpret_cast<float*>(ci + nq * (size_t)k);
        uint32_t* ctrl = reinterpret_cast<uint32_t*>(s->own_block);
        SLHA_TRY(score_topk_device(c, tiles, nullptr, h_segs, n_segs, d_qc, d_qs, nq, k, ci, csc, nullptr));
        uint32_t* const* tabs = reinterpret_cast<uint32_t* const*>(s->d_tables);
        shard_signal_kernel<<<1, 64, 0, c->stream>>>(tabs + 2 * W, W, s->rank, ctrl + 64);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
        if (s->timed) {
            SLHA_CUDA(cudaEventRecord(s->ev[1], c->stream));
            SLHA_CUDA(cudaEventRecord(s->ev[2], c->stream));  // (no all-gather: the merge reads the peers' blocks itself)
        }
        SLHA_TRY(launch_topk_merge_peers(c, reinterpret_cast<const uint32_t* const*>(tabs + (size_t)parity * W), (uint32_t)W, (uint32_t)nq, k,
                                         ctrl, ctrl + 64, ctrl + 65, ctrl + 66, d_out_index, d_out_score));
        if (s->timed) {
            SLHA_CUDA(cudaEventRecord(s->ev[3], c->stream));
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
        // (every rank makes the same calls with the same shapes, so all take the same branch here)
        if (s->peers_wanted && (!s->peers_tried || (s->peers_ok && pad256(block * 4) > s->block_bytes))) SLHA_TRY(peers_setup(c, s, block * 4));
        if (!s->peers_ok) {
            const void *p0 = s->cand.p, *p1 = s->gathered.p;
            SLHA_TRY(s->cand.ensure(block * 4));
            SLHA_TRY(s->gathered.ensure(block * 4 * (size_t)s->world));
            if (p0 != s->cand.p || p1 != s->gathered.p) {  // (a captured step names the old buffers)
                s->graph_key[0].clear();
                s->graph_key[1].clear();
            }
        }
    }
    const int gp = s->peers_ok ? (int)(s->step_no & 1) : 0;  // which captured step: the peer exchange alternates its buffers
    struct StepDone {  // the parity advances with every step that was enqueued
        Shard* s;
        ~StepDone() { ++s->step_no; }
    } step_done{s};
    if (s->timed || s->graphs_off || timing_active()) return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
    // the call's identity: every pointer and size the enqueued work depends on
    std::vector<unsigned char> key(sizeof(SlhaB200Segment) * n_segs + 8 * 8);
    const uint64_t head[8] = {(uint64_t)(uintptr_t)tiles, (uint64_t)(uintptr_t)d_qc, (uint64_t)(uintptr_t)d_qs,
                              (uint64_t)(uintptr_t)d_out_index, (uint64_t)(uintptr_t)d_out_score, (uint64_t)nq, (uint64_t)k,
                              (uint64_t)(uintptr_t)c->stream};
    std::memcpy(key.data(), head, sizeof(head));
    std::memcpy(key.data() + sizeof(head), h_segs, sizeof(SlhaB200Segment) * n_segs);
    if (s->graph_exec[gp] && key == s->graph_key[gp]) {
        SLHA_CUDA(cudaGraphLaunch(s->graph_exec[gp], c->stream));
        count_launch(s->graph_launches);
        return Status();
    }
    if (key != s->seen_key[gp]) {  // first call of this shape: plain (it also sizes the plan's buffers, which a capture may not)
        s->seen_key[gp] = key;
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
        if (s->graph_exec[gp]) cudaGraphExecDestroy(s->graph_exec[gp]);
        s->graph_exec[gp] = exec;
        s->graph_key[gp] = key;
        s->graph_launches = launches;
        cudaGraphDestroy(graph);
        SLHA_CUDA(cudaGraphLaunch(s->graph_exec[gp], c->stream));
        return Status();
    }
    // the capture did not work out (nothing of it ran): enqueue the step the plain way from now on
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    s->graphs_off = true;
    return shard_enqueue(c, s, tiles, h_segs, n_segs, d_qc, d_qs, nq, k, d_out_index, d_out_score);
}

}  // namespace slha
