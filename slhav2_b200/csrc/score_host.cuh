// Host side of the scoring path: work decomposition ("plan"), kernel launches.
// Included by score.cu.
#pragma once

#include <memory>

namespace slha {

namespace {

constexpr size_t MAX_SMEM = 227 * 1024;

// slha_b200_debug_force_generic_score: the calling thread's score_topk calls skip the
// tensor-core kernel (a checking aid: both kernels must give the same answers).
thread_local bool g_force_generic = false;
struct Plan;
thread_local const Plan* g_last_stream_plan = nullptr;  // the calling thread's latest tensor-core call (for its counters)

size_t mma_smem_bytes(int nwarps, bool nf4_table) {  // (keep in step with the kernel's layout)
    // nf4 table | stage ring | B fragments | sign words, thresholds, bucket mappings, flag
    return (size_t)(nf4_table ? NF4_LUT_BYTES : 0) + (size_t)nwarps * MMA_DEPTH * MMA_SET_STRIDE + MMA_BQ_BYTES + 128 + 16 + 32 + 32 + 16;
}
constexpr int STREAM_THREADS = SLHA_STREAM_THREADS;

size_t score_smem_bytes(int G, int nwarps, bool topk, uint32_t cap) {
    size_t b = (size_t)G * D_C * 4 + 16 * 32 * 4 + (size_t)nwarps * DEPTH * BLK_BYTES;
    if (topk) b += (size_t)G * cap * 8;
    b += (size_t)G * 8 + (size_t)G * 4 + 260 * 4 + 16;
    return b;
}

template <int G, bool TOPK>
Status launch_score_t(Ctx* c, const ScoreArgs& a, uint32_t grid, int threads, size_t smem) {
    static thread_local size_t configured[16] = {0};
    int dev = c->device & 15;
    if (configured[dev] < smem) {
        SLHA_CUDA(cudaFuncSetAttribute(score_kernel<G, TOPK>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        // every kernel of a scoring call asks for the same shared-memory / L1 split, so that an SM does not have to
        // be drained and reconfigured between the kernels of one call
        SLHA_CUDA(cudaFuncSetAttribute(score_kernel<G, TOPK>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured[dev] = MAX_SMEM;
    }
    score_kernel<G, TOPK><<<grid, threads, smem, c->stream>>>(a);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

template <bool TOPK>
Status launch_score(Ctx* c, int G, const ScoreArgs& a, uint32_t grid, int threads, size_t smem) {
    switch (G) {
        case 1: return launch_score_t<1, TOPK>(c, a, grid, threads, smem);
        case 2: return launch_score_t<2, TOPK>(c, a, grid, threads, smem);
        default: return launch_score_t<4, TOPK>(c, a, grid, threads, smem);
    }
}

int group_width(uint32_t nq) { return nq >= 3 ? 4 : (int)nq; }

// shared-memory candidate slots of the merge kernel for at most `total` candidates per query
// (k results wanted, kp2 = k rounded up to a power of two).  kp2 + k slots let the merge kernel order
// its winners by bucket placement next to them; more buys nothing: longer inputs go through the
// kernel's bucket pre-filter, which gathers only k plus one bucket of candidates, and a small buffer
// lets more CTAs share an SM.
uint32_t merge_cap(uint64_t total, uint32_t kp2, uint32_t k) {
    // (and room to order up to 1.5 k gathered keys next to themselves: the merge's sort-all path)
    const uint64_t enough = (std::max<uint64_t>((uint64_t)kp2 + k + 256, 2 * ((uint64_t)k + k / 2) + 512) + 255) / 256 * 256;
    return (uint32_t)std::min<uint64_t>(enough, 24576);
}
int merge_threads(uint32_t cap_s) { return cap_s > 4096 ? 512 : 256; }
size_t merge_smem(uint32_t cap_s, uint32_t kp2) {
    return (size_t)cap_s * 8 + 8 + (size_t)(std::max(SEL_HIST_INTS, merge_buckets(kp2, (uint32_t)merge_threads(cap_s)) + 48) + 4) * 4;
}

// Optional per-call CUDA-event timing of the two kernels of score_topk
// (slha_b200_timing_begin / _end).  Events are recorded on the launching stream.
struct Timing {
    std::vector<cudaEvent_t> ev;  // 3 per call: before score, after score, after merge
    uint32_t max_calls = 0, calls = 0;
};
thread_local Timing g_timing;

// Grow-only device buffer owned by a plan (kept when the plan object is recycled).
struct DevBuf {
    void* p = nullptr;
    size_t cap = 0;
    Status ensure(size_t need) {
        need = std::max<size_t>(need, 256);
        if (need <= cap) return Status();
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        const size_t want = need + need / 2;
        void* q = nullptr;
        SLHA_CUDA(cudaMalloc(&q, want));  // (on failure the buffer stays empty: p == nullptr, cap == 0)
        p = q;
        cap = want;
        return Status();
    }
    ~DevBuf() { cudaFree(p); }
};

// The cached decomposition of one score_topk call shape.
struct Plan {
    std::vector<unsigned char> key;
    int device = -1;
    uint32_t k = 0, cap = 0, kp2 = 0, nq = 0, n_lists = 0;
    int threads = 128;
    struct Class { int G; uint32_t first, count; };
    std::vector<Class> classes;
    WorkItem* d_items = nullptr;
    uint32_t* d_q_list_begin = nullptr;
    uint32_t* d_q_list_count = nullptr;
    uint64_t* d_cand_keys = nullptr;
    uint32_t* d_cand_cnt = nullptr;
    uint32_t* d_cta_begin = nullptr;  // tensor-core kernel: items [cta_begin[b], cta_begin[b+1]) belong to CTA b
    unsigned long long* d_gpivot = nullptr;  // per query: streaming top-k state (threshold, mapping, count, flag, histogram)
    uint64_t* d_gbuf = nullptr;              // per query: gcap candidate keys of the tensor-core kernel
    uint32_t gcap = 0;
    size_t gstate_bytes = 0;
    bool state_clean = false;  // the previous call's merge left the streaming state cleared (see StreamLists::finish)
    uint32_t compact_splits = 0, selcap = 0;  // optional compaction pass before the merge (few rows, long buffers)
    // wide scoring (16 or more queries per segment, INT4 / TQ3 launches): work items of up to 64 query rows for score_wide_kernel
    bool wide = false, allow_wide_in = false;
    WorkItem* d_wide_items = nullptr;
    WorkItem* d_stream_items = nullptr;  // interleaved description of every CTA's work for score_stream_kernel (null: the work items themselves)
    uint32_t* d_wide_cta = nullptr;
    uint32_t wide_grid = 0, n_wide_items = 0;
    uint32_t n_items = 0;
    uint32_t max_parts = 1;  // most candidate lists any query has
    uint32_t list_cap = 0;   // slots per candidate list: k plus the slack the tensor-core kernel's last selection may leave
    bool use_mma = false;
    bool nf4_table = true;
    bool mixed = false;
    bool tq3 = false;
    int codec_hint_in = -1;
    bool force_generic_in = false;
    int mma_threads = STREAM_THREADS;
    uint32_t mma_grid = 0;
    size_t mma_smem = 0;
    DevBuf b_stream_items, b_items, b_qbegin, b_qcount, b_keys, b_cnt, b_cta, b_gpivot, b_gbuf, b_gsel, b_vq, b_tmp, b_wide_items, b_wide_cta;
    // Two-level merge for calls with few queries and many candidate lists per query (a pool scored
    // by one GQA group: 148 lists each): groups of `group_parts` lists are merged by a CTA each into
    // `n_groups` intermediate (index, score) lists per query, which a second launch merges.
    uint32_t n_groups = 0, group_parts = 0;
    uint32_t* d_vq_begin = nullptr;
    uint32_t* d_vq_count = nullptr;
    uint32_t* d_tmp_index = nullptr;
    float* d_tmp_score = nullptr;
    uint64_t last_use = 0;
};

size_t wide_smem_bytes() { return 3 * WIDE_A_BYTES + 2 * WIDE_RAW_BYTES + 2048 + 256 + 256 + 512 + 512 + 64 + 2048 + 1024; }

Status build_plan(Ctx* c, const SciRustSlhaTile* tiles, const SlhaB200Segment* segs, size_t n_segs, size_t nq,
                  uint32_t k, int codec_hint, bool allow_wide, Plan** out) {
    std::vector<unsigned char> key(sizeof(SlhaB200Segment) * n_segs + 16);
    std::memcpy(key.data(), segs, sizeof(SlhaB200Segment) * n_segs);
    uint64_t nq64 = nq;
    std::memcpy(key.data() + sizeof(SlhaB200Segment) * n_segs, &nq64, 8);
    std::memcpy(key.data() + sizeof(SlhaB200Segment) * n_segs + 8, &k, 4);
    // small per-thread cache of plans (call shapes alternate in practice: appends
    // change a pool's length, layers differ); a recycled plan keeps its device buffers
    static thread_local std::vector<std::unique_ptr<Plan>> cache;
    static thread_local uint64_t tick = 0;
    ++tick;
    for (auto& e : cache)
        if (e->device == c->device && e->codec_hint_in == codec_hint && e->force_generic_in == g_force_generic && e->allow_wide_in == allow_wide && e->key == key) {
            e->last_use = tick;
            *out = e.get();
            return Status();
        }
    Plan* p;
    if (cache.size() < 4) {
        cache.push_back(std::make_unique<Plan>());
        p = cache.back().get();
    } else {
        p = cache[0].get();
        for (auto& e : cache)
            if (e->last_use < p->last_use) p = e.get();
        p->classes.clear();
        p->max_parts = 1;
    }
    // The plan is published (key + device set) only once it is complete: any early return
    // below leaves a slot that no later call can match.
    p->key.clear();
    p->device = -1;
    p->last_use = tick;
    p->codec_hint_in = codec_hint;
    p->force_generic_in = g_force_generic;
    p->allow_wide_in = allow_wide;
    p->wide = false;
    p->k = k;
    p->n_lists = 0;
    p->nq = (uint32_t)nq;
    p->kp2 = 2;
    while (p->kp2 < k) p->kp2 <<= 1;
    p->threads = k > 1024 ? 256 : 128;
    const int nwarps = p->threads / 32;
    const uint32_t round = (uint32_t)nwarps * BLK_TILES;
    uint32_t cap = std::max<uint32_t>(2 * k, k + 2 * round);
    while (cap > k + round && score_smem_bytes(4, nwarps, true, cap) > MAX_SMEM) cap -= round;
    if (score_smem_bytes(4, nwarps, true, cap) > MAX_SMEM || (size_t)p->kp2 * 8 + 2048 > MAX_SMEM)
        return Status(SLHA_ERR_CAPACITY, "top-k: k is too large for the shared-memory selection state");
    p->cap = cap;

    // tensor-core kernel: one persistent CTA per SM
    p->mma_threads = STREAM_THREADS;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
    {
        const int mw = p->mma_threads / 32;
        // Codec hint: the flags of the first tile of the first non-empty segment decide
        // whether the NF4 table occupies shared memory.  A wrong hint costs speed only
        // (NF4 tiles met without the table are handed to the generic kernel).
        // (hint: -1 = look at the first tile, else bit 0 = NF4 tiles expected, bit 1 = mixed 8/4 tiles only,
        //  bit 2 = TQ3 tiles only)
        p->nf4_table = codec_hint < 0 || (codec_hint & 1);
        p->mixed = codec_hint > 0 && (codec_hint & 2);
        p->tq3 = codec_hint > 0 && (codec_hint & 4);
        for (size_t i = 0; i < n_segs && codec_hint < 0; ++i)
            if (segs[i].n_tiles) {
                uint16_t flags = 0;
                const unsigned char* t0 = reinterpret_cast<const unsigned char*>(tiles) + segs[i].tile_begin * TILE_BYTES;
                SLHA_CUDA(cudaMemcpyAsync(&flags, t0 + 118, 2, cudaMemcpyDeviceToHost, c->stream));
                SLHA_CUDA(cudaStreamSynchronize(c->stream));
                p->nf4_table = (flags & F_NF4) != 0;
                p->mixed = (flags & F_MIXED) != 0;
                p->tq3 = (flags & F_TQ3) != 0;
                break;
            }
        p->mma_smem = mma_smem_bytes(mw, p->nf4_table);
        p->use_mma = !g_force_generic && p->mma_smem <= MAX_SMEM;
        p->mma_grid = (uint32_t)sms;
    }

    // Work items.  Generic kernel: fixed-size runs, large enough that candidate
    // traffic stays a few percent of the tile stream and small enough to balance
    // the SMs through the hardware CTA scheduler.  Tensor-core kernel: the
    // concatenated tile stream is cut into one equal share per persistent CTA
    // (and at segment ends), so per-item costs are paid once per ~total/grid tiles.
    uint64_t total = 0;
    for (size_t i = 0; i < n_segs; ++i) total += (uint64_t)segs[i].n_tiles * ((segs[i].n_queries + 3) / 4);
    uint32_t item_tiles = std::max<uint32_t>(8192, 8 * k);
    while (item_tiles > 2048 && total / item_tiles < 592) item_tiles /= 2;
    item_tiles = std::max(round, (item_tiles + round - 1) / round * round);
    uint64_t share = (total + p->mma_grid - 1) / std::max<uint32_t>(p->mma_grid, 1);
    share = std::max<uint64_t>(2048, (share + MMA_SET_TILES - 1) / MMA_SET_TILES * MMA_SET_TILES);
    const uint64_t snap = std::min<uint64_t>(share / 16, 2048);
    uint64_t spare = share * std::max<uint32_t>(p->mma_grid, 1) > total ? share * std::max<uint32_t>(p->mma_grid, 1) - total : 0;  // room the equal shares leave
    uint64_t filled = 0;  // tiles already given to the current CTA (tensor-core mode)
    std::vector<uint32_t> cta_begin(1, 0);
    // Few long streams (a stream = one segment's tiles for one group of up to four query rows; at most half as many as
    // there are CTAs): every stream gets whole CTAs in proportion to its tiles, and the CTAs of a stream take its tiles
    // interleaved -- CTA c of C takes the 24-set chunks c, c + C, c + 2 C .. -- instead of one contiguous range each.
    // Equal ranges are not equal work: where the scores are high (recent tokens) a CTA appends far more candidates, and
    // the CTA with the densest range ended 13 us after the median one; interleaved, every CTA sees the same mix.  The
    // work items below stay contiguous ranges (one per CTA): they are what the generic kernel scores when a row is
    // handed back; the tensor-core kernel reads the interleaved description of the same CTA from `stream_items`.
    std::vector<uint32_t> stream_ctas;
    std::vector<WorkItem> stream_items;
    if (p->use_mma && total > 0) {
        std::vector<uint64_t> st_tiles;
        for (size_t i = 0; i < n_segs; ++i)
            for (uint32_t q0 = 0; q0 < segs[i].n_queries; q0 += 4)
                if (segs[i].n_tiles) st_tiles.push_back(segs[i].n_tiles);
        // Only for short shares (less than 20 000 tiles per CTA: shards of a long context, measured at 7 k and 14 k tiles
        // per CTA): with whole CTAs per stream the streams' CTA counts differ by one (18 or 19 of 148 for eight streams),
        // which costs the slower streams 5 % -- less than the second set-up of a CTA that works on two streams when a
        // share lasts 40 us, more when it lasts 200 us.
        if (!st_tiles.empty() && st_tiles.size() * 2 <= p->mma_grid && total / p->mma_grid < 20000) {
            stream_ctas.resize(st_tiles.size());
            uint32_t used = 0;
            for (size_t j = 0; j < st_tiles.size(); ++j) {
                const uint64_t most = (st_tiles[j] + 2047) / 2048;  // (no CTA for less than 2048 tiles)
                stream_ctas[j] = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(most, st_tiles[j] * p->mma_grid / total));
                used += stream_ctas[j];
            }
            while (used < p->mma_grid) {  // the CTAs left over go where a CTA has the most tiles
                size_t best = st_tiles.size();
                uint64_t worst = 0;
                for (size_t j = 0; j < st_tiles.size(); ++j) {
                    const uint64_t per = st_tiles[j] / stream_ctas[j];
                    if (per > worst && (uint64_t)stream_ctas[j] < (st_tiles[j] + 2047) / 2048) { worst = per; best = j; }
                }
                if (best == st_tiles.size()) break;
                ++stream_ctas[best];
                ++used;
            }
        }
    }
    size_t stream_no = 0;

    std::vector<WorkItem> items[3];  // by class G = 1, 2, 4 (generic mode); all in [2] in tensor-core mode
    std::vector<uint32_t> q_begin(nq, 0), q_count(nq, 0);
    uint32_t n_lists = 0;
    for (size_t i = 0; i < n_segs; ++i) {
        const SlhaB200Segment& s = segs[i];
        if ((uint64_t)s.query_begin + s.n_queries > nq)
            return Status(SLHA_ERR_DIMENSION, "segment query range exceeds n_queries");
        for (uint32_t q0 = 0; q0 < s.n_queries; q0 += 4) {
            const uint32_t gq = std::min<uint32_t>(4, s.n_queries - q0);
            const int G = group_width(gq);
            // cut points of this (segment, query group) stream
            std::vector<std::pair<uint32_t, uint32_t>> cuts;  // (offset, length)
            if (!stream_ctas.empty() && s.n_tiles) {
                uint32_t ctas = stream_ctas[stream_no++];
                const uint32_t per = (uint32_t)(((uint64_t)s.n_tiles + ctas - 1) / ctas + MMA_SET_TILES - 1) / MMA_SET_TILES * MMA_SET_TILES;
                ctas = (s.n_tiles + per - 1) / per;  // (rounding to whole sets can leave the last CTA nothing)
                for (uint32_t part = 0; part < ctas; ++part) {
                    cuts.push_back({part * per, std::min<uint32_t>(per, s.n_tiles - part * per)});
                    cta_begin.push_back((uint32_t)items[2].size() + (uint32_t)cuts.size());
                    WorkItem w{};
                    w.tile_begin = s.tile_begin;
                    w.n_tiles = s.n_tiles;
                    w.index_base = s.index_base;
                    w.query_begin = s.query_begin + q0;
                    w.n_queries = gq;
                    w.list_begin = part;                              // this CTA's place among the stream's CTAs
                    w.pad = gq | (ctas << 8) | 0x80000000u;           // their number; bit 31: interleaved
                    stream_items.push_back(w);
                }
            }
            for (uint32_t pos = 0; stream_ctas.empty() && pos < s.n_tiles;) {
                uint32_t take;
                if (p->use_mma) {
                    // A work item costs its set-up and first set (several microseconds) whatever its length, so cuts that
                    // would leave a sliver are moved to the segment's end: a CTA with little room left does not start the
                    // next segment, and a cut that would leave a short rest of a segment takes the rest along.
                    if (pos == 0 && filled > 0 && share - filled < snap && spare >= share - filled) {
                        spare -= share - filled;  // (the grid must not grow beyond one CTA per SM)
                        filled = 0;
                        cta_begin.push_back((uint32_t)items[2].size() + (uint32_t)cuts.size());
                    }
                    take = (uint32_t)std::min<uint64_t>(s.n_tiles - pos, share - filled);
                    const uint32_t rest = s.n_tiles - pos - take;
                    if (rest > 0 && rest < snap) {
                        take += rest;
                        spare += rest;
                    }
                    filled += take;
                } else {
                    take = std::min<uint32_t>(item_tiles, s.n_tiles - pos);
                }
                cuts.push_back({pos, take});
                pos += take;
                if (p->use_mma && filled >= share) {
                    filled = 0;
                    cta_begin.push_back((uint32_t)items[2].size() + (uint32_t)cuts.size());
                }
            }
            const uint32_t parts = (uint32_t)cuts.size();
            p->max_parts = std::max(p->max_parts, parts);
            for (uint32_t g = 0; g < gq; ++g) {
                const uint32_t Q = s.query_begin + q0 + g;
                if (q_count[Q]) return Status(SLHA_ERR_DIMENSION, "a query row belongs to two segments");
                q_begin[Q] = n_lists + g;  // lists of one item are consecutive: stride gq per part
                q_count[Q] = parts;
            }
            for (uint32_t part = 0; part < parts; ++part) {
                WorkItem w;
                w.tile_begin = s.tile_begin + cuts[part].first;
                w.n_tiles = cuts[part].second;
                w.index_base = s.index_base + cuts[part].first;
                w.query_begin = s.query_begin + q0;
                w.n_queries = gq;
                w.list_begin = n_lists + part * gq;
                w.pad = gq | (std::min<uint32_t>(parts, 0xFFFFFFu) << 8);  // low byte: list stride between parts (merge accessor); above: parts of the row group
                items[p->use_mma ? 2 : (G == 1 ? 0 : (G == 2 ? 1 : 2))].push_back(w);
            }
            n_lists += parts * gq;
        }
    }
    p->n_lists = n_lists;
    std::vector<WorkItem> all;
    for (int cls = 0; cls < 3; ++cls) {
        if (items[cls].empty()) continue;
        p->classes.push_back({cls == 0 ? 1 : (cls == 1 ? 2 : 4), (uint32_t)all.size(), (uint32_t)items[cls].size()});
        all.insert(all.end(), items[cls].begin(), items[cls].end());
    }
    if (cta_begin.back() != (uint32_t)all.size()) cta_begin.push_back((uint32_t)all.size());
    if (all.empty()) p->use_mma = false;
    p->mma_grid = (uint32_t)cta_begin.size() - 1;
    // per query: list id of part p is q_begin + p * stride; store stride in the count's high bits
    std::vector<uint32_t> q_stride(nq, 1);
    for (const WorkItem& w : all)
        for (uint32_t g = 0; g < w.n_queries; ++g) q_stride[w.query_begin + g] = w.pad & 0xFFu;
    SLHA_TRY(p->b_items.ensure(all.size() * sizeof(WorkItem)));
    if (!stream_items.empty() && stream_items.size() != all.size()) return Status(SLHA_ERR_PANIC, "score plan: stream items out of step");
    SLHA_TRY(p->b_stream_items.ensure(stream_items.size() * sizeof(WorkItem)));
    p->d_stream_items = stream_items.empty() ? nullptr : (WorkItem*)p->b_stream_items.p;
    if (p->d_stream_items)
        SLHA_CUDA(cudaMemcpyAsync(p->d_stream_items, stream_items.data(), stream_items.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
    SLHA_TRY(p->b_qbegin.ensure(nq * 4));
    SLHA_TRY(p->b_qcount.ensure(nq * 4));
    p->list_cap = (k + std::max<uint32_t>(64, k / 2) + 31) / 32 * 32;
    SLHA_TRY(p->b_keys.ensure((size_t)n_lists * p->list_cap * 8));
    SLHA_TRY(p->b_cnt.ensure((size_t)n_lists * 4));
    SLHA_TRY(p->b_cta.ensure(cta_begin.size() * 4));
    // Wide scoring: every segment brings 16 or more queries and the launch holds INT4 / MX-INT4 or TQ3 tiles.  Work items
    // of up to 64 query rows; the (segment, row group) streams are cut into one share per CTA, in whole 128-tile blocks.
    uint32_t wide_parts = 1;
    {
        bool all_wide = p->use_mma && allow_wide && n_segs > 0 && (p->mixed || p->tq3 || !p->nf4_table);
        uint64_t wtotal = 0;
        for (size_t i = 0; i < n_segs && all_wide; ++i) {
            all_wide = segs[i].n_queries >= 16 || segs[i].n_tiles == 0;
            wtotal += (uint64_t)segs[i].n_tiles * ((segs[i].n_queries + WIDE_NQ - 1) / WIDE_NQ);
        }
        if (all_wide && wtotal > 0 && wide_smem_bytes() <= MAX_SMEM) {
            uint64_t wshare = (wtotal + sms - 1) / sms;
            wshare = std::max<uint64_t>(WIDE_M, (wshare + WIDE_M - 1) / WIDE_M * WIDE_M);
            std::vector<WorkItem> wi;
            std::vector<uint32_t> wcta(1, 0);
            uint64_t wfilled = 0;
            for (size_t i = 0; i < n_segs; ++i) {
                const SlhaB200Segment& s = segs[i];
                for (uint32_t q0 = 0; q0 < s.n_queries; q0 += WIDE_NQ) {
                    uint32_t parts = 0;
                    for (uint32_t pos = 0; pos < s.n_tiles;) {
                        const uint32_t take = (uint32_t)std::min<uint64_t>(s.n_tiles - pos, wshare - wfilled);
                        WorkItem w{};
                        w.tile_begin = s.tile_begin + pos;
                        w.n_tiles = take;
                        w.index_base = s.index_base + pos;
                        w.query_begin = s.query_begin + q0;
                        w.n_queries = std::min<uint32_t>(WIDE_NQ, s.n_queries - q0);
                        wi.push_back(w);
                        ++parts;
                        pos += take;
                        wfilled += take;
                        if (wfilled >= wshare) {
                            wfilled = 0;
                            wcta.push_back((uint32_t)wi.size());
                        }
                    }
                    wide_parts = std::max(wide_parts, parts);
                }
            }
            if (wcta.back() != (uint32_t)wi.size()) wcta.push_back((uint32_t)wi.size());
            SLHA_TRY(p->b_wide_items.ensure(wi.size() * sizeof(WorkItem)));
            SLHA_TRY(p->b_wide_cta.ensure(wcta.size() * 4));
            p->d_wide_items = (WorkItem*)p->b_wide_items.p;
            p->d_wide_cta = (uint32_t*)p->b_wide_cta.p;
            SLHA_CUDA(cudaMemcpyAsync(p->d_wide_items, wi.data(), wi.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
            SLHA_CUDA(cudaMemcpyAsync(p->d_wide_cta, wcta.data(), wcta.size() * 4, cudaMemcpyHostToDevice, c->stream));
            p->n_wide_items = (uint32_t)wi.size();
            p->wide_grid = (uint32_t)wcta.size() - 1;
            p->wide = true;
        }
    }
    // Streaming top-k state per query row: threshold, bucket mapping, count, flag, 256 bucket counts; and
    // the row's candidate buffer.  In random order about k (1 + ln(n / k)) tiles pass the rising threshold
    // plus the unfiltered first sets of every warp; 16 k slots (at most the longest segment) leave a wide
    // margin, and a row that fills its buffer all the same is scored by the generic kernel.
    // (a warp reserves slots in chunks of 16 per row and work item, so up to 16 slots per warp and item stay unused)
    uint32_t longest = 0;
    for (size_t i = 0; i < n_segs; ++i) longest = std::max(longest, segs[i].n_tiles);
    const uint64_t all_of_a_row = (uint64_t)longest + (uint64_t)MMA_CHUNK * (uint64_t)(p->mma_threads / 32) * p->max_parts + 64;
    // (the first set of every warp that scans a row is appended unfiltered: 16 slots per warp and item, twice over)
    const uint64_t first_sets = (uint64_t)(16 + MMA_CHUNK) * (uint64_t)(p->mma_threads / 32) * p->max_parts;
    p->gcap = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(std::max<uint64_t>(16ull * k, 4096), first_sets + 4ull * k), all_of_a_row / 64 * 64);
    // (wide scoring: the first 128-tile block of every item is appended unfiltered, and a CTA sees few blocks)
    if (p->wide) p->gcap = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(p->gcap, 4ull * WIDE_M * wide_parts + 16ull * k), ((uint64_t)longest + 63) / 64 * 64);
    p->gstate_bytes = nq * (1024 + 8 + 8 + 4 + 4 + 4 + 8);  // histogram, threshold, mapping, count, flag, compacted count, statistics
    p->state_clean = false;
    // few rows with long buffers: several CTAs per row compact the survivors before the merge
    // (a slice of at most 1024 slots per CTA: one round of four keys per thread)
    p->compact_splits = (p->use_mma && nq < 128 && p->gcap >= 8192) ? (uint32_t)std::min<size_t>(64, std::max<size_t>((296 + nq - 1) / nq, (p->gcap + 1023) / 1024)) : 0;
    p->selcap = merge_cap((uint64_t)p->gcap, p->kp2, k);
    if (p->compact_splits) SLHA_TRY(p->b_gsel.ensure(nq * (size_t)p->selcap * 8));
    SLHA_TRY(p->b_gpivot.ensure(p->gstate_bytes));
    if (p->use_mma) SLHA_TRY(p->b_gbuf.ensure(nq * (size_t)p->gcap * 8));
    p->d_gbuf = (uint64_t*)p->b_gbuf.p;
    p->d_items = (WorkItem*)p->b_items.p;
    p->d_q_list_begin = (uint32_t*)p->b_qbegin.p;
    p->d_q_list_count = (uint32_t*)p->b_qcount.p;
    p->d_cand_keys = (uint64_t*)p->b_keys.p;
    p->d_cand_cnt = (uint32_t*)p->b_cnt.p;
    p->d_cta_begin = (uint32_t*)p->b_cta.p;
    p->d_gpivot = (unsigned long long*)p->b_gpivot.p;
    p->n_items = (uint32_t)all.size();
    // (pageable sources: cudaMemcpyAsync returns once they are staged, so the vectors may die)
    SLHA_CUDA(cudaMemcpyAsync(p->d_cta_begin, cta_begin.data(), cta_begin.size() * 4, cudaMemcpyHostToDevice, c->stream));
    p->n_groups = 0;
    if (nq <= 64 && p->max_parts >= 24 && !p->use_mma) {
        uint32_t G = 1;
        while (G * G < p->max_parts) ++G;
        const uint32_t ng = (p->max_parts + G - 1) / G;
        std::vector<uint32_t> vq(2 * (size_t)ng * nq);
        for (uint32_t g = 0; g < ng; ++g)
            for (size_t Q = 0; Q < nq; ++Q) {
                const uint32_t parts = q_count[Q], lo = g * G;
                vq[g * nq + Q] = q_begin[Q] + lo * q_stride[Q];
                vq[(size_t)ng * nq + g * nq + Q] = (parts > lo ? std::min(G, parts - lo) : 0u) | (q_stride[Q] << 24);
            }
        SLHA_TRY(p->b_vq.ensure(vq.size() * 4));
        SLHA_TRY(p->b_tmp.ensure((size_t)ng * nq * k * 8));
        p->d_vq_begin = (uint32_t*)p->b_vq.p;
        p->d_vq_count = p->d_vq_begin + (size_t)ng * nq;
        p->d_tmp_index = (uint32_t*)p->b_tmp.p;
        p->d_tmp_score = reinterpret_cast<float*>(p->d_tmp_index + (size_t)ng * nq * k);
        SLHA_CUDA(cudaMemcpyAsync(p->d_vq_begin, vq.data(), vq.size() * 4, cudaMemcpyHostToDevice, c->stream));
        p->n_groups = ng;
        p->group_parts = G;
    }
    for (size_t Q = 0; Q < nq; ++Q) q_count[Q] |= q_stride[Q] << 24;
    SLHA_CUDA(cudaMemcpyAsync(p->d_items, all.data(), all.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaMemcpyAsync(p->d_q_list_begin, q_begin.data(), nq * 4, cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaMemcpyAsync(p->d_q_list_count, q_count.data(), nq * 4, cudaMemcpyHostToDevice, c->stream));
    p->key = std::move(key);
    p->device = c->device;
    *out = p;
    return Status();
}

}  // namespace

namespace {
// slha-c/src/lib.rs:244-286 per tile; status = min over bad tiles of (index << 8 | -code)
__global__ void validate_tiles_kernel(const unsigned char* tiles, uint64_t n, unsigned long long* status) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned char* t = tiles + i * TILE_BYTES;
    const uint32_t flags = *reinterpret_cast<const uint16_t*>(t + 118);
    const float sc = *reinterpret_cast<const float*>(t + 96), lam = *reinterpret_cast<const float*>(t + 100),
                sg = *reinterpret_cast<const float*>(t + 104);
    int code = 0;
    if (flags & ~0x3Fu) code = 6;
    else if (__popc(flags & (F_NF4 | F_MIXED | F_TQ3 | F_MIX3)) > 1) code = 6;
    else if ((flags & F_NOCORR) && !(flags & (F_TQ3 | F_MIX3))) code = 6;
    else if (!isfinite(sc) || !isfinite(lam) || !isfinite(sg)) code = 5;
    else if (sc < 0.0f || lam < 0.0f || sg < 0.0f) code = 6;
    if (code) atomicMin(status, (unsigned long long)((i << 8) | (uint64_t)code));
}
}  // namespace

Status launch_validate_tiles(Ctx* c, const SciRustSlhaTile* tiles, size_t n, unsigned long long* d_status) {
    if (n == 0) return Status();
    validate_tiles_kernel<<<(uint32_t)((n + 255) / 256), 256, 0, c->stream>>>(
        reinterpret_cast<const unsigned char*>(tiles), n, d_status);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

Status launch_score_full(Ctx* c, const SciRustSlhaTile* tiles, const uint8_t* state, size_t n,
                         const float* q_coarse, const uint64_t* q_sign, size_t nq, float* scores, int codec_hint) {
    if (n == 0 || nq == 0) return Status();
    // Long arenas: the streaming tensor-core kernel in its dense mode (all query groups of four in one launch, every CTA an
    // equal share of the tiles), then the generic kernel for the rows of work items it handed back (a codec it does not
    // decode, a query outside the fp16 split).  codec_hint as for score_topk_device: -1 = look at the first tile, -2 = generic.
    if (n >= 32768 && n < 0xFFFFFFFFull && codec_hint != -2 && !g_force_generic) {
        bool nf4 = codec_hint < 0 || (codec_hint & 1), mixed = codec_hint > 0 && (codec_hint & 2), tq3 = codec_hint > 0 && (codec_hint & 4), other = false;
        if (codec_hint < 0) {
            uint16_t flags = 0;
            SLHA_CUDA(cudaMemcpyAsync(&flags, reinterpret_cast<const unsigned char*>(tiles) + 118, 2, cudaMemcpyDeviceToHost, c->stream));
            SLHA_CUDA(cudaStreamSynchronize(c->stream));
            nf4 = (flags & F_NF4) != 0;
            mixed = (flags & F_MIXED) != 0;
            tq3 = (flags & F_TQ3) != 0;
            other = (flags & F_MIX3) != 0;
        }
        const int kind = tq3 ? 2 : (mixed ? 1 : (nf4 ? 0 : 3));
        const int mw = STREAM_THREADS / 32;
        const size_t smem = mma_smem_bytes(mw, kind == 0);
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
        if (!other && smem <= MAX_SMEM) {
            const uint32_t groups = (uint32_t)((nq + 3) / 4);
            const uint64_t total = (uint64_t)n * groups;
            uint64_t share = (total + sms - 1) / sms;
            share = std::max<uint64_t>(2048, (share + MMA_SET_TILES - 1) / MMA_SET_TILES * MMA_SET_TILES);
            std::vector<WorkItem> items;
            std::vector<uint32_t> cta(1, 0);
            uint64_t filled = 0;
            for (uint32_t grp = 0; grp < groups; ++grp)
                for (uint64_t pos = 0; pos < n;) {
                    const uint32_t take = (uint32_t)std::min<uint64_t>(n - pos, share - filled);
                    WorkItem w{};
                    w.tile_begin = pos;
                    w.n_tiles = take;
                    w.index_base = (uint32_t)pos;
                    w.query_begin = 4 * grp;
                    w.n_queries = (uint32_t)std::min<size_t>(4, nq - 4 * (size_t)grp);
                    w.pad = w.n_queries;
                    items.push_back(w);
                    pos += take;
                    filled += take;
                    if (filled >= share) {
                        filled = 0;
                        cta.push_back((uint32_t)items.size());
                    }
                }
            if (cta.back() != (uint32_t)items.size()) cta.push_back((uint32_t)items.size());
            WorkItem* d_items;
            uint32_t *d_cta, *d_gflag;
            SLHA_TRY(ctx_device_scratch(c, items.size() * sizeof(WorkItem), (void**)&d_items));
            SLHA_TRY(ctx_device_scratch(c, cta.size() * 4, (void**)&d_cta));
            SLHA_TRY(ctx_device_scratch(c, nq * 4, (void**)&d_gflag));
            SLHA_CUDA(cudaMemcpyAsync(d_items, items.data(), items.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
            SLHA_CUDA(cudaMemcpyAsync(d_cta, cta.data(), cta.size() * 4, cudaMemcpyHostToDevice, c->stream));
            SLHA_CUDA(cudaMemsetAsync(d_gflag, 0, nq * 4, c->stream));
            SLHA_CUDA(cudaStreamSynchronize(c->stream));  // (the host vectors go away)
            static thread_local bool configured[16] = {false};
            if (!configured[c->device & 15]) {
#define SLHA_DENSE_SMEM(K) SLHA_CUDA(cudaFuncSetAttribute(score_stream_kernel<K, STREAM_THREADS, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM))
                SLHA_DENSE_SMEM(0); SLHA_DENSE_SMEM(1); SLHA_DENSE_SMEM(2); SLHA_DENSE_SMEM(3);
#undef SLHA_DENSE_SMEM
                configured[c->device & 15] = true;
            }
            ScoreArgs a{};
            a.tiles = reinterpret_cast<const unsigned char*>(tiles);
            a.state = state;
            a.items = d_items;
            a.stream_items = d_items;
            a.n_items = (uint32_t)items.size();
            a.cta_begin = d_cta;
            a.q_coarse = q_coarse;
            a.q_sign = reinterpret_cast<const uint32_t*>(q_sign);
            a.scores = scores;
            a.score_stride = n;
            a.gflag = d_gflag;
            a.nf4_table = kind == 0 ? 1u : 0u;
            a.mixed = kind == 1 ? 1u : 0u;
            const uint32_t grid = (uint32_t)cta.size() - 1;
#define SLHA_LAUNCH_DENSE(K) score_stream_kernel<K, STREAM_THREADS, false, true><<<grid, STREAM_THREADS, smem, c->stream>>>(a)
            if (kind == 3) SLHA_LAUNCH_DENSE(3); else if (kind == 2) SLHA_LAUNCH_DENSE(2); else if (kind == 1) SLHA_LAUNCH_DENSE(1); else SLHA_LAUNCH_DENSE(0);
#undef SLHA_LAUNCH_DENSE
            count_launch();
            SLHA_CUDA(cudaGetLastError());
            // the generic kernel over the same work items, only those whose rows were handed back
            const int threads = 128, nwarps = threads / 32;
            return launch_score<false>(c, 4, a, (uint32_t)items.size(), threads, score_smem_bytes(4, nwarps, false, 0));
        }
    }
    const int threads = 128, nwarps = threads / 32;
    const uint32_t item_tiles = 4096;
    const uint32_t chunks = (uint32_t)((n + item_tiles - 1) / item_tiles);
    size_t q0 = 0;
    while (q0 < nq) {
        const size_t gq = std::min<size_t>(4, nq - q0);
        const int G = group_width((uint32_t)gq);
        ScoreArgs a{};
        a.tiles = reinterpret_cast<const unsigned char*>(tiles);
        a.state = state;
        a.items = nullptr;
        a.q_coarse = q_coarse + q0 * D_C;
        a.q_sign = reinterpret_cast<const uint32_t*>(q_sign + q0 * 4);
        a.scores = scores + q0 * n;
        a.score_stride = n;
        a.total_tiles = n;
        a.item_tiles = item_tiles;
        a.nq_launch = (uint32_t)gq;
        SLHA_TRY(launch_score<false>(c, G, a, chunks, threads, score_smem_bytes(G, nwarps, false, 0)));
        q0 += gq;
    }
    return Status();
}

// Dense scores of whole segments in one launch: every query row of a segment against every tile of the segment,
// row q written at scores + row_offsets[q] + index_base + tile, the rest of the row up to row_len set to `fill`.
// Work items: (segment, group of up to four query rows, run of 4096 tiles) on the generic kernel.
// fill of the rows' tails [tail_begin[q], row_len) (one CTA per row)
__global__ void fill_rows_kernel(float* scores, const unsigned long long* row_offset, const uint32_t* tail_begin, uint32_t row_len, float fill) {
    float* row = scores + row_offset[blockIdx.x];
    for (uint32_t e = tail_begin[blockIdx.x] + threadIdx.x; e < row_len; e += blockDim.x) row[e] = fill;
}

Status launch_score_segments(Ctx* c, const SciRustSlhaTile* tiles, const SlhaB200Segment* segs, size_t n_segs, const float* d_q_coarse,
                             const uint64_t* d_q_sign, size_t nq, float* d_scores, const unsigned long long* d_row_offsets,
                             uint32_t row_len, float fill) {
    // Sixteen or more query rows per segment and INT4 / MX-INT4, TQ3 or mixed 8/4 tiles (by the first tile): the contraction runs on the
    // tensor cores (score_wide_kernel in its dense mode); rows it cannot score (a tile of another codec, a query outside the
    // fp16 split) are flagged and the generic kernel below scores them.
    bool wide = n_segs > 0 && wide_smem_bytes() <= MAX_SMEM;
    uint64_t wtotal = 0;
    for (size_t i = 0; i < n_segs && wide; ++i) {
        wide = segs[i].n_queries >= 16 || segs[i].n_tiles == 0;
        wtotal += (uint64_t)segs[i].n_tiles * ((segs[i].n_queries + WIDE_NQ - 1) / WIDE_NQ);
    }
    int kindw = -1;
    for (size_t i = 0; i < n_segs && wide && wtotal && kindw < 0; ++i)
        if (segs[i].n_tiles) {
            uint16_t flags = 0;
            const unsigned char* t0 = reinterpret_cast<const unsigned char*>(tiles) + segs[i].tile_begin * TILE_BYTES;
            SLHA_CUDA(cudaMemcpyAsync(&flags, t0 + 118, 2, cudaMemcpyDeviceToHost, c->stream));
            SLHA_CUDA(cudaStreamSynchronize(c->stream));
            kindw = (flags & (F_NF4 | F_MIX3)) ? 3 : ((flags & F_MIXED) ? 2 : ((flags & F_TQ3) ? 1 : 0));
        }
    wide = wide && wtotal > 0 && kindw >= 0 && kindw <= 2;
    uint32_t* d_gflag = nullptr;
    if (wide) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
        uint64_t wshare = (wtotal + sms - 1) / sms;
        wshare = std::max<uint64_t>(WIDE_M, (wshare + WIDE_M - 1) / WIDE_M * WIDE_M);
        std::vector<WorkItem> wi;
        std::vector<uint32_t> wcta(1, 0), tail(nq, row_len);
        uint64_t wfilled = 0;
        for (size_t i = 0; i < n_segs; ++i) {
            const SlhaB200Segment& s = segs[i];
            if ((uint64_t)s.query_begin + s.n_queries > nq) return Status(SLHA_ERR_DIMENSION, "segment query range exceeds n_queries");
            if ((uint64_t)s.index_base + s.n_tiles > row_len) return Status(SLHA_ERR_DIMENSION, "segment does not fit a row of row_len scores");
            for (uint32_t q = 0; q < s.n_queries; ++q) tail[s.query_begin + q] = s.index_base + s.n_tiles;
            for (uint32_t q0 = 0; q0 < s.n_queries; q0 += WIDE_NQ)
                for (uint32_t pos = 0; pos < s.n_tiles;) {
                    const uint32_t take = (uint32_t)std::min<uint64_t>(s.n_tiles - pos, wshare - wfilled);
                    WorkItem w{};
                    w.tile_begin = s.tile_begin + pos;
                    w.n_tiles = take;
                    w.index_base = s.index_base + pos;
                    w.query_begin = s.query_begin + q0;
                    w.n_queries = std::min<uint32_t>(WIDE_NQ, s.n_queries - q0);
                    wi.push_back(w);
                    pos += take;
                    wfilled += take;
                    if (wfilled >= wshare) {
                        wfilled = 0;
                        wcta.push_back((uint32_t)wi.size());
                    }
                }
        }
        if (wcta.back() != (uint32_t)wi.size()) wcta.push_back((uint32_t)wi.size());
        WorkItem* d_wi;
        uint32_t *d_wcta, *d_tail;
        SLHA_TRY(ctx_device_scratch(c, wi.size() * sizeof(WorkItem), (void**)&d_wi));
        SLHA_TRY(ctx_device_scratch(c, wcta.size() * 4, (void**)&d_wcta));
        SLHA_TRY(ctx_device_scratch(c, nq * 4, (void**)&d_tail));
        SLHA_TRY(ctx_device_scratch(c, nq * 4, (void**)&d_gflag));
        SLHA_CUDA(cudaMemcpyAsync(d_wi, wi.data(), wi.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
        SLHA_CUDA(cudaMemcpyAsync(d_wcta, wcta.data(), wcta.size() * 4, cudaMemcpyHostToDevice, c->stream));
        SLHA_CUDA(cudaMemcpyAsync(d_tail, tail.data(), nq * 4, cudaMemcpyHostToDevice, c->stream));
        SLHA_CUDA(cudaMemsetAsync(d_gflag, 0, nq * 4, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));  // (the host vectors go away)
        static thread_local bool configured[16] = {false};
        if (!configured[c->device & 15]) {
            SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
            SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
            SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
            configured[c->device & 15] = true;
        }
        ScoreArgs a{};
        a.tiles = reinterpret_cast<const unsigned char*>(tiles);
        a.items = d_wi;
        a.n_items = (uint32_t)wi.size();
        a.cta_begin = d_wcta;
        a.q_coarse = d_q_coarse;
        a.q_sign = reinterpret_cast<const uint32_t*>(d_q_sign);
        a.scores = d_scores;
        a.row_offset = d_row_offsets;
        a.gflag = d_gflag;
        const uint32_t grid = (uint32_t)wcta.size() - 1;
        if (kindw == 1) score_wide_kernel<1, true><<<grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
        else if (kindw == 2) score_wide_kernel<2, true><<<grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
        else score_wide_kernel<0, true><<<grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
        fill_rows_kernel<<<(uint32_t)nq, 256, 0, c->stream>>>(d_scores, d_row_offsets, d_tail, row_len, fill);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
    }
    const uint32_t item_tiles = 4096;
    std::vector<WorkItem> items;
    for (size_t i = 0; i < n_segs; ++i) {
        const SlhaB200Segment& s = segs[i];
        if ((uint64_t)s.query_begin + s.n_queries > nq) return Status(SLHA_ERR_DIMENSION, "segment query range exceeds n_queries");
        if ((uint64_t)s.index_base + s.n_tiles > row_len) return Status(SLHA_ERR_DIMENSION, "segment does not fit a row of row_len scores");
        for (uint32_t q0 = 0; q0 < s.n_queries; q0 += 4) {
            uint32_t pos = 0;
            do {  // (a segment without tiles still fills its rows)
                WorkItem w{};
                w.tile_begin = s.tile_begin + pos;
                w.n_tiles = std::min<uint32_t>(item_tiles, s.n_tiles - pos);
                w.index_base = s.index_base + pos;
                w.query_begin = s.query_begin + q0;
                w.n_queries = std::min<uint32_t>(4, s.n_queries - q0);
                pos += w.n_tiles;
                w.pad = (pos >= s.n_tiles && !wide) ? 1u : 0u;  // (the rows' tails: filled above when the tensor-core kernel ran)
                items.push_back(w);
            } while (pos < s.n_tiles);
        }
    }
    if (items.empty()) return Status();
    WorkItem* d_items;
    SLHA_TRY(ctx_device_scratch(c, items.size() * sizeof(WorkItem), (void**)&d_items));
    SLHA_CUDA(cudaMemcpyAsync(d_items, items.data(), items.size() * sizeof(WorkItem), cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));  // (the host vector goes away)
    const int threads = 128, nwarps = threads / 32;
    ScoreArgs a{};
    a.tiles = reinterpret_cast<const unsigned char*>(tiles);
    a.items = d_items;
    a.q_coarse = d_q_coarse;
    a.q_sign = reinterpret_cast<const uint32_t*>(d_q_sign);
    a.scores = d_scores;
    a.row_offset = d_row_offsets;
    a.row_len = row_len;
    a.row_fill = fill;
    a.gflag = d_gflag;  // (behind the tensor-core kernel: only the work items of rows it handed back)
    return launch_score<false>(c, 4, a, (uint32_t)items.size(), threads, score_smem_bytes(4, nwarps, false, 0));
}

Status score_topk_device(Ctx* c, const SciRustSlhaTile* tiles, const uint8_t* state,
                         const SlhaB200Segment* segs, size_t n_segs, const float* d_q_coarse,
                         const uint64_t* d_q_sign, size_t nq, uint32_t k, uint32_t* d_out_index,
                         float* d_out_score, uint32_t* d_out_count, bool prefer_generic, int codec_hint) {
    if (nq == 0) return Status();
    // (4096 winners per row is what the generic kernel's block-wide selection state holds in shared memory beside its
    // tile ring; the plan builder checks the exact figure)
    if (k == 0 || k > 4096) return Status(SLHA_ERR_DIMENSION, "top-k: k must be in 1..4096");
    Plan* p = nullptr;
    SLHA_TRY(build_plan(c, tiles, segs, n_segs, nq, k, codec_hint, /*allow_wide=*/state == nullptr, &p));
    const int nwarps = p->threads / 32;
    const bool timed = g_timing.calls < g_timing.max_calls;
    cudaEvent_t* tev = timed ? &g_timing.ev[3 * g_timing.calls] : nullptr;
    if (timed) SLHA_CUDA(cudaEventRecord(tev[0], c->stream));
    const bool mma = p->use_mma && !prefer_generic;
    ScoreArgs am{};
    if (mma) g_last_stream_plan = p;
    if (mma) {
        if (!p->state_clean) SLHA_CUDA(cudaMemsetAsync(p->d_gpivot, 0, p->gstate_bytes, c->stream));
        p->state_clean = false;
        ScoreArgs& a = am;
        a.tiles = reinterpret_cast<const unsigned char*>(tiles);
        a.state = state;
        a.items = p->d_items;
        a.stream_items = p->d_stream_items ? p->d_stream_items : p->d_items;
        a.n_items = p->n_items;
        a.cta_begin = p->d_cta_begin;
        // (histograms first: they are read with 16-byte loads)
        a.ghist = reinterpret_cast<uint32_t*>(p->d_gpivot);
        a.gpivot = p->d_gpivot + 128 * nq;
        a.grange = a.gpivot + nq;
        a.gcount = reinterpret_cast<uint32_t*>(a.grange + nq);
        a.gflag = a.gcount + nq;
        a.gbuf = p->d_gbuf;
        a.gcap = p->gcap;
        a.nf4_table = p->nf4_table ? 1u : 0u;
        a.mixed = p->mixed ? 1u : 0u;
        a.q_coarse = d_q_coarse;
        a.q_sign = reinterpret_cast<const uint32_t*>(d_q_sign);
        a.k = k;
        static thread_local bool mma_configured[16] = {false};  // the attribute is per device
        if (!mma_configured[c->device & 15]) {
#define SLHA_STREAM_SMEM(K, I) SLHA_CUDA(cudaFuncSetAttribute(score_stream_kernel<K, STREAM_THREADS, I>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM))
            SLHA_STREAM_SMEM(0, false); SLHA_STREAM_SMEM(1, false); SLHA_STREAM_SMEM(2, false); SLHA_STREAM_SMEM(3, false);
            SLHA_STREAM_SMEM(0, true); SLHA_STREAM_SMEM(1, true); SLHA_STREAM_SMEM(2, true); SLHA_STREAM_SMEM(3, true);
#undef SLHA_STREAM_SMEM
            mma_configured[c->device & 15] = true;
        }
        // 3: no NF4 tile is expected, so the launch holds INT4 / MX-INT4 tiles only (any other tile hands its rows back)
        const int kind = p->tq3 ? 2 : (p->mixed ? 1 : (p->nf4_table ? 0 : 3));
        if (p->wide) {
            static thread_local bool wide_configured[16] = {false};
            if (!wide_configured[c->device & 15]) {
                SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
                SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
                SLHA_CUDA(cudaFuncSetAttribute(score_wide_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
                wide_configured[c->device & 15] = true;
            }
            a.items = p->d_wide_items;
            a.n_items = p->n_wide_items;
            a.cta_begin = p->d_wide_cta;
            if (kind == 2) score_wide_kernel<1, false><<<p->wide_grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
            else if (kind == 1) score_wide_kernel<2, false><<<p->wide_grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
            else score_wide_kernel<0, false><<<p->wide_grid, WIDE_THREADS, wide_smem_bytes(), c->stream>>>(a);
        } else {
#define SLHA_LAUNCH_MMA(K)                                                                                             \
    do {                                                                                                               \
        if (p->d_stream_items) score_stream_kernel<K, STREAM_THREADS, true><<<p->mma_grid, p->mma_threads, p->mma_smem, c->stream>>>(a); \
        else score_stream_kernel<K, STREAM_THREADS, false><<<p->mma_grid, p->mma_threads, p->mma_smem, c->stream>>>(a); \
    } while (0)
            if (kind == 3) SLHA_LAUNCH_MMA(3); else if (kind == 2) SLHA_LAUNCH_MMA(2); else if (kind == 1) SLHA_LAUNCH_MMA(1); else SLHA_LAUNCH_MMA(0);
#undef SLHA_LAUNCH_MMA
        }
        count_launch();
        SLHA_CUDA(cudaGetLastError());
        // (timing: the first bracket is the tensor-core kernel alone; the generic kernel's pass over handed-back rows, an
        // early exit when there are none, counts with the compaction and the merge)
        if (timed) SLHA_CUDA(cudaEventRecord(tev[1], c->stream));
    }
    for (const Plan::Class& cl : p->classes) {
        ScoreArgs a{};
        a.gflag = mma ? am.gflag : nullptr;  // after the tensor-core kernel: only the work items of rows it handed back
        a.tiles = reinterpret_cast<const unsigned char*>(tiles);
        a.state = state;
        a.items = p->d_items + cl.first;
        a.q_coarse = d_q_coarse;
        a.q_sign = reinterpret_cast<const uint32_t*>(d_q_sign);
        a.k = k;
        a.list_cap = p->list_cap;
        a.cap = p->cap;
        a.cand_keys = p->d_cand_keys;
        a.cand_cnt = p->d_cand_cnt;
        SLHA_TRY(launch_score<true>(c, cl.G, a, cl.count, p->threads, score_smem_bytes(cl.G, nwarps, true, p->cap)));
    }
    if (timed && !mma) SLHA_CUDA(cudaEventRecord(tev[1], c->stream));
    static thread_local bool configured[16] = {false};  // the attribute is per device
    if (!configured[c->device & 15]) {
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<CompLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<PairLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<StreamLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<CompLists>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<PairLists>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<StreamLists>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        SLHA_CUDA(cudaFuncSetAttribute(stream_compact_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured[c->device & 15] = true;
    }
    if (mma) {
        uint32_t* gselcnt = am.gflag + nq;
        const uint32_t cap_s = p->selcap;
        if (p->compact_splits) {
            stream_compact_kernel<<<dim3(p->compact_splits, (uint32_t)nq), 256, 0, c->stream>>>(
                p->d_gbuf, am.gcount, am.gflag, am.gpivot, p->gcap, (uint64_t*)p->b_gsel.p, gselcnt, cap_s, p->compact_splits);
            count_launch();
            SLHA_CUDA(cudaGetLastError());
        }
        StreamLists L{p->d_gbuf, am.gcount, am.gflag, am.gpivot, p->gcap,
                      p->compact_splits ? (const uint64_t*)p->b_gsel.p : nullptr, gselcnt, cap_s,
                      CompLists{p->d_cand_keys, p->d_cand_cnt, p->d_q_list_begin, p->d_q_list_count, p->list_cap},
                      am.ghist, gselcnt + nq};
        topk_merge_kernel<StreamLists><<<(uint32_t)nq, merge_threads(cap_s), merge_smem(cap_s, p->kp2), c->stream>>>(
            L, k, p->kp2, cap_s, d_out_index, d_out_score, d_out_count);
        p->state_clean = cudaPeekAtLastError() == cudaSuccess;
    } else if (p->n_groups) {
        // few queries, many lists each: groups of lists first, then the groups' results
        CompLists L1{p->d_cand_keys, p->d_cand_cnt, p->d_vq_begin, p->d_vq_count, p->list_cap};
        const uint32_t cap1 = merge_cap((uint64_t)p->group_parts * p->list_cap, p->kp2, k);
        topk_merge_kernel<CompLists><<<p->n_groups * (uint32_t)nq, merge_threads(cap1), merge_smem(cap1, p->kp2), c->stream>>>(
            L1, k, p->kp2, cap1, p->d_tmp_index, p->d_tmp_score, nullptr);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
        PairLists L2{p->d_tmp_index, p->d_tmp_score, p->n_groups, (uint32_t)nq, k, (uint64_t)nq * k, 1u, nullptr, nullptr, nullptr, nullptr, nullptr};
        const uint32_t cap2 = merge_cap((uint64_t)p->n_groups * k, p->kp2, k);
        topk_merge_kernel<PairLists><<<(uint32_t)nq, merge_threads(cap2), merge_smem(cap2, p->kp2), c->stream>>>(
            L2, k, p->kp2, cap2, d_out_index, d_out_score, d_out_count);
    } else {
        CompLists L{p->d_cand_keys, p->d_cand_cnt, p->d_q_list_begin, p->d_q_list_count, p->list_cap};
        const uint32_t cap_s = merge_cap((uint64_t)p->max_parts * p->list_cap, p->kp2, k);
        topk_merge_kernel<CompLists><<<(uint32_t)nq, merge_threads(cap_s), merge_smem(cap_s, p->kp2), c->stream>>>(
            L, k, p->kp2, cap_s, d_out_index, d_out_score, d_out_count);
    }
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    if (timed) {
        SLHA_CUDA(cudaEventRecord(tev[2], c->stream));
        ++g_timing.calls;
    }
    return Status();
}

void debug_force_generic_score(bool on) { g_force_generic = on; }
bool debug_general_paths() { return g_force_generic; }

// Counters of the calling thread's latest score_topk call that used the tensor-core kernel.
Status last_score_stats(Ctx* c, uint64_t* out4) {
    out4[0] = out4[1] = out4[2] = out4[3] = 0;
    const Plan* p = g_last_stream_plan;
    if (!p || p->device != c->device || !p->use_mma) return Status();
    const size_t nq = p->nq;
    std::vector<uint32_t> h(2 * nq);
    const uint32_t* stats = reinterpret_cast<const uint32_t*>(p->d_gpivot + 128 * nq + 2 * nq) + 3 * nq;  // kept by the merge
    SLHA_CUDA(cudaMemcpyAsync(h.data(), stats, 8 * nq, cudaMemcpyDeviceToHost, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    out4[0] = nq;
    for (size_t q = 0; q < nq; ++q) {
        out4[1] += h[2 * q + 1] != 0;
        out4[2] += h[2 * q];
    }
    out4[3] = p->gcap;
    return Status();
}

bool timing_active() { return g_timing.calls < g_timing.max_calls; }

Status timing_begin(uint32_t max_calls) {
    for (cudaEvent_t e : g_timing.ev) cudaEventDestroy(e);
    g_timing.ev.assign((size_t)3 * max_calls, nullptr);
    for (cudaEvent_t& e : g_timing.ev) SLHA_CUDA(cudaEventCreate(&e));
    g_timing.max_calls = max_calls;
    g_timing.calls = 0;
    return Status();
}

Status timing_end(Ctx* c, float* score_ms, float* merge_ms, uint32_t capacity, uint32_t* n_out) {
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    const uint32_t n = std::min(g_timing.calls, capacity);
    for (uint32_t i = 0; i < n; ++i) {
        float a = 0, b = 0;
        SLHA_CUDA(cudaEventElapsedTime(&a, g_timing.ev[3 * i], g_timing.ev[3 * i + 1]));
        SLHA_CUDA(cudaEventElapsedTime(&b, g_timing.ev[3 * i + 1], g_timing.ev[3 * i + 2]));
        if (score_ms) score_ms[i] = a;
        if (merge_ms) merge_ms[i] = b;
    }
    if (n_out) *n_out = g_timing.calls;
    for (cudaEvent_t e : g_timing.ev) cudaEventDestroy(e);
    g_timing.ev.clear();
    g_timing.max_calls = g_timing.calls = 0;
    return Status();
}

Status launch_topk_merge_pairs(Ctx* c, const uint32_t* cand_index, const float* cand_score,
                               uint32_t n_lists, uint64_t list_stride, uint32_t n_queries, uint32_t k_in,
                               uint32_t k_out, uint32_t* out_index, float* out_score, bool lists_sorted) {
    if (n_queries == 0) return Status();
    if (k_out == 0 || k_out > 8192) return Status(SLHA_ERR_DIMENSION, "merge: k_out must be in 1..8192");
    uint32_t kp2 = 2;
    while (kp2 < k_out) kp2 <<= 1;
    PairLists L{cand_index, cand_score, n_lists, n_queries, k_in, list_stride, lists_sorted ? 1u : 0u, nullptr, nullptr, nullptr, nullptr, nullptr};
    static thread_local bool configured[16] = {false};  // the attribute is per device
    if (!configured[c->device & 15]) {
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<PairLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        configured[c->device & 15] = true;
    }
    const uint32_t cap_s = merge_cap((uint64_t)n_lists * k_in, kp2, k_out);
    topk_merge_kernel<PairLists><<<n_queries, merge_threads(cap_s), merge_smem(cap_s, kp2), c->stream>>>(L, k_out, kp2, cap_s, out_index, out_score, nullptr);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

// The merge of a sharded step whose lists lie in their owners' memory (see PairLists::bases): lists ordered best first.
Status launch_topk_merge_peers(Ctx* c, const uint32_t* const* d_bases, uint32_t n_lists, uint32_t n_queries, uint32_t k, const uint32_t* d_ready,
                               uint32_t* d_step, uint32_t* d_done, uint32_t* d_status, uint32_t* out_index, float* out_score) {
    if (n_queries == 0) return Status();
    if (k == 0 || k > 8192) return Status(SLHA_ERR_DIMENSION, "merge: k must be in 1..8192");
    uint32_t kp2 = 2;
    while (kp2 < k) kp2 <<= 1;
    PairLists L{nullptr, nullptr, n_lists, n_queries, k, 0, 1u, d_bases, d_ready, d_step, d_done, d_status};
    static thread_local bool configured[16] = {false};  // the attribute is per device
    if (!configured[c->device & 15]) {
        SLHA_CUDA(cudaFuncSetAttribute(topk_merge_kernel<PairLists>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_SMEM));
        configured[c->device & 15] = true;
    }
    const uint32_t cap_s = merge_cap((uint64_t)n_lists * k, kp2, k);
    topk_merge_kernel<PairLists><<<n_queries, merge_threads(cap_s), merge_smem(cap_s, kp2), c->stream>>>(L, k, kp2, cap_s, out_index, out_score, nullptr);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

}  // namespace slha
