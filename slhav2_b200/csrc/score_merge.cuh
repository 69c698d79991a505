// Second stage of the top-k: one CTA per query merges candidate lists (the
// per-work-item survivors of score_kernel, or per-shard results gathered from
// other GPUs) into the final k entries, sorted by score descending with ties
// towards the lower index (ordering of scirust/src/metrics.rs:186-192).
// Included by score.cu.
#pragma once

namespace slha {
namespace {

#ifdef SLHA_STREAM_PROBE
__device__ unsigned long long g_merge_probe[64][12];
#define MPROBE(i) do { if (threadIdx.x == 0 && blockIdx.x < 64) g_merge_probe[blockIdx.x][i] = probe_now(); } while (0)
#define MPROBE_VAL(i, v) do { if (threadIdx.x == 0 && blockIdx.x < 64) g_merge_probe[blockIdx.x][i] = (unsigned long long)(v); } while (0)
#else
#define MPROBE(i)
#define MPROBE_VAL(i, v)
#endif
// A list as the gathering loop wants it: when `p` is set, its keys are p[0 .. len) and a key counts when it is
// at least `pivot` (everything the accessors below would re-read per key, read once); else the loop asks at().
struct ListView {
    const uint64_t* p;
    uint64_t pivot;
    uint32_t len;
};

// Candidate accessors: element e of query Q as a composite key, 0 = absent.
struct CompLists {  // lists written by score_kernel
    static constexpr bool kFiltered = false;
    const uint64_t* keys;      // [n_lists][k] (k here = slots per list, >= the k asked for)
    const uint32_t* cnt;       // [n_lists]
    const uint32_t* q_list_begin;  // [nq]
    const uint32_t* q_list_count;  // [nq]: parts in bits 0..23, list stride between parts in bits 24..31
    uint32_t k;
    __device__ uint32_t size(uint32_t Q) const { return (q_list_count[Q] & 0xFFFFFFu) * k; }
    __device__ uint32_t lists(uint32_t Q) const { return q_list_count[Q] & 0xFFFFFFu; }
    __device__ uint32_t list_len(uint32_t Q, uint32_t part) const {
        return cnt[q_list_begin[Q] + part * (q_list_count[Q] >> 24)];
    }
    __device__ uint64_t at(uint32_t Q, uint32_t part, uint32_t j) const {
        return keys[(size_t)(q_list_begin[Q] + part * (q_list_count[Q] >> 24)) * k + j];
    }
    __device__ uint64_t get(uint32_t Q, uint32_t e) const {
        const uint32_t l = q_list_begin[Q] + (e / k) * (q_list_count[Q] >> 24), j = e % k;
        return j < cnt[l] ? keys[(size_t)l * k + j] : 0ull;
    }
    __device__ void finish(uint32_t) const {}
    __device__ bool wait_ready(int*) const { return true; }
    __device__ uint64_t floor_key(uint32_t, uint32_t, uint64_t*, uint32_t, int*) const { return 0ull; }
    __device__ ListView view(uint32_t Q, uint32_t part) const {
        const uint32_t l = q_list_begin[Q] + part * (q_list_count[Q] >> 24);
        return ListView{keys + (size_t)l * k, 0ull, cnt[l]};
    }
};
// Candidates of the streaming tensor-core kernel: one buffer per query row (keys below the row's
// final threshold count as absent), or - for rows that kernel handed to the generic kernel - the
// generic kernel's per-work-item lists.
struct StreamLists {
    static constexpr bool kFiltered = true;
    const uint64_t* gbuf;                // [nq][gcap]
    const uint32_t* gcount;              // [nq]
    const uint32_t* gflag;               // [nq]
    const unsigned long long* gpivot;    // [nq]
    uint32_t gcap;
    // optional: the survivors of every row's buffer, compacted by stream_compact_kernel
    const uint64_t* gsel;                // [nq][selcap] or null
    const uint32_t* gselcnt;             // [nq]
    uint32_t selcap;
    CompLists items;
    __device__ bool compacted(uint32_t Q) const { return gsel != nullptr && gselcnt[Q] <= selcap; }
    __device__ uint32_t len0(uint32_t Q) const { return compacted(Q) ? gselcnt[Q] : min(gcount[Q], gcap); }
    __device__ uint32_t size(uint32_t Q) const { return gflag[Q] ? items.size(Q) : len0(Q); }
    __device__ uint32_t lists(uint32_t Q) const { return gflag[Q] ? items.lists(Q) : 1u; }
    __device__ uint32_t list_len(uint32_t Q, uint32_t part) const { return gflag[Q] ? items.list_len(Q, part) : len0(Q); }
    __device__ uint64_t at(uint32_t Q, uint32_t part, uint32_t j) const {
        if (gflag[Q]) return items.at(Q, part, j);
        if (compacted(Q)) return gsel[(size_t)Q * selcap + j];
        const uint64_t key = gbuf[(size_t)Q * gcap + j];
        return key >= gpivot[Q] ? key : 0ull;
    }
    __device__ uint64_t get(uint32_t Q, uint32_t e) const { return gflag[Q] ? items.get(Q, e) : (e < len0(Q) ? at(Q, 0, e) : 0ull); }
    // The merge is the last reader of a row's streaming state: it leaves the state cleared for the next call
    // (which then needs no memset in front of its score kernel) and keeps the row's figures for the statistics call.
    __device__ uint64_t floor_key(uint32_t, uint32_t, uint64_t*, uint32_t, int*) const { return 0ull; }  // (the row's threshold filters already)
    __device__ bool wait_ready(int*) const { return true; }
    __device__ ListView view(uint32_t Q, uint32_t part) const {
        if (gflag[Q]) return items.view(Q, part);
        if (compacted(Q)) return ListView{gsel + (size_t)Q * selcap, 0ull, gselcnt[Q]};
        return ListView{gbuf + (size_t)Q * gcap, gpivot[Q], min(gcount[Q], gcap)};
    }
    uint32_t* ghist;     // [nq][256]; the state arrays follow it in one allocation
    uint32_t* stats;     // [nq][2] candidates appended, handed to the generic kernel
    __device__ void finish(uint32_t Q) const {
        for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) ghist[(size_t)Q * 256 + i] = 0u;
        if (threadIdx.x == 0) {
            stats[2 * Q] = gcount[Q];
            stats[2 * Q + 1] = gflag[Q];
            const_cast<unsigned long long*>(gpivot)[Q] = 0ull;
            const_cast<unsigned long long*>(gpivot)[gridDim.x + Q] = 0ull;  // (the bucket mapping lies behind the thresholds)
            const_cast<uint32_t*>(gcount)[Q] = 0u;
            const_cast<uint32_t*>(gflag)[Q] = 0u;
            const_cast<uint32_t*>(gselcnt)[Q] = 0u;
        }
    }
};
struct PairLists {  // (index, score) lists laid out [list][query][k_in]
    static constexpr bool kFiltered = false;
    const uint32_t* idx;
    const float* score;
    uint32_t n_lists, n_queries, k_in;
    uint64_t list_stride;  // elements between the blocks of consecutive lists
    uint32_t sorted;       // every list is ordered best first (lists this library produced)
    // Lists that lie where their owners wrote them, in the memory of other GPUs of the node (token-range sharding without
    // an all-gather: the merge reads the few entries it needs over NVLink).  bases[l] = list l's index block, its score
    // block n_queries * k_in words behind it; ready[l] (this GPU's memory, written by list l's owner) must have reached
    // *step before list l is read; the last CTA to finish advances *step.  All null for lists in one local buffer.
    const uint32_t* const* bases;
    const uint32_t* ready;
    uint32_t* step;
    uint32_t* done;
    uint32_t* status;
    __device__ ListView view(uint32_t, uint32_t) const { return ListView{nullptr, 0ull, k_in}; }
    // false when an owner's flag did not arrive within ten seconds (*status is set; the caller writes an empty row)
    __device__ bool wait_ready(int* ok_s_ptr) const {  // ok_s_ptr: one word of shared memory
        if (!ready) return true;
        int& ok_s = *ok_s_ptr;
        if (threadIdx.x == 0) {
            const uint32_t want = *reinterpret_cast<volatile uint32_t*>(step);
            unsigned long long t0, t1;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t0));
            int ok = 1;
            for (uint32_t l = 0; l < n_lists && ok; ++l) {
                for (;;) {
                    uint32_t v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(ready + l) : "memory");
                    if ((int32_t)(v - want) >= 0) break;
                    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t1));
                    if (t1 - t0 > 10000000000ull) {  // ten seconds: the owner is gone
                        ok = 0;
                        atomicExch(status, 1u);
                        break;
                    }
                    __nanosleep(200);
                }
            }
            ok_s = ok;
        }
        __syncthreads();
        const bool all_ok = ok_s != 0;
        __syncthreads();  // (the word belongs to the merge's buffer from here on)
        return all_ok;
    }
    // A key that at least k candidates reach -- and few more -- from sorted lists alone.  Every list is sampled at every
    // `stride`-th entry (stride = k / (8 n_lists)); a sample certifies that `stride` more entries of its list are at
    // least as large.  For a sample v, L(v) = stride x (samples of all lists >= v) entries reach v for certain; the
    // largest sample with L >= k is the floor.  Fewer than stride (n_lists + 1) further entries can lie above it, so
    // the merge gathers fewer than k + k / 8 + stride keys instead of n_lists * k, however unevenly the lists share the
    // k best (token-range shards do: recent tokens score higher).  All threads of the block call this; `scratch` is
    // shared memory of `slots` keys.  Zero: no bound (unsorted lists, too few entries, no room).  With a floor,
    // prefix[0 .. n_lists] receives the exclusive prefix sums of how many leading entries of every list can reach it
    // (the list's first sample below the floor ends them), so that only those are read.
    __device__ uint64_t floor_key(uint32_t Q, uint32_t k, uint64_t* scratch, uint32_t slots, int* prefix) const {
        if (!sorted || n_lists < 2 || n_lists > 64) return 0ull;
        const uint32_t stride = max(1u, k / (8u * n_lists)), m = k_in / stride, S = n_lists * m;
        if (m == 0 || S + 1 > slots) return 0ull;
        const uint32_t tid = threadIdx.x, nt = blockDim.x;
        for (uint32_t i = tid; i < S; i += nt) scratch[i] = at(Q, i / m, stride * (i % m + 1) - 1);  // (an absent entry is key 0)
        if (tid == 0) scratch[S] = 0ull;
        __syncthreads();
        for (uint32_t i = tid; i < S; i += nt) {
            const uint64_t v = scratch[i];
            if (!v) continue;
            uint32_t reach = 0;
            for (uint32_t l = 0; l < n_lists; ++l) {
                // samples of list l that are >= v: the list is ordered best first
                const uint64_t* a = scratch + l * m;
                uint32_t lo = 0, hi = m;
                while (lo < hi) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (a[mid] >= v) lo = mid + 1;
                    else hi = mid;
                }
                reach += lo;
            }
            if ((uint64_t)reach * stride >= k) atomicMax(reinterpret_cast<unsigned long long*>(scratch + S), (unsigned long long)v);
        }
        __syncthreads();
        const uint64_t f = scratch[S];
        if (f && tid == 0) {
            int run = 0;
            for (uint32_t l = 0; l < n_lists; ++l) {
                const uint64_t* a = scratch + l * m;
                uint32_t lo = 0, hi = m;
                while (lo < hi) {  // samples of list l that are >= f
                    const uint32_t mid = (lo + hi) >> 1;
                    if (a[mid] >= f) lo = mid + 1;
                    else hi = mid;
                }
                prefix[l] = run;
                run += (int)min(k_in, stride * (lo + 1));
            }
            prefix[n_lists] = run;
        }
        __syncthreads();
        return f;
    }
    __device__ uint32_t size(uint32_t) const { return n_lists * k_in; }
    __device__ uint32_t lists(uint32_t) const { return n_lists; }
    __device__ uint32_t list_len(uint32_t, uint32_t) const { return k_in; }
    __device__ uint64_t at(uint32_t Q, uint32_t part, uint32_t j) const {
        if (bases) {  // (another GPU's memory: read past the L1)
            const uint32_t* b = bases[part] + (size_t)Q * k_in + j;
            const uint32_t i = __ldcg(b);
            return i == 0xFFFFFFFFu ? 0ull : make_comp(__uint_as_float(__ldcg(b + (size_t)n_queries * k_in)), i);
        }
        const size_t o = (size_t)part * list_stride + (size_t)Q * k_in + j;
        const uint32_t i = idx[o];
        return i == 0xFFFFFFFFu ? 0ull : make_comp(score[o], i);
    }
    __device__ uint64_t get(uint32_t Q, uint32_t e) const { return at(Q, e / k_in, e % k_in); }
    __device__ void finish(uint32_t) const {
        if (!step) return;
        if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) {  // every CTA has read *step at its start
            *done = 0u;
            *reinterpret_cast<volatile uint32_t*>(step) = *reinterpret_cast<volatile uint32_t*>(step) + 1u;
        }
    }
};

// Calls with few query rows (a long context scored by a handful of heads) leave every row tens of
// thousands of buffered candidates, most of them below the row's final threshold, and one merge CTA
// per row would read them alone.  Here `splits` CTAs per row each filter a slice of the row's buffer
// and append the survivors (keys at or above the threshold) to a compact list; a row whose survivors
// exceed `selcap` keeps a count above it, which sends the merge back to the full buffer.
__global__ void __launch_bounds__(256) stream_compact_kernel(const uint64_t* gbuf, const uint32_t* gcount, const uint32_t* gflag,
                                                             const unsigned long long* gpivot, uint32_t gcap, uint64_t* gsel,
                                                             uint32_t* gselcnt, uint32_t selcap, uint32_t splits) {
    const uint32_t Q = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    if (gflag[Q]) return;
    const uint32_t len = min(gcount[Q], gcap);
    const uint32_t per = ((len + splits - 1) / splits + 3) & ~3u;
    const uint32_t lo = blockIdx.x * per, hi = min(len, lo + per);
    const uint64_t pv = gpivot[Q];
    const uint64_t* src = gbuf + (size_t)Q * gcap;
    uint64_t* dst = gsel + (size_t)Q * selcap;
    for (uint32_t j0 = lo; j0 < hi; j0 += 4 * blockDim.x) {
        uint64_t key[4];
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t j = j0 + u * blockDim.x + tid;
            key[u] = j < hi ? src[j] : 0ull;
        }
        // one reservation per warp for the four keys of its lanes (the slice of a CTA is one such round when the
        // launch has enough splits, so a CTA pays one load and one atomic round trip)
        unsigned bal[4];
        uint32_t tot = 0;
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            bal[u] = __ballot_sync(0xFFFFFFFFu, key[u] != 0ull && key[u] >= pv);
            tot += (uint32_t)__popc(bal[u]);
        }
        if (!tot) continue;
        uint32_t base = 0;
        if (lane == 0) base = atomicAdd(gselcnt + Q, tot);
        base = __shfl_sync(0xFFFFFFFFu, base, 0);
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t at = base + (uint32_t)__popc(bal[u] & ((1u << lane) - 1u));
            if ((bal[u] >> lane & 1u) && at < selcap) dst[at] = key[u];
            base += (uint32_t)__popc(bal[u]);
        }
    }
}

// Orders buf[0..m) descending into out[0..m) by bucket placement: NB (1024 or 2048) score buckets between the
// smallest and the largest score (highest first, widths shrinking towards the dense low end), a counting pass, an exclusive scan, a
// scatter, and an insertion sort inside every bucket by one thread.  The winners of a top-k are a
// thin tail, a handful of keys per bucket, so this replaces the 55 dependent stages of a bitonic
// sort of 1024 keys by six barriers.  Returns false (nothing written that matters) when a bucket
// would hold more than 16 keys or the scores cannot be bucketed; the caller then sorts bitonically.
// hist: NB + 48 ints, NB a multiple of the thread count and at most four times it.  All threads of the block.
__device__ bool bucket_sort(const uint64_t* buf, uint64_t* out, uint32_t m, int* hist, const int NB) {
    const uint32_t tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
    uint32_t* st = reinterpret_cast<uint32_t*>(hist + NB);  // 0 min, 1 max, 2 largest bucket, 8.. warp totals
    if (tid == 0) { st[0] = 0xFFFFFFFFu; st[1] = 0u; st[2] = 0u; }
    for (int b = (int)tid; b < NB; b += (int)nt) hist[b] = 0;
    __syncthreads();
    uint32_t mn = 0xFFFFFFFFu, mx = 0u;
    for (uint32_t i = tid; i < m; i += nt) {
        const uint32_t h = (uint32_t)(buf[i] >> 32);
        mn = min(mn, h);
        mx = max(mx, h);
    }
    mn = __reduce_min_sync(0xFFFFFFFFu, mn);
    mx = __reduce_max_sync(0xFFFFFFFFu, mx);
    if (lane == 0) { atomicMin(&st[0], mn); atomicMax(&st[1], mx); }
    __syncthreads();
    const float smin = key_score(st[0]), smax = key_score(st[1]);
    const float inv = 1.0f / (smax - smin);
    MPROBE(4);
    if (!(st[1] > st[0]) || !isfinite(smin) || !isfinite(smax) || !isfinite(inv)) return false;
    // The best of a long list thin out towards the top: most keys sit just above the smallest.  Bucketing the
    // square root of the normalised score (every step monotone: subtraction, multiplication by a positive
    // constant, the correctly rounded square root, truncation) spreads that dense end over more buckets.
    auto bucket = [&](uint64_t key) {
        const float v = sqrtf(fmaxf((key_score((uint32_t)(key >> 32)) - smin) * inv, 0.0f));  // 1 = highest score
        const int b = (int)((1.0f - v) * (float)NB);                                            // -> bucket 0
        return b < 0 ? 0 : (b > NB - 1 ? NB - 1 : b);
    };
    for (uint32_t i = tid; i < m; i += nt) atomicAdd(&hist[bucket(buf[i])], 1);
    __syncthreads();
    // exclusive scan of the bucket counts: thread t owns NB / nt consecutive buckets
    const uint32_t per = (uint32_t)NB / nt;  // 2 or 4
    int c[4], sum = 0, big = 0;
#pragma unroll
    for (uint32_t jj = 0; jj < 4; ++jj) {
        c[jj] = jj < per ? hist[tid * per + jj] : 0;
        sum += c[jj];
        big = max(big, c[jj]);
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if ((int)lane >= o) incl += y;
    }
    big = __reduce_max_sync(0xFFFFFFFFu, big);
    if (lane == 31) st[8 + warp] = (uint32_t)incl;
    if (lane == 0) atomicMax(&st[2], (uint32_t)big);
    __syncthreads();
    MPROBE(5);
    MPROBE_VAL(3, st[2]);
    if (st[2] > 16u) return false;
    int base = incl - sum;
    for (uint32_t w = 0; w < warp; ++w) base += (int)st[8 + w];
#pragma unroll
    for (uint32_t jj = 0; jj < 4; ++jj) {
        if (jj < per) {
            hist[tid * per + jj] = base;  // start of the bucket; becomes its end during the scatter
            base += c[jj];
        }
    }
    __syncthreads();
    for (uint32_t i = tid; i < m; i += nt) {
        const uint64_t key = buf[i];
        out[atomicAdd(&hist[bucket(key)], 1)] = key;
    }
    __syncthreads();
    MPROBE(6);
    for (int b = (int)tid; b < NB; b += (int)nt) {
        const int s0 = b ? hist[b - 1] : 0, e0 = hist[b];
        for (int x = s0 + 1; x < e0; ++x) {
            const uint64_t key = out[x];
            int y = x - 1;
            while (y >= s0 && out[y] < key) { out[y + 1] = out[y]; --y; }
            out[y + 1] = key;
        }
    }
    __syncthreads();
    return true;
}

// Buckets of bucket_sort for a merge of kp2 (k rounded up to a power of two) results by nt threads.
__host__ __device__ inline int merge_buckets(uint32_t kp2, uint32_t nt) {
    const uint32_t nb = kp2 < 1024u ? 1024u : kp2;
    return (int)(nb > 4u * nt ? 4u * nt : nb);
}

// The k outputs of query Q from keys sorted descending, the first m of them valid.
__device__ __forceinline__ void emit_sorted(const uint64_t* sorted, uint32_t m, uint32_t k, uint32_t Q, uint32_t* out_index, float* out_score,
                                            uint32_t* out_count) {
    for (uint32_t r = threadIdx.x; r < k; r += blockDim.x) {
        const bool v = r < m;
        const uint64_t key = v ? sorted[r] : 0ull;
        out_index[(size_t)Q * k + r] = v ? 0xFFFFFFFFu - (uint32_t)key : 0xFFFFFFFFu;
        out_score[(size_t)Q * k + r] = v ? key_score((uint32_t)(key >> 32)) : -INFINITY;
    }
    if (out_count && threadIdx.x == 0) out_count[Q] = m;
}

// Sort the m winners in buf[0..m) (buf[m..kp2) is zero) descending and write the k outputs of
// query Q.  buf has cap_s >= kp2 slots; with m more beyond kp2 the bucket placement above is used,
// otherwise (or when it declines) a bitonic sort of buf[0..kp2), kp2 a power of two.
__device__ void sort_and_emit(uint64_t* buf, uint32_t cap_s, int* hist, uint32_t kp2, uint32_t m, uint32_t k, uint32_t Q,
                              uint32_t* out_index, float* out_score, uint32_t* out_count) {
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    const uint64_t* sorted = buf;
    if (m >= 64 && kp2 + m <= cap_s && (nt == 256 || nt == 512) && bucket_sort(buf, buf + kp2, m, hist, merge_buckets(kp2, nt))) {
        sorted = buf + kp2;
    } else {
        // Comparator i of a stage with stride <= 32 touches only elements [64 (i / 32), +64): the 32
        // comparators a warp executes together stay inside one 64-element chunk, so those stages need no
        // block barrier, only the stages that cross chunks (and the step into or out of them) do.
        for (uint32_t size = 2; size <= kp2; size <<= 1) {
            for (uint32_t stride = size >> 1; stride; stride >>= 1) {
                for (uint32_t i = tid; i < kp2 / 2; i += nt) {
                    const uint32_t lo = 2 * i - (i & (stride - 1));
                    const uint32_t hi = lo + stride;
                    const bool desc = (lo & size) == 0;
                    const uint64_t x = buf[lo], y = buf[hi];
                    if ((x < y) == desc) { buf[lo] = y; buf[hi] = x; }
                }
                const uint32_t next_stride = stride > 1 ? stride >> 1 : size;
                if (stride > 32 || next_stride > 32) __syncthreads();
                else __syncwarp();
            }
        }
        __syncthreads();
    }
    emit_sorted(sorted, m, k, Q, out_index, out_score, out_count);
}

// cap_s: candidate slots of the shared-memory buffer (>= kp2).  When the query's
// candidates fit they are gathered once and selected / sorted in shared memory;
// otherwise the radix select runs over global memory.
template <typename Lists>
__device__ __forceinline__ void topk_merge_body(const Lists& L, uint32_t k, uint32_t kp2, uint32_t cap_s, uint32_t* out_index,
                                                float* out_score, uint32_t* out_count, unsigned char* smem) {
    uint64_t* buf = reinterpret_cast<uint64_t*>(smem);  // [cap_s]
    uint64_t* pivot_s = buf + cap_s;                    // [1]
    int* hist = reinterpret_cast<int*>(pivot_s + 1);    // max(SEL_HIST_INTS, buckets of bucket_sort + 48)
    int* n_s = hist + max(SEL_HIST_INTS, merge_buckets(kp2, blockDim.x) + 48);
    const uint32_t Q = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    MPROBE(0);
    const uint32_t T = L.size(Q);

    // upper bound of the number of candidates
    uint32_t total = 0;
    for (uint32_t l = 0; l < L.lists(Q); ++l) total += L.list_len(Q, l);
    // Lists that drop keys below a known threshold while they are read (Lists::kFiltered) hold far
    // fewer present keys than slots: one gathering pass usually fits them into shared memory.
    bool gathered = false;
    const uint64_t floor_key = L.floor_key(Q, k, buf, cap_s, hist);  // (the same in every thread; buf and hist are free until the gathering)
    const bool filtered = Lists::kFiltered || floor_key != 0ull;
    MPROBE(1);
    if (total <= cap_s || filtered) {
        if (tid == 0) *n_s = 0;
        __syncthreads();
        const uint32_t n_lists_q = L.lists(Q);
        if (floor_key != 0ull) {
            // lists ordered best first: only the leading entries that can reach the floor, all lists in one sweep
            const uint32_t total_pre = (uint32_t)hist[n_lists_q];
            for (uint32_t e0 = 0; e0 < total_pre; e0 += 4 * nt) {
                uint64_t key[4];
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t e = e0 + u * nt + tid;
                    key[u] = 0ull;
                    if (e < total_pre) {
                        uint32_t l = 0;
                        while (l + 1 < n_lists_q && (uint32_t)hist[l + 1] <= e) ++l;
                        key[u] = L.at(Q, l, e - (uint32_t)hist[l]);
                        if (key[u] < floor_key) key[u] = 0ull;
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const unsigned bal = __ballot_sync(0xFFFFFFFFu, key[u] != 0ull);
                    if (!bal) continue;
                    int base = 0;
                    if ((tid & 31) == 0) base = atomicAdd(n_s, __popc(bal));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    const uint32_t at = (uint32_t)base + __popc(bal & ((1u << (tid & 31)) - 1));
                    if (key[u] && at < cap_s) buf[at] = key[u];
                }
            }
        }
        for (uint32_t l = 0; floor_key == 0ull && l < n_lists_q; ++l) {
            const ListView V = L.view(Q, l);
            const uint32_t len = V.len;
            const uint64_t low = V.p ? (V.pivot > floor_key ? V.pivot : floor_key) : floor_key;
            // four keys per round: the loads go out together, then the compaction
            for (uint32_t j0 = 0; j0 < len; j0 += 4 * nt) {
                uint64_t key[4];
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t j = j0 + u * nt + tid;
                    key[u] = j < len ? (V.p ? V.p[j] : L.at(Q, l, j)) : 0ull;
                    if (key[u] < low) key[u] = 0ull;
                }
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const unsigned bal = __ballot_sync(0xFFFFFFFFu, key[u] != 0ull);
                    if (!bal) continue;
                    int base = 0;
                    if ((tid & 31) == 0) base = atomicAdd(n_s, __popc(bal));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    const uint32_t at = (uint32_t)base + __popc(bal & ((1u << (tid & 31)) - 1));
                    if (key[u] && at < cap_s) buf[at] = key[u];
                }
            }
        }
        __syncthreads();
        gathered = (uint32_t)*n_s <= cap_s;
        __syncthreads();
        MPROBE(2);
    }
    if (gathered) {
        const uint32_t present = (uint32_t)*n_s;
        __syncthreads();
        MPROBE_VAL(11, present);
        if (present > k) {
            // Lists filtered by a threshold that is proven to keep k candidates hold little more than k (up to 1.5 k here):
            // ordering them all and writing the first k is cheaper than selecting the k first.
            const uint32_t pa = (present + 1u) & ~1u;
            if (filtered && present <= k + (k >> 1) && 2 * pa <= cap_s && (nt == 256 || nt == 512) &&
                bucket_sort(buf, buf + pa, present, hist, merge_buckets(kp2, nt))) {
                MPROBE(7);
                emit_sorted(buf + pa, k, k, Q, out_index, out_score, out_count);
                MPROBE(8);
                return;
            }
            __syncthreads();
            // bucket selection on the score word; equal scores around the k-th place
            // fall back to the exact radix selection, which also orders by index
            if (tid == 0) *pivot_s = 0ull;
            __syncthreads();
            if (block_select_multi(buf, cap_s, n_s, 1, k, 0u, (int)k, pivot_s, hist)) block_select_topk(buf, n_s, k, pivot_s, hist);
        }
        const uint32_t m = present < k ? present : k;
        for (uint32_t i = m + tid; i < kp2; i += nt) buf[i] = 0ull;
        __syncthreads();
        sort_and_emit(buf, cap_s, hist, kp2, m, k, Q, out_index, out_score, out_count);
        return;
    }

    // Too many candidates for shared memory: one bucket pass over the lists where
    // they lie (256 equal-width score buckets between the smallest and the largest
    // score) finds a score bound that at least k candidates reach; when those fit,
    // they alone are gathered and the selection finishes in shared memory.
    {
        uint32_t* rng = reinterpret_cast<uint32_t*>(hist + 1024);  // [0] min, [1] max, [2] gathered
        if (tid == 0) { rng[0] = 0xFFFFFFFFu; rng[1] = 0u; rng[2] = 0u; *n_s = 0; }
        for (uint32_t b = tid; b < 256; b += nt) hist[b] = 0;
        __syncthreads();
        uint32_t mn = 0xFFFFFFFFu, mx = 0u;
        for (uint32_t l = 0; l < L.lists(Q); ++l) {
            const uint32_t len = L.list_len(Q, l);
            for (uint32_t j = tid; j < len; j += nt) {
                const uint64_t key = L.at(Q, l, j);
                if (key) { const uint32_t h = (uint32_t)(key >> 32); mn = min(mn, h); mx = max(mx, h); }
            }
        }
        mn = __reduce_min_sync(0xFFFFFFFFu, mn);
        mx = __reduce_max_sync(0xFFFFFFFFu, mx);
        if ((tid & 31) == 0) { atomicMin(&rng[0], mn); atomicMax(&rng[1], mx); }
        __syncthreads();
        float smin, inv;
        const uint32_t lo = rng[0], hi = rng[1];
        if (sel_range(lo, hi, smin, inv)) {
            for (uint32_t l = 0; l < L.lists(Q); ++l) {
                const uint32_t len = L.list_len(Q, l);
                for (uint32_t j = tid; j < len; j += nt) {
                    const uint64_t key = L.at(Q, l, j);
                    if (key) atomicAdd(&hist[sel_bucket((uint32_t)(key >> 32), smin, inv)], 1);
                }
            }
            __syncthreads();
            if (tid < 32) {
                // lane l owns buckets 255-8l .. 248-8l (descending)
                int c[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * tid - j]; tot += c[j]; }
                int incl = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if ((int)tid >= o) incl += y;
                }
                const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= (int)k);
                int bsel = -1, kept = 0;  // fewer than k present: everything stays
                if (ok) {
                    const int src = __ffs(ok) - 1;
                    if ((int)tid == src) {
                        int run = incl - tot;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (run + c[j] >= (int)k) { bsel = 255 - 8 * tid - j; kept = run + c[j]; break; }
                            run += c[j];
                        }
                    }
                    bsel = __shfl_sync(0xFFFFFFFFu, bsel, src);
                    kept = __shfl_sync(0xFFFFFFFFu, kept, src);
                } else {
                    kept = __shfl_sync(0xFFFFFFFFu, incl, 31);
                    bsel = 0;
                }
                if (tid == 0) { hist[256] = bsel; hist[257] = kept; }
            }
            __syncthreads();
            const int bsel = hist[256];
            const uint32_t kept = (uint32_t)hist[257];
            if (kept <= cap_s) {
                for (uint32_t l = 0; l < L.lists(Q); ++l) {
                    const uint32_t len = L.list_len(Q, l);
                    for (uint32_t j0 = 0; j0 < len; j0 += nt) {
                        const uint32_t j = j0 + tid;
                        const uint64_t key = j < len ? L.at(Q, l, j) : 0ull;
                        const bool keep = key != 0ull && sel_bucket((uint32_t)(key >> 32), smin, inv) >= bsel;
                        const unsigned bal = __ballot_sync(0xFFFFFFFFu, keep);
                        int base = 0;
                        if ((tid & 31) == 0 && bal) base = atomicAdd(n_s, __popc(bal));
                        base = __shfl_sync(0xFFFFFFFFu, base, 0);
                        if (keep) buf[base + __popc(bal & ((1u << (tid & 31)) - 1))] = key;
                    }
                }
                __syncthreads();
                const uint32_t present = (uint32_t)*n_s;
                __syncthreads();
                if (present > k) {
                    if (tid == 0) *pivot_s = 0ull;
                    __syncthreads();
                    if (block_select_multi(buf, cap_s, n_s, 1, k, 0u, (int)k, pivot_s, hist))
                        block_select_topk(buf, n_s, k, pivot_s, hist);
                }
                const uint32_t m = present < k ? present : k;
                for (uint32_t i = m + tid; i < kp2; i += nt) buf[i] = 0ull;
                __syncthreads();
                sort_and_emit(buf, cap_s, hist, kp2, m, k, Q, out_index, out_score, out_count);
                return;
            }
        }
        __syncthreads();
    }

    // last resort (scores piled up in one bucket, or non-finite): radix selection over the lists
    // number of present candidates
    if (tid == 0) hist[259] = 0;
    __syncthreads();
    int local = 0;
    for (uint32_t e = tid; e < T; e += nt) local += L.get(Q, e) != 0ull;
    for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xFFFFFFFFu, local, o);
    if ((tid & 31) == 0 && local) atomicAdd(&hist[259], local);
    __syncthreads();
    const uint32_t present = (uint32_t)hist[259];
    __syncthreads();

    uint64_t pivot = 1;  // every present candidate (>= 1) wins when present <= k
    if (present > k) {
        uint64_t prefix = 0;
        uint32_t need = k;
        int shift = 56;
        for (;; shift -= 8) {
            for (uint32_t b = tid; b < 256; b += nt) hist[b] = 0;
            __syncthreads();
            for (uint32_t e = tid; e < T; e += nt) {
                const uint64_t key = L.get(Q, e);
                if (key && (shift == 56 || (key >> (shift + 8)) == prefix))
                    atomicAdd(&hist[(key >> shift) & 255], 1);
            }
            __syncthreads();
            if (tid < 32) {
                int c[8], tot = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * tid - j]; tot += c[j]; }
                int incl = tot;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int y = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if ((int)tid >= o) incl += y;
                }
                const unsigned ok = __ballot_sync(0xFFFFFFFFu, incl >= (int)need);
                if ((int)tid == __ffs(ok) - 1) {
                    int run = incl - tot;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (run + c[j] >= (int)need) {
                            hist[256] = 255 - 8 * tid - j;
                            hist[257] = run;
                            hist[258] = c[j];
                            break;
                        }
                        run += c[j];
                    }
                }
            }
            __syncthreads();
            const int digit = hist[256], above = hist[257], binc = hist[258];
            __syncthreads();
            need -= (uint32_t)above;
            prefix = (prefix << 8) | (uint64_t)digit;
            if ((uint32_t)binc == need || shift == 0) break;
        }
        pivot = prefix << shift;
    }
    const uint32_t m = present < k ? present : k;

    // gather the winners, pad, sort descending
    if (tid == 0) hist[259] = 0;
    for (uint32_t i = tid; i < kp2; i += nt) buf[i] = 0ull;
    __syncthreads();
    for (uint32_t e = tid; e < T; e += nt) {
        const uint64_t key = L.get(Q, e);
        if (key >= pivot && key) buf[atomicAdd(&hist[259], 1)] = key;
    }
    __syncthreads();
    sort_and_emit(buf, cap_s, hist, kp2, m, k, Q, out_index, out_score, out_count);
}
template <typename Lists>
__global__ void __launch_bounds__(512) topk_merge_kernel(Lists L, uint32_t k, uint32_t kp2, uint32_t cap_s,
                                                         uint32_t* out_index, float* out_score,
                                                         uint32_t* out_count) {
    extern __shared__ __align__(16) unsigned char smem[];
    if (L.wait_ready(reinterpret_cast<int*>(smem))) {
        topk_merge_body(L, k, kp2, cap_s, out_index, out_score, out_count, smem);
    } else {
        for (uint32_t r = threadIdx.x; r < k; r += blockDim.x) {  // a list's owner did not answer: an empty row
            out_index[(size_t)blockIdx.x * k + r] = 0xFFFFFFFFu;
            out_score[(size_t)blockIdx.x * k + r] = -INFINITY;
        }
        if (out_count && threadIdx.x == 0) out_count[blockIdx.x] = 0;
    }
    __syncthreads();
    MPROBE(9);
    L.finish(blockIdx.x);
    MPROBE(10);
}

}  // namespace
}  // namespace slha
