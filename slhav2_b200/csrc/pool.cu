// Device-resident CCOS elastic tile pool: the ElasticKvCache of
// scirust/src/ccos.rs with its arena, per-slot state/seq/importance arrays,
// LIFO free list and logical byte counter all kept in HBM.  Every transition
// (insert, page_out, drop_correction, evict, enforce_budget, observe_scores)
// runs as kernels; the host only reads back a 64-byte counter block.
//
// enforce_budget reproduces the reference's four ordered phases
// (ccos.rs:555-614).  A phase sorts its candidates by the reference's key
// (cub::DeviceRadixSort on a unique 64-bit key), prefix-sums the bytes each
// candidate would free, and applies the operation to exactly the prefix the
// reference's sequential loop would have reached.
#include <cooperative_groups.h>
#include <cub/block/block_radix_sort.cuh>
#include <cub/block/block_scan.cuh>
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <vector>

#include "common.cuh"
#include "pool.cuh"

namespace slha {
namespace {

__device__ __forceinline__ uint32_t f32_total_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t corr_bytes(uint32_t flags) {  // tile.rs:118-126
    return (flags & F_TQ3) ? 16u : ((flags & F_MIX3) ? 14u : 0u);
}
__device__ __forceinline__ uint32_t live_bytes_of(uint8_t st, uint32_t flags) {  // ccos.rs:468-482
    if (st == ST_COLD) return 0;
    const uint32_t base = st == ST_HOT ? 128u : 96u;
    return base - ((flags & F_NOCORR) ? corr_bytes(flags) : 0u);
}
__device__ __forceinline__ uint32_t tile_flags(const unsigned char* tiles, uint64_t slot) {
    return *reinterpret_cast<const uint16_t*>(tiles + slot * TILE_BYTES + 118);
}

// ---- insert (ccos.rs:217-259) ------------------------------------------------
// Tile j of the batch takes free_list[free_len-1-j] while the free list lasts
// (LIFO pops), then fresh slots len, len+1, ...
__global__ void insert_kernel(PoolDev p, const unsigned char* src, uint64_t n, uint64_t pops,
                              uint64_t len0, uint64_t free0, uint64_t seq0, uint32_t* slots_out) {
    const uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t bytes = 0;
    if (j < n) {
        const uint32_t slot = j < pops ? p.free_list[free0 - 1 - j] : (uint32_t)(len0 + (j - pops));
        uint32_t flags = 0;
        if (src) flags = *reinterpret_cast<const uint16_t*>(src + j * TILE_BYTES + 118);
        const uint8_t st = (flags & F_WARM) ? ST_WARM : ST_HOT;
        p.state[slot] = st;
        p.seq[slot] = seq0 + j;
        p.importance[slot] = 0.0f;
        slots_out[j] = slot;
        bytes = live_bytes_of(st, flags);
    }
    for (int o = 16; o; o >>= 1) bytes += __shfl_xor_sync(0xFFFFFFFFu, bytes, o);
    if ((threadIdx.x & 31) == 0 && bytes) atomicAdd((unsigned long long*)&p.cnt->live, (unsigned long long)bytes);
    if (j == 0) {
        p.cnt->free_len = free0 - pops;
        p.cnt->len = len0 + (n - pops);
        p.cnt->next_seq = seq0 + n;
    }
}
__global__ void scatter_tiles_kernel(unsigned char* tiles, const unsigned char* src,
                                     const uint32_t* slots, uint64_t n) {
    const uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e < n * 8) {
        const uint64_t j = e >> 3, c = e & 7;
        reinterpret_cast<uint4*>(tiles + (uint64_t)slots[j] * TILE_BYTES)[c] =
            reinterpret_cast<const uint4*>(src + j * TILE_BYTES)[c];
    }
}

// ---- single-slot transitions ---------------------------------------------------
__device__ bool do_page_out(const PoolDev& p, uint32_t slot, int64_t* delta) {  // ccos.rs:365-380
    if (p.state[slot] != ST_HOT) return false;
    unsigned char* t = p.tiles + (uint64_t)slot * TILE_BYTES;
    uint4 z = make_uint4(0, 0, 0, 0);
    reinterpret_cast<uint4*>(t + 64)[0] = z;
    reinterpret_cast<uint4*>(t + 64)[1] = z;
    *reinterpret_cast<float*>(t + 100) = 0.0f;
    *reinterpret_cast<uint16_t*>(t + 118) |= F_WARM;
    p.state[slot] = ST_WARM;
    *delta -= 32;
    return true;
}
__device__ bool do_drop_correction(const PoolDev& p, uint32_t slot, int64_t* delta) {  // ccos.rs:386-397
    unsigned char* t = p.tiles + (uint64_t)slot * TILE_BYTES;
    const uint32_t flags = *reinterpret_cast<uint16_t*>(t + 118);
    const uint32_t nb = corr_bytes(flags);
    if (p.state[slot] == ST_COLD || nb == 0 || (flags & F_NOCORR)) return false;
    for (uint32_t b = 64 - nb; b < 64; ++b) t[b] = 0;
    *reinterpret_cast<uint16_t*>(t + 118) = (uint16_t)(flags | F_NOCORR);
    *delta -= (int64_t)nb;
    return true;
}
__global__ void single_op_kernel(PoolDev p, int op, uint32_t slot, int32_t* result) {
    int64_t delta = 0;
    bool done = false;
    if (slot < p.cnt->len) {
        if (op == 0) done = do_page_out(p, slot, &delta);
        else if (op == 1) done = do_drop_correction(p, slot, &delta);
        else if (p.state[slot] != ST_COLD) {  // evict, ccos.rs:404-438 (no event log)
            delta = -(int64_t)live_bytes_of(p.state[slot], tile_flags(p.tiles, slot));
            p.state[slot] = ST_COLD;
            p.free_list[p.cnt->free_len++] = slot;
            done = true;
        }
    }
    p.cnt->live = (uint64_t)((int64_t)p.cnt->live + delta);
    *result = done ? 1 : 0;
}

// ---- enforce_budget phases -------------------------------------------------------
enum Phase { PH_CORR_HOT = 0, PH_PAGE = 1, PH_CORR_WARM = 2, PH_EVICT = 3, PH_EVICT_PINNED = 4 };
constexpr uint64_t SENTINEL = ~0ull;

// max live position (for the recent-window extension)
__global__ void max_pos_kernel(PoolDev p) {
    const uint64_t len = p.cnt->len;
    uint32_t m = 0;
    for (uint64_t s = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; s < len; s += (uint64_t)gridDim.x * blockDim.x)
        if (p.state[s] != ST_COLD) m = max(m, *reinterpret_cast<const uint32_t*>(p.tiles + s * TILE_BYTES + 112));
    for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(&p.cnt->max_pos, m);
}

__device__ __forceinline__ bool is_pinned(const PoolDev& p, uint32_t pos, uint32_t max_pos) {
    if (pos < p.sink_window) return true;  // ccos.rs:592-594
    return p.recent_window && (max_pos - pos) < p.recent_window;
}

// the sort key of slot s in `phase`, or SENTINEL when the phase cannot act on it
__device__ __forceinline__ uint64_t phase_key(const PoolDev& p, int phase, uint64_t s, uint32_t max_pos) {
    const uint8_t st = p.state[s];
    if (st == ST_COLD) return SENTINEL;
    const unsigned char* t = p.tiles + s * TILE_BYTES;
    const uint32_t flags = *reinterpret_cast<const uint16_t*>(t + 118);
    bool cand = false;
    if (phase == PH_CORR_HOT) cand = st == ST_HOT && corr_bytes(flags) && !(flags & F_NOCORR);
    else if (phase == PH_PAGE) cand = st == ST_HOT;
    else if (phase == PH_CORR_WARM) cand = st == ST_WARM && corr_bytes(flags) && !(flags & F_NOCORR);
    else {
        const bool pin = p.evict_policy == SLHA_B200_EVICT_IMPORTANCE &&
                         is_pinned(p, *reinterpret_cast<const uint32_t*>(t + 112), max_pos);
        cand = (phase == PH_EVICT_PINNED) == pin;
    }
    if (!cand) return SENTINEL;
    const uint32_t seq32 = (uint32_t)p.seq[s];
    if (phase <= PH_CORR_WARM) {
        // slots_in_paging_order, ccos.rs:526-539: stable sort of the
        // slot-ascending list by sigma (total order) or by seq
        return p.page_policy == SLHA_B200_PAGE_LOWEST_IMPACT_FIRST
                   ? ((uint64_t)f32_total_key(*reinterpret_cast<const float*>(t + 104)) << 32) | (uint32_t)s
                   : (uint64_t)seq32;
    }
    // ccos.rs:586-603: causal = by seq; importance = (importance, seq)
    return p.evict_policy == SLHA_B200_EVICT_CAUSAL ? (uint64_t)seq32 : ((uint64_t)f32_total_key(p.importance[s]) << 32) | seq32;
}

// candidate (key, slot) pairs of one phase, compacted in arbitrary order (keys are unique, so the
// sort that follows gives one order): only the slots a phase can act on are sorted, e.g. the few
// HOT tiles just appended for the page-out phase.  n_cand is zero when the kernel starts.
__global__ void phase_build_kernel(PoolDev p, int phase, uint64_t* keys, uint32_t* vals) {
    const uint64_t len = p.cnt->len;
    const bool over = p.cnt->live > p.cnt->budget;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.cnt->phase_deficit = over ? p.cnt->live - p.cnt->budget : 0;
        p.cnt->phase_applied = 0;
    }
    const uint32_t max_pos = p.cnt->max_pos;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t rounds = over ? (len + stride - 1) / stride : 0;  // whole warps stay together for the ballot
    for (uint64_t r = 0; r < rounds; ++r) {
        const uint64_t s = r * stride + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
        uint64_t key = SENTINEL;
        if (s < len) key = phase_key(p, phase, s, max_pos);
        const unsigned hit = __ballot_sync(0xFFFFFFFFu, key != SENTINEL);
        if (hit) {
            const int lane = threadIdx.x & 31;
            uint32_t base = 0;
            if (lane == 0) base = atomicAdd(&p.cnt->n_cand, (uint32_t)__popc(hit));
            base = __shfl_sync(0xFFFFFFFFu, base, 0);
            if (key != SENTINEL) {
                const uint32_t i = base + (uint32_t)__popc(hit & ((1u << lane) - 1u));
                keys[i] = key;
                vals[i] = (uint32_t)s;
            }
        }
    }
}

// Pre-filter of a long candidate list: a phase stops once the bytes it has freed reach the deficit,
// and every operation of a phase frees at least `min_freed` bytes (14 for a dropped correction
// plane, 32 for a page-out, 80 for an eviction), so only the M = deficit / min_freed + 1 smallest
// keys can be reached.  A histogram over the keys' 12 high bits gives the smallest bin prefix that
// holds M candidates; only those candidates are sorted.
constexpr uint32_t PREFILTER_BINS = 4096, PREFILTER_MIN = 65536;
__global__ void phase_hist_kernel(PoolDev p, const uint64_t* keys, uint32_t* hist) {
    __shared__ uint32_t h[PREFILTER_BINS];
    for (uint32_t b = threadIdx.x; b < PREFILTER_BINS; b += blockDim.x) h[b] = 0;
    __syncthreads();
    const uint64_t n = p.cnt->n_cand;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        atomicAdd(&h[(uint32_t)(keys[i] >> 52)], 1u);
    __syncthreads();
    for (uint32_t b = threadIdx.x; b < PREFILTER_BINS; b += blockDim.x)
        if (h[b]) atomicAdd(&hist[b], h[b]);
}
// keeps the candidates whose bin is at most `last_bin`; n_cand becomes their number (out_n, then copied)
__global__ void phase_filter_kernel(PoolDev p, const uint64_t* keys, const uint32_t* vals, uint32_t last_bin,
                                    uint64_t* keys_out, uint32_t* vals_out, uint32_t* out_n) {
    const uint64_t n = p.cnt->n_cand;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t rounds = (n + stride - 1) / stride;
    for (uint64_t r = 0; r < rounds; ++r) {
        const uint64_t i = r * stride + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
        const bool keep = i < n && (uint32_t)(keys[i] >> 52) <= last_bin;
        const unsigned hit = __ballot_sync(0xFFFFFFFFu, keep);
        if (hit) {
            const int lane = threadIdx.x & 31;
            uint32_t base = 0;
            if (lane == 0) base = atomicAdd(out_n, (uint32_t)__popc(hit));
            base = __shfl_sync(0xFFFFFFFFu, base, 0);
            if (keep) {
                const uint32_t o = base + (uint32_t)__popc(hit & ((1u << lane) - 1u));
                keys_out[o] = keys[i];
                vals_out[o] = vals[i];
            }
        }
    }
}
__global__ void phase_set_ncand_kernel(PoolDev p, const uint32_t* n) { p.cnt->n_cand = *n; }

__global__ void phase_weights_kernel(PoolDev p, int phase, const uint64_t* keys_sorted,
                                     const uint32_t* slots_sorted, uint32_t* w) {
    const uint64_t len = p.cnt->n_cand;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t bytes = 0;
        if (keys_sorted[i] != SENTINEL) {
            const uint32_t s = slots_sorted[i];
            const uint32_t flags = tile_flags(p.tiles, s);
            if (phase == PH_PAGE) bytes = 32;
            else if (phase <= PH_CORR_WARM) bytes = corr_bytes(flags);
            else bytes = live_bytes_of(p.state[s], flags);
        }
        w[i] = bytes;
    }
}

// Apply the phase operation to the sorted prefix whose exclusive byte prefix is
// below the deficit: exactly the items the reference's `for s in order { if
// live <= budget {return}; op(s) }` loop reaches.
__global__ void phase_apply_kernel(PoolDev p, int phase, const uint64_t* keys_sorted,
                                   const uint32_t* slots_sorted, const uint32_t* w,
                                   const uint64_t* excl, uint64_t limit) {
    const uint64_t len = p.cnt->n_cand;
    const uint64_t deficit = p.cnt->phase_deficit;
    const uint64_t free0 = p.cnt->free_len;
    int64_t delta = 0;
    uint32_t applied = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (uint64_t)gridDim.x * blockDim.x) {
        if (keys_sorted[i] == SENTINEL || deficit == 0 || excl[i] >= deficit || i >= limit) continue;
        const uint32_t s = slots_sorted[i];
        if (phase == PH_PAGE) do_page_out(p, s, &delta);
        else if (phase <= PH_CORR_WARM) do_drop_correction(p, s, &delta);
        else {
            delta -= (int64_t)w[i];
            p.state[s] = ST_COLD;
            p.free_list[free0 + i] = s;  // pushes happen in sorted order (applied items are a prefix)
            ++applied;
        }
    }
    for (int o = 16; o; o >>= 1) {
        delta += __shfl_xor_sync(0xFFFFFFFFu, delta, o);
        applied += __shfl_xor_sync(0xFFFFFFFFu, applied, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (delta) atomicAdd((unsigned long long*)&p.cnt->live_delta, (unsigned long long)delta);
        if (applied) atomicAdd((unsigned long long*)&p.cnt->phase_applied, (unsigned long long)applied);
    }
}
// With an event log attached: (seq, slot, tile) of the slots an eviction phase is about to turn COLD,
// in eviction order (the applied items are a prefix of the sorted candidates), for the host to append.
__global__ void phase_journal_kernel(PoolDev p, const uint64_t* keys_sorted, const uint32_t* slots_sorted, const uint64_t* excl,
                                     unsigned long long* count, uint64_t* seq_out, uint32_t* slot_out, uint4* tiles_out) {
    const uint64_t len = p.cnt->n_cand, deficit = p.cnt->phase_deficit;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (uint64_t)gridDim.x * blockDim.x) {
        if (keys_sorted[i] == SENTINEL || deficit == 0 || excl[i] >= deficit) continue;
        const uint32_t s = slots_sorted[i];
        seq_out[i] = p.seq[s];
        slot_out[i] = s;
        const uint4* src = reinterpret_cast<const uint4*>(p.tiles + (size_t)s * TILE_BYTES);
        for (int j = 0; j < 8; ++j) tiles_out[i * 8 + j] = src[j];
        atomicMax(count, (unsigned long long)(i + 1));
    }
}
__global__ void phase_commit_kernel(PoolDev p) {
    p.cnt->live = (uint64_t)((int64_t)p.cnt->live + (int64_t)p.cnt->live_delta);
    p.cnt->live_delta = 0;
    p.cnt->free_len += p.cnt->phase_applied;
    p.cnt->phase_applied = 0;
}

// ---- enforce_budget in one cooperative launch --------------------------------------
// The host-driven phases above need the candidate count (for the sort) and the prefilter cut on the
// host, one stream round trip each.  When no event log is attached nothing of a phase needs the
// host: this kernel runs every phase with grid-wide barriers in between.  Per phase
//   build    candidates (key, slot) compacted as above, with the smallest and largest key;
//   select   when there are more than EB_CAP candidates, a radix select (12 key bits per level,
//            starting at the highest bit in which the keys differ) finds a key bound below which at
//            least `reach` = deficit / min_freed + 1 and at most EB_CAP candidates lie -- no more
//            than `reach` can be reached before the deficit is covered;
//   finish   one block sorts those (cub::BlockRadixSort), prefix-sums the bytes each would free and
//            applies the operation to exactly the prefix the reference's loop reaches.
// A phase the select cannot bound (a deficit worth more than EB_CAP operations) raises `overflow`
// and ends the kernel; the phases already finished are complete, and the host-driven path then
// continues from the state they left (a finished phase has no candidates left or met the budget).
constexpr int EB_THREADS = 512, EB_ITEMS = 8, EB_CAP = EB_THREADS * EB_ITEMS, EB_LEVELS = 6, EB_BINS = 4096;
struct EnforceState {
    unsigned long long inv_min_key, max_key;  // ~min and max over the phase's candidates (zero = none yet)
    uint32_t n_keep, overflow, pad[2];
    uint32_t hist[5][EB_LEVELS][EB_BINS];
};

__global__ void __launch_bounds__(EB_THREADS) enforce_kernel(PoolDev p, uint32_t phase_mask, uint64_t* keys, uint32_t* vals,
                                                             uint64_t* skeys, uint32_t* svals, EnforceState* es) {
    namespace cg = cooperative_groups;
    cg::grid_group grid = cg::this_grid();
    using Sort = cub::BlockRadixSort<uint64_t, EB_THREADS, EB_ITEMS, uint32_t>;
    using Scan64 = cub::BlockScan<uint64_t, EB_THREADS>;
    using Scan32 = cub::BlockScan<uint32_t, EB_THREADS>;
    __shared__ union {
        typename Sort::TempStorage sort;
        typename Scan64::TempStorage scan64;
        typename Scan32::TempStorage scan32;
        uint32_t hist[EB_BINS];
    } sm;
    __shared__ uint32_t cut_bin, cut_hist;
    __shared__ unsigned long long cut_cum, fin_applied;
    __shared__ long long fin_delta;
    volatile PoolCounters* cnt = p.cnt;
    const uint64_t len = cnt->len;
    const uint64_t gtid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (uint64_t)gridDim.x * blockDim.x;
    const int lane = threadIdx.x & 31;
    if (cnt->live <= cnt->budget) return;  // (nothing has been written yet: every block sees the same)
    if (p.recent_window) {
        uint32_t m = 0;
        for (uint64_t s = gtid; s < len; s += stride)
            if (p.state[s] != ST_COLD) m = max(m, *reinterpret_cast<const uint32_t*>(p.tiles + s * TILE_BYTES + 112));
        for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        if (lane == 0 && m) atomicMax(&p.cnt->max_pos, m);
        grid.sync();
    }
    const uint32_t max_pos = cnt->max_pos;
    for (int phase = 0; phase < 5; ++phase) {
        if (!((phase_mask >> phase) & 1u)) continue;
        const uint64_t live = cnt->live, budget = cnt->budget;
        if (live <= budget) break;
        const uint64_t deficit = live - budget;
        // ---- build
        {
            uint64_t kmin = SENTINEL, kmax = 0;
            const uint64_t rounds = (len + stride - 1) / stride;
            for (uint64_t r = 0; r < rounds; ++r) {
                const uint64_t s = r * stride + gtid;
                uint64_t key = SENTINEL;
                if (s < len) key = phase_key(p, phase, s, max_pos);
                const unsigned hit = __ballot_sync(0xFFFFFFFFu, key != SENTINEL);
                if (hit) {
                    uint32_t base = 0;
                    if (lane == 0) base = atomicAdd(&p.cnt->n_cand, (uint32_t)__popc(hit));
                    base = __shfl_sync(0xFFFFFFFFu, base, 0);
                    if (key != SENTINEL) {
                        const uint32_t i = base + (uint32_t)__popc(hit & ((1u << lane) - 1u));
                        keys[i] = key;
                        vals[i] = (uint32_t)s;
                        kmin = min(kmin, key);
                        kmax = max(kmax, key);
                    }
                }
            }
            for (int o = 16; o; o >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(0xFFFFFFFFu, kmin, o));
                kmax = max(kmax, __shfl_xor_sync(0xFFFFFFFFu, kmax, o));
            }
            if (lane == 0 && kmin != SENTINEL) {
                atomicMax(&es->inv_min_key, ~kmin);
                atomicMax(&es->max_key, kmax);
            }
        }
        grid.sync();
        const uint64_t nc = cnt->n_cand;
        if (nc) {
            const uint64_t min_freed = phase == PH_PAGE ? 32 : (phase >= PH_EVICT ? 80 : 14);
            const uint64_t reach = deficit / min_freed + 1;
            const bool take_all = nc <= (uint64_t)EB_CAP;
            uint64_t base = ~*(volatile unsigned long long*)&es->inv_min_key, thr_rel = ~0ull, below = 0;
            bool bounded = take_all;
            if (!take_all && reach <= (uint64_t)EB_CAP) {
                const uint64_t span = *(volatile unsigned long long*)&es->max_key - base;
                int shift = max(0, 64 - __clzll((long long)span) - 12);
                for (int level = 0; level < EB_LEVELS && !bounded; ++level) {
                    uint32_t* ghist = es->hist[phase][level];
                    for (uint32_t b = threadIdx.x; b < EB_BINS; b += EB_THREADS) sm.hist[b] = 0;
                    __syncthreads();
                    for (uint64_t i = gtid; i < nc; i += stride) {
                        const uint64_t k = keys[i];
                        if (k >= base && ((k - base) >> shift) < (uint64_t)EB_BINS) atomicAdd(&sm.hist[(uint32_t)((k - base) >> shift)], 1u);
                    }
                    __syncthreads();
                    for (uint32_t b = threadIdx.x; b < EB_BINS; b += EB_THREADS)
                        if (sm.hist[b]) atomicAdd(&ghist[b], sm.hist[b]);
                    grid.sync();
                    // every block finds the cut itself: the first bin at which `below` + the running count reaches `reach`
                    uint32_t h[EB_ITEMS], mine = 0;
                    for (int j = 0; j < EB_ITEMS; ++j) {
                        h[j] = *(volatile uint32_t*)&ghist[threadIdx.x * EB_ITEMS + j];
                        mine += h[j];
                    }
                    if (threadIdx.x == 0) cut_bin = 0xFFFFFFFFu;
                    __syncthreads();
                    uint32_t before;
                    Scan32(sm.scan32).ExclusiveSum(mine, before);
                    uint64_t cum = below + before;
                    if (cum < reach && cum + mine >= reach) {
                        for (int j = 0; j < EB_ITEMS; ++j) {
                            cum += h[j];
                            if (cum >= reach) {
                                cut_bin = threadIdx.x * EB_ITEMS + j;
                                cut_hist = h[j];
                                cut_cum = cum;
                                break;
                            }
                        }
                    }
                    __syncthreads();
                    const uint32_t b = cut_bin;
                    const uint64_t kept = cut_cum;
                    const uint32_t hb = cut_hist;
                    __syncthreads();
                    if (b == 0xFFFFFFFFu) break;  // fewer candidates than `reach`: all of them are needed, and they do not fit
                    if (kept <= (uint64_t)EB_CAP) {
                        thr_rel = (((uint64_t)b + 1) << shift) - 1;
                        bounded = true;
                    } else if (shift == 0) {
                        break;  // equal keys beyond the block sort's capacity
                    } else {
                        below = kept - hb;
                        base += (uint64_t)b << shift;
                        shift = max(0, shift - 12);
                    }
                }
            }
            if (!bounded) {
                if (gtid == 0) es->overflow = 1;
                return;  // every block takes this branch
            }
            if (!take_all) {
                const uint64_t rounds = (nc + stride - 1) / stride;
                for (uint64_t r = 0; r < rounds; ++r) {
                    const uint64_t i = r * stride + gtid;
                    uint64_t k = 0;
                    bool keep = false;
                    if (i < nc) {
                        k = keys[i];
                        keep = k < base || (k - base) <= thr_rel;
                    }
                    const unsigned hit = __ballot_sync(0xFFFFFFFFu, keep);
                    if (hit) {
                        uint32_t o = 0;
                        if (lane == 0) o = atomicAdd(&es->n_keep, (uint32_t)__popc(hit));
                        o = __shfl_sync(0xFFFFFFFFu, o, 0) + (uint32_t)__popc(hit & ((1u << lane) - 1u));
                        if (keep && o < (uint32_t)EB_CAP) {
                            skeys[o] = k;
                            svals[o] = vals[i];
                        }
                    }
                }
                grid.sync();
            }
            // ---- finish (block 0)
            if (blockIdx.x == 0) {
                const uint64_t* ks = take_all ? keys : skeys;
                const uint32_t* vs = take_all ? vals : svals;
                const uint32_t n = take_all ? (uint32_t)nc : min(*(volatile uint32_t*)&es->n_keep, (uint32_t)EB_CAP);
                uint64_t k[EB_ITEMS];
                uint32_t v[EB_ITEMS];
                for (int j = 0; j < EB_ITEMS; ++j) {
                    const uint32_t i = threadIdx.x * EB_ITEMS + j;
                    k[j] = i < n ? ks[i] : SENTINEL;
                    v[j] = i < n ? vs[i] : 0u;
                }
                if (threadIdx.x == 0) {
                    fin_applied = 0;
                    fin_delta = 0;
                }
                __syncthreads();
                Sort(sm.sort).Sort(k, v);
                __syncthreads();
                uint64_t w[EB_ITEMS], excl[EB_ITEMS];
                for (int j = 0; j < EB_ITEMS; ++j) {
                    uint32_t bytes = 0;
                    if (k[j] != SENTINEL) {
                        const uint32_t flags = tile_flags(p.tiles, v[j]);
                        if (phase == PH_PAGE) bytes = 32;
                        else if (phase <= PH_CORR_WARM) bytes = corr_bytes(flags);
                        else bytes = live_bytes_of(p.state[v[j]], flags);
                    }
                    w[j] = bytes;
                }
                Scan64(sm.scan64).ExclusiveSum(w, excl);
                const uint64_t free0 = cnt->free_len;
                int64_t delta = 0;
                uint32_t applied = 0;
                for (int j = 0; j < EB_ITEMS; ++j) {
                    if (k[j] == SENTINEL || excl[j] >= deficit) continue;
                    const uint32_t s = v[j];
                    if (phase == PH_PAGE) do_page_out(p, s, &delta);
                    else if (phase <= PH_CORR_WARM) do_drop_correction(p, s, &delta);
                    else {
                        delta -= (int64_t)w[j];
                        p.state[s] = ST_COLD;
                        p.free_list[free0 + threadIdx.x * EB_ITEMS + j] = s;  // applied items are a prefix of the sorted order
                        ++applied;
                    }
                }
                for (int o = 16; o; o >>= 1) {
                    delta += __shfl_xor_sync(0xFFFFFFFFu, delta, o);
                    applied += __shfl_xor_sync(0xFFFFFFFFu, applied, o);
                }
                if (lane == 0) {
                    if (delta) atomicAdd((unsigned long long*)&fin_delta, (unsigned long long)delta);
                    if (applied) atomicAdd(&fin_applied, (unsigned long long)applied);
                }
                __syncthreads();
                if (threadIdx.x == 0) {
                    cnt->live = (uint64_t)((int64_t)live + fin_delta);
                    cnt->free_len = free0 + fin_applied;
                    cnt->n_cand = 0;
                    es->inv_min_key = 0;
                    es->max_key = 0;
                    es->n_keep = 0;
                    __threadfence();
                }
            }
        }
        grid.sync();
    }
}

// ---- observe_scores (ccos.rs:275-314) -----------------------------------------
struct ObserveTmp {
    uint32_t max_key;   // order-preserving key of the max live score
    uint32_t bad;       // a live score is non-finite
    uint32_t live;      // number of live entries
    uint32_t pad;
    float sum;
};
__global__ void observe_pass1(PoolDev p, const uint32_t* slots, const float* scores, uint64_t n, ObserveTmp* tmp) {
    const uint64_t len = p.cnt->len;
    uint32_t mk = 0, bad = 0, live = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t s = slots ? slots[i] : (uint32_t)i;
        if (s < len && p.state[s] != ST_COLD) {
            const float v = scores[i];
            ++live;
            if (!isfinite(v)) bad = 1;
            mk = max(mk, f32_total_key(v));
        }
    }
    for (int o = 16; o; o >>= 1) {
        mk = max(mk, __shfl_xor_sync(0xFFFFFFFFu, mk, o));
        bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
        live += __shfl_xor_sync(0xFFFFFFFFu, live, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(&tmp->max_key, mk);
        if (bad) atomicOr(&tmp->bad, 1u);
        if (live) atomicAdd(&tmp->live, live);
    }
}
__device__ __forceinline__ float key_to_f32(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
// per-CTA partial sums of exp((s-m)/T) in a fixed order (deterministic)
__global__ void observe_pass2(PoolDev p, const uint32_t* slots, const float* scores, uint64_t n,
                              float temperature, const ObserveTmp* tmp, float* partial) {
    __shared__ float red[32];
    const uint64_t len = p.cnt->len;
    const float m = key_to_f32(tmp->max_key);
    float acc = 0.0f;
    if (!tmp->bad && tmp->live) {
        const uint64_t per = (n + gridDim.x - 1) / gridDim.x;
        const uint64_t lo = (uint64_t)blockIdx.x * per, hi = min(n, lo + per);
        for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const uint32_t s = slots ? slots[i] : (uint32_t)i;
            if (s < len && p.state[s] != ST_COLD) acc += expf((scores[i] - m) / temperature);
        }
    }
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}
__global__ void observe_pass3(PoolDev p, const uint32_t* slots, const float* scores, uint64_t n,
                              float temperature, ObserveTmp* tmp, const float* partial, int n_partial) {
    __shared__ float s_inv;
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (int i = 0; i < n_partial; ++i) sum += partial[i];
        s_inv = (tmp->bad || !tmp->live || !isfinite(sum) || sum <= 0.0f) ? 0.0f : 1.0f / sum;
    }
    __syncthreads();
    const float inv = s_inv;
    if (inv == 0.0f) return;
    const uint64_t len = p.cnt->len;
    const float m = key_to_f32(tmp->max_key);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t s = slots ? slots[i] : (uint32_t)i;
        if (s < len && p.state[s] != ST_COLD) atomicAdd(&p.importance[s], expf((scores[i] - m) / temperature) * inv);
    }
}

// ---- stats / compaction ---------------------------------------------------------
__global__ void stats_kernel(PoolDev p, unsigned long long* out) {
    const uint64_t len = p.cnt->len;
    unsigned long long h = 0, w = 0, c = 0, nc = 0, rec = 0;
    for (uint64_t s = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; s < len; s += (uint64_t)gridDim.x * blockDim.x) {
        const uint8_t st = p.state[s];
        if (st == ST_HOT) ++h; else if (st == ST_WARM) ++w; else ++c;
        const uint32_t flags = tile_flags(p.tiles, s);
        if (st != ST_COLD && (flags & F_NOCORR)) { ++nc; rec += corr_bytes(flags); }
    }
    for (int o = 16; o; o >>= 1) {
        h += __shfl_xor_sync(0xFFFFFFFFu, h, o); w += __shfl_xor_sync(0xFFFFFFFFu, w, o);
        c += __shfl_xor_sync(0xFFFFFFFFu, c, o); nc += __shfl_xor_sync(0xFFFFFFFFu, nc, o);
        rec += __shfl_xor_sync(0xFFFFFFFFu, rec, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&out[2], h); atomicAdd(&out[3], w); atomicAdd(&out[4], c);
        atomicAdd(&out[5], nc); atomicAdd(&out[6], rec);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        out[0] = p.cnt->len; out[1] = p.cnt->live; out[7] = p.cnt->free_len;
    }
}
// ordered compaction of the non-COLD (slot, score) pairs; one CTA
__global__ void compact_live_kernel(PoolDev p, const float* scores, uint32_t* slots_out,
                                    float* scores_out, unsigned long long* n_out) {
    __shared__ uint32_t warp_tot[32];
    __shared__ uint32_t base_s;
    const uint64_t len = p.cnt->len;
    if (threadIdx.x == 0) base_s = 0;
    __syncthreads();
    for (uint64_t b = 0; b < len; b += blockDim.x) {
        const uint64_t s = b + threadIdx.x;
        const bool live = s < len && p.state[s] != ST_COLD;
        const unsigned bal = __ballot_sync(0xFFFFFFFFu, live);
        const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
        if (lane == 0) warp_tot[wp] = __popc(bal);
        __syncthreads();
        uint32_t off = base_s;
        for (int w = 0; w < wp; ++w) off += warp_tot[w];
        if (live) {
            const uint32_t o = off + __popc(bal & ((1u << lane) - 1));
            slots_out[o] = (uint32_t)s;
            scores_out[o] = scores[s];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t t = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += warp_tot[w];
            base_s += t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_out = base_s;
}

inline uint32_t grid_for(uint64_t n, int threads = 256) {
    return (uint32_t)std::min<uint64_t>(std::max<uint64_t>(1, (n + threads - 1) / threads), 148 * 8);
}

}  // namespace

Status pool_sync_counters(Ctx* c, Pool* pl) {
    SLHA_CUDA(cudaMemcpyAsync(&pl->h_cnt, pl->dev.cnt, sizeof(PoolCounters), cudaMemcpyDeviceToHost, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    return Status();
}

Status pool_create(Ctx* c, const SlhaB200PoolConfig& cfg, Pool** out) {
    auto* pl = new Pool();
    pl->cfg = cfg;
    pl->device = c->device;
    const uint64_t cap = cfg.capacity_tiles;
    PoolDev& d = pl->dev;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) { if (e == cudaSuccess) e = cudaMalloc(p, std::max<size_t>(bytes, 256)); };
    alloc((void**)&d.tiles, cap * TILE_BYTES);
    alloc((void**)&d.state, cap);
    alloc((void**)&d.seq, cap * 8);
    alloc((void**)&d.importance, cap * 4);
    alloc((void**)&d.free_list, cap * 4);
    alloc((void**)&d.cnt, sizeof(PoolCounters));
    if (e != cudaSuccess) {
        pool_destroy(pl);
        return cuda_status(e, "cudaMalloc(pool)");
    }
    d.page_policy = cfg.page_policy;
    d.evict_policy = cfg.evict_policy;
    d.sink_window = cfg.sink_window;
    d.recent_window = cfg.recent_window;
    PoolCounters z{};
    z.budget = cfg.budget_bytes;
    pl->h_cnt = z;
    SLHA_CUDA(cudaMemcpyAsync(d.cnt, &pl->h_cnt, sizeof(z), cudaMemcpyHostToDevice, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    *out = pl;
    return Status();
}

void pool_destroy(Pool* pl) {
    if (!pl) return;
    cudaFree(pl->dev.tiles);
    cudaFree(pl->dev.state);
    cudaFree(pl->dev.seq);
    cudaFree(pl->dev.importance);
    cudaFree(pl->dev.free_list);
    cudaFree(pl->dev.cnt);
    cudaFree(pl->d_observe);
    if (pl->log) eventlog_close(pl->log);
    delete pl;
}

// Reserve slots for n tiles (bookkeeping only); d_slots receives the slot ids.
Status pool_reserve(Ctx* c, Pool* pl, const unsigned char* d_src_tiles, uint64_t n, uint32_t* d_slots) {
    PoolCounters& h = pl->h_cnt;
    if (h.next_seq + n > 0xFFFFFFFFull)
        return Status(SLHA_ERR_CAPACITY, "pool: insertion counter exhausted (2^32 inserts)");
    const uint64_t pops = std::min<uint64_t>(n, h.free_len);
    if (h.len + (n - pops) > pl->cfg.capacity_tiles)
        return Status(SLHA_ERR_CAPACITY, "pool: capacity_tiles exceeded");
    insert_kernel<<<(uint32_t)((n + 255) / 256), 256, 0, c->stream>>>(pl->dev, d_src_tiles, n, pops, h.len,
                                                                      h.free_len, h.next_seq, d_slots);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    h.free_len -= pops;
    h.len += n - pops;
    h.next_seq += n;
    return Status();
}

Status pool_scatter(Ctx* c, Pool* pl, const unsigned char* d_src_tiles, const uint32_t* d_slots, uint64_t n) {
    scatter_tiles_kernel<<<(uint32_t)((n * 8 + 255) / 256), 256, 0, c->stream>>>(pl->dev.tiles, d_src_tiles, d_slots, n);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

Status pool_single_op(Ctx* c, Pool* pl, int op, uint32_t slot, int32_t* result) {
    if (op == 2 && (pl->log || pl->require_durable)) {
        // evict with an event log attached (ccos.rs:404-438): persist the record, then (and only then) go COLD
        SLHA_TRY(pool_sync_counters(c, pl));
        uint8_t st = ST_COLD;
        if (slot < pl->h_cnt.len) SLHA_CUDA(cudaMemcpyAsync(&st, pl->dev.state + slot, 1, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        if (st == ST_COLD) {
            *result = 0;
            return Status();
        }
        uint64_t seq = 0;
        unsigned char tile[TILE_BYTES];
        SLHA_CUDA(cudaMemcpyAsync(&seq, pl->dev.seq + slot, 8, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaMemcpyAsync(tile, pl->dev.tiles + (size_t)slot * TILE_BYTES, TILE_BYTES, cudaMemcpyDeviceToHost, c->stream));
        SLHA_CUDA(cudaStreamSynchronize(c->stream));
        const bool ok = pl->log && eventlog_append(pl->log, seq, slot, tile, pl->require_durable).ok();
        if (!ok) {
            if (pl->log) ++pl->log_errors;
            if (pl->require_durable) {
                ++pl->blocked_evictions;
                *result = 0;
                return Status();
            }
        }
    }
    int32_t* d_res;
    SLHA_TRY(ctx_device_scratch(c, 256, (void**)&d_res));
    single_op_kernel<<<1, 1, 0, c->stream>>>(pl->dev, op, slot, d_res);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    SLHA_CUDA(cudaMemcpyAsync(result, d_res, 4, cudaMemcpyDeviceToHost, c->stream));
    return pool_sync_counters(c, pl);
}

// One cooperative launch for all phases, one read-back of the counters.  Sets *done when the
// budget question is settled; leaves it clear when a phase needs the host-driven path.
static Status pool_enforce_budget_fused(Ctx* c, Pool* pl, int32_t* within, bool* done) {
    *done = false;
    static int blocks_per_sm[64] = {0}, sms[64] = {0};
    const int dev = pl->device & 63;
    if (!blocks_per_sm[dev]) {
        int coop = 0, n = 0, b = 0;
        SLHA_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, pl->device));
        SLHA_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, pl->device));
        SLHA_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, enforce_kernel, EB_THREADS, 0));
        sms[dev] = n;
        blocks_per_sm[dev] = coop && b > 0 ? std::min(b, 2) : -1;
    }
    if (blocks_per_sm[dev] < 0) return Status();
    const uint64_t len = pl->h_cnt.len;  // (the host mirror of len is exact: only inserts move it)
    if (len == 0) return Status();
    Scratch sc{c};
    SLHA_TRY(sc.reserve(pad256(len * 8) + pad256(len * 4) + pad256(EB_CAP * 8) + pad256(EB_CAP * 4) + pad256(sizeof(EnforceState)) + 4096));
    uint64_t* keys = sc.take<uint64_t>(len);
    uint32_t* vals = sc.take<uint32_t>(len);
    uint64_t* skeys = sc.take<uint64_t>(EB_CAP);
    uint32_t* svals = sc.take<uint32_t>(EB_CAP);
    EnforceState* es = sc.take<EnforceState>(1);
    uint32_t mask = 0x1Fu;
    if (pl->cfg.evict_policy != SLHA_B200_EVICT_IMPORTANCE) mask &= ~(1u << PH_EVICT_PINNED);
    const uint32_t cm = pl->codec_mask;
    if (cm && !(cm & 0x80000000u) && !(cm & ((1u << SLHA_CODEC_TQ3) | (1u << SLHA_CODEC_MIX3))))
        mask &= ~((1u << PH_CORR_HOT) | (1u << PH_CORR_WARM));  // no tile with a correction plane can be in the pool
    SLHA_CUDA(cudaMemsetAsync(es, 0, sizeof(EnforceState), c->stream));
    SLHA_CUDA(cudaMemsetAsync(&pl->dev.cnt->max_pos, 0, 8, c->stream));  // max_pos and n_cand
    PoolDev d = pl->dev;
    void* args[] = {&d, &mask, &keys, &vals, &skeys, &svals, &es};
    const uint64_t want = (len + EB_THREADS - 1) / EB_THREADS;
    const unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(want, (uint64_t)sms[dev] * blocks_per_sm[dev]));
    SLHA_CUDA(cudaLaunchCooperativeKernel((const void*)enforce_kernel, dim3(grid), dim3(EB_THREADS), args, 0, c->stream));
    count_launch();
    uint32_t overflow = 0;
    SLHA_CUDA(cudaMemcpyAsync(&overflow, &es->overflow, 4, cudaMemcpyDeviceToHost, c->stream));
    SLHA_TRY(pool_sync_counters(c, pl));
    if (overflow) return Status();
    *within = pl->h_cnt.live <= pl->h_cnt.budget ? 1 : 0;
    *done = true;
    return Status();
}

Status pool_enforce_budget(Ctx* c, Pool* pl, int32_t* within) {
    if (!pl->log && !pl->require_durable && !debug_general_paths()) {
        bool done = false;
        SLHA_TRY(pool_enforce_budget_fused(c, pl, within, &done));
        if (done) return Status();
    }
    SLHA_TRY(pool_sync_counters(c, pl));
    PoolCounters& h = pl->h_cnt;
    if (h.live <= h.budget) {
        *within = 1;
        return Status();
    }
    const uint64_t len = h.len;
    size_t tmp_sort = 0, tmp_scan = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tmp_sort, (uint64_t*)nullptr, (uint64_t*)nullptr,
                                    (uint32_t*)nullptr, (uint32_t*)nullptr, (int)len);
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_scan, (uint32_t*)nullptr, (uint64_t*)nullptr, (int)len);
    const size_t tmp_bytes = std::max(tmp_sort, tmp_scan);
    Scratch sc{c};
    SLHA_TRY(sc.reserve(pad256(len * 8) * 3 + pad256(len * 4) * 3 + pad256(tmp_bytes) + 4096));
    uint64_t* keys = sc.take<uint64_t>(len);
    uint64_t* keys_s = sc.take<uint64_t>(len);
    uint64_t* excl = sc.take<uint64_t>(len);
    uint32_t* vals = sc.take<uint32_t>(len);
    uint32_t* vals_s = sc.take<uint32_t>(len);
    uint32_t* w = sc.take<uint32_t>(len);
    void* tmp = sc.take<unsigned char>(tmp_bytes);
    const uint32_t grid = grid_for(len);

    SLHA_CUDA(cudaMemsetAsync(&pl->dev.cnt->max_pos, 0, 4, c->stream));
    if (pl->cfg.recent_window) {
        max_pos_kernel<<<grid, 256, 0, c->stream>>>(pl->dev);
        count_launch();
    }
    const int phases[5] = {PH_CORR_HOT, PH_PAGE, PH_CORR_WARM, PH_EVICT, PH_EVICT_PINNED};
    for (int ph : phases) {
        if (ph == PH_EVICT_PINNED && pl->cfg.evict_policy != SLHA_B200_EVICT_IMPORTANCE) continue;
        // a pool that has only ever been appended to with codecs without a correction plane (every
        // codec but TQ3 and MIX3) has no candidate for the two correction phases: no scan for them
        const uint32_t cm = pl->codec_mask;
        const bool no_corr_planes = cm && !(cm & 0x80000000u) && !(cm & ((1u << SLHA_CODEC_TQ3) | (1u << SLHA_CODEC_MIX3)));
        if (no_corr_planes && (ph == PH_CORR_HOT || ph == PH_CORR_WARM)) continue;
        SLHA_CUDA(cudaMemsetAsync(&pl->dev.cnt->n_cand, 0, 4, c->stream));
        phase_build_kernel<<<grid, 256, 0, c->stream>>>(pl->dev, ph, keys, vals);
        count_launch();
        SLHA_CUDA(cudaGetLastError());
        // the host needs the candidate count for the sort (and learns whether the budget is met)
        SLHA_TRY(pool_sync_counters(c, pl));
        if (pl->h_cnt.live <= pl->h_cnt.budget) break;
        int nc = (int)pl->h_cnt.n_cand;
        if (nc == 0) continue;
        uint64_t* keys_in = keys;
        uint32_t* vals_in = vals;
        if ((uint32_t)nc >= PREFILTER_MIN) {
            // only the smallest keys can be reached before the deficit is covered (see phase_hist_kernel)
            const uint64_t min_freed = ph == PH_PAGE ? 32 : (ph >= PH_EVICT ? 80 : 14);
            const uint64_t reach = (pl->h_cnt.live - pl->h_cnt.budget) / min_freed + 1;
            uint32_t* d_hist = reinterpret_cast<uint32_t*>(excl);  // (free until the scan; 8 bytes x len >= 16 KB + 4 here)
            SLHA_CUDA(cudaMemsetAsync(d_hist, 0, (PREFILTER_BINS + 1) * 4, c->stream));
            phase_hist_kernel<<<grid_for((uint64_t)nc), 256, 0, c->stream>>>(pl->dev, keys, d_hist);
            std::vector<uint32_t> hh(PREFILTER_BINS);
            SLHA_CUDA(cudaMemcpyAsync(hh.data(), d_hist, PREFILTER_BINS * 4, cudaMemcpyDeviceToHost, c->stream));
            SLHA_CUDA(cudaStreamSynchronize(c->stream));
            uint64_t cum = 0;
            uint32_t last = PREFILTER_BINS - 1;
            for (uint32_t b = 0; b < PREFILTER_BINS; ++b) {
                cum += hh[b];
                if (cum >= reach) { last = b; break; }
            }
            if (cum < (uint64_t)nc) {  // the filter drops something: compact into the sorted-side buffers, sort back
                phase_filter_kernel<<<grid_for((uint64_t)nc), 256, 0, c->stream>>>(pl->dev, keys, vals, last, keys_s, vals_s, d_hist + PREFILTER_BINS);
                phase_set_ncand_kernel<<<1, 1, 0, c->stream>>>(pl->dev, d_hist + PREFILTER_BINS);
                count_launch(3);
                SLHA_CUDA(cudaGetLastError());
                nc = (int)cum;
                std::swap(keys, keys_s);
                std::swap(vals, vals_s);
                keys_in = keys;
                vals_in = vals;
            }
        }
        const uint32_t cgrid = grid_for((uint64_t)nc);
        size_t tb = tmp_bytes;
        SLHA_CUDA(cub::DeviceRadixSort::SortPairs(tmp, tb, keys_in, keys_s, vals_in, vals_s, nc, 0, 64, c->stream));
        phase_weights_kernel<<<cgrid, 256, 0, c->stream>>>(pl->dev, ph, keys_s, vals_s, w);
        tb = tmp_bytes;
        SLHA_CUDA(cub::DeviceScan::ExclusiveSum(tmp, tb, w, excl, nc, c->stream));
        uint64_t limit = ~0ull;
        if (ph >= PH_EVICT && (pl->log || pl->require_durable)) {
            // persist first (ccos.rs:411-432): the records of the slots this phase will evict, in order
            unsigned long long* d_cnt;
            uint64_t* d_seq;
            uint32_t* d_slot;
            uint4* d_tiles;
            SLHA_TRY(ctx_device_scratch(c, 256, (void**)&d_cnt));
            SLHA_TRY(ctx_device_scratch(c, (size_t)nc * 8, (void**)&d_seq));
            SLHA_TRY(ctx_device_scratch(c, (size_t)nc * 4, (void**)&d_slot));
            SLHA_TRY(ctx_device_scratch(c, (size_t)nc * TILE_BYTES, (void**)&d_tiles));
            SLHA_CUDA(cudaMemsetAsync(d_cnt, 0, 8, c->stream));
            phase_journal_kernel<<<cgrid, 256, 0, c->stream>>>(pl->dev, keys_s, vals_s, excl, d_cnt, d_seq, d_slot, d_tiles);
            count_launch();
            unsigned long long m = 0;
            SLHA_CUDA(cudaMemcpyAsync(&m, d_cnt, 8, cudaMemcpyDeviceToHost, c->stream));
            SLHA_CUDA(cudaStreamSynchronize(c->stream));
            std::vector<uint64_t> hseq(m);
            std::vector<uint32_t> hslot(m);
            std::vector<unsigned char> htiles((size_t)m * TILE_BYTES);
            if (m) {
                SLHA_CUDA(cudaMemcpyAsync(hseq.data(), d_seq, m * 8, cudaMemcpyDeviceToHost, c->stream));
                SLHA_CUDA(cudaMemcpyAsync(hslot.data(), d_slot, m * 4, cudaMemcpyDeviceToHost, c->stream));
                SLHA_CUDA(cudaMemcpyAsync(htiles.data(), d_tiles, (size_t)m * TILE_BYTES, cudaMemcpyDeviceToHost, c->stream));
                SLHA_CUDA(cudaStreamSynchronize(c->stream));
            }
            // all records of the phase in one write (the same bytes in the same order as one append per eviction)
            uint64_t written = 0;
            const bool ok = m == 0 || (pl->log && eventlog_append_batch(pl->log, m, hseq.data(), hslot.data(), htiles.data(), pl->require_durable, &written).ok());
            if (!ok) {
                if (pl->log) ++pl->log_errors;
                if (pl->require_durable) {
                    // record `written` could not be persisted: its slot stays live; the reference goes on to try (and be
                    // refused) every remaining live slot
                    limit = written;
                    pl->blocked_evictions += (uint64_t)nc - written;
                    if (pl->log) pl->log_errors += (uint64_t)nc - written - 1;
                }
            }
        }
        phase_apply_kernel<<<cgrid, 256, 0, c->stream>>>(pl->dev, ph, keys_s, vals_s, w, excl, limit);
        phase_commit_kernel<<<1, 1, 0, c->stream>>>(pl->dev);
        count_launch(3);
        SLHA_CUDA(cudaGetLastError());
    }
    SLHA_TRY(pool_sync_counters(c, pl));
    *within = pl->h_cnt.live <= pl->h_cnt.budget ? 1 : 0;
    return Status();
}

Status pool_observe(Ctx* c, Pool* pl, const uint32_t* d_slots, const float* d_scores, uint64_t n, float temperature) {
    if (n == 0 || !std::isfinite(temperature) || temperature <= 0.0f) return Status();
    const int nparts = 256;
    if (!pl->d_observe) SLHA_CUDA(cudaMalloc(&pl->d_observe, sizeof(ObserveTmp) + nparts * 4));
    ObserveTmp* tmp = reinterpret_cast<ObserveTmp*>(pl->d_observe);
    float* partial = reinterpret_cast<float*>(tmp + 1);
    SLHA_CUDA(cudaMemsetAsync(tmp, 0, sizeof(ObserveTmp), c->stream));
    observe_pass1<<<grid_for(n), 256, 0, c->stream>>>(pl->dev, d_slots, d_scores, n, tmp);
    observe_pass2<<<nparts, 256, 0, c->stream>>>(pl->dev, d_slots, d_scores, n, temperature, tmp, partial);
    observe_pass3<<<grid_for(n), 256, 0, c->stream>>>(pl->dev, d_slots, d_scores, n, temperature, tmp, partial, nparts);
    count_launch(3);
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

Status pool_stats(Ctx* c, Pool* pl, uint64_t out[8]) {
    unsigned long long* d;
    SLHA_TRY(ctx_device_scratch(c, 256, (void**)&d));
    SLHA_CUDA(cudaMemsetAsync(d, 0, 64, c->stream));
    stats_kernel<<<grid_for(std::max<uint64_t>(pl->h_cnt.len, 1)), 256, 0, c->stream>>>(pl->dev, d);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    SLHA_CUDA(cudaMemcpyAsync(out, d, 64, cudaMemcpyDeviceToHost, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    return Status();
}

Status pool_compact_live(Ctx* c, Pool* pl, const float* d_scores, uint32_t* d_slots_out, float* d_scores_out,
                         unsigned long long* d_n_out) {
    compact_live_kernel<<<1, 1024, 0, c->stream>>>(pl->dev, d_scores, d_slots_out, d_scores_out, d_n_out);
    count_launch();
    SLHA_CUDA(cudaGetLastError());
    return Status();
}

}  // namespace slha

namespace slha {
// ElasticKvCache::rehydrate (ccos.rs:451-466): the most recent record with that eviction seq comes back as a
// fresh admission (new seq, importance 0), WARM when its tile carries the WARM flag, else HOT.
Status pool_rehydrate(Ctx* c, Pool* pl, uint64_t seq, int64_t* slot_out) {
    *slot_out = -1;
    if (!pl->log) return Status();
    bool found = false;
    uint32_t old_slot = 0;
    unsigned char tile[TILE_BYTES];
    SLHA_TRY(eventlog_fetch_by_seq(pl->log, seq, &found, &old_slot, tile));
    if (!found) return Status();
    unsigned char* d_tile;
    uint32_t* d_slot;
    SLHA_TRY(ctx_device_scratch(c, TILE_BYTES, (void**)&d_tile));
    SLHA_TRY(ctx_device_scratch(c, 256, (void**)&d_slot));
    SLHA_CUDA(cudaMemcpyAsync(d_tile, tile, TILE_BYTES, cudaMemcpyHostToDevice, c->stream));
    SLHA_TRY(pool_reserve(c, pl, d_tile, 1, d_slot));
    SLHA_TRY(pool_scatter(c, pl, d_tile, d_slot, 1));
    uint32_t slot = 0;
    SLHA_CUDA(cudaMemcpyAsync(&slot, d_slot, 4, cudaMemcpyDeviceToHost, c->stream));
    SLHA_CUDA(cudaStreamSynchronize(c->stream));
    pl->codec_mask |= 0x80000000u;
    *slot_out = (int64_t)slot;
    return Status();
}
}  // namespace slha
