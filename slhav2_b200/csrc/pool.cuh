// Device-resident CCOS pool: shared declarations (pool.cu, capi.cu).
#pragma once

#include "common.cuh"

namespace slha {

// 64-byte counter block living in device memory (mirrored on the host after
// every call that can change it in a data-dependent way).
struct PoolCounters {
    uint64_t len;        // slots ever allocated (arena high-water mark)
    uint64_t free_len;   // entries in the LIFO free list
    uint64_t next_seq;   // insertion counter (ccos.rs `next_seq`)
    uint64_t live;       // logical live bytes (ccos.rs `live_bytes_counter`)
    uint64_t budget;     // byte budget
    uint64_t phase_deficit;
    uint64_t phase_applied;
    int64_t live_delta;
    uint32_t max_pos;
    uint32_t n_cand;     // candidates of the enforce_budget phase being built
};

struct PoolDev {
    unsigned char* tiles = nullptr;  // [capacity][128]
    uint8_t* state = nullptr;        // HOT / WARM / COLD per slot
    uint64_t* seq = nullptr;         // insertion order per slot
    float* importance = nullptr;     // accumulated H2O importance per slot
    uint32_t* free_list = nullptr;   // LIFO stack of COLD slots
    PoolCounters* cnt = nullptr;
    int32_t page_policy = 0, evict_policy = 0;
    uint32_t sink_window = 0, recent_window = 0;
};

// COLD persistence (eventlog.cu): the reference's EventLog file format
struct EventLog;
Status eventlog_open(const char* path, int mode, EventLog** out);
void eventlog_close(EventLog* log);
uint64_t eventlog_records(const EventLog* log);
Status eventlog_append(EventLog* log, uint64_t seq, uint32_t slot, const unsigned char* tile, bool durable);
Status eventlog_append_batch(EventLog* log, uint64_t n, const uint64_t* seq, const uint32_t* slot, const unsigned char* tiles,
                             bool durable, uint64_t* written);
Status eventlog_fetch_by_seq(EventLog* log, uint64_t seq, bool* found, uint32_t* slot, unsigned char* tile);

struct Pool {
    SlhaB200PoolConfig cfg;
    int device = 0;
    PoolDev dev;
    PoolCounters h_cnt;      // host mirror
    void* d_observe = nullptr;  // scratch of observe_scores (reduction cell + partial sums)
    // codecs the pool may hold: bit i = codec id i appended through append_keys; bit 31 = tiles of
    // unknown codec were inserted. Lets the scorer pick its kernel variant without reading tiles back.
    uint32_t codec_mask = 0;
    // attached event log (ccos.rs:155-170): evicted tiles are appended before their slots go COLD
    EventLog* log = nullptr;
    bool require_durable = false;            // EvictionDurability::RequireDurable
    uint64_t log_errors = 0, blocked_evictions = 0;  // ccos.rs:173-181
};

Status pool_create(Ctx* c, const SlhaB200PoolConfig& cfg, Pool** out);
void pool_destroy(Pool* pl);
Status pool_sync_counters(Ctx* c, Pool* pl);
Status pool_reserve(Ctx* c, Pool* pl, const unsigned char* d_src_tiles, uint64_t n, uint32_t* d_slots);
Status pool_scatter(Ctx* c, Pool* pl, const unsigned char* d_src_tiles, const uint32_t* d_slots, uint64_t n);
Status pool_single_op(Ctx* c, Pool* pl, int op, uint32_t slot, int32_t* result);
Status pool_enforce_budget(Ctx* c, Pool* pl, int32_t* within);
Status pool_observe(Ctx* c, Pool* pl, const uint32_t* d_slots, const float* d_scores, uint64_t n, float temperature);
Status pool_stats(Ctx* c, Pool* pl, uint64_t out[8]);
Status pool_rehydrate(Ctx* c, Pool* pl, uint64_t seq, int64_t* slot_out);
Status pool_compact_live(Ctx* c, Pool* pl, const float* d_scores, uint32_t* d_slots_out, float* d_scores_out,
                         unsigned long long* d_n_out);

}  // namespace slha
