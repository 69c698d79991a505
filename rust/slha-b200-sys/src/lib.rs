//! FFI declarations of `libslha_b200` (`include/slha_b200.h`) and thin safe wrappers named after the
//! scirust items they stand in for (`LearnedModel`, `ElasticKvCache`, `compute_score` ...).
//!
//! Part 1 of the header is the reference's own C ABI (`slha-c/include/slha.h`, 20 functions); a host
//! that links `libslha` today links this library instead and keeps calling the same symbols.  Part 2
//! adds the batched / device-resident entry points.  This crate has not been compiled where it was
//! written (no Rust toolchain there); it is kept in step with the header by review, and
//! `tests/test_abi_cpu.py` checks that every function named here is exported by the library.
#![allow(non_camel_case_types, clippy::missing_safety_doc, clippy::too_many_arguments)]

use core::ffi::{c_char, c_void};

pub mod safe;

pub const SLHA_ABI_VERSION: u32 = 1;
pub const SLHA_D_C: usize = 128;
pub const SLHA_D_S: usize = 256;

pub const SLHA_OK: i32 = 0;
pub const SLHA_ERR_NULL: i32 = -1;
pub const SLHA_ERR_PANIC: i32 = -2;
pub const SLHA_ERR_DIMENSION: i32 = -3;
pub const SLHA_ERR_CODEC: i32 = -4;
pub const SLHA_ERR_NONFINITE: i32 = -5;
pub const SLHA_ERR_INVALID_TILE: i32 = -6;
pub const SLHA_ERR_INVALID_HANDLE: i32 = -7;
pub const SLHA_ERR_IO: i32 = -8;
pub const SLHA_ERR_UTF8: i32 = -9;
pub const SLHA_ERR_DEVICE: i32 = -100;
pub const SLHA_ERR_CAPACITY: i32 = -101;

pub const SLHA_CODEC_INT4_SINGLE: i32 = 0;
pub const SLHA_CODEC_INT4_GROUPED: i32 = 1;
pub const SLHA_CODEC_NF4: i32 = 2;
pub const SLHA_CODEC_MIXED: i32 = 3;
pub const SLHA_CODEC_TQ3: i32 = 4;
pub const SLHA_CODEC_MIX3: i32 = 5;
pub const SLHA_B200_CODEC_INT4_GROUPED32: i32 = 6;

pub const SLHA_FLAG_WARM: u16 = 1 << 0;
pub const SLHA_FLAG_NF4: u16 = 1 << 1;
pub const SLHA_FLAG_MIXED: u16 = 1 << 2;
pub const SLHA_FLAG_TQ3: u16 = 1 << 3;
pub const SLHA_FLAG_TQ3_NOCORR: u16 = 1 << 4;
pub const SLHA_FLAG_MIX3: u16 = 1 << 5;

pub const SLHA_B200_F32: i32 = 0;
pub const SLHA_B200_BF16: i32 = 1;
pub const SLHA_B200_STATE_HOT: u8 = 0;
pub const SLHA_B200_STATE_WARM: u8 = 1;
pub const SLHA_B200_STATE_COLD: u8 = 2;
pub const SLHA_B200_PAGE_LOWEST_IMPACT_FIRST: i32 = 0;
pub const SLHA_B200_PAGE_OLDEST_FIRST: i32 = 1;
pub const SLHA_B200_EVICT_CAUSAL: i32 = 0;
pub const SLHA_B200_EVICT_IMPORTANCE: i32 = 1;

/// The 128-byte tile (`scirust/src/attention/slha_v2/tile.rs:52-77`, `slha.h:87-110`).
#[repr(C, align(64))]
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct SciRustSlhaTile {
    pub latent_kv: [u8; 64],
    pub residual_bitmap: [u64; 4],
    pub scale: f32,
    pub dynamic_lambda: f32,
    pub residual_sigma: f32,
    pub token_id: u32,
    pub position: u32,
    pub head_id: u16,
    pub flags: u16,
    pub group_scales: [u8; 8],
}
const _: () = assert!(core::mem::size_of::<SciRustSlhaTile>() == 128);
const _: () = assert!(core::mem::align_of::<SciRustSlhaTile>() == 64);

#[repr(C)]
pub struct SlhaContext {
    _private: [u8; 0],
}
#[repr(C)]
pub struct SlhaModel {
    _private: [u8; 0],
}
#[repr(C)]
pub struct SlhaB200Pool {
    _private: [u8; 0],
}
#[repr(C)]
pub struct SlhaB200Shard {
    _private: [u8; 0],
}

/// A contiguous run of tiles scored by a contiguous group of query rows.
#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct SlhaB200Segment {
    pub tile_begin: u64,
    pub n_tiles: u32,
    pub query_begin: u32,
    pub n_queries: u32,
    pub index_base: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct SlhaB200PoolConfig {
    pub capacity_tiles: u64,
    pub budget_bytes: u64,
    pub page_policy: i32,
    pub evict_policy: i32,
    pub sink_window: u32,
    pub recent_window: u32,
}

extern "C" {
    // ---- part 1: slha-c/include/slha.h:123-278 -------------------------------------------------
    pub fn slha_abi_version() -> u32;
    pub fn slha_tile_size() -> usize;
    pub fn slha_tile_align() -> usize;
    pub fn slha_last_error_message() -> *const c_char;
    pub fn slha_clear_error();
    pub fn slha_init() -> *mut SlhaContext;
    pub fn slha_shutdown(context: *mut SlhaContext) -> i32;
    pub fn slha_process_tile(tile: *const SciRustSlhaTile, q_coarse: *const f32, q_sign: *const u64, score_out: *mut f32) -> i32;
    pub fn slha_prepare_query(model: *const SlhaModel, q: *const f32, d: usize, q_coarse: *mut f32, q_sign: *mut u64) -> i32;
    pub fn slha_score_tile(model: *const SlhaModel, tile: *const SciRustSlhaTile, q_coarse: *const f32, q_sign: *const u64, score_out: *mut f32) -> i32;
    pub fn slha_score_tiles(model: *const SlhaModel, tiles: *const SciRustSlhaTile, n_tiles: usize, q_coarse: *const f32, q_sign: *const u64, scores_out: *mut f32) -> i32;
    pub fn slha_audit() -> *mut c_char;
    pub fn slha_free_string(string: *mut c_char);
    pub fn slha_weights_load(path: *const c_char) -> *mut SlhaModel;
    pub fn slha_model_dim(model: *const SlhaModel) -> usize;
    pub fn slha_encode_key(model: *const SlhaModel, key: *const f32, d: usize, position: u32, codec: i32, out_tile: *mut SciRustSlhaTile) -> i32;
    pub fn slha_decode_latent(model: *const SlhaModel, tile: *const SciRustSlhaTile, out: *mut f32, d: usize) -> i32;
    pub fn slha_decode_key(model: *const SlhaModel, tile: *const SciRustSlhaTile, out: *mut f32, d: usize) -> i32;
    pub fn slha_weights_release(model: *mut SlhaModel) -> i32;
    pub fn slha_weights_free(model: *mut SlhaModel);

    // ---- part 2: batched and device-resident entry points ---------------------------------------
    pub fn slha_b200_device_count() -> i32;
    pub fn slha_b200_set_device(device: i32) -> i32;
    pub fn slha_b200_set_stream(cuda_stream: *mut c_void) -> i32;
    pub fn slha_b200_launch_count() -> u64;
    pub fn slha_b200_debug_force_generic_score(on: i32) -> i32;
    pub fn slha_b200_last_score_stats(out: *mut u64) -> i32;
    pub fn slha_b200_timing_begin(max_calls: u32) -> i32;
    pub fn slha_b200_timing_end(score_ms: *mut f32, merge_ms: *mut f32, capacity: u32, n_out: *mut u32) -> i32;
    pub fn slha_b200_malloc(bytes: usize, out: *mut *mut c_void) -> i32;
    pub fn slha_b200_free(ptr: *mut c_void) -> i32;
    pub fn slha_b200_memcpy(dst: *mut c_void, src: *const c_void, bytes: usize) -> i32;
    pub fn slha_b200_synchronize() -> i32;
    pub fn slha_b200_model_create(projection: *const f32, d: usize, seed: u64, rht: i32, scale: *const f32, z: *const f32) -> *mut SlhaModel;
    pub fn slha_b200_encode_keys(model: *const SlhaModel, keys: *const c_void, key_dtype: i32, n: usize, positions: *const u32, position_base: u32, head_ids: *const u16, codec: i32, tiles_out: *mut SciRustSlhaTile) -> i32;
    pub fn slha_b200_prepare_queries(model: *const SlhaModel, q: *const f32, nq: usize, q_coarse_out: *mut f32, q_sign_out: *mut u64) -> i32;
    pub fn slha_b200_score_tiles(tiles: *const SciRustSlhaTile, n: usize, q_coarse: *const f32, q_sign: *const u64, nq: usize, scores_out: *mut f32) -> i32;
    pub fn slha_b200_score_topk(tiles: *const SciRustSlhaTile, segments: *const SlhaB200Segment, n_segments: usize, q_coarse: *const f32, q_sign: *const u64, n_queries: usize, k: u32, out_index: *mut u32, out_score: *mut f32, out_count: *mut u32) -> i32;
    pub fn slha_b200_score_topk_noalloc(tiles: *const SciRustSlhaTile, segments: *const SlhaB200Segment, n_segments: usize, q_coarse: *const f32, q_sign: *const u64, n_queries: usize, k: u32, out_index: *mut u32, out_score: *mut f32, out_count: *mut u32) -> i32;
    pub fn slha_b200_score_segments(tiles: *const SciRustSlhaTile, segments: *const SlhaB200Segment, n_segments: usize, q_coarse: *const f32, q_sign: *const u64, n_queries: usize, scores_out: *mut f32, scores_len: usize, row_offsets: *const u64, row_len: u32, fill: f32) -> i32;
    pub fn slha_b200_attend_topk(top_index: *const u32, top_score: *const f32, top_count: *const u32, n_queries: usize, k: u32, scale: f32, values: *const c_void, value_dtype: i32, d_v: usize, value_row_stride: usize, value_row_base: *const u64, out: *mut f32, weights_out: *mut f32) -> i32;
    pub fn slha_b200_shard_unique_id(id_out: *mut c_void) -> i32;
    pub fn slha_b200_shard_init(nccl_unique_id: *const c_void, rank: i32, world: i32, out: *mut *mut SlhaB200Shard) -> i32;
    pub fn slha_b200_shard_destroy(shard: *mut SlhaB200Shard) -> i32;
    pub fn slha_b200_shard_score_topk(shard: *mut SlhaB200Shard, tiles: *const SciRustSlhaTile, segments: *const SlhaB200Segment, n_segments: usize, q_coarse: *const f32, q_sign: *const u64, n_queries: usize, k: u32, out_index: *mut u32, out_score: *mut f32) -> i32;
    pub fn slha_b200_shard_set_timing(shard: *mut SlhaB200Shard, on: i32) -> i32;
    pub fn slha_b200_shard_last_times(shard: *mut SlhaB200Shard, ms_out: *mut f32) -> i32;
    pub fn slha_b200_shard_status(shard: *mut SlhaB200Shard, out: *mut u64) -> i32;
    pub fn slha_b200_shard_set_exchange(shard: *mut SlhaB200Shard, mode: i32) -> i32;
    pub fn slha_b200_topk_merge(cand_index: *const u32, cand_score: *const f32, n_lists: u32, n_queries: u32, k_in: u32, k_out: u32, out_index: *mut u32, out_score: *mut f32) -> i32;
    pub fn slha_b200_topk_merge_strided(cand_index: *const u32, cand_score: *const f32, n_lists: u32, list_stride: u64, n_queries: u32, k_in: u32, k_out: u32, out_index: *mut u32, out_score: *mut f32) -> i32;
    pub fn slha_b200_topk_merge_sorted_strided(cand_index: *const u32, cand_score: *const f32, n_lists: u32, list_stride: u64, n_queries: u32, k_in: u32, k_out: u32, out_index: *mut u32, out_score: *mut f32) -> i32;
    pub fn slha_b200_pool_create(config: *const SlhaB200PoolConfig, out: *mut *mut SlhaB200Pool) -> i32;
    pub fn slha_b200_pool_destroy(pool: *mut SlhaB200Pool) -> i32;
    pub fn slha_b200_pool_insert_tiles(pool: *mut SlhaB200Pool, tiles: *const SciRustSlhaTile, n: usize, slots_out: *mut u32) -> i32;
    pub fn slha_b200_pool_append_keys(pool: *mut SlhaB200Pool, model: *const SlhaModel, keys: *const c_void, key_dtype: i32, n: usize, positions: *const u32, position_base: u32, head_ids: *const u16, codec: i32, slots_out: *mut u32) -> i32;
    pub fn slha_b200_pool_score_all(pool: *mut SlhaB200Pool, q_coarse: *const f32, q_sign: *const u64, slots_out: *mut u32, scores_out: *mut f32, n_out: *mut u64) -> i32;
    pub fn slha_b200_pool_score_topk(pool: *mut SlhaB200Pool, q_coarse: *const f32, q_sign: *const u64, nq: usize, k: u32, out_slot: *mut u32, out_score: *mut f32, out_count: *mut u32) -> i32;
    pub fn slha_b200_pool_observe_scores(pool: *mut SlhaB200Pool, slots: *const u32, scores: *const f32, n: usize, temperature: f32) -> i32;
    pub fn slha_b200_pool_observe_query(pool: *mut SlhaB200Pool, q_coarse: *const f32, q_sign: *const u64, temperature: f32) -> i32;
    pub fn slha_b200_pool_page_out(pool: *mut SlhaB200Pool, slot: u32) -> i32;
    pub fn slha_b200_pool_drop_correction(pool: *mut SlhaB200Pool, slot: u32, dropped: *mut i32) -> i32;
    pub fn slha_b200_pool_evict(pool: *mut SlhaB200Pool, slot: u32, evicted: *mut i32) -> i32;
    pub fn slha_b200_pool_attach_event_log(pool: *mut SlhaB200Pool, path: *const c_char, mode: i32, require_durable: i32) -> i32;
    pub fn slha_b200_pool_rehydrate(pool: *mut SlhaB200Pool, seq: u64, slot_out: *mut i64) -> i32;
    pub fn slha_b200_pool_event_log_stats(pool: *mut SlhaB200Pool, out: *mut u64) -> i32;
    pub fn slha_b200_pool_enforce_budget(pool: *mut SlhaB200Pool, within_budget: *mut i32) -> i32;
    pub fn slha_b200_pool_set_budget(pool: *mut SlhaB200Pool, budget_bytes: u64) -> i32;
    pub fn slha_b200_pool_stats(pool: *mut SlhaB200Pool, out: *mut u64) -> i32;
    pub fn slha_b200_pool_read(pool: *mut SlhaB200Pool, first: u64, n: u64, tiles_out: *mut SciRustSlhaTile, state_out: *mut u8, importance_out: *mut f32, seq_out: *mut u64) -> i32;
    pub fn slha_b200_pool_tiles_device(pool: *mut SlhaB200Pool) -> *const SciRustSlhaTile;
}
