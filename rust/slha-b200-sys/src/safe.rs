//! Safe wrappers with the names of the scirust items they replace on the GPU path.
//!
//! | here | scirust |
//! |---|---|
//! | [`LearnedModel`] | `scirust::learned::LearnedModel` (`try_from_projection_with`, `encode_with`, `query_coarse` + `sign_bits`) |
//! | [`compute_scores`] | `SciRustSlhaTile::compute_score` over a batch |
//! | [`score_topk`] | scoring + the ordering of `metrics::topk` (no reference function) |
//! | [`ElasticKvCache`] | `scirust::ccos::ElasticKvCache` |
//! | [`ShardedScorer`] | none (token-range sharding over NCCL) |
//!
//! Host slices go in and come out; the library stages them.  Device-resident use goes through the raw
//! functions with device pointers.

use crate::*;
use std::ffi::CStr;

#[derive(Debug, Clone, PartialEq, Eq)]
pub struct SlhaError {
    pub code: i32,
    pub message: String,
}
impl std::fmt::Display for SlhaError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "SLHA status {}: {}", self.code, self.message)
    }
}
impl std::error::Error for SlhaError {}
pub type Result<T> = std::result::Result<T, SlhaError>;

fn check(code: i32) -> Result<()> {
    if code == SLHA_OK {
        return Ok(());
    }
    // SAFETY: the library returns a pointer to a NUL-terminated thread-local buffer that stays valid until the next call.
    let message = unsafe { CStr::from_ptr(slha_last_error_message()) }.to_string_lossy().into_owned();
    Err(SlhaError { code, message })
}

/// `LearnedModel::try_from_projection_with` (`scirust/src/learned.rs:204-238`) resident on the GPU.
pub struct LearnedModel {
    handle: *mut SlhaModel,
    d: usize,
}
// SAFETY: the handle is a registry token; the library is re-entrant for a given model.
unsafe impl Send for LearnedModel {}
unsafe impl Sync for LearnedModel {}

impl LearnedModel {
    pub fn try_from_projection_with(projection: &[f32], d: usize, seed: u64, rht: bool) -> Result<Self> {
        if projection.len() != SLHA_D_C * d {
            return Err(SlhaError { code: SLHA_ERR_DIMENSION, message: "projection must be 128 x d".into() });
        }
        // SAFETY: the slice holds 128 * d floats; NULL scale / z select the reference defaults.
        let handle = unsafe { slha_b200_model_create(projection.as_ptr(), d, seed, rht as i32, core::ptr::null(), core::ptr::null()) };
        if handle.is_null() {
            check(SLHA_ERR_PANIC)?;
        }
        Ok(Self { handle, d })
    }
    pub fn d(&self) -> usize {
        self.d
    }
    pub fn as_ptr(&self) -> *const SlhaModel {
        self.handle
    }
    /// `encode_with` over a batch of `keys.len() / d` keys (`learned.rs:353-408`); tile bytes equal the scalar encoder's.
    pub fn encode_with(&self, keys: &[f32], position_base: u32, codec: i32) -> Result<Vec<SciRustSlhaTile>> {
        let n = keys.len() / self.d;
        let mut tiles = vec![unsafe { core::mem::zeroed::<SciRustSlhaTile>() }; n];
        // SAFETY: n keys of d floats in, n tiles out; NULL positions / heads select position_base + i and head 0.
        check(unsafe {
            slha_b200_encode_keys(self.handle, keys.as_ptr().cast(), SLHA_B200_F32, n, core::ptr::null(), position_base, core::ptr::null(), codec, tiles.as_mut_ptr())
        })?;
        Ok(tiles)
    }
    /// `query_coarse` + `sign_bits` (`learned.rs:267-273`, `:326-347`) for `q.len() / d` queries.
    pub fn prepare_queries(&self, q: &[f32]) -> Result<(Vec<f32>, Vec<u64>)> {
        let nq = q.len() / self.d;
        let (mut qc, mut qs) = (vec![0f32; nq * SLHA_D_C], vec![0u64; nq * 4]);
        // SAFETY: buffer sizes follow the header.
        check(unsafe { slha_b200_prepare_queries(self.handle, q.as_ptr(), nq, qc.as_mut_ptr(), qs.as_mut_ptr()) })?;
        Ok((qc, qs))
    }
}
impl Drop for LearnedModel {
    fn drop(&mut self) {
        // SAFETY: the handle came from slha_b200_model_create and is released once.
        unsafe { slha_weights_release(self.handle) };
    }
}

/// `SciRustSlhaTile::compute_score` (`tile.rs:267-281`) of every tile against `nq` prepared queries:
/// `scores[j * tiles.len() + i]`.
pub fn compute_scores(tiles: &[SciRustSlhaTile], q_coarse: &[f32], q_sign: &[u64]) -> Result<Vec<f32>> {
    let nq = q_coarse.len() / SLHA_D_C;
    let mut scores = vec![0f32; nq * tiles.len()];
    // SAFETY: buffer sizes follow the header.
    check(unsafe { slha_b200_score_tiles(tiles.as_ptr(), tiles.len(), q_coarse.as_ptr(), q_sign.as_ptr(), nq, scores.as_mut_ptr()) })?;
    Ok(scores)
}

/// Device memory owned through the library (`slha_b200_malloc`).
pub struct DeviceTiles {
    ptr: *mut SciRustSlhaTile,
    len: usize,
}
impl DeviceTiles {
    pub fn upload(tiles: &[SciRustSlhaTile]) -> Result<Self> {
        let mut p: *mut core::ffi::c_void = core::ptr::null_mut();
        // SAFETY: plain allocation and a synchronous copy of tiles.len() * 128 bytes.
        check(unsafe { slha_b200_malloc(tiles.len().max(1) * 128, &mut p) })?;
        check(unsafe { slha_b200_memcpy(p, tiles.as_ptr().cast(), tiles.len() * 128) })?;
        Ok(Self { ptr: p.cast(), len: tiles.len() })
    }
    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn as_ptr(&self) -> *const SciRustSlhaTile {
        self.ptr
    }
}
impl Drop for DeviceTiles {
    fn drop(&mut self) {
        // SAFETY: allocated by slha_b200_malloc above.
        unsafe { slha_b200_free(self.ptr.cast()) };
    }
}

/// Fused scoring + top-k: for every query row of every segment its `k` best (index, score) pairs, score
/// descending, ties towards the lower index (`scirust/src/metrics.rs:186-192`).
pub fn score_topk(tiles: &DeviceTiles, segments: &[SlhaB200Segment], q_coarse: &[f32], q_sign: &[u64], k: u32) -> Result<(Vec<u32>, Vec<f32>, Vec<u32>)> {
    let nq = q_coarse.len() / SLHA_D_C;
    let (mut idx, mut sc, mut cnt) = (vec![0u32; nq * k as usize], vec![0f32; nq * k as usize], vec![0u32; nq]);
    // SAFETY: tiles is device memory of tiles.len() tiles; the other buffers are host slices of the documented sizes.
    check(unsafe {
        slha_b200_score_topk(tiles.as_ptr(), segments.as_ptr(), segments.len(), q_coarse.as_ptr(), q_sign.as_ptr(), nq, k, idx.as_mut_ptr(), sc.as_mut_ptr(), cnt.as_mut_ptr())
    })?;
    Ok((idx, sc, cnt))
}

/// `scirust::ccos::ElasticKvCache` (`ccos.rs:132-614`) with its arena in HBM.
pub struct ElasticKvCache {
    pool: *mut SlhaB200Pool,
}
unsafe impl Send for ElasticKvCache {}

#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct Counts {
    pub len: u64,
    pub live_bytes: u64,
    pub hot: u64,
    pub warm: u64,
    pub cold: u64,
    pub nocorr: u64,
    pub reclaimed_correction_bytes: u64,
    pub free_len: u64,
}

impl ElasticKvCache {
    pub fn with_eviction(capacity_tiles: u64, budget_bytes: u64, page_policy: i32, evict_policy: i32, sink_window: u32) -> Result<Self> {
        let cfg = SlhaB200PoolConfig { capacity_tiles, budget_bytes, page_policy, evict_policy, sink_window, recent_window: 0 };
        let mut pool = core::ptr::null_mut();
        // SAFETY: cfg outlives the call; pool receives the handle.
        check(unsafe { slha_b200_pool_create(&cfg, &mut pool) })?;
        Ok(Self { pool })
    }
    /// `insert` (`ccos.rs:217-259`) for ready-made tiles; returns their slots.
    pub fn insert(&mut self, tiles: &[SciRustSlhaTile]) -> Result<Vec<u32>> {
        let mut slots = vec![0u32; tiles.len()];
        check(unsafe { slha_b200_pool_insert_tiles(self.pool, tiles.as_ptr(), tiles.len(), slots.as_mut_ptr()) })?;
        Ok(slots)
    }
    /// `encode_with` + `insert` without the tiles leaving HBM.
    pub fn append_keys(&mut self, model: &LearnedModel, keys: &[f32], position_base: u32, codec: i32) -> Result<Vec<u32>> {
        let n = keys.len() / model.d();
        let mut slots = vec![0u32; n];
        check(unsafe {
            slha_b200_pool_append_keys(self.pool, model.as_ptr(), keys.as_ptr().cast(), SLHA_B200_F32, n, core::ptr::null(), position_base, core::ptr::null(), codec, slots.as_mut_ptr())
        })?;
        Ok(slots)
    }
    /// `score_all` (`ccos.rs:346-355`): (slot, score) of every non-COLD slot.
    pub fn score_all(&self, q_coarse: &[f32], q_sign: &[u64]) -> Result<Vec<(u32, f32)>> {
        let len = self.counts()?.len as usize;
        let (mut slots, mut scores, mut n) = (vec![0u32; len], vec![0f32; len], 0u64);
        check(unsafe { slha_b200_pool_score_all(self.pool, q_coarse.as_ptr(), q_sign.as_ptr(), slots.as_mut_ptr(), scores.as_mut_ptr(), &mut n) })?;
        Ok(slots.into_iter().zip(scores).take(n as usize).collect())
    }
    pub fn score_topk(&self, q_coarse: &[f32], q_sign: &[u64], k: u32) -> Result<(Vec<u32>, Vec<f32>, Vec<u32>)> {
        let nq = q_coarse.len() / SLHA_D_C;
        let (mut idx, mut sc, mut cnt) = (vec![0u32; nq * k as usize], vec![0f32; nq * k as usize], vec![0u32; nq]);
        check(unsafe { slha_b200_pool_score_topk(self.pool, q_coarse.as_ptr(), q_sign.as_ptr(), nq, k, idx.as_mut_ptr(), sc.as_mut_ptr(), cnt.as_mut_ptr()) })?;
        Ok((idx, sc, cnt))
    }
    /// `observe_scores` (`ccos.rs:275-314`).
    pub fn observe_scores(&mut self, slots: &[u32], scores: &[f32], temperature: f32) -> Result<()> {
        check(unsafe { slha_b200_pool_observe_scores(self.pool, slots.as_ptr(), scores.as_ptr(), slots.len().min(scores.len()), temperature) })
    }
    pub fn page_out(&mut self, slot: u32) -> Result<()> {
        check(unsafe { slha_b200_pool_page_out(self.pool, slot) })
    }
    pub fn drop_correction(&mut self, slot: u32) -> Result<bool> {
        let mut dropped = 0;
        check(unsafe { slha_b200_pool_drop_correction(self.pool, slot, &mut dropped) })?;
        Ok(dropped != 0)
    }
    pub fn evict(&mut self, slot: u32) -> Result<bool> {
        let mut evicted = 0;
        check(unsafe { slha_b200_pool_evict(self.pool, slot, &mut evicted) })?;
        Ok(evicted != 0)
    }
    /// `enforce_budget` (`ccos.rs:555-614`); true when the pool is within its budget afterwards.
    pub fn enforce_budget(&mut self) -> Result<bool> {
        let mut ok = 0;
        check(unsafe { slha_b200_pool_enforce_budget(self.pool, &mut ok) })?;
        Ok(ok != 0)
    }
    pub fn counts(&self) -> Result<Counts> {
        let mut o = [0u64; 8];
        check(unsafe { slha_b200_pool_stats(self.pool, o.as_mut_ptr()) })?;
        Ok(Counts { len: o[0], live_bytes: o[1], hot: o[2], warm: o[3], cold: o[4], nocorr: o[5], reclaimed_correction_bytes: o[6], free_len: o[7] })
    }
    pub fn live_bytes(&self) -> Result<u64> {
        Ok(self.counts()?.live_bytes)
    }
}
impl Drop for ElasticKvCache {
    fn drop(&mut self) {
        // SAFETY: created by slha_b200_pool_create, destroyed once.
        unsafe { slha_b200_pool_destroy(self.pool) };
    }
}

/// One rank of the token-range sharded scorer (`slha_b200_shard_*`): local fused score + top-k, one
/// NCCL all-gather, merge.  Rank 0 obtains [`ShardedScorer::unique_id`] and hands the 128 bytes to the
/// other ranks by any transport the host has.
pub struct ShardedScorer {
    shard: *mut SlhaB200Shard,
}
unsafe impl Send for ShardedScorer {}

impl ShardedScorer {
    pub fn unique_id() -> Result<[u8; 128]> {
        let mut id = [0u8; 128];
        check(unsafe { slha_b200_shard_unique_id(id.as_mut_ptr().cast()) })?;
        Ok(id)
    }
    pub fn init(unique_id: Option<&[u8; 128]>, rank: i32, world: i32) -> Result<Self> {
        let mut shard = core::ptr::null_mut();
        let id = unique_id.map_or(core::ptr::null(), |b| b.as_ptr().cast());
        check(unsafe { slha_b200_shard_init(id, rank, world, &mut shard) })?;
        Ok(Self { shard })
    }
    /// One sharded decode step (collective): this rank's tiles and segment table, everybody's queries.
    pub fn score_topk(&mut self, tiles: &DeviceTiles, segments: &[SlhaB200Segment], q_coarse: &[f32], q_sign: &[u64], k: u32) -> Result<(Vec<u32>, Vec<f32>)> {
        let nq = q_coarse.len() / SLHA_D_C;
        let (mut idx, mut sc) = (vec![0u32; nq * k as usize], vec![0f32; nq * k as usize]);
        check(unsafe {
            slha_b200_shard_score_topk(self.shard, tiles.as_ptr(), segments.as_ptr(), segments.len(), q_coarse.as_ptr(), q_sign.as_ptr(), nq, k, idx.as_mut_ptr(), sc.as_mut_ptr())
        })?;
        Ok((idx, sc))
    }
}
impl Drop for ShardedScorer {
    fn drop(&mut self) {
        // SAFETY: created by slha_b200_shard_init, destroyed once.
        unsafe { slha_b200_shard_destroy(self.shard) };
    }
}
