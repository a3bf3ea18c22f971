//! hyprstream-attn-sys: bindings of libhs_attn.so, the B200 (sm_100a) attention + quantised KV-cache kernels.
//!
//! NOT COMPILED IN THE BUILD ENVIRONMENT OF THIS REPOSITORY (no cargo / rustc): source for a maintainer.  The same C ABI
//! is exercised from Python (hyprstream_b200/ffi.py) by the repository's tests, and `gen_bindings.py --check` keeps
//! `bindings.rs` in step with include/hs_attn.h.
//!
//! Shape of the crate follows crates/bitsandbytes-sys/src/lib.rs: the raw bindings re-exported, an error type
//! (lib.rs:48-74), safe wrappers for what only touches the host (lib.rs:212-402), and thin `unsafe fn` forwards for the
//! entry points that take device pointers (lib.rs:443-572).  Every call returns a status instead of `void`; a non-zero
//! status becomes `AttnError` with the library's thread-local message.
#![cfg(hs_attn_cuda)]

mod bindings;
pub use bindings::*;

use std::ffi::{c_void, CStr};
use std::ptr;

/// A non-zero status from the library: negative = argument error found on the host before any launch,
/// positive = a `cudaError_t`.
#[derive(Debug, Clone)]
pub struct AttnError {
    pub code: i32,
    pub message: String,
}

impl AttnError {
    /// The typed, fail-soft pool exhaustion (kv_cache.rs:482-505): a scheduler defers admission instead of failing.
    pub fn is_pool_exhausted(&self) -> bool {
        self.code == HS_ERR_POOL_EXHAUSTED
    }
}

impl std::fmt::Display for AttnError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "hs_attn status {}: {}", self.code, self.message)
    }
}

impl std::error::Error for AttnError {}

pub type Result<T> = std::result::Result<T, AttnError>;

/// Status -> Result, with the library's thread-local message.
pub fn check(status: i32) -> Result<()> {
    if status == HS_OK {
        return Ok(());
    }
    // SAFETY: hs_attn_last_error returns a pointer to a thread-local, NUL-terminated buffer that lives as long as the thread
    let message = unsafe {
        let p = hs_attn_last_error();
        if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    };
    Err(AttnError { code: status, message })
}

/// Library version (100 = 1.0.0).
pub fn version() -> i32 {
    // SAFETY: no arguments, no state
    unsafe { hs_attn_version() }
}

/// Ok if `device` (or the current device when negative) is compute capability 10.x.
pub fn device_check(device: i32) -> Result<()> {
    // SAFETY: host-only query
    check(unsafe { hs_attn_device_check(device) })
}

/// Flags recorded by kernels that refused an index or ran out of a bounded wait (HS_DEVERR_*); synchronises, clears.
pub fn take_device_error() -> Result<i32> {
    let mut flags = 0i32;
    // SAFETY: `flags` is a valid out-pointer
    check(unsafe { hs_attn_take_device_error(&mut flags) })?;
    Ok(flags)
}

/// Scratch bytes hs_attn_decode needs for a batch of `n_seqs` sequences.
pub fn decode_workspace_bytes(n_seqs: i32, n_q_heads: i32, head_dim: i32) -> Result<i64> {
    // SAFETY: host-only arithmetic
    let n = unsafe { hs_attn_decode_workspace_bytes(n_seqs, n_q_heads, head_dim) };
    if n < 0 { check(n as i32)?; }
    Ok(n)
}

/// KVQuantType {None, Int8, Nf4, Fp4} (crates/hyprstream-rpc-std/schema/model.capnp:252-257) as the library's kind codes.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum KvKind {
    Bf16 = HS_KV_BF16 as isize,
    Int8 = HS_KV_INT8 as isize,
    Nf4 = HS_KV_NF4 as isize,
    Fp4 = HS_KV_FP4 as isize,
}

/// BlockPool (kv_cache.rs:515-680): pages of `page_tokens` tokens, LIFO free list, owner tags.  Owns device memory.
pub struct Pool {
    raw: *mut hs_pool,
}

impl Pool {
    pub fn new(n_blocks: i32, page_tokens: i32, kind: KvKind, block: i32, scale_dtype: i32, n_kv_heads: i32, head_dim: i32) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer; the library validates the rest
        check(unsafe { hs_pool_create(n_blocks, page_tokens, kind as i32, block, scale_dtype, n_kv_heads, head_dim, &mut raw) })?;
        Ok(Pool { raw })
    }
    pub fn num_free(&self) -> i32 {
        // SAFETY: `raw` is a live handle
        unsafe { hs_pool_num_free(self.raw) }
    }
    pub fn as_raw(&self) -> *mut hs_pool {
        self.raw
    }
}

impl Drop for Pool {
    fn drop(&mut self) {
        // SAFETY: the handle is live and dropped once; caches created from the pool must have been dropped before it
        unsafe { hs_pool_destroy(self.raw) }
    }
}

/// LayerKVCache (kv_cache.rs:1029-1900) over device-resident, token-granular storage.  `!Send`, like tch::Tensor: all calls
/// on one cache come from the engine's thread (inference/local.rs:84-85).
pub struct Cache {
    raw: *mut hs_cache,
}

impl Cache {
    /// LayerKVCache::new: contiguous storage grown in 1024-token chunks.
    pub fn new(max_seq_len: i32, kind: KvKind, block: i32, scale_dtype: i32, n_kv_heads: i32, head_dim: i32) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: valid out-pointer
        check(unsafe { hs_cache_create(max_seq_len, kind as i32, block, scale_dtype, n_kv_heads, head_dim, &mut raw) })?;
        Ok(Cache { raw })
    }
    /// LayerKVCache::new_paged: pages from a shared pool, tagged with `owner`.
    pub fn new_paged(max_seq_len: i32, pool: &Pool, owner: i64) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: the pool handle is live; valid out-pointer
        check(unsafe { hs_cache_create_paged(max_seq_len, pool.as_raw(), owner, &mut raw) })?;
        Ok(Cache { raw })
    }
    /// LayerKVCache::update.  SAFETY: `k_new`, `v_new` are device pointers to bf16 [1, n_tokens, n_kv_heads, head_dim]; `sin` / `cos`
    /// are null or device bf16 tables; `stream` is a live CUDA stream of the cache's device (null = default stream).
    pub unsafe fn update(&mut self, k_new: *const c_void, v_new: *const c_void, n_tokens: i32, start_pos: i32, sin: *const c_void,
                         cos: *const c_void, rotary_dim: i32, n_positions: i32, stream: hs_stream_t) -> Result<()> {
        check(hs_cache_update(self.raw, k_new, v_new, n_tokens, start_pos, sin, cos, rotary_dim, n_positions, stream))
    }
    pub fn reserve(&mut self, n_tokens: i32) -> Result<()> {
        // SAFETY: live handle
        check(unsafe { hs_cache_reserve(self.raw, n_tokens) })
    }
    pub fn clear(&mut self) -> Result<()> {
        // SAFETY: live handle
        check(unsafe { hs_cache_clear(self.raw) })
    }
    pub fn truncate_to(&mut self, n_tokens: i32) -> Result<()> {
        // SAFETY: live handle
        check(unsafe { hs_cache_truncate_to(self.raw, n_tokens) })
    }
    pub fn seq_pos(&self) -> i32 {
        // SAFETY: live handle
        unsafe { hs_cache_seq_pos(self.raw) }
    }
    pub fn memory_usage(&self) -> i64 {
        // SAFETY: live handle
        unsafe { hs_cache_memory_usage(self.raw) }
    }
    pub fn as_raw(&self) -> *mut hs_cache {
        self.raw
    }
}

impl Drop for Cache {
    fn drop(&mut self) {
        // SAFETY: live handle, dropped once; pages go back to the pool (kv_cache.rs:1889-1898)
        unsafe { hs_cache_destroy(self.raw) }
    }
}

/// One hs_kv_view over the caches of a batch; owns the device pointer tables.  Stale after any call that releases or
/// replaces a member's storage (see include/hs_attn.h at hs_view_create): check `is_current` or rebuild.
pub struct View {
    raw: *mut hs_view,
}

impl View {
    pub fn new(caches: &[&Cache]) -> Result<Self> {
        let handles: Vec<*mut hs_cache> = caches.iter().map(|c| c.as_raw()).collect();
        let mut raw = ptr::null_mut();
        // SAFETY: `handles` outlives the call; valid out-pointer
        check(unsafe { hs_view_create(handles.as_ptr(), handles.len() as i32, &mut raw) })?;
        Ok(View { raw })
    }
    pub fn get(&self) -> *const hs_kv_view {
        // SAFETY: live handle
        unsafe { hs_view_get(self.raw) }
    }
    pub fn is_current(&self) -> bool {
        // SAFETY: live handle; the member caches must still exist
        unsafe { hs_view_is_current(self.raw) == HS_OK }
    }
}

impl Drop for View {
    fn drop(&mut self) {
        // SAFETY: live handle, dropped once
        unsafe { hs_view_destroy(self.raw) }
    }
}

/// Fused decode attention (replaces cache.get() + GQA expansion + compute_attention_masked for q_len == 1:
/// llama.rs:605-640,710-844,1023-1119; qwen3_5.rs:992-1059 with `gate`).
/// SAFETY: every pointer is a device pointer of the current device with the extent include/hs_attn.h states; `view` comes
/// from a `View` that is current; `stream` is live; no other decode launch is in flight on the device.
pub unsafe fn attn_decode(q: *const c_void, view: *const hs_kv_view, seq_lens: *const i32, n_seqs: i32, n_q_heads: i32, softmax_scale: f32,
                          out: *mut c_void, gate: *const c_void, workspace: *mut c_void, workspace_bytes: i64, stream: hs_stream_t) -> Result<()> {
    check(hs_attn_decode(q, view, seq_lens, n_seqs, n_q_heads, softmax_scale, out, gate, workspace, workspace_bytes, ptr::null_mut(), ptr::null_mut(), stream))
}

/// LayerKVCache::update for a batch through a view (quantise-on-write, optional fused K RoPE).  SAFETY: as `attn_decode`.
pub unsafe fn kv_quantize_write(view: *const hs_kv_view, k_new: *const c_void, v_new: *const c_void, n_seqs: i32, n_tokens: i32,
                                dst_pos: *const i32, sin: *const c_void, cos: *const c_void, rotary_dim: i32, n_positions: i32,
                                stream: hs_stream_t) -> Result<()> {
    check(hs_kv_quantize_write(view, k_new, v_new, n_seqs, n_tokens, dst_pos, sin, cos, rotary_dim, n_positions, stream))
}

/// compute_attention_masked for q_len > 1 (llama.rs:1023-1119; qwen3_5.rs:1012-1059 with `gate`).  SAFETY: as `attn_decode`.
pub unsafe fn attn_prefill_causal(q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, gate: *const c_void, n_seqs: i32,
                                  q_len: i32, kv_len: i32, n_q_heads: i32, n_kv_heads: i32, head_dim: i32, softmax_scale: f32,
                                  stream: hs_stream_t) -> Result<()> {
    check(hs_attn_prefill_causal(q, k, v, out, gate, n_seqs, q_len, kv_len, n_q_heads, n_kv_heads, head_dim, softmax_scale, stream))
}

/// The continuous-batching scheduler (hs_sched_*): see include/hs_attn.h for the loop it expects.
pub struct Scheduler {
    raw: *mut hs_sched,
}

impl Scheduler {
    pub fn new(pool: &Pool, continuous_batch_max: i32, max_seq_len: i32) -> Result<Self> {
        let mut raw = ptr::null_mut();
        // SAFETY: live pool handle, valid out-pointer; the pool must outlive the scheduler
        check(unsafe { hs_sched_create(pool.as_raw(), continuous_batch_max, max_seq_len, &mut raw) })?;
        Ok(Scheduler { raw })
    }
    pub fn submit(&mut self, seq_id: i64, prompt_len: i32, max_new_tokens: i32) -> Result<()> {
        // SAFETY: live handle
        check(unsafe { hs_sched_submit(self.raw, seq_id, prompt_len, max_new_tokens) })
    }
    /// SAFETY: with HS_SCHED_DEVICE_OBJECTS the scheduler's device is current and `stream` is live; the plan's pointers are
    /// valid until the next plan or commit.
    pub unsafe fn plan_step(&mut self, flags: i32, stream: hs_stream_t) -> Result<hs_sched_plan> {
        let mut plan: hs_sched_plan = std::mem::zeroed();
        check(hs_sched_plan_step(self.raw, flags, &mut plan, stream))?;
        Ok(plan)
    }
    pub fn commit_step(&mut self, finished: &[i64]) -> Result<()> {
        // SAFETY: live handle; the slice outlives the call
        check(unsafe { hs_sched_commit_step(self.raw, finished.as_ptr(), finished.len() as i32) })
    }
    pub fn cancel(&mut self, seq_id: i64) -> Result<()> {
        // SAFETY: live handle
        check(unsafe { hs_sched_cancel(self.raw, seq_id) })
    }
}

impl Drop for Scheduler {
    fn drop(&mut self) {
        // SAFETY: live handle, dropped once
        unsafe { hs_sched_destroy(self.raw) }
    }
}
