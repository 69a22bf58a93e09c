//! GPU workers behind tempura's own disaggregated-serving traits.
//!
//! `GpuPrefillWorker` and `GpuDecodeWorker` implement `PrefillWorker` and `DecodeWorker`
//! (engine/src/disaggregated.rs:7-19), so `DisaggregatedPipeline::new(Box::new(prefill), Box::new(decode))`
//! (engine/src/disaggregated.rs:135-151) is unchanged.  What changes is what travels: the reference's
//! `SessionTransfer.cache` holds every layer's K and V as `Vec<f32>` (engine/src/kv_cache.rs:514-522); here the
//! K/V stay in the prefill GPU's paged pool, `cache.k_data` / `cache.v_data` stay empty, and the block table that
//! names the sequence's pages crosses through a ticket queue the two workers of a pair share.  `decode` allocates
//! destination pages, plans the handoff, and one kernel on the prefill GPU gathers through the source table and
//! stores into the decode pool (same GPU, or a peer over NVLink).
//!
//! Source only: this file was written in an environment without `cargo` / `rustc` and has never been compiled.
//! `tests/test_rust_shim.py` checks every `tkv_sys::` call below against include/tkv.h (name, argument count).

use std::collections::VecDeque;
use std::ffi::{c_void, CStr};
use std::sync::{Arc, Mutex};

use tempura_engine::disaggregated::{DecodeWorker, PrefillWorker};
use tempura_engine::kv_cache::KvCacheTransfer;
use tempura_engine::session::SessionTransfer;
use tempura_kernel_api::KernelError;
use tempura_kernels::SamplingParams;
use tkv_sys::*;

/// Status code of the C ABI -> `KernelError` (kernel-api/src/lib.rs:5-13).  Code 1 carries
/// "dimension mismatch: expected E, got G" in its text, which is parsed back into the typed variant; every other
/// non-zero code folds into `InvalidConfig` with the library's text, the way the reference folds a driver `rc`
/// (kernels/src/kv_scatter_write.rs:855-859).
pub fn status(rc: i32) -> Result<(), KernelError> {
    if rc == TKV_OK {
        return Ok(());
    }
    let mut buf = [0 as std::os::raw::c_char; 512];
    unsafe { tkv_last_error(buf.as_mut_ptr(), buf.len()) };
    let msg = unsafe { CStr::from_ptr(buf.as_ptr()) }.to_string_lossy().into_owned();
    if rc == TKV_ERR_DIMENSION_MISMATCH {
        if let Some((expected, got)) = parse_expected_got(&msg) {
            return Err(KernelError::DimensionMismatch { expected, got });
        }
    }
    Err(KernelError::InvalidConfig(format!("tkv status {rc}: {msg}")))
}

fn parse_expected_got(msg: &str) -> Option<(usize, usize)> {
    let rest = msg.split("expected ").nth(1)?;
    let (e, rest) = rest.split_once(", got ")?;
    let g: String = rest.chars().take_while(|c| c.is_ascii_digit()).collect();
    Some((e.trim().parse().ok()?, g.parse().ok()?))
}

/// A paged KV pool on one GPU in the layout of `GpuKvPagePool` (engine/src/cutile_kv_cache.rs:1584-1602): per layer
/// one K and one V tensor `[page][token_in_page][kv_head][head_dim]`.  Owns the pointer arrays `TkvPool` points at.
pub struct PoolDesc {
    pub device: i32,
    pub dtype: i32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub block_size: u32,
    pub total_blocks: u32,
    pub k_layer_ptrs: Vec<u64>,
    pub v_layer_ptrs: Vec<u64>,
    pub k_scales: u64,
    pub v_scales: u64,
    pub refcounts: u64,
}

impl PoolDesc {
    fn as_c(&self) -> TkvPool {
        TkvPool {
            device: self.device,
            dtype: self.dtype,
            n_layers: self.k_layer_ptrs.len() as u32,
            n_kv_heads: self.n_kv_heads,
            head_dim: self.head_dim,
            block_size: self.block_size,
            total_blocks: self.total_blocks,
            reserved: 0,
            k_layer_ptrs: self.k_layer_ptrs.as_ptr(),
            v_layer_ptrs: self.v_layer_ptrs.as_ptr(),
            k_scales: self.k_scales,
            v_scales: self.v_scales,
            refcounts: self.refcounts,
        }
    }
}

/// What `prefill` leaves for `decode`: which pages of the prefill pool hold the sequence.
struct Ticket {
    seed: u64,
    position: usize,
    block_table: Vec<u32>,
}

/// The queue one prefill / decode pair shares (`DisaggregatedPipeline::generate` calls `prefill` then `decode`
/// on the same thread, so the queue is FIFO with at most a few entries).
#[derive(Default)]
pub struct HandoffQueue(Mutex<VecDeque<Ticket>>);

/// The model side of a prefill worker: runs the prompt on its GPU, K/V written into `pool`'s pages.
pub trait PrefillEngine: Send + Sync {
    /// Returns the sequence's block table (page ids in `pool`, logical order) and the last logits.
    fn run_prompt(&self, token_ids: &[u32], seed: u64) -> (Vec<u32>, Vec<f32>);
    fn pool(&self) -> &PoolDesc;
    fn dims(&self) -> (usize, usize, usize); // (num_layers, num_kv_heads, head_dim)
}

/// The model side of a decode worker: owns the destination pool and its page allocator, and decodes from it.
pub trait DecodeEngine: Send + Sync {
    fn pool(&self) -> &PoolDesc;
    /// `PageAllocator::allocate` (engine/src/kv_cache.rs:776-778) n times, or a `PageRunAllocator` run.
    fn allocate_pages(&self, n: usize) -> Result<Vec<u32>, KernelError>;
    /// CUDA stream of the PREFILL GPU on which the handoff kernel is enqueued.
    fn handoff_stream(&self) -> *mut c_void;
    /// u32 completion flag in page-locked host memory, and the next generation value to publish there.
    fn completion_flag(&self) -> (u64, u32);
    /// Ordinary decoding over the adopted pages (engine/src/disaggregated.rs:82-126).
    fn decode_from_pool(
        &self,
        block_table: &[u32],
        transfer: SessionTransfer,
        max_new_tokens: usize,
        params: &SamplingParams,
        eos_token: Option<u32>,
    ) -> Vec<u32>;
}

pub struct GpuPrefillWorker<E: PrefillEngine> {
    engine: E,
    queue: Arc<HandoffQueue>,
}

impl<E: PrefillEngine> GpuPrefillWorker<E> {
    pub fn new(engine: E, queue: Arc<HandoffQueue>) -> Self {
        Self { engine, queue }
    }
}

impl<E: PrefillEngine> PrefillWorker for GpuPrefillWorker<E> {
    fn prefill(&self, token_ids: &[u32], seed: u64) -> SessionTransfer {
        let (block_table, last_logits) = self.engine.run_prompt(token_ids, seed);
        let (num_layers, num_kv_heads, head_dim) = self.engine.dims();
        self.queue.0.lock().unwrap().push_back(Ticket { seed, position: token_ids.len(), block_table });
        SessionTransfer {
            // geometry only: the K/V never leave the GPUs (engine/src/kv_cache.rs:514-522)
            cache: KvCacheTransfer {
                k_data: Vec::new(),
                v_data: Vec::new(),
                seq_len: token_ids.len(),
                num_layers,
                num_kv_heads,
                head_dim,
            },
            position: token_ids.len(),
            seed,
            last_logits,
        }
    }
}

pub struct GpuDecodeWorker<D: DecodeEngine> {
    engine: D,
    src_pool: Arc<PoolDesc>,
    queue: Arc<HandoffQueue>,
    timeout_us: u64,
}

impl<D: DecodeEngine> GpuDecodeWorker<D> {
    /// `devices`: the CUDA ordinals of the pair; peer access is enabled once (`tkv_init`).
    pub fn new(engine: D, src_pool: Arc<PoolDesc>, queue: Arc<HandoffQueue>, devices: &[i32]) -> Result<Self, KernelError> {
        status(unsafe { tkv_init(devices.as_ptr(), devices.len() as i32) })?;
        Ok(Self { engine, src_pool, queue, timeout_us: 10_000_000 })
    }

    /// `KvCache::from_transfer` (engine/src/kv_cache.rs:419-431) as one planned GPU move.
    fn adopt(&self, ticket: &Ticket) -> Result<Vec<u32>, KernelError> {
        let bs = self.src_pool.block_size as usize;
        let n_blocks = (ticket.position + bs - 1) / bs;
        if ticket.block_table.len() < n_blocks {
            return Err(KernelError::DimensionMismatch { expected: n_blocks, got: ticket.block_table.len() });
        }
        let dst_table = self.engine.allocate_pages(n_blocks)?;
        let seq_lens = [ticket.position as u32];
        let (src, dst) = (self.src_pool.as_c(), self.engine.pool().as_c());
        let batch = TkvBatch {
            n_seqs: 1,
            table_stride: n_blocks as u32,
            table_layer_stride: 0,
            reserved: 0,
            seq_lens: seq_lens.as_ptr(),
            prefix_lens: std::ptr::null(),
            src_tables: ticket.block_table.as_ptr(),
            dst_tables: dst_table.as_ptr(),
        };
        let mut plan: *mut tkv_plan = std::ptr::null_mut();
        status(unsafe { tkv_plan_create(&src, &dst, &batch, std::ptr::null(), TKV_PLAN_DEFAULT, &mut plan) })?;
        let (flag, generation) = self.engine.completion_flag();
        let sent = status(unsafe { tkv_handoff_enqueue(plan, self.engine.handoff_stream(), flag, generation) })
            .and_then(|_| status(unsafe { tkv_flag_wait_host(self.src_pool.device, flag, generation, self.timeout_us) }));
        unsafe { tkv_plan_destroy(plan) };
        sent.map(|_| dst_table)
    }
}

impl<D: DecodeEngine> DecodeWorker for GpuDecodeWorker<D> {
    fn decode(
        &self,
        transfer: SessionTransfer,
        max_new_tokens: usize,
        params: &SamplingParams,
        eos_token: Option<u32>,
    ) -> Vec<u32> {
        let ticket = {
            let mut q = self.queue.0.lock().unwrap();
            let at = q
                .iter()
                .position(|t| t.seed == transfer.seed && t.position == transfer.position)
                .expect("decode called without a matching prefill");
            q.remove(at).unwrap()
        };
        // the reference's workers panic on a failed allocation (engine/src/kv_cache.rs:980); so does this one
        let dst_table = self.adopt(&ticket).expect("KV handoff failed");
        self.engine.decode_from_pool(&dst_table, transfer, max_new_tokens, params, eos_token)
    }
}
