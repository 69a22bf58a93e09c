/*
 * tkv.h -- C ABI of the B200 (sm_100a) prefill->decode KV-cache handoff.
 *
 * This is the boundary a tempura build links through `build.rs`: plain pointers
 * and sizes, POD structs, int32_t status codes.  Device memory is addressed as
 * raw uint64_t CUdeviceptr values and streams as raw CUstream/cudaStream_t
 * handles (void*), the conventions of the reference's own launchers
 * (kernels/src/kv_scatter_write.rs:822-861, engine/src/cutile_kv_cache.rs:92-126).
 * The library never allocates or frees pool memory; the caller keeps pools,
 * tables and streams alive until the stream work completes.  One host thread
 * per device, as in the reference (engine/src/cutile_kv_cache.rs:217-220).
 *
 * Citations are paths inside the tempura repository.
 */
#ifndef TKV_H
#define TKV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  1 and 2 map onto kernel-api/src/lib.rs:5-13 (KernelError::
 * DimensionMismatch / InvalidConfig); 3 carries a CUDA error the way
 * kernels/src/kv_scatter_write.rs:855-859 folds `rc` into InvalidConfig;
 * 5 is the recoverable PoolExhausted of engine/src/cutile_kv_cache.rs:27-44. */
enum {
    TKV_OK = 0,
    TKV_ERR_DIMENSION_MISMATCH = 1,
    TKV_ERR_INVALID_CONFIG = 2,
    TKV_ERR_CUDA = 3,
    TKV_ERR_TIMEOUT = 4,
    TKV_ERR_POOL_EXHAUSTED = 5
};

/* engine/src/cutile_kv_cache.rs:57-62 (KvDtype) */
enum { TKV_DTYPE_F32 = 0, TKV_DTYPE_F16 = 1, TKV_DTYPE_E4M3 = 2 };

/* A paged KV pool on one device.  Layout per layer, separately for K and V:
 * [block][token_in_block][kv_head][head_dim], i.e. the byte offset of a block
 * is block * block_size * n_kv_heads * head_dim * elem
 * (engine/src/cutile_kv_cache.rs:1584-1602, engine/src/kv_cache.rs:925-936;
 * row formula kernels/src/attention.rs:472-484).                             */
typedef struct TkvPool {
    int32_t device;               /* CUDA ordinal that owns the memory            */
    int32_t dtype;                /* TKV_DTYPE_*                                   */
    uint32_t n_layers;            /* layers held by this pool                      */
    uint32_t n_kv_heads;          /* kv heads held by this pool                    */
    uint32_t head_dim;
    uint32_t block_size;          /* tokens per block (reference constant: 16)     */
    uint32_t total_blocks;
    uint32_t reserved;
    const uint64_t* k_layer_ptrs; /* HOST array [n_layers] of device addresses     */
    const uint64_t* v_layer_ptrs;
    uint64_t k_scales;            /* E4M3 pools: device float[n_layers][total_blocks][n_kv_heads] */
    uint64_t v_scales;            /*   (0 for other dtypes, or for unscaled E4M3)  */
    uint64_t refcounts;           /* device uint32_t[total_blocks], or 0           */
} TkvPool;

/* One batch of finished prompts.  Tables hold physical block ids, logical
 * block i of sequence q at tables[q*table_stride + i]
 * (BlockTable, engine/src/kv_cache.rs:836-893).  Tokens
 * [prefix_lens[q], seq_lens[q]) move; tokens below prefix_lens[q] are shared
 * prefix blocks already resident on the destination (prefix_lens must be a
 * multiple of block_size).                                                    */
typedef struct TkvBatch {
    uint32_t n_seqs;
    uint32_t table_stride;
    uint32_t table_layer_stride;  /* 0: one table per sequence for all layers (GPU pool,
                                     engine/src/cutile_kv_cache.rs:1054-1072); else layer l's
                                     tables start l*table_layer_stride entries further
                                     (per-layer tables, engine/src/kv_cache.rs:925-936) */
    uint32_t reserved;
    const uint32_t* seq_lens;     /* HOST arrays */
    const uint32_t* prefix_lens;  /* may be NULL (all zero) */
    const uint32_t* src_tables;
    const uint32_t* dst_tables;
} TkvBatch;

/* Which heads and layers one prefill->decode pair moves. */
typedef struct TkvShard {
    uint32_t src_head_begin, dst_head_begin, n_heads;
    uint32_t src_layer_begin, dst_layer_begin, n_layers;
} TkvShard;

typedef struct TkvPairing {
    int32_t prefill_device;
    int32_t decode_device;
    TkvShard shard;               /* head/layer ranges in GLOBAL (unsharded) numbering:
                                     src_* == dst_* */
} TkvPairing;

typedef struct TkvStats {
    uint64_t payload_bytes;       /* source bytes of the moved tokens                    */
    uint64_t bytes_read;          /* algorithmic bytes read per enqueue                  */
    uint64_t bytes_written;       /* algorithmic bytes written per enqueue (incl. scales) */
    uint64_t n_blocks;            /* (src block, dst block) pairs in the work list        */
    uint64_t n_chunks;            /* blocks * layers * 2 (K and V)                        */
    uint64_t n_tokens;
    uint64_t n_prefix_refs;       /* shared prefix block references in the batch          */
    uint64_t worklist_bytes;      /* host->device bytes uploaded by plan create/update    */
    uint32_t grid, block;         /* launch shape of the handoff kernel                   */
    uint32_t kernel_variant;      /* TKV_VARIANT_* actually selected                      */
    uint32_t peer;                /* 1 when destination is another device                 */
} TkvStats;

/* A contiguous transfer buffer: the batch form of KvCacheTransfer{k_data, v_data}
 * (engine/src/kv_cache.rs:514-522).  For each moved layer, K then V, it holds the moved
 * blocks of sequence 0, 1, ... in work-list order, each block `block_size` rows of
 * [kv_head][head_dim] restricted to the shard's heads; one sequence's rows are therefore
 * contiguous [token][kv_head][head_dim], which is what k_data[layer] is.  With n moved
 * blocks, layer l's K plane starts at data + (2l) * n * block_bytes and its V plane one
 * plane later.  An E4M3 buffer may carry scales: float[K|V][layer][block][kv_head].
 * `device` is the GPU whose kernel touches the buffer.  host_memory == 0: the buffer is
 * device memory of that GPU.  host_memory == 1: it is page-locked host memory that GPU can
 * address (cudaHostAlloc / cudaHostRegister); the kernel then reads or writes it over PCIe
 * directly, which is the DRAM swap tier of engine/src/cutile_kv_cache.rs:1127-1368 without
 * a staging copy.                                                                    */
typedef struct TkvTransfer {
    int32_t device;
    int32_t dtype;                /* TKV_DTYPE_* of the buffer                          */
    uint32_t host_memory;
    uint32_t reserved;
    uint64_t data;
    uint64_t bytes;               /* capacity; at least tkv_transfer_bytes(...)          */
    uint64_t scales;              /* 0, or the scale array described above               */
} TkvTransfer;

typedef struct tkv_plan tkv_plan;

/* Plan flags */
enum {
    TKV_PLAN_DEFAULT = 0,
    TKV_PLAN_ALLOW_SHARED_DST = 1,  /* skip the "destination block ids are unique" check   */
    TKV_PLAN_FORCE_VECTOR = 2,      /* use the register kernels (vector copy, warp-per-head FP8, element-wide F32 casts) */
    TKV_PLAN_FORCE_BULK = 4,        /* use the shared-memory bulk-copy pipelines (copy ring, staged FP8) */
    TKV_PLAN_INT_QUANTIZER = 8,     /* FP8: integer bit-math encoder instead of cvt + flush */
    TKV_PLAN_PEER_BULK_STORES = 16, /* same-dtype move to a peer: use the bulk-copy ring (bulk stores
                                       shared -> peer global) instead of register stores; measured
                                       equal over NVLink, so it is opt-in.  The staged FP8 kernel
                                       always stores whole rows in bulk, local or peer.            */
    TKV_PLAN_PULL = 32              /* pools on two devices, same dtype: the kernel runs on the DESTINATION
                                       pool's device (enqueue on one of its streams), fetches the source
                                       blocks with ordinary loads over the peer mapping and stores locally;
                                       the completion flag is then local to the receiver.  Needs the
                                       destination device to reach the source pool (tkv_init, or
                                       tkv_ipc_import on the destination side).                     */,
    TKV_PLAN_STAGE_HOST = 64        /* from_transfer plans whose buffer is page-locked host memory: instead of the kernel
                                       reading host memory over PCIe (51 GB/s measured), the copy engine brings one layer at a
                                       time (several where a layer is under 4 MiB) into two device buffers of the plan
                                       (55.6 GB/s measured) while the previous layer's kernel runs.  The plan owns those
                                       buffers and a stream; not for buffers that carry scales.                      */
};
enum { TKV_VARIANT_VECTOR = 1, TKV_VARIANT_BULK = 2, TKV_VARIANT_FP8_WARP = 3, TKV_VARIANT_FP8_GENERIC = 4,
       TKV_VARIANT_CAST_GENERIC = 5, TKV_VARIANT_FP8_STAGED = 6, TKV_VARIANT_DEQUANT = 7, TKV_VARIANT_CAST_VEC = 8,
       TKV_VARIANT_WIDE = 9 /* the register copy with 32-byte accesses (tkv_plan_tune_vector; the default of a pulled plan) */ };

/* ---- library -------------------------------------------------------------- */
/* Copies the calling thread's last error text (NUL-terminated) into buf. */
void tkv_last_error(char* buf, size_t len);
int32_t tkv_last_cuda_error(void);
const char* tkv_version(void);

/* Enables peer access between every ordered pair of `devices` that supports it.
 * Replaces nothing in the reference (it has no multi-device path:
 * kernels/src/allreduce.rs:38-43); needed once per process before a plan whose
 * pools live on two devices.                                                  */
int32_t tkv_init(const int32_t* devices, int32_t n_devices);
int32_t tkv_shutdown(void);

/* ---- the handoff ---------------------------------------------------------- */
/* Validates shapes, tables and refcount rules, builds the (src block, dst
 * block, valid tokens) work list and uploads it to the source device.
 * Replaces the gather half KvCache::to_transfer / PagedKvCache::k_contiguous
 * (engine/src/kv_cache.rs:402-417,1032-1060) and the scatter half
 * KvCache::from_transfer / PagedKvCache::append_kv / Fp8PagedKvCache::append_kv
 * (engine/src/kv_cache.rs:419-431,986-1004,1204-1225) as one planned move.
 * dtype pairs: same dtype (byte copy), F16->E4M3 (per-block scales when the
 * destination has scale arrays, else unscaled as kernels/src/kv_scatter_write.rs:
 * 176-273), F32->F16 and F32->E4M3 (append_kv's casts, engine/src/kv_cache.rs:
 * 209-221; kernels/src/cutile_elementwise.rs:82-178), and E4M3->F16 / E4M3->F32,
 * the reader's side of the FP8 cache (Fp8PagedKvCache::k_contiguous,
 * engine/src/kv_cache.rs:1241-1271): exact decode of kernels/src/e4m3.rs:27-41 times
 * the source pool's per-block scale when it has scale arrays.                  */
int32_t tkv_plan_create(const TkvPool* src, const TkvPool* dst, const TkvBatch* batch,
                        const TkvShard* shard /* NULL = everything */, uint32_t flags,
                        tkv_plan** out);
/* The two halves on their own, against a contiguous transfer buffer.
 * to_transfer: gather through the source tables into the buffer (KvCache::to_transfer,
 * PagedKvCache::k_contiguous / v_contiguous, engine/src/kv_cache.rs:402-417,1032-1060;
 * swap_out, engine/src/cutile_kv_cache.rs:1127-1230); batch->dst_tables is not read.
 * A buffer dtype narrower than the pool's casts on the way (F16 pool -> E4M3 buffer with
 * scales is the "cast before the wire" form).
 * from_transfer: scatter the buffer into the destination pool through the destination
 * tables (KvCache::from_transfer, append_kv, engine/src/kv_cache.rs:419-431,986-1004;
 * swap_in, engine/src/cutile_kv_cache.rs:1232-1368); batch->src_tables is not read, and an
 * E4M3 buffer with scales lands in an E4M3 pool with scales.  The shard's head and layer
 * ranges apply to the pool; the buffer holds exactly the shard.  to_transfer runs with
 * tkv_handoff_enqueue on a stream of the source pool's device, from_transfer on a stream
 * of the buffer's device (xfer->device), which stores into the pool locally or as a peer. */
int32_t tkv_plan_create_to_transfer(const TkvPool* src, const TkvTransfer* xfer, const TkvBatch* batch,
                                    const TkvShard* shard /* NULL = everything */, uint32_t flags,
                                    tkv_plan** out);
int32_t tkv_plan_create_from_transfer(const TkvTransfer* xfer, const TkvPool* dst, const TkvBatch* batch,
                                      const TkvShard* shard /* NULL = everything */, uint32_t flags,
                                      tkv_plan** out);
/* Bytes a transfer buffer needs for n_blocks moved blocks, and the number of blocks a
 * batch moves (sum over sequences of ceil(seq_len / block_size) - prefix_len / block_size). */
uint64_t tkv_transfer_bytes(uint32_t n_layers, uint32_t n_heads, uint32_t head_dim, uint32_t block_size,
                            int32_t dtype, uint64_t n_blocks);
uint64_t tkv_batch_blocks(const TkvBatch* batch, uint32_t block_size);

/* Re-validates a new batch into an existing plan (same pools, shard and flags; no allocation
 * unless the work list outgrew its capacity).  The work list travels to the device in stream
 * order at the head of the next tkv_handoff_enqueue, so an update may be issued while the
 * plan's previous handoff is still running on that same stream.                          */
int32_t tkv_plan_update(tkv_plan* plan, const TkvBatch* batch);
int32_t tkv_plan_destroy(tkv_plan* plan);
int32_t tkv_plan_stats(const tkv_plan* plan, TkvStats* out);

/* Asynchronous on `stream` (a stream of the SOURCE device): gathers through the
 * source tables, converts if asked, and stores straight into the destination
 * pool (local or peer).  If done_flag != 0 the last CTA to finish stores
 * flag_value there (system-scope release) after all payload stores.
 * Launch convention follows kernels/src/kv_scatter_write.rs:822-861.          */
int32_t tkv_handoff_enqueue(tkv_plan* plan, void* stream, uint64_t done_flag, uint32_t flag_value);

/* No counterpart in the reference.  A same-dtype handoff (gather through the source
 * tables, store into the destination pool) for callers that must not allocate device
 * memory at handoff time: an engine whose KV pools already own nearly all of HBM, so a
 * late cudaMalloc can fail; a serving loop that cannot afford the device-wide stall a
 * cudaMalloc/cudaFree causes while other streams are decoding; a host that hands this
 * library a fixed memory budget.  Instead of a plan's device buffer, the layer
 * pointers and the work list live in ONE fixed array compiled into the library
 * (TKV_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads it, held until
 * the process exits).  The call checks its arguments the way tkv_plan_create does
 * (geometry, shard, table ids, duplicate and shared-prefix destinations, and that a
 * destination on another device was mapped by tkv_init or tkv_ipc_import), copies the
 * work list into that array on `stream` and launches the copy kernel behind it; it
 * calls no cudaMalloc, cudaFree or other allocating routine.  What it does not do that
 * a plan does: casts (both pools must have one dtype), E4M3 pools with scale arrays
 * (refused; a plan carries the scales along), completion flags, reference counts.
 *   - Limits: at most TKV_NOALLOC_MAX_BLOCK_PAIRS (source block, destination block)
 *     pairs and TKV_NOALLOC_MAX_LAYERS layers per call; more is refused with
 *     TKV_ERR_INVALID_CONFIG and nothing is launched.
 *   - The first call on a device looks up the array's device address; make that call
 *     before any stream capture begins on that device.  A call on a stream that is being
 *     captured is refused with TKV_ERR_INVALID_CONFIG: the work list is uploaded from host
 *     memory that the next call rewrites.
 *   - Every call on a device shares the array and overwrites the previous call's
 *     contents: calls whose GPU work may overlap (different streams, or different
 *     threads) race on it.  Order them on one stream or with events.
 *   - `stream` belongs to the SOURCE pool's device.                              */
#define TKV_NOALLOC_MAX_BLOCK_PAIRS 16384u
#define TKV_NOALLOC_MAX_LAYERS 128u
#define TKV_NOALLOC_SCRATCH_BYTES (4u * TKV_NOALLOC_MAX_LAYERS * 8u + 256u + TKV_NOALLOC_MAX_BLOCK_PAIRS * 16u)
int32_t tkv_handoff_noalloc(const TkvPool* src, const TkvPool* dst, const TkvBatch* batch,
                            const TkvShard* shard /* NULL = everything */, void* stream);

/* Tuning of the bulk-copy variant (ring depth per CTA, CTAs per SM, bytes per ring
 * stage; without this call 32 KiB, or 8 KiB for a batch with fewer than four chunks per SM); ctas_per_sm 0 derives it from
 * the stage size.  The staged FP8 kernel takes the
 * ring depth and the CTA cap from the same call (its stage is one chunk).  No reference
 * counterpart.
 * Takes effect at the next enqueue.                                             */
int32_t tkv_plan_tune_bulk(tkv_plan* plan, uint32_t stages, uint32_t ctas_per_sm, uint32_t stage_bytes);
/* The register copy kernel's access shape: bytes per load / store (16, or 32 where every address keeps
 * 32-byte alignment and chunks are contiguous; 0 = the library's choice), loads a thread keeps in flight
 * (4, 8, 16; the 32-byte kernel only), cache policy of the stores (0 default, 1 streaming, 2 no L1
 * allocation; the 32-byte kernel only).  No reference counterpart.  Takes effect at the next enqueue. */
int32_t tkv_plan_tune_vector(tkv_plan* plan, uint32_t bytes_per_access, uint32_t unroll, uint32_t store_hint);
/* Two choices that matter to small handoffs.  flag_mode: who writes the completion flag -- 0 the library's choice
 * (a stream-ordered 32-bit write behind the kernel where the launching device's stream can reach the word: its own
 * memory or page-locked host memory; the kernel's last CTA for a peer GPU's word and inside a stream capture), 1 always
 * the kernel's last CTA, 2 the stream write wherever it is possible.  inline_list: 0 the library's choice (a host-built
 * work list of at most 256 pairs and 64 layers rides in the kernel's parameter block when the batch has few chunks per
 * SM, and nothing is uploaded for it), 1 never, 2 whenever it fits.  No reference counterpart. */
int32_t tkv_plan_tune_small(tkv_plan* plan, uint32_t flag_mode, uint32_t inline_list);
/* Caps the resident CTAs per SM of the register (non-bulk) kernels; 0 = as many as fit. */
int32_t tkv_plan_tune_grid(tkv_plan* plan, uint32_t ctas_per_sm);
/* Reads the plan's device-side error word (synchronous): 0, or 1 when a kernel of
 * this plan gave up on one of its own bounded waits.                            */
int32_t tkv_plan_error(const tkv_plan* plan, uint32_t* device_error);

/* Bounded waits on a completion flag (uint32_t in device memory of the
 * waiting side).  Flag values are generations: successive handoffs publish increasing
 * values, and a wait for `expected` returns once the flag has reached OR PASSED it
 * ((int32_t)(flag - expected) >= 0), so a waiter that polls late cannot miss a
 * generation that a following handoff has already overwritten.  The host form also accepts
 * a flag in page-locked host memory (the kernel's system-scope store lands there) and then
 * reads it in place instead of copying.  Host form polls with small device->host copies; device form
 * enqueues a one-thread kernel that spins at most max_spins times and records
 * TKV_OK or TKV_ERR_TIMEOUT in *status (device uint32_t).  Neither can hang.   */
int32_t tkv_flag_wait_host(int32_t device, uint64_t flag, uint32_t expected, uint64_t timeout_us);
int32_t tkv_flag_wait_enqueue(void* stream, uint64_t flag, uint32_t expected, uint64_t max_spins,
                              uint64_t status);

/* refcounts[block] += 1 (delta > 0) or saturating -= 1 (delta < 0) for every
 * shared prefix block reference of the plan's batch, on the destination pool's
 * refcount array.  PrefixCacheTable::probe / release
 * (engine/src/kv_cache.rs:622-647,688-693), RadixTree::lookup / release
 * (engine/src/prefix_cache.rs:58-97), at block granularity.                    */
int32_t tkv_refcount_apply(tkv_plan* plan, int32_t delta, void* stream);

/* Prefill GPU i <-> decode GPU i + P, P = max(1, n_gpus / 2); KV heads split
 * evenly over the P pairs, layers when there are fewer heads than pairs.  With
 * n_gpus == 1 the single device plays both roles.  `out` holds P entries.
 * (No reference counterpart: engine/src/disaggregated.rs:21-62 pairs two local
 * workers in one process.)                                                     */
int32_t tkv_pairing_make(int32_t n_gpus, uint32_t n_layers, uint32_t n_kv_heads, TkvPairing* out,
                         int32_t out_cap, int32_t* n_pairs);

/* ---- element casts (kernels/src/cutile_elementwise.rs:82-212) -------------- */
int32_t tkv_cast(uint64_t src, int32_t src_dtype, uint64_t dst, int32_t dst_dtype, uint64_t n,
                 void* stream);
/* Device self-check of the FP8 encoder used on the fast path against the
 * integer bit-math port of kernels/src/e4m3.rs:50-94 over every f32 whose low
 * `skip_bits` bits are zero (0 = all 2^32).  Writes the mismatch count.        */
int32_t tkv_selfcheck_e4m3(uint32_t skip_bits, uint64_t* mismatches);
/* Device self-check of the scaled fast path (flush threshold on the F16 magnitude +
 * hardware conversion) against the integer port applied to the same FP32 product, for
 * every finite non-zero block amax and every F16 value of magnitude <= amax.       */
int32_t tkv_selfcheck_scaled_quant(uint64_t* mismatches);

/* ---- contiguous copies (engine/src/cutile_kv_cache.rs:449-468,619-631) ------- */
/* The copy-engine route: one asynchronous copy of `bytes` on `stream` between any two
 * addresses the stream's device can reach (its own memory, a peer pool mapped by tkv_init
 * or tkv_ipc_import, page-locked host memory).  This is what the reference's per-layer
 * cuMemcpyDtoDAsync / DtoHAsync / HtoDAsync calls are; contiguous runs (a GpuKvRun's live
 * prefix) can keep using it, and the benchmark uses it as its peer-copy yardstick.       */
int32_t tkv_memcpy_enqueue(uint64_t dst, uint64_t src, uint64_t bytes, void* stream);

/* ---- bits checksum (engine/src/cutile_kv_cache.rs:1274-1368) --------------- */
/* Wrapping sum of the f32 bit patterns of n elements (narrow dtypes widened). */
int32_t tkv_bits_checksum(uint64_t data, int32_t dtype, uint64_t n, void* stream, uint64_t* out);

/* ---- cross-process mapping of a destination pool --------------------------- */
/* One process per GPU: the decode process exports its pool allocation, the
 * prefill process imports it and uses the mapped address in TkvPool.  The
 * import is made on the current device and its address range is remembered:
 * a plan whose destination layer pointers lie inside it passes the peer check
 * whatever ordinal the pool gives the owning device.                          */
int32_t tkv_ipc_export(uint64_t devptr, uint8_t handle[64], uint64_t* offset_in_allocation);
int32_t tkv_ipc_import(const uint8_t handle[64], uint64_t offset_in_allocation, uint64_t* devptr);
int32_t tkv_ipc_close(uint64_t devptr, uint64_t offset_in_allocation);

/* ---- decode attention over the paged pool (the FP8 cache's consumer) ---------- */
/* One query token per sequence, grouped-query heads, K/V rows resolved through the block
 * table, for one layer of an F16 or E4M3 pool; an E4M3 pool with scale arrays reads as
 * decode(byte) * scale[layer][block][kv_head].  Replaces the reference's per-dtype decode
 * twins OxideDecodeAttn::forward_d2d_ptrs_{f16,e4m3} / forward_batch_d2d_ptrs_{f16,e4m3}
 * (kernels/src/oxide_decode_attn_host.rs:198-260,682-760), which read a contiguous run
 * and assume unscaled E4M3; the arithmetic is paged_flash_attention
 * (kernels/src/attention.rs:486-590) to FP16-input, FP32-accumulate tolerance.
 * As there, kv_lens is a DEVICE array whose values are read when the kernel runs;
 * max_kv_len (host) sizes the grid, the table rows and the scratch, and bounds every length read.  head_dim 128, 16-token blocks,
 * 1..8 query heads per kv head.  All pointers are device memory of pool->device.       */
typedef struct TkvDecodeAttn {
    uint32_t n_seqs, n_q_heads, table_stride, layer, max_kv_len;
    float sm_scale;               /* usually 1 / sqrt(head_dim)                              */
    uint32_t split_tokens;        /* cached tokens per CTA, a multiple of 64 (of 32 in the
                                     whole-block form); 0 = library's choice */
    uint32_t flags;               /* TKV_ATTN_*                                               */
    uint64_t q;                   /* f32 [n_seqs][n_q_heads][head_dim]                        */
    uint64_t out;                 /* f32, same shape                                          */
    uint64_t tables;              /* u32 [n_seqs][table_stride] block ids                     */
    uint64_t kv_lens;             /* u32 [n_seqs]                                             */
    uint64_t scratch;             /* tkv_decode_attn_scratch_bytes(...) bytes of device memory  */
    uint64_t scratch_bytes;
    uint64_t total_kv_tokens;     /* optional hint: sum of kv_lens as the host knows it (0 = unknown);
                                     lets the library size the token ranges: one wave of CTAs for a
                                     few sequences, several waves of short ranges for many            */
    uint64_t status;              /* 0, or a device u32 (zero it before the launch) that receives the first
                                     failure: TKV_ERR_TIMEOUT if a bounded wait gave up, TKV_ERR_INVALID_CONFIG
                                     if kv_lens held a value above max_kv_len (clamped to it) or a table entry
                                     named a block outside the pool (never read); the output is then not valid */
} TkvDecodeAttn;
enum { TKV_ATTN_DEFAULT = 0,
       TKV_ATTN_PER_HEAD_CTAS = 1, /* one CTA per (sequence, kv head, split) with per-lane copies, the
                                      form used when a pool has more than 8 kv heads               */
       TKV_ATTN_MMA_SYNC = 2       /* whole-block form on warp-level mma.sync instead of tcgen05 with
                                      tensor-memory accumulators (the default where the shape allows:
                                      8 kv heads, 4 query heads per kv head)                        */ };
/* Scratch for the partial results: two per token range and query head (running maximum, row sum, head_dim
 * numerators each), sized for the smallest range the library may choose unless split_tokens fixes one.  */
uint64_t tkv_decode_attn_scratch_bytes(uint32_t n_seqs, uint32_t n_q_heads, uint32_t head_dim, uint32_t max_kv_len,
                                       uint32_t split_tokens /* 0 = default */);
int32_t tkv_decode_attn_enqueue(const TkvPool* pool, const TkvDecodeAttn* args, void* stream);

/* The prefill-side twin: causal attention of n_tokens NEW tokens of ONE sequence over its paged cache, their K/V rows
 * already written at positions start_pos .. start_pos + n_tokens - 1; query token t attends to positions
 * 0 .. start_pos + t (paged_flash_attention, kernels/src/attention.rs:486-590, with a causal bound per query token; the
 * reference's kernel for the FP8 pool, cutile_flash_attn_heads_paged_e4m3, kernels/src/cutile_flash_attention.rs:868, reads
 * unscaled bytes, this one applies the per-(layer, block, kv-head) scales).  Runs on the tcgen05 tensor cores; built for
 * the benchmark's geometry only: 8 kv heads of 128 dims, 32 query heads, 16-token blocks, F16 or E4M3 pool
 * (TKV_ERR_DIMENSION_MISMATCH otherwise).  All pointers are device memory of pool->device.                          */
typedef struct TkvPrefillAttn {
    uint32_t n_tokens, n_q_heads, layer, start_pos;
    uint32_t table_len;           /* entries of `table`; at least ceil((start_pos + n_tokens) / 16) */
    float sm_scale;               /* usually 1 / sqrt(head_dim)                                     */
    uint32_t flags, reserved;     /* TKV_PREFILL_*; 0                                               */
    uint64_t q;                   /* f32 [n_tokens][n_q_heads][128]                                 */
    uint64_t out;                 /* f32, same shape                                                */
    uint64_t table;               /* u32 [table_len] block ids of the sequence                      */
    uint64_t status;              /* 0, or a device u32 (zero it before the launch): TKV_ERR_TIMEOUT if a bounded wait gave
                                     up, TKV_ERR_INVALID_CONFIG if a table entry named a block outside the pool      */
} TkvPrefillAttn;
enum { TKV_PREFILL_DEFAULT = 0,
       TKV_PREFILL_SINGLE_TILE = 1, /* one query tile (32 tokens) per CTA */
       TKV_PREFILL_TWO_TILES = 2    /* two query tiles per CTA, their softmax groups out of step; without either flag the library
                                       chooses (two from 1 536 new tokens on) */ };
int32_t tkv_prefill_attn_enqueue(const TkvPool* pool, const TkvPrefillAttn* args, void* stream);
/* Device self-check of the tcgen05 path's operand plumbing (tensor-map copy with the 128-byte swizzle,
 * shared-memory and instruction descriptors, tensor-memory reads) on operands of small dyadic values whose
 * products and sums are exact: mismatches[0..3] count wrong accumulators for E4M3 K-major, E4M3 x E5M2
 * MN-major, F16 K-major and F16 MN-major operands.  No reference counterpart.                        */
int32_t tkv_selfcheck_tensor_cores(uint64_t mismatches[4]);

/* ---- the handoff's metadata on the wire -------------------------------------- */
/* SessionTransfer {cache, position, seed, last_logits} (engine/src/session.rs:194-200)
 * for a prefill and a decode process without a common address space: the cache is
 * reduced to its geometry and the block table that names its blocks in the prefill
 * pool (the K/V bytes travel through the handoff kernels, not through this message).
 * Little-endian; layout: "TKVS", version, this header, n_blocks block ids, n_logits
 * floats, FNV-1a-64 of everything before it.  A sequence may be announced in pieces:
 * piece_index of piece_count names blocks [block_begin, block_begin + n_blocks).
 * The reference derives serde traits and fixes no byte format (session.rs:194).     */
typedef struct TkvSessionHeader {
    uint64_t position;            /* tokens already in the cache                       */
    uint64_t seed;                /* sampler RNG seed (StdRng::seed_from_u64)           */
    uint32_t seq_len;
    uint32_t n_layers, n_kv_heads, head_dim, block_size;
    uint32_t kv_dtype;            /* TKV_DTYPE_* of the prefill pool                    */
    uint32_t block_begin, n_blocks;
    uint32_t piece_index, piece_count;
    uint32_t n_logits;            /* last_logits (vocab_size floats), usually in the last piece */
    uint32_t reserved;
} TkvSessionHeader;
size_t tkv_session_wire_size(const TkvSessionHeader* h);
int32_t tkv_session_pack(const TkvSessionHeader* h, const uint32_t* blocks, const float* logits, uint8_t* out,
                         size_t cap, size_t* written);
/* `blocks` and `logits` point into `in` (4-byte aligned when `in` is). */
int32_t tkv_session_unpack(const uint8_t* in, size_t len, TkvSessionHeader* h, const uint32_t** blocks,
                           const float** logits);

/* ---- host-side block bookkeeping ------------------------------------------- */
/* PageAllocator (engine/src/kv_cache.rs:762-793) */
typedef struct tkv_page_allocator tkv_page_allocator;
tkv_page_allocator* tkv_page_allocator_new(size_t total_pages);
void tkv_page_allocator_delete(tkv_page_allocator*);
int32_t tkv_page_allocator_allocate(tkv_page_allocator*, size_t* page); /* TKV_ERR_POOL_EXHAUSTED when empty */
void tkv_page_allocator_free(tkv_page_allocator*, size_t page);
size_t tkv_page_allocator_available(const tkv_page_allocator*);
size_t tkv_page_allocator_in_use(const tkv_page_allocator*);
size_t tkv_page_allocator_total(const tkv_page_allocator*);

/* BlockTable (engine/src/kv_cache.rs:836-893) */
typedef struct tkv_block_table tkv_block_table;
tkv_block_table* tkv_block_table_new(size_t max_blocks);
void tkv_block_table_delete(tkv_block_table*);
int32_t tkv_block_table_set_block(tkv_block_table*, size_t logical, size_t page);
int32_t tkv_block_table_get_block(const tkv_block_table*, size_t logical, size_t* page); /* 1 = Some */
size_t tkv_block_table_num_blocks(const tkv_block_table*);
size_t tkv_block_table_max_blocks(const tkv_block_table*);
const uint32_t* tkv_block_table_as_slice(const tkv_block_table*);
size_t tkv_block_table_clear(tkv_block_table*, size_t* freed, size_t cap);

/* PageRunAllocator (engine/src/gpu_page_pool.rs:34-218) */
typedef struct tkv_run_allocator tkv_run_allocator;
tkv_run_allocator* tkv_run_allocator_new(size_t total_pages);
void tkv_run_allocator_delete(tkv_run_allocator*);
int32_t tkv_run_allocator_alloc(tkv_run_allocator*, size_t pages, size_t* start); /* 1 = Some */
int32_t tkv_run_allocator_free(tkv_run_allocator*, size_t start, size_t pages);
int32_t tkv_run_allocator_try_extend(tkv_run_allocator*, size_t start, size_t pages, size_t target);
size_t tkv_run_allocator_free_pages(const tkv_run_allocator*);
size_t tkv_run_allocator_allocated_pages(const tkv_run_allocator*);
size_t tkv_run_allocator_free_runs(const tkv_run_allocator*, size_t* starts, size_t* pages, size_t cap);

/* RadixTree (engine/src/prefix_cache.rs:17-149) */
typedef struct tkv_radix_tree tkv_radix_tree;
tkv_radix_tree* tkv_radix_tree_new(void);
void tkv_radix_tree_delete(tkv_radix_tree*);
void tkv_radix_tree_insert(tkv_radix_tree*, const uint32_t* tokens, size_t n, const size_t* pages, size_t n_pages);
size_t tkv_radix_tree_lookup(tkv_radix_tree*, const uint32_t* tokens, size_t n, size_t* pages_out,
                             size_t cap, size_t* n_pages);
void tkv_radix_tree_release(tkv_radix_tree*, const uint32_t* tokens, size_t n);
size_t tkv_radix_tree_evict_lru(tkv_radix_tree*, size_t* freed, size_t cap);
uint64_t tkv_radix_tree_hit_count(const tkv_radix_tree*);
uint64_t tkv_radix_tree_tokens_saved(const tkv_radix_tree*);
size_t tkv_radix_tree_node_count(const tkv_radix_tree*);

/* PrefixCacheTable (engine/src/kv_cache.rs:581-730); entries name destination
 * block ids instead of holding cloned K/V vectors.                            */
typedef struct tkv_prefix_table tkv_prefix_table;
tkv_prefix_table* tkv_prefix_table_new(size_t max_entries);
void tkv_prefix_table_delete(tkv_prefix_table*);
void tkv_prefix_table_store(tkv_prefix_table*, const uint32_t* tokens, size_t n, const char* salt,
                            const uint32_t* blocks, size_t n_blocks, size_t seq_len);
size_t tkv_prefix_table_probe(tkv_prefix_table*, const uint32_t* tokens, size_t n, const char* salt,
                              uint32_t* blocks_out, size_t cap, size_t* n_blocks);
void tkv_prefix_table_release(tkv_prefix_table*, const uint32_t* tokens, size_t n, const char* salt);
size_t tkv_prefix_table_len(const tkv_prefix_table*);
uint64_t tkv_prefix_table_hit_count(const tkv_prefix_table*);
uint64_t tkv_prefix_table_tokens_saved(const tkv_prefix_table*);

/* ---- device-resident prefix index --------------------------------------------- */
/* RadixTree (engine/src/prefix_cache.rs:17-149) kept in HBM and walked by the GPU, one CTA per
 * sequence and one thread per node, so a batch of prompts resolves its cached prefix (length, page ids, reference
 * counts, LRU stamps) in one launch.  A node is `group_tokens` consecutive token ids below its
 * parent (1 = the reference's per-token nodes, 16 = one node per KV block), named by a 64-bit
 * hash chained from the root; only whole groups are indexed.  One call is one tick of the
 * reference's clock, and its result is that of the reference's method applied to the
 * sequences in index order at that tick.  Calls on one index must be stream-ordered.
 * Departure kept from the host mirror above: an unlinked node is never reported twice.      */
typedef struct tkv_prefix_index tkv_prefix_index;
typedef struct TkvPrefixBatch {
    uint32_t n_seqs, stride, page_stride, reserved;
    uint64_t tokens;              /* device u32 [n_seqs][stride] token ids                        */
    uint64_t lens;                /* device u32 [n_seqs] tokens per sequence (<= stride)         */
    uint64_t pages;               /* insert: device u32 [n_seqs][page_stride], page of node i of a
                                     sequence at [i]; 0 = insert without pages                  */
    uint64_t page_lens;           /* insert: device u32 [n_seqs] valid entries per row; 0 = rows are full */
} TkvPrefixBatch;
typedef struct TkvPrefixIndexStats {
    uint64_t hits, tokens_saved;  /* RadixTree::hit_count / tokens_saved                         */
    uint64_t live_nodes, tombstones, capacity, ticks;
    uint32_t group_tokens;
    uint32_t table_full;          /* 1 once an insert found no free slot (nodes of that call are missing) */
    uint64_t key_collisions;      /* walks that found their 64-bit key on a node whose first / last token id differ from
                                     theirs: treated as a miss instead of adopting the other prefix's page             */
} TkvPrefixIndexStats;
#define TKV_PREFIX_NO_PAGE 0xFFFFFFFFu
int32_t tkv_prefix_index_create(int32_t device, uint64_t capacity /* power of two */, uint32_t group_tokens, tkv_prefix_index** out);
void tkv_prefix_index_destroy(tkv_prefix_index*);
/* Test hook for the collision guard: cut the node keys to `bits` bits ([4, 64]) so that prefixes collide; only before the
 * first insert / lookup.  Lookups then match less (a collision is a checked miss) but never return another prefix's page. */
int32_t tkv_prefix_index_set_key_bits(tkv_prefix_index*, uint32_t bits);
/* RadixTree::insert for every sequence of the batch */
int32_t tkv_prefix_index_insert(tkv_prefix_index*, const TkvPrefixBatch*, void* stream);
/* RadixTree::lookup: out_matched[s] = matched nodes of sequence s (times group_tokens = its prefix
 * length, the handoff batch's prefix_lens); out_pages[s][i] = page of matched node i or
 * TKV_PREFIX_NO_PAGE (entries past the match are left alone).  Either output may be 0.        */
int32_t tkv_prefix_index_lookup(tkv_prefix_index*, const TkvPrefixBatch*, uint64_t out_pages /* device u32 [n_seqs][out_stride] */,
                                uint32_t out_stride, uint64_t out_matched /* device u32 [n_seqs] */, void* stream);
/* RadixTree::release */
int32_t tkv_prefix_index_release(tkv_prefix_index*, const TkvPrefixBatch*, void* stream);
/* RadixTree::evict_lru, up to max_nodes times: *out_count = pages written to out_pages (device u32
 * [out_cap]), *out_nodes (optional) = nodes unlinked.                                            */
int32_t tkv_prefix_index_evict_lru(tkv_prefix_index*, uint32_t max_nodes, uint64_t out_pages, uint32_t out_cap,
                                   uint64_t out_count /* device u32 */, uint64_t out_nodes /* device u32 or 0 */, void* stream);
/* synchronises the stream */
int32_t tkv_prefix_index_stats(tkv_prefix_index*, void* stream, TkvPrefixIndexStats* out);

/* ---- device-side page allocator ----------------------------------------------- */
/* PageAllocator (engine/src/kv_cache.rs:762-797), a LIFO stack of free page ids, kept in HBM so
 * that the decode side places a batch's blocks without a host round trip and without needing
 * contiguous runs (the reference's GPU pool hands out PageRunAllocator runs,
 * engine/src/gpu_page_pool.rs:1-10).  One launch per batch: sequence s takes counts[s] pages
 * into tables[s][first[s] ...] (first = its matched prefix nodes, say) and gets exactly the ids
 * allocate() would pop for the sequences in index order; free pushes them back in table order.
 * A batch asking for more than is free gets nothing: *status = TKV_ERR_POOL_EXHAUSTED.
 * Rows that would overrun table_stride, or more pages returned than were handed out:
 * *status = TKV_ERR_INVALID_CONFIG and nothing changes.  Calls must be stream-ordered.       */
typedef struct tkv_device_page_allocator tkv_device_page_allocator;
typedef struct TkvPageBatch {
    uint32_t n_seqs, table_stride;
    uint64_t tables;              /* device u32 [n_seqs][table_stride]                            */
    uint64_t first;               /* device u32 [n_seqs] first entry of each row to fill; 0 = entry 0 */
    uint64_t counts;              /* device u32 [n_seqs] pages per sequence; 0 = derive them:      */
    uint64_t seq_lens;            /* device u32 [n_seqs] tokens: counts[s] = ceil(seq_lens[s] /    */
    uint32_t block_size, reserved;/*   block_size) - first[s] (the blocks a lookup did not match)  */
} TkvPageBatch;
int32_t tkv_device_page_allocator_create(int32_t device, uint32_t total_pages, tkv_device_page_allocator** out);
void tkv_device_page_allocator_destroy(tkv_device_page_allocator*);
int32_t tkv_device_page_allocator_allocate(tkv_device_page_allocator*, const TkvPageBatch*, uint64_t status /* device u32 or 0 */, void* stream);
int32_t tkv_device_page_allocator_free(tkv_device_page_allocator*, const TkvPageBatch*, uint64_t status /* device u32 or 0 */, void* stream);
int32_t tkv_device_page_allocator_available(tkv_device_page_allocator*, void* stream, uint32_t* out); /* synchronises the stream */

/* ---- handoff from block tables that live on the device ------------------------ */
/* The same kernels as tkv_handoff_enqueue, but the work list is built ON THE DEVICE, in stream
 * order, from tables the device prefix index and page allocator have just filled: no block id,
 * length or prefix length crosses to the host.  `plan` supplies the geometry and the CAPACITY:
 * create it from a host batch with as many block pairs as a device batch may ever have (its own
 * table contents are not used here).  Sequence q moves its blocks past prefix_lens[q], in table
 * order, as the host path would; with apply_refcounts each shared-prefix block of each sequence
 * gets +1 in the destination pool's refcount array (RadixTree::lookup's count).  Nothing is
 * trusted: a misaligned or over-long prefix, a sequence longer than a table row, a block id
 * outside a pool, or more pairs than the capacity leave an empty list -- nothing moves, no
 * count changes, the flag is still published -- and *status = TKV_ERR_INVALID_CONFIG or
 * TKV_ERR_DIMENSION_MISMATCH (capacity).  Destination ids are NOT checked for duplicates here.
 * Not for transfer-buffer plans or per-layer tables.  tkv_plan_stats keeps describing the plan's
 * capacity batch, not the device batch.                                                       */
typedef struct TkvDeviceBatch {
    uint32_t n_seqs, table_stride, apply_refcounts, reserved;
    uint64_t seq_lens;            /* device u32 [n_seqs]                                          */
    uint64_t prefix_lens;         /* device u32 [n_seqs] tokens already resident; 0 = none, or see prefix_blocks */
    uint64_t src_tables;          /* device u32 [n_seqs][table_stride]                            */
    uint64_t dst_tables;          /* device u32 [n_seqs][table_stride]                            */
    uint64_t status;              /* device u32 or 0                                              */
    uint64_t prefix_blocks;       /* used when prefix_lens is 0: device u32 [n_seqs] BLOCKS already resident
                                     (tkv_prefix_index_lookup's out_matched with group_tokens = block_size) */
} TkvDeviceBatch;
int32_t tkv_handoff_enqueue_device_tables(tkv_plan* plan, const TkvDeviceBatch* batch, void* stream, uint64_t done_flag, uint32_t flag_value);
/* The prefix reference counts of a device batch alone (+1 or -1 per sequence and shared block, never below zero),
 * launched on the pool's own device: for a destination pool on a peer GPU, whose counts the prefill side's
 * handoff does not touch (apply_refcounts is for same-device plans), and for giving the references back.
 * Reads dst_tables and prefix_lens or prefix_blocks of `batch`; ids outside the pool are skipped and set
 * *status = TKV_ERR_INVALID_CONFIG.                                                                          */
int32_t tkv_refcount_apply_device_tables(const TkvPool* dst, const TkvDeviceBatch* batch, int32_t delta, void* stream);

/* ---- handoff coordinator (host logic, no CUDA) --------------------------------- */
/* The bookkeeping a disaggregated server keeps around the handoff: which prefill worker takes a
 * new request, which decode worker receives its cache and only when that worker's pool has the
 * pages (the reference gates admission on pool headroom, server/src/engine_task.rs:618-660, and
 * tracks requests in BatchScheduler, server/src/batch.rs:13-56), which handoffs are overdue, and
 * when to give up on one and let the decode worker prefill the prompt itself.
 *   QUEUED -> PREFILL -> WAITING -> ADMITTED -> TRANSFER -> DECODE -> (finish)
 *                                      ^------- failed, attempts left
 *                                   TRANSFER -> failed, none left -> REPREFILL -> DECODE
 * The caller reports what the device calls said: free pages (tkv_device_page_allocator_available
 * or the host allocator), completion (tkv_flag_wait_*), failures (a status word, a timeout).    */
typedef struct tkv_coordinator tkv_coordinator;
typedef struct TkvCoordinatorConfig {
    uint32_t n_prefill, n_decode, block_size;
    uint32_t max_inflight_per_decode;   /* handoffs admitted and not yet complete per decode worker; 0 = no limit */
    uint32_t max_retries;               /* handoff attempts after the first before falling back to re-prefill     */
    uint32_t headroom_blocks;           /* pages every decode pool keeps free for the growth of running sequences  */
    uint64_t handoff_timeout;           /* in the caller's clock units; 0 = handoffs never time out                */
} TkvCoordinatorConfig;
enum { TKV_REQ_QUEUED = 0, TKV_REQ_PREFILL = 1, TKV_REQ_WAITING = 2, TKV_REQ_ADMITTED = 3, TKV_REQ_TRANSFER = 4,
       TKV_REQ_DECODE = 5, TKV_REQ_REPREFILL = 6 };
enum { TKV_RETRY_HANDOFF = 1, TKV_REPREFILL = 2 };
typedef struct TkvAdmission {
    uint64_t request_id;
    uint32_t prefill_worker, decode_worker;
    uint32_t blocks;                    /* pages to take from the decode worker's allocator (prompt + max_new_tokens, less the resident prefix) */
    uint32_t prefix_tokens;
} TkvAdmission;
typedef struct TkvRequestInfo {
    uint64_t request_id;
    uint32_t state, prefill_worker, decode_worker, reserved_blocks, prefix_tokens, attempts;
} TkvRequestInfo;
typedef struct TkvCoordinatorStats {
    uint64_t submitted, admitted, handoffs_completed, handoffs_failed, retries, fallbacks, finished;
    uint64_t in_system, waiting, reserved_blocks;
} TkvCoordinatorStats;
tkv_coordinator* tkv_coordinator_new(const TkvCoordinatorConfig*);
void tkv_coordinator_delete(tkv_coordinator*);
int32_t tkv_coordinator_set_headroom(tkv_coordinator*, uint32_t decode_worker, uint64_t free_blocks);
/* least-loaded prefill worker (prompt tokens queued or running), lowest index on a tie */
int32_t tkv_coordinator_submit(tkv_coordinator*, uint64_t request_id, uint32_t n_tokens, uint32_t max_new_tokens, uint32_t priority,
                               uint32_t* prefill_worker);
/* 1 = *request_id is the worker's next prompt (highest priority, then oldest); 0 = its queue is empty; -1 = error */
int32_t tkv_coordinator_next_prefill(tkv_coordinator*, uint32_t prefill_worker, uint64_t* request_id);
int32_t tkv_coordinator_prefill_done(tkv_coordinator*, uint64_t request_id, uint32_t prefix_tokens_resident);
/* oldest first; to the decode worker paired with the prefill worker (index mod n_decode) when it fits there, else to
 * the one with the most room; a request that fits nowhere waits without blocking smaller ones behind it */
size_t tkv_coordinator_admit(tkv_coordinator*, TkvAdmission* out, size_t cap);
/* the pages were taken and the handoff enqueued; report the pool's new headroom before the next admit */
int32_t tkv_coordinator_handoff_started(tkv_coordinator*, uint64_t request_id, uint64_t now);
int32_t tkv_coordinator_handoff_complete(tkv_coordinator*, uint64_t request_id);
int32_t tkv_coordinator_handoff_failed(tkv_coordinator*, uint64_t request_id, uint32_t* action /* TKV_RETRY_HANDOFF | TKV_REPREFILL */);
size_t tkv_coordinator_timed_out(tkv_coordinator*, uint64_t now, uint64_t* request_ids, size_t cap);
int32_t tkv_coordinator_reprefill_done(tkv_coordinator*, uint64_t request_id);
int32_t tkv_coordinator_finish(tkv_coordinator*, uint64_t request_id);                 /* from any state */
int32_t tkv_coordinator_request(const tkv_coordinator*, uint64_t request_id, TkvRequestInfo* out);   /* 1 = found */
int32_t tkv_coordinator_stats(const tkv_coordinator*, TkvCoordinatorStats* out);

#ifdef __cplusplus
}
#endif
#endif /* TKV_H */
