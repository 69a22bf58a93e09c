/*
 * tkv_oracle.h -- CPU restatement of tempura's prefill->decode KV-cache handoff.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls
 * this code; it exists so the tests, the smoke check and the benchmark's CPU
 * baseline leg have an independent statement of what the reference computes.
 *
 * Every function cites the reference file:line (paths inside the tempura
 * repository) whose behaviour it restates.  The reference is Rust and cannot be
 * compiled in an image without cargo/rustc, so this file is pinned against the
 * reference's own known-answer tests (restated in tests/test_oracle_golden.py)
 * instead of against a compiled copy of the reference.
 *
 * PARITY UNPINNED for exactly one rule: the per-(layer, kv-head, block) absmax
 * scale of the FP8 destination cache.  The reference stores unscaled FP8 bytes
 * (engine/src/kv_cache.rs:1149-1160) and has no test that pins a scaled form;
 * orc_block_scale() below freezes the arithmetic and tests/golden/ holds vectors
 * generated from it.  The element quantizer itself (orc_f32_to_e4m3) IS pinned by
 * kernels/src/e4m3.rs:100-174.
 *
 * Deliberate reinterpretation: the reference counts prefix references per hash
 * entry (engine/src/kv_cache.rs:635) or per trie node, one node per token
 * (engine/src/prefix_cache.rs:41-45,64-70).  All tokens of a block move together,
 * so the block-level rule here keeps one u32 per destination block.
 */
#ifndef TKV_ORACLE_H
#define TKV_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- element conversions ------------------------------------------------ */
uint8_t orc_f32_to_e4m3(float x);          /* kernels/src/e4m3.rs:50-94  */
float orc_e4m3_to_f32(uint8_t b);          /* kernels/src/e4m3.rs:27-41  */
uint8_t orc_f32_to_e4m3_legacy(float x);   /* engine/src/kv_cache.rs:1078-1123 (NOT the oracle quantizer) */
uint16_t orc_f32_to_f16(float x);          /* engine/src/kv_cache.rs:29-47 (vcvtps2ph, RNE) */
float orc_f16_to_f32(uint16_t h);          /* engine/src/kv_cache.rs:49-67 (vcvtph2ps, exact) */
uint16_t orc_f32_to_f16_scalar_fallback(float x); /* engine/src/kv_cache.rs:77-89 (truncating) */

/* amax rule + scale arithmetic frozen for the FP8 destination cache.
 * amax_bits = max(bits & 0x7FFF) over the valid F16 elements of one
 * (layer, K|V, block, kv-head).  Returns the stored FP32 scale (dequant
 * multiplier) and writes the quantisation multiplier to *inv.            */
float orc_block_scale(uint16_t amax_bits, float* inv);
uint8_t orc_quantize_scaled(uint16_t h, float inv);

/* ---- index formula ------------------------------------------------------ */
/* kernels/src/attention.rs:472-484 */
size_t orc_paged_row_offset(const uint32_t* block_table, size_t block_size, size_t stride,
                            size_t token, size_t kv_h, size_t head_dim);

/* ---- PageAllocator (engine/src/kv_cache.rs:762-793) --------------------- */
typedef struct orc_page_allocator orc_page_allocator;
orc_page_allocator* orc_pa_new(size_t total_pages);
void orc_pa_delete(orc_page_allocator*);
int64_t orc_pa_allocate(orc_page_allocator*);      /* -1 == None */
void orc_pa_free(orc_page_allocator*, size_t page);
size_t orc_pa_available(const orc_page_allocator*);
size_t orc_pa_in_use(const orc_page_allocator*);

/* ---- BlockTable (engine/src/kv_cache.rs:836-893) ------------------------ */
typedef struct orc_block_table orc_block_table;
orc_block_table* orc_bt_new(size_t max_blocks);
void orc_bt_delete(orc_block_table*);
void orc_bt_set_block(orc_block_table*, size_t logical, size_t page);
int64_t orc_bt_get_block(const orc_block_table*, size_t logical);  /* -1 == None */
size_t orc_bt_num_blocks(const orc_block_table*);
const uint32_t* orc_bt_as_slice(const orc_block_table*);
size_t orc_bt_clear(orc_block_table*, size_t* freed_out, size_t cap);

/* ---- paged gather / scatter (PagedKvCache) ------------------------------ */
/* k_contiguous / v_contiguous: engine/src/kv_cache.rs:1032-1060 */
void orc_paged_gather(const void* pool_layer, const uint32_t* table, size_t block_size,
                      size_t stride_elems, size_t elem_size, size_t kv_len, void* out);
/* append_kv copy loop: engine/src/kv_cache.rs:991-1003 (table already populated) */
void orc_paged_scatter(void* pool_layer, const uint32_t* table, size_t block_size,
                       size_t stride_elems, size_t elem_size, size_t seq_len_before,
                       size_t n_new_tokens, const void* src);

/* ---- contiguous transfer (KvCache::to_transfer / from_transfer) --------- */
/* engine/src/kv_cache.rs:402-431; dst_f16 != 0 takes the use_f16 branch of
 * append_kv (:209-221).  src is F32 [seq_len*stride]; dst is F32 or F16.    */
void orc_transfer_layer(const float* src_layer, size_t seq_len, size_t stride, int dst_f16,
                        void* dst_layer);

/* ---- the handoff, batch form ------------------------------------------- */
typedef struct {
    uint32_t n_layers;      /* layers held by this pool                         */
    uint32_t n_kv_heads;    /* kv heads held by this pool (row = heads*head_dim) */
    uint32_t head_dim;
    uint32_t block_size;
    uint32_t total_blocks;
    uint32_t elem_size;     /* 4 = F32, 2 = F16, 1 = E4M3                        */
    void* const* k_layers;  /* [n_layers] -> [total_blocks*block_size*heads*dim] */
    void* const* v_layers;
    float* k_scales;        /* E4M3 only: [n_layers][total_blocks][n_kv_heads]   */
    float* v_scales;
} orc_pool;

typedef struct {
    uint32_t n_seqs;
    const uint32_t* seq_lens;     /* tokens per sequence                         */
    const uint32_t* prefix_lens;  /* tokens already resident on dst (NULL = 0)   */
    const uint32_t* src_tables;   /* [n_seqs][table_stride]                      */
    const uint32_t* dst_tables;
    uint32_t table_stride;
    uint32_t table_layer_stride;  /* 0: one table per sequence shared by all layers (GPU pool
                                     convention, engine/src/cutile_kv_cache.rs:1054-1072);
                                     else layer l's tables start l*table_layer_stride entries in
                                     (per-layer tables of PagedKvCache, engine/src/kv_cache.rs:925-936) */
} orc_batch;

typedef struct {
    uint32_t src_head_begin, dst_head_begin, n_heads;
    uint32_t src_layer_begin, dst_layer_begin, n_layers;
} orc_shard;

/* Same-dtype handoff: gather each sequence's [prefix_len, seq_len) tokens
 * through src table, scatter through dst table.  n_threads > 1 spreads the
 * (sequence, layer, K|V) units over OpenMP threads.  Returns 0, or a
 * negative code for an invalid argument.                                    */
int orc_handoff_copy(const orc_pool* src, const orc_pool* dst, const orc_batch* batch,
                     const orc_shard* shard, int n_threads);
/* F16 source, E4M3 destination with per-(layer, kv-head, block) scales; a
 * destination without scale arrays receives unscaled e4m3 bytes.             */
int orc_handoff_f16_to_e4m3(const orc_pool* src, const orc_pool* dst, const orc_batch* batch,
                            const orc_shard* shard, int n_threads);
/* F32 source, F16 destination (from_transfer into a use_f16 cache).          */
int orc_handoff_f32_to_f16(const orc_pool* src, const orc_pool* dst, const orc_batch* batch,
                           const orc_shard* shard, int n_threads);
/* the reader's side of the FP8 cache: gather + widen (engine/src/kv_cache.rs:1241-1271),
 * element decode kernels/src/e4m3.rs:27-41, times the source block scale if present */
int orc_handoff_e4m3_to_f16(const orc_pool* src, const orc_pool* dst, const orc_batch* b,
                            const orc_shard* sh, int n_threads);
/* F32 rows into an unscaled E4M3 pool (kernels/src/kv_scatter_write.rs:172-273, element rule e4m3.rs:50-94) */
int orc_handoff_f32_to_e4m3(const orc_pool* src, const orc_pool* dst, const orc_batch* b,
                            const orc_shard* sh, int n_threads);
int orc_handoff_e4m3_to_f32(const orc_pool* src, const orc_pool* dst, const orc_batch* b,
                            const orc_shard* sh, int n_threads);

/* Block-level prefix refcounts: +1 (delta>0) on every dst block that lies
 * wholly inside a sequence's prefix_len, saturating -1 (delta<0).
 * engine/src/kv_cache.rs:635,691; engine/src/prefix_cache.rs:68,92.          */
void orc_refcount_apply(uint32_t* refcounts, const orc_batch* batch, uint32_t block_size,
                        int delta);

/* bits checksum idiom: engine/src/cutile_kv_cache.rs:1274-1286 */
uint64_t orc_bits_checksum_f32(const float* v, size_t n);
uint64_t orc_bits_checksum_f16_as_f32(const uint16_t* v, size_t n);
uint64_t orc_bits_checksum_e4m3_as_f32(const uint8_t* v, size_t n);

/* ---- decode attention over a paged pool ---------------------------------------- */
/* kernels/src/attention.rs:486-590 with one query token per sequence; q and out are
 * [n_seqs][num_heads][head_dim] f32; E4M3 pools read as decode x block scale.      */
int orc_paged_decode_attention(const orc_pool* pool, uint32_t layer, const float* q, const uint32_t* tables,
                               uint32_t table_stride, const uint32_t* kv_lens, uint32_t n_seqs,
                               uint32_t num_heads, float scale, float* out);

/* ---- RadixTree (engine/src/prefix_cache.rs:17-149) ---------------------- */
typedef struct orc_radix orc_radix;
orc_radix* orc_radix_new(void);
void orc_radix_delete(orc_radix*);
void orc_radix_insert(orc_radix*, const uint32_t* tokens, size_t n, const size_t* pages, size_t n_pages);
size_t orc_radix_lookup(orc_radix*, const uint32_t* tokens, size_t n, size_t* pages_out,
                        size_t cap, size_t* n_pages_out);
void orc_radix_release(orc_radix*, const uint32_t* tokens, size_t n);
size_t orc_radix_evict_lru(orc_radix*, size_t* freed_out, size_t cap);
uint64_t orc_radix_hit_count(const orc_radix*);
uint64_t orc_radix_tokens_saved(const orc_radix*);
size_t orc_radix_node_count(const orc_radix*);
/* test accessor: ref_count of the node reached by walking `tokens` (or -1) */
int64_t orc_radix_ref_count(const orc_radix*, const uint32_t* tokens, size_t n);

/* ---- PrefixCacheTable, block-id form (engine/src/kv_cache.rs:581-730) ---- */
typedef struct orc_prefix_table orc_prefix_table;
orc_prefix_table* orc_pt_new(size_t max_entries);
void orc_pt_delete(orc_prefix_table*);
void orc_pt_store(orc_prefix_table*, const uint32_t* tokens, size_t n, const char* salt,
                  const uint32_t* blocks, size_t n_blocks, size_t seq_len);
/* returns matched_len (0 = miss); copies the entry's block ids */
size_t orc_pt_probe(orc_prefix_table*, const uint32_t* tokens, size_t n, const char* salt,
                    uint32_t* blocks_out, size_t cap, size_t* n_blocks_out);
void orc_pt_release(orc_prefix_table*, const uint32_t* tokens, size_t n, const char* salt);
size_t orc_pt_len(const orc_prefix_table*);
uint64_t orc_pt_hit_count(const orc_prefix_table*);
uint64_t orc_pt_tokens_saved(const orc_prefix_table*);
int64_t orc_pt_ref_count(const orc_prefix_table*, const uint32_t* tokens, size_t n, const char* salt);

/* ---- PageRunAllocator (engine/src/gpu_page_pool.rs:34-218) -------------- */
typedef struct orc_run_allocator orc_run_allocator;
orc_run_allocator* orc_ra_new(size_t total_pages);
void orc_ra_delete(orc_run_allocator*);
int orc_ra_alloc(orc_run_allocator*, size_t pages, size_t* start_out);   /* 1 = Some */
void orc_ra_free(orc_run_allocator*, size_t start, size_t pages);
int orc_ra_try_extend(orc_run_allocator*, size_t start, size_t pages, size_t target);
size_t orc_ra_free_pages(const orc_run_allocator*);
size_t orc_ra_allocated_pages(const orc_run_allocator*);
size_t orc_ra_free_runs(const orc_run_allocator*, size_t* starts, size_t* pages, size_t cap);

/* ---- deterministic synthetic inputs (no reference counterpart) ---------- */
uint64_t orc_mix64(uint64_t seed, uint64_t stream, uint64_t index);
/* N(0, sigma) rounded to F16 (RNE); `outlier_channels`/`n_outliers` name
 * head_dim channel indices scaled by `outlier_gain` (config 3).            */
void orc_gen_normal_f16(uint16_t* out, size_t n, uint64_t seed, uint64_t stream, double sigma,
                        uint32_t head_dim, const uint32_t* outlier_channels, uint32_t n_outliers,
                        double outlier_gain, size_t first_index);
void orc_gen_permutation(uint32_t* out, uint32_t n, uint64_t seed, uint64_t stream);
void orc_gen_lengths(uint32_t* out, uint32_t n, uint32_t lo, uint32_t hi, uint64_t seed,
                     uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TKV_ORACLE_H */
