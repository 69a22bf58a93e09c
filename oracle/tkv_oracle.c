/*
 * tkv_oracle.c -- CPU restatement of tempura's KV handoff (see tkv_oracle.h).
 * TEST INFRASTRUCTURE ONLY: never linked into, loaded by or called from the
 * shipped library.  Plain C99 + optional OpenMP for the all-cores timing form.
 */
#include "tkv_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f32_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

/* ======================================================================= */
/* element conversions                                                      */
/* ======================================================================= */

/* kernels/src/e4m3.rs:27-41.  exp == 0 reads as signed zero (subnormal
 * flush); exp == 15 goes through the normal path, as the reference says.   */
float orc_e4m3_to_f32(uint8_t b8) {
    uint32_t b = b8;
    uint32_t sign = (b & 0x80u) << 24;
    uint32_t exp = (b >> 3) & 0x0Fu;
    uint32_t man = b & 0x07u;
    if (exp == 0) return bits_f32(sign);
    return bits_f32(sign | ((exp + 120u) << 23) | (man << 20));
}

/* kernels/src/e4m3.rs:50-94.  NaN -> 0x7F; clamp to +-448; f32 exponent
 * below 121 -> signed zero; RNE on the 20 dropped bits with carry into the
 * exponent field.                                                          */
uint8_t orc_f32_to_e4m3(float x) {
    uint32_t bits = f32_bits(x);
    uint32_t sign = (bits >> 24) & 0x80u;
    uint32_t abs = bits & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return 0x7F;
    if (x > 448.0f) x = 448.0f;
    else if (x < -448.0f) x = -448.0f;
    bits = f32_bits(x);
    abs = bits & 0x7FFFFFFFu;
    uint32_t exp = (abs >> 23) & 0xFFu;
    if (exp < 121u) return (uint8_t)sign;
    uint32_t man = abs & 0x7FFFFFu;
    uint32_t e2 = exp - 120u;
    uint32_t kept = man >> 20;
    uint32_t dropped = man & 0xFFFFFu;
    int round_up = dropped > 0x80000u || (dropped == 0x80000u && (kept & 1u) == 1u);
    if (round_up) {
        if (kept == 7u) {
            e2 += 1u;
            kept = 0u;
        } else {
            kept += 1u;
        }
    }
    return (uint8_t)(sign | (e2 << 3) | kept);
}

/* engine/src/kv_cache.rs:1078-1123 -- the engine's private quantizer.  Kept
 * only so a test can document where it departs from e4m3.rs (round-half-up,
 * [256, 448) -> 448, NaN/Inf -> 0x7E, subnormal range truncated to zero by
 * the e4m3_exp <= 0 test).  It is not used by any handoff function.         */
uint8_t orc_f32_to_e4m3_legacy(float x) {
    uint8_t sign = (f32_bits(x) >> 31) ? 0x80 : 0;
    float a = fabsf(x);
    if (a == 0.0f) return sign;
    if (isnan(a) || isinf(a)) return sign | 0x7E;
    if (a >= 448.0f) return sign | 0x7E;
    if (a < 0.001953125f) return sign;
    uint32_t bits = f32_bits(a);
    int32_t f32_exp = (int32_t)((bits >> 23) & 0xFF);
    uint32_t frac = bits & 0x7FFFFFu;
    int32_t e = f32_exp - 127 + 7;
    if (e <= 0) return sign;
    if (e > 14) return sign | 0x7E;
    uint32_t m = (frac + (1u << 19)) >> 20;
    if (m >= 8u) {
        int32_t ne = e + 1;
        if (ne > 14) return sign | 0x7E;
        return sign | (uint8_t)(ne << 3);
    }
    return sign | (uint8_t)(e << 3) | (uint8_t)m;
}

/* engine/src/kv_cache.rs:29-47: _mm256_cvtps_ph(_MM_FROUND_TO_NEAREST_INT).
 * IEEE-754 binary32 -> binary16, round to nearest even, overflow to Inf,
 * gradual underflow.  NaN follows the x86 instruction: sign kept, quiet bit
 * set, top ten payload bits kept.  (A GPU cvt.rn.f16.f32 yields 0x7FFF for
 * NaN instead: tools/bench-gpu/src/bench_decode_ops.rs:711-726.)            */
uint16_t orc_f32_to_f16(float x) {
    uint32_t b = f32_bits(x);
    uint32_t sign = (b >> 16) & 0x8000u;
    uint32_t abs = b & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((abs >> 13) & 0x1FFu));
    if (abs >= 0x47800000u) {            /* >= 65536 (incl. Inf) -> Inf          */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (abs >= 0x38800000u) {            /* normal half range (>= 2^-14)         */
        uint32_t v = abs - 0x38000000u;  /* rebias exponent 127 -> 15            */
        uint32_t kept = v >> 13;
        uint32_t dropped = v & 0x1FFFu;
        if (dropped > 0x1000u || (dropped == 0x1000u && (kept & 1u))) kept += 1u;
        return (uint16_t)(sign | kept);  /* carry may roll into Inf = correct    */
    }
    if (abs < 0x33000000u) return (uint16_t)sign;   /* < 2^-25 -> zero           */
    /* subnormal half: value = m * 2^-24, m in [0, 1024) */
    uint32_t exp = abs >> 23;                        /* 102..112                 */
    uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;    /* 24-bit significand       */
    uint32_t shift = 126u - exp;                     /* 14..24                   */
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (kept & 1u))) kept += 1u;
    return (uint16_t)(sign | kept);
}

/* engine/src/kv_cache.rs:49-67: _mm256_cvtph_ps -- exact widening. */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1Fu) return bits_f32(sign | 0x7F800000u | (man << 13) | (man ? 0x400000u : 0u));
    if (exp != 0) return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
    if (man == 0) return bits_f32(sign);
    int e = -1;
    do {
        man <<= 1;
        e++;
    } while (!(man & 0x400u));
    return bits_f32(sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3FFu) << 13));
}

/* engine/src/kv_cache.rs:77-89: the non-F16C fallback (mantissa truncation,
 * subnormals flushed, overflow to Inf).  Restated for completeness; x86
 * hosts with F16C never take it.                                            */
uint16_t orc_f32_to_f16_scalar_fallback(float x) {
    uint32_t bits = f32_bits(x);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exp = (int32_t)((bits >> 23) & 0xFF) - 127 + 15;
    uint32_t frac = (bits >> 13) & 0x3FFu;
    if (exp <= 0) return (uint16_t)sign;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)exp << 10) | frac);
}

/* Frozen scale rule (no reference test pins it).  Precedent for absmax scaling
 * and for the unscaled fallback on a zero or non-finite amax:
 * kernels/src/fp8_sim.rs:262-286.  Target is 448 (full e4m3 range) because the
 * element quantizer already saturates.                                       */
float orc_block_scale(uint16_t amax_bits, float* inv) {
    if (amax_bits == 0 || amax_bits >= 0x7C00u) {
        *inv = 1.0f;
        return 1.0f;
    }
    volatile float amax = orc_f16_to_f32(amax_bits);
    volatile float scale = amax / 448.0f;
    volatile float iv = 448.0f / amax;
    *inv = iv;
    return scale;
}

uint8_t orc_quantize_scaled(uint16_t h, float inv) {
    volatile float x = orc_f16_to_f32(h);
    volatile float y = x * inv;     /* one RN multiply; volatile blocks contraction */
    return orc_f32_to_e4m3(y);
}

/* ======================================================================= */
/* index formula: kernels/src/attention.rs:472-484                          */
/* ======================================================================= */
size_t orc_paged_row_offset(const uint32_t* block_table, size_t block_size, size_t stride,
                            size_t token, size_t kv_h, size_t head_dim) {
    size_t block_idx = token / block_size;
    size_t page = block_table[block_idx];
    size_t block_offset = token % block_size;
    return (page * block_size + block_offset) * stride + kv_h * head_dim;
}

/* ======================================================================= */
/* PageAllocator: engine/src/kv_cache.rs:762-793 (free list popped from the */
/* back; initial list is total-1 .. 0 so the first page handed out is 0)    */
/* ======================================================================= */
struct orc_page_allocator {
    size_t* free_pages;
    size_t n_free, total;
};
orc_page_allocator* orc_pa_new(size_t total) {
    orc_page_allocator* a = malloc(sizeof *a);
    a->free_pages = malloc(sizeof(size_t) * (total ? total * 2 : 1));
    a->total = total;
    a->n_free = total;
    for (size_t i = 0; i < total; i++) a->free_pages[i] = total - 1 - i;
    return a;
}
void orc_pa_delete(orc_page_allocator* a) {
    if (a) {
        free(a->free_pages);
        free(a);
    }
}
int64_t orc_pa_allocate(orc_page_allocator* a) {
    if (a->n_free == 0) return -1;
    return (int64_t)a->free_pages[--a->n_free];
}
void orc_pa_free(orc_page_allocator* a, size_t page) {
    if (a->n_free < a->total * 2) a->free_pages[a->n_free++] = page;
}
size_t orc_pa_available(const orc_page_allocator* a) { return a->n_free; }
size_t orc_pa_in_use(const orc_page_allocator* a) { return a->total - a->n_free; }

/* ======================================================================= */
/* BlockTable: engine/src/kv_cache.rs:836-893                               */
/* ======================================================================= */
struct orc_block_table {
    uint32_t* table;
    size_t max_blocks, num_blocks;
};
orc_block_table* orc_bt_new(size_t max_blocks) {
    orc_block_table* t = malloc(sizeof *t);
    t->table = malloc(sizeof(uint32_t) * (max_blocks ? max_blocks : 1));
    for (size_t i = 0; i < max_blocks; i++) t->table[i] = UINT32_MAX;
    t->max_blocks = max_blocks;
    t->num_blocks = 0;
    return t;
}
void orc_bt_delete(orc_block_table* t) {
    if (t) {
        free(t->table);
        free(t);
    }
}
void orc_bt_set_block(orc_block_table* t, size_t logical, size_t page) {
    t->table[logical] = (uint32_t)page;
    if (logical >= t->num_blocks) t->num_blocks = logical + 1;
}
int64_t orc_bt_get_block(const orc_block_table* t, size_t logical) {
    if (logical < t->num_blocks && t->table[logical] != UINT32_MAX) return t->table[logical];
    return -1;
}
size_t orc_bt_num_blocks(const orc_block_table* t) { return t->num_blocks; }
const uint32_t* orc_bt_as_slice(const orc_block_table* t) { return t->table; }
size_t orc_bt_clear(orc_block_table* t, size_t* freed_out, size_t cap) {
    size_t n = 0;
    for (size_t i = 0; i < t->num_blocks; i++)
        if (t->table[i] != UINT32_MAX) {
            if (n < cap) freed_out[n] = t->table[i];
            n++;
        }
    for (size_t i = 0; i < t->max_blocks; i++) t->table[i] = UINT32_MAX;
    t->num_blocks = 0;
    return n;
}

/* ======================================================================= */
/* PagedKvCache gather / scatter                                            */
/* ======================================================================= */

/* engine/src/kv_cache.rs:1032-1060: per token, block_idx = pos / bs,
 * off = pos % bs, page_base = page * page_stride + off * stride.           */
void orc_paged_gather(const void* pool_layer, const uint32_t* table, size_t block_size,
                      size_t stride, size_t elem, size_t kv_len, void* out) {
    size_t page_stride = block_size * stride;
    for (size_t pos = 0; pos < kv_len; pos++) {
        size_t block_idx = pos / block_size, block_offset = pos % block_size;
        size_t page_base = (size_t)table[block_idx] * page_stride + block_offset * stride;
        memcpy((char*)out + pos * stride * elem, (const char*)pool_layer + page_base * elem,
               stride * elem);
    }
}

/* engine/src/kv_cache.rs:991-1003: global_pos = seq_len + t. */
void orc_paged_scatter(void* pool_layer, const uint32_t* table, size_t block_size, size_t stride,
                       size_t elem, size_t seq_len_before, size_t n_new, const void* src) {
    size_t page_stride = block_size * stride;
    for (size_t t = 0; t < n_new; t++) {
        size_t g = seq_len_before + t;
        size_t block_idx = g / block_size, block_offset = g % block_size;
        size_t page_base = (size_t)table[block_idx] * page_stride + block_offset * stride;
        memcpy((char*)pool_layer + page_base * elem, (const char*)src + t * stride * elem,
               stride * elem);
    }
}

/* engine/src/kv_cache.rs:402-431 with append_kv's dtype branch (:209-226). */
void orc_transfer_layer(const float* src, size_t seq_len, size_t stride, int dst_f16, void* dst) {
    size_t n = seq_len * stride;
    if (dst_f16) {
        uint16_t* d = dst;
        for (size_t i = 0; i < n; i++) d[i] = orc_f32_to_f16(src[i]);
    } else {
        memcpy(dst, src, n * sizeof(float));
    }
}

/* ---- batch handoff ------------------------------------------------------ */

static int check_args(const orc_pool* s, const orc_pool* d, const orc_batch* b, const orc_shard* sh) {
    if (!s || !d || !b || !sh) return -1;
    if (s->head_dim != d->head_dim || s->block_size != d->block_size) return -2;
    if (sh->src_head_begin + sh->n_heads > s->n_kv_heads) return -3;
    if (sh->dst_head_begin + sh->n_heads > d->n_kv_heads) return -3;
    if (sh->src_layer_begin + sh->n_layers > s->n_layers) return -4;
    if (sh->dst_layer_begin + sh->n_layers > d->n_layers) return -4;
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        uint32_t pre = b->prefix_lens ? b->prefix_lens[q] : 0;
        if (pre > b->seq_lens[q] || pre % s->block_size) return -5;
        uint32_t nb = (b->seq_lens[q] + s->block_size - 1) / s->block_size;
        if (nb > b->table_stride) return -6;
        uint32_t n_tab = b->table_layer_stride ? sh->n_layers : 1;
        for (uint32_t l = 0; l < n_tab; l++)
            for (uint32_t i = pre / s->block_size; i < nb; i++) {
                size_t so = (size_t)(sh->src_layer_begin + l) * b->table_layer_stride;
                size_t dof = (size_t)(sh->dst_layer_begin + l) * b->table_layer_stride;
                if (b->src_tables[so + (size_t)q * b->table_stride + i] >= s->total_blocks) return -7;
                if (b->dst_tables[dof + (size_t)q * b->table_stride + i] >= d->total_blocks) return -7;
            }
    }
    return 0;
}

enum { MODE_COPY = 0, MODE_F16_E4M3 = 1, MODE_F32_F16 = 2, MODE_E4M3_F16 = 3, MODE_E4M3_F32 = 4, MODE_F32_E4M3 = 5 };

/* One (sequence, layer, K|V) unit: gather the suffix tokens of the selected
 * heads into a contiguous buffer (k_contiguous, restricted to the shard's
 * heads), convert, scatter through the destination table (append_kv).       */
static void handoff_unit(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                         const orc_shard* sh, uint32_t q, uint32_t l, int is_v, int mode) {
    const uint32_t bs = s->block_size, D = s->head_dim;
    const uint32_t pre = b->prefix_lens ? b->prefix_lens[q] : 0;
    const uint32_t len = b->seq_lens[q];
    if (len <= pre) return;
    const uint32_t* st = b->src_tables + (size_t)q * b->table_stride +
                         (size_t)(sh->src_layer_begin + l) * b->table_layer_stride;
    const uint32_t* dt = b->dst_tables + (size_t)q * b->table_stride +
                         (size_t)(sh->dst_layer_begin + l) * b->table_layer_stride;
    const size_t s_stride = (size_t)s->n_kv_heads * D, d_stride = (size_t)d->n_kv_heads * D;
    const char* sp = (is_v ? s->v_layers : s->k_layers)[sh->src_layer_begin + l];
    char* dp = (is_v ? d->v_layers : d->k_layers)[sh->dst_layer_begin + l];
    const uint32_t dl = sh->dst_layer_begin + l;
    const size_t n_tok = len - pre, row = (size_t)sh->n_heads * D;

    /* gather (src elem size) */
    char* tmp = malloc(n_tok * row * s->elem_size);
    for (size_t t = 0; t < n_tok; t++) {
        size_t off = orc_paged_row_offset(st, bs, s_stride, pre + t, sh->src_head_begin, D);
        memcpy(tmp + t * row * s->elem_size, sp + off * s->elem_size, row * s->elem_size);
    }

    if (mode == MODE_COPY) {
        for (size_t t = 0; t < n_tok; t++) {
            size_t off = orc_paged_row_offset(dt, bs, d_stride, pre + t, sh->dst_head_begin, D);
            memcpy(dp + off * d->elem_size, tmp + t * row * d->elem_size, row * d->elem_size);
        }
    } else if (mode == MODE_F32_F16) {
        const float* f = (const float*)tmp;
        for (size_t t = 0; t < n_tok; t++) {
            size_t off = orc_paged_row_offset(dt, bs, d_stride, pre + t, sh->dst_head_begin, D);
            uint16_t* o = (uint16_t*)dp + off;
            for (size_t i = 0; i < row; i++) o[i] = orc_f32_to_f16(f[t * row + i]);
        }
    } else if (mode == MODE_F32_E4M3) {
        /* the e4m3 row writer of the GPU pool (kernels/src/kv_scatter_write.rs:172-273): each element through
         * kernels/src/e4m3.rs:50-94, no scale                                                                */
        const float* f = (const float*)tmp;
        for (size_t t = 0; t < n_tok; t++) {
            size_t off = orc_paged_row_offset(dt, bs, d_stride, pre + t, sh->dst_head_begin, D);
            uint8_t* o = (uint8_t*)dp + off;
            for (size_t i = 0; i < row; i++) o[i] = orc_f32_to_e4m3(f[t * row + i]);
        }
    } else if (mode == MODE_E4M3_F16 || mode == MODE_E4M3_F32) {
        /* Fp8PagedKvCache::k_contiguous / v_contiguous (engine/src/kv_cache.rs:1241-1271) widen
         * while they gather; the element decode is kernels/src/e4m3.rs:27-41 (the quantizer's
         * own inverse, not the cache's private decoder), times the block's scale when the
         * source pool has scale arrays: one round-to-nearest multiply, then RNE for F16.    */
        const uint8_t* bsrc = (const uint8_t*)tmp;
        const float* scales = is_v ? s->v_scales : s->k_scales;
        const uint32_t sl = sh->src_layer_begin + l;
        for (size_t t = 0; t < n_tok; t++) {
            size_t off = orc_paged_row_offset(dt, bs, d_stride, pre + t, sh->dst_head_begin, D);
            uint32_t blk = (uint32_t)((pre + t) / bs);
            for (uint32_t h = 0; h < sh->n_heads; h++) {
                float scale = scales ? scales[((size_t)sl * s->total_blocks + st[blk]) * s->n_kv_heads +
                                              sh->src_head_begin + h]
                                     : 1.0f;
                for (uint32_t i = 0; i < D; i++) {
                    volatile float x = orc_e4m3_to_f32(bsrc[t * row + (size_t)h * D + i]) * scale;
                    if (mode == MODE_E4M3_F16) ((uint16_t*)dp)[off + (size_t)h * D + i] = orc_f32_to_f16(x);
                    else ((float*)dp)[off + (size_t)h * D + i] = x;
                }
            }
        }
    } else { /* MODE_F16_E4M3 */
        const uint16_t* hsrc = (const uint16_t*)tmp;
        float* scales = is_v ? d->v_scales : d->k_scales;
        for (uint32_t blk = pre / bs; blk * bs < len; blk++) {
            uint32_t t0 = blk * bs, t1 = t0 + bs < len ? t0 + bs : len;   /* valid tokens */
            for (uint32_t h = 0; h < sh->n_heads; h++) {
                uint16_t amax = 0;
                for (uint32_t t = t0; t < t1; t++)
                    for (uint32_t i = 0; i < D; i++) {
                        uint16_t a = hsrc[(size_t)(t - pre) * row + (size_t)h * D + i] & 0x7FFFu;
                        if (a > amax) amax = a;
                    }
                /* A pool without scale arrays stores raw e4m3 bytes, as the reference's own
                 * pools do (engine/src/cutile_kv_cache.rs:1593-1595; element rule as the
                 * e4m3 row writer, kernels/src/kv_scatter_write.rs:172-273).               */
                float inv = 1.0f;
                if (scales) {
                    float scale = orc_block_scale(amax, &inv);
                    scales[((size_t)dl * d->total_blocks + dt[blk]) * d->n_kv_heads +
                           sh->dst_head_begin + h] = scale;
                }
                for (uint32_t t = t0; t < t1; t++) {
                    size_t off = orc_paged_row_offset(dt, bs, d_stride, t, sh->dst_head_begin + h, D);
                    uint8_t* o = (uint8_t*)dp + off;
                    for (uint32_t i = 0; i < D; i++)
                        o[i] = orc_quantize_scaled(hsrc[(size_t)(t - pre) * row + (size_t)h * D + i], inv);
                }
            }
        }
    }
    free(tmp);
}

static int handoff_run(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                       const orc_shard* sh, int n_threads, int mode) {
    int rc = check_args(s, d, b, sh);
    if (rc) return rc;
    if (mode == MODE_COPY && s->elem_size != d->elem_size) return -8;
    if (mode == MODE_F16_E4M3 && (s->elem_size != 2 || d->elem_size != 1 || (!d->k_scales != !d->v_scales)))
        return -8;
    if (mode == MODE_F32_F16 && (s->elem_size != 4 || d->elem_size != 2)) return -8;
    if (mode == MODE_F32_E4M3 && (s->elem_size != 4 || d->elem_size != 1)) return -8;
    if (mode == MODE_E4M3_F16 && (s->elem_size != 1 || d->elem_size != 2)) return -8;
    if (mode == MODE_E4M3_F32 && (s->elem_size != 1 || d->elem_size != 4)) return -8;
    const long units = (long)b->n_seqs * sh->n_layers * 2;
    if (n_threads <= 1) {
        /* faithful order: the reference walks layers, K then V, with plain
         * iterators and no thread pool (engine/src/kv_cache.rs:402-431).     */
        for (long u = 0; u < units; u++)
            handoff_unit(s, d, b, sh, (uint32_t)(u / (sh->n_layers * 2)),
                         (uint32_t)((u / 2) % sh->n_layers), (int)(u & 1), mode);
    } else {
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(n_threads)
#endif
        for (long u = 0; u < units; u++)
            handoff_unit(s, d, b, sh, (uint32_t)(u / (sh->n_layers * 2)),
                         (uint32_t)((u / 2) % sh->n_layers), (int)(u & 1), mode);
    }
    return 0;
}

int orc_handoff_copy(const orc_pool* s, const orc_pool* d, const orc_batch* b, const orc_shard* sh,
                     int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_COPY);
}
int orc_handoff_f16_to_e4m3(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                            const orc_shard* sh, int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_F16_E4M3);
}
int orc_handoff_f32_to_f16(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                           const orc_shard* sh, int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_F32_F16);
}

int orc_handoff_f32_to_e4m3(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                            const orc_shard* sh, int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_F32_E4M3);
}
int orc_handoff_e4m3_to_f16(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                            const orc_shard* sh, int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_E4M3_F16);
}
int orc_handoff_e4m3_to_f32(const orc_pool* s, const orc_pool* d, const orc_batch* b,
                            const orc_shard* sh, int n_threads) {
    return handoff_run(s, d, b, sh, n_threads, MODE_E4M3_F32);
}

/* ---- decode attention over a paged pool (the FP8 cache's consumer) -------------------
 * kernels/src/attention.rs:486-590 (paged_flash_attention) with seq_len == 1: tiles of
 * FLASH_BC = 32 cached tokens (:343), online softmax in the reference's update order, K/V rows
 * resolved through the block table by paged_row_offset (:472-484), GQA head h reading kv head
 * h / (num_heads / num_kv_heads).  The pool may be F32, F16 or E4M3; an E4M3 element reads as
 * orc_e4m3_to_f32(byte) times the block's scale when the pool has scale arrays (the rule of
 * orc_handoff_e4m3_to_f32).  exp is libm's expf where the reference uses its own polynomial
 * (kernels/src/portable_math.rs:5-40); the comparison with the GPU kernel is by tolerance. */
static float pool_elem(const orc_pool* p, const char* layer, const float* scales, uint32_t l,
                       const uint32_t* table, size_t tok, uint32_t kv_h, uint32_t d) {
    size_t off = orc_paged_row_offset(table, p->block_size, (size_t)p->n_kv_heads * p->head_dim, tok, kv_h, p->head_dim) + d;
    if (p->elem_size == 4) return ((const float*)layer)[off];
    if (p->elem_size == 2) return orc_f16_to_f32(((const uint16_t*)layer)[off]);
    float sc = scales ? scales[((size_t)l * p->total_blocks + table[tok / p->block_size]) * p->n_kv_heads + kv_h] : 1.0f;
    volatile float x = orc_e4m3_to_f32(((const uint8_t*)layer)[off]) * sc;
    return x;
}

int orc_paged_decode_attention(const orc_pool* p, uint32_t layer, const float* q, const uint32_t* tables,
                               uint32_t table_stride, const uint32_t* kv_lens, uint32_t n_seqs,
                               uint32_t num_heads, float scale, float* out) {
    if (!p || !q || !tables || !kv_lens || !out || layer >= p->n_layers) return -1;
    if (!num_heads || num_heads % p->n_kv_heads) return -2;
    const uint32_t D = p->head_dim, hpg = num_heads / p->n_kv_heads, BC = 32;
    const char* kl = p->k_layers[layer];
    const char* vl = p->v_layers[layer];
    float* o_acc = malloc(sizeof(float) * D);
    float tile_scores[32];
    for (uint32_t s = 0; s < n_seqs; s++) {
        const uint32_t* table = tables + (size_t)s * table_stride;
        const uint32_t kv_len = kv_lens[s];
        if ((kv_len + p->block_size - 1) / p->block_size > table_stride) { free(o_acc); return -3; }
        for (uint32_t h = 0; h < num_heads; h++) {
            const uint32_t kv_h = h / hpg;
            const float* qv = q + ((size_t)s * num_heads + h) * D;
            float row_max = -INFINITY, row_sum = 0.0f;
            for (uint32_t d = 0; d < D; d++) o_acc[d] = 0.0f;
            for (uint32_t t0 = 0; t0 < kv_len; t0 += BC) {
                const uint32_t t1 = t0 + BC < kv_len ? t0 + BC : kv_len;
                float tile_max = -INFINITY;
                for (uint32_t t = t0; t < t1; t++) {
                    float dot = 0.0f;
                    for (uint32_t d = 0; d < D; d++) dot += qv[d] * pool_elem(p, kl, p->k_scales, layer, table, t, kv_h, d);
                    tile_scores[t - t0] = dot * scale;
                    if (tile_scores[t - t0] > tile_max) tile_max = tile_scores[t - t0];
                }
                const float new_max = row_max > tile_max ? row_max : tile_max;
                const float corr = row_max > -INFINITY ? expf(row_max - new_max) : 0.0f;
                for (uint32_t d = 0; d < D; d++) o_acc[d] *= corr;
                row_sum *= corr;
                float tile_sum = 0.0f;
                for (uint32_t t = t0; t < t1; t++) {
                    tile_scores[t - t0] = expf(tile_scores[t - t0] - new_max);
                    tile_sum += tile_scores[t - t0];
                }
                for (uint32_t t = t0; t < t1; t++) {
                    const float w = tile_scores[t - t0];
                    if (w == 0.0f) continue;
                    for (uint32_t d = 0; d < D; d++) o_acc[d] += w * pool_elem(p, vl, p->v_scales, layer, table, t, kv_h, d);
                }
                row_sum += tile_sum;
                row_max = new_max;
            }
            const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
            float* ov = out + ((size_t)s * num_heads + h) * D;
            for (uint32_t d = 0; d < D; d++) ov[d] = o_acc[d] * inv;
        }
    }
    free(o_acc);
    return 0;
}

/* Block-level collapse of ref_count += 1 on lookup/probe
 * (engine/src/prefix_cache.rs:68, engine/src/kv_cache.rs:635) and
 * saturating_sub(1) on release (prefix_cache.rs:92, kv_cache.rs:691).       */
void orc_refcount_apply(uint32_t* rc, const orc_batch* b, uint32_t block_size, int delta) {
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        uint32_t pre = b->prefix_lens ? b->prefix_lens[q] : 0;
        for (uint32_t i = 0; i < pre / block_size; i++) {
            uint32_t id = b->dst_tables[(size_t)q * b->table_stride + i];
            if (delta > 0) rc[id] += 1u;
            else if (delta < 0 && rc[id] > 0) rc[id] -= 1u;
        }
    }
}

/* engine/src/cutile_kv_cache.rs:1274-1286 and :1294-1368: wrapping sum of the
 * f32 bit patterns; narrower pools are widened first.                       */
uint64_t orc_bits_checksum_f32(const float* v, size_t n) {
    uint64_t cs = 0;
    for (size_t i = 0; i < n; i++) cs += f32_bits(v[i]);
    return cs;
}
uint64_t orc_bits_checksum_f16_as_f32(const uint16_t* v, size_t n) {
    uint64_t cs = 0;
    for (size_t i = 0; i < n; i++) cs += f32_bits(orc_f16_to_f32(v[i]));
    return cs;
}
uint64_t orc_bits_checksum_e4m3_as_f32(const uint8_t* v, size_t n) {
    uint64_t cs = 0;
    for (size_t i = 0; i < n; i++) cs += f32_bits(orc_e4m3_to_f32(v[i]));
    return cs;
}

/* ======================================================================= */
/* RadixTree: engine/src/prefix_cache.rs:17-149                             */
/* ======================================================================= */
typedef struct {
    uint32_t* child_tok;
    size_t* child_idx;
    size_t n_children, cap_children;
    size_t page_id;
    int has_page;
    size_t ref_count;
    uint64_t last_used;
} rnode;
struct orc_radix {
    rnode* nodes;
    size_t n, cap;
    uint64_t tick, hits, tokens_saved;
};
static size_t radix_push(orc_radix* r) {
    if (r->n == r->cap) {
        r->cap = r->cap ? r->cap * 2 : 16;
        r->nodes = realloc(r->nodes, r->cap * sizeof(rnode));
    }
    memset(&r->nodes[r->n], 0, sizeof(rnode));
    return r->n++;
}
static int64_t radix_child(const orc_radix* r, size_t node, uint32_t tok) {
    const rnode* nd = &r->nodes[node];
    for (size_t i = 0; i < nd->n_children; i++)
        if (nd->child_tok[i] == tok) return (int64_t)nd->child_idx[i];
    return -1;
}
orc_radix* orc_radix_new(void) {
    orc_radix* r = calloc(1, sizeof *r);
    radix_push(r); /* root */
    return r;
}
void orc_radix_delete(orc_radix* r) {
    if (!r) return;
    for (size_t i = 0; i < r->n; i++) {
        free(r->nodes[i].child_tok);
        free(r->nodes[i].child_idx);
    }
    free(r->nodes);
    free(r);
}
/* :32-56 -- a page id is attached to token i only when a NEW node is made. */
void orc_radix_insert(orc_radix* r, const uint32_t* tokens, size_t n, const size_t* pages,
                      size_t n_pages) {
    r->tick++;
    size_t node = 0;
    for (size_t i = 0; i < n; i++) {
        int64_t c = radix_child(r, node, tokens[i]);
        if (c >= 0) {
            node = (size_t)c;
            r->nodes[node].last_used = r->tick;
        } else {
            size_t nn = radix_push(r);
            if (i < n_pages) {
                r->nodes[nn].has_page = 1;
                r->nodes[nn].page_id = pages[i];
            }
            r->nodes[nn].last_used = r->tick;
            rnode* p = &r->nodes[node];
            if (p->n_children == p->cap_children) {
                p->cap_children = p->cap_children ? p->cap_children * 2 : 4;
                p->child_tok = realloc(p->child_tok, p->cap_children * sizeof(uint32_t));
                p->child_idx = realloc(p->child_idx, p->cap_children * sizeof(size_t));
            }
            p->child_tok[p->n_children] = tokens[i];
            p->child_idx[p->n_children++] = nn;
            node = nn;
        }
    }
}
/* :58-85 */
size_t orc_radix_lookup(orc_radix* r, const uint32_t* tokens, size_t n, size_t* pages_out,
                        size_t cap, size_t* n_pages_out) {
    r->tick++;
    size_t node = 0, matched = 0, np = 0;
    for (size_t i = 0; i < n; i++) {
        int64_t c = radix_child(r, node, tokens[i]);
        if (c < 0) break;
        node = (size_t)c;
        r->nodes[node].last_used = r->tick;
        r->nodes[node].ref_count += 1;
        matched++;
        if (r->nodes[node].has_page) {
            if (np < cap && pages_out) pages_out[np] = r->nodes[node].page_id;
            np++;
        }
    }
    if (matched > 0) {
        r->hits++;
        r->tokens_saved += matched;
    }
    if (n_pages_out) *n_pages_out = np;
    return matched;
}
/* :87-97 */
void orc_radix_release(orc_radix* r, const uint32_t* tokens, size_t n) {
    size_t node = 0;
    for (size_t i = 0; i < n; i++) {
        int64_t c = radix_child(r, node, tokens[i]);
        if (c < 0) break;
        node = (size_t)c;
        if (r->nodes[node].ref_count > 0) r->nodes[node].ref_count -= 1;
    }
}
/* :99-125 -- only the oldest unreferenced leaf is unlinked; its pages are
 * returned.  The node itself stays in the arena (node_count never shrinks). */
size_t orc_radix_evict_lru(orc_radix* r, size_t* freed_out, size_t cap) {
    int64_t oldest = -1;
    for (size_t i = 1; i < r->n; i++) {
        rnode* nd = &r->nodes[i];
        if (nd->ref_count == 0 && nd->n_children == 0)
            if (oldest < 0 || nd->last_used < r->nodes[oldest].last_used) oldest = (int64_t)i;
    }
    if (oldest < 0) return 0;
    size_t nf = 0;
    if (r->nodes[oldest].has_page) {
        if (cap > 0 && freed_out) freed_out[0] = r->nodes[oldest].page_id;
        nf = 1;
    }
    for (size_t i = 0; i < r->n; i++) {
        rnode* nd = &r->nodes[i];
        size_t w = 0;
        for (size_t k = 0; k < nd->n_children; k++)
            if (nd->child_idx[k] != (size_t)oldest) {
                nd->child_tok[w] = nd->child_tok[k];
                nd->child_idx[w++] = nd->child_idx[k];
            }
        nd->n_children = w;
    }
    /* As in the reference, the unlinked node stays in the arena with
     * ref_count 0 and no children, so a second call selects it again and
     * reports the same page a second time.                                  */
    return nf;
}
uint64_t orc_radix_hit_count(const orc_radix* r) { return r->hits; }
uint64_t orc_radix_tokens_saved(const orc_radix* r) { return r->tokens_saved; }
size_t orc_radix_node_count(const orc_radix* r) { return r->n; }
int64_t orc_radix_ref_count(const orc_radix* r, const uint32_t* tokens, size_t n) {
    size_t node = 0;
    for (size_t i = 0; i < n; i++) {
        int64_t c = radix_child(r, node, tokens[i]);
        if (c < 0) return -1;
        node = (size_t)c;
    }
    return (int64_t)r->nodes[node].ref_count;
}

/* ======================================================================= */
/* PrefixCacheTable: engine/src/kv_cache.rs:581-730.  The reference keys a   */
/* HashMap by a 64-bit hash of (salt, tokens) and then compares the tokens;  */
/* this restatement keys by the (salt, tokens) pair itself, which is the     */
/* same map whenever two different keys do not share a hash.  Entries hold   */
/* destination block ids instead of cloned K/V vectors.                      */
/* ======================================================================= */
typedef struct {
    uint32_t* tokens;
    size_t n_tokens;
    char* salt; /* NULL == None */
    uint32_t* blocks;
    size_t n_blocks, seq_len, ref_count;
    uint64_t last_used;
} pentry;
struct orc_prefix_table {
    pentry* e;
    size_t n, cap, max_entries;
    uint64_t tick, hits, tokens_saved;
};
static int salt_eq(const char* a, const char* b) {
    if (!a || !b) return a == b;
    return strcmp(a, b) == 0;
}
static int64_t pt_find(const orc_prefix_table* t, const uint32_t* tok, size_t n, const char* salt) {
    for (size_t i = 0; i < t->n; i++)
        if (t->e[i].n_tokens == n && salt_eq(t->e[i].salt, salt) &&
            memcmp(t->e[i].tokens, tok, n * sizeof(uint32_t)) == 0)
            return (int64_t)i;
    return -1;
}
static void pt_drop(orc_prefix_table* t, size_t i) {
    free(t->e[i].tokens);
    free(t->e[i].salt);
    free(t->e[i].blocks);
    t->e[i] = t->e[t->n - 1];
    t->n--;
}
orc_prefix_table* orc_pt_new(size_t max_entries) {
    orc_prefix_table* t = calloc(1, sizeof *t);
    t->max_entries = max_entries;
    return t;
}
void orc_pt_delete(orc_prefix_table* t) {
    if (!t) return;
    while (t->n) pt_drop(t, t->n - 1);
    free(t->e);
    free(t);
}
/* :695-706 */
static void pt_evict_lru(orc_prefix_table* t) {
    int64_t best = -1;
    for (size_t i = 0; i < t->n; i++)
        if (t->e[i].ref_count == 0 && (best < 0 || t->e[i].last_used < t->e[best].last_used))
            best = (int64_t)i;
    if (best >= 0) pt_drop(t, (size_t)best);
}
/* :651-682 */
void orc_pt_store(orc_prefix_table* t, const uint32_t* tok, size_t n, const char* salt,
                  const uint32_t* blocks, size_t n_blocks, size_t seq_len) {
    if (n == 0 || seq_len == 0) return;
    t->tick++;
    if (t->n >= t->max_entries) pt_evict_lru(t);
    int64_t old = pt_find(t, tok, n, salt);
    if (old >= 0) pt_drop(t, (size_t)old); /* HashMap::insert replaces */
    if (t->n == t->cap) {
        t->cap = t->cap ? t->cap * 2 : 8;
        t->e = realloc(t->e, t->cap * sizeof(pentry));
    }
    pentry* p = &t->e[t->n++];
    p->tokens = malloc(n * sizeof(uint32_t));
    memcpy(p->tokens, tok, n * sizeof(uint32_t));
    p->n_tokens = n;
    p->salt = salt ? strdup(salt) : NULL;
    p->blocks = malloc((n_blocks ? n_blocks : 1) * sizeof(uint32_t));
    if (n_blocks) memcpy(p->blocks, blocks, n_blocks * sizeof(uint32_t));
    p->n_blocks = n_blocks;
    p->seq_len = seq_len;
    p->ref_count = 0;
    p->last_used = t->tick;
}
/* :622-647 -- longest prefix first */
size_t orc_pt_probe(orc_prefix_table* t, const uint32_t* tok, size_t n, const char* salt,
                    uint32_t* blocks_out, size_t cap, size_t* n_blocks_out) {
    t->tick++;
    for (size_t len = n; len >= 1; len--) {
        int64_t i = pt_find(t, tok, len, salt);
        if (i >= 0) {
            pentry* p = &t->e[i];
            p->last_used = t->tick;
            p->ref_count += 1;
            t->hits++;
            t->tokens_saved += len;
            if (n_blocks_out) *n_blocks_out = p->n_blocks;
            for (size_t k = 0; k < p->n_blocks && k < cap; k++) blocks_out[k] = p->blocks[k];
            return p->seq_len;
        }
    }
    if (n_blocks_out) *n_blocks_out = 0;
    return 0;
}
/* :688-693 */
void orc_pt_release(orc_prefix_table* t, const uint32_t* tok, size_t n, const char* salt) {
    int64_t i = pt_find(t, tok, n, salt);
    if (i >= 0 && t->e[i].ref_count > 0) t->e[i].ref_count -= 1;
}
size_t orc_pt_len(const orc_prefix_table* t) { return t->n; }
uint64_t orc_pt_hit_count(const orc_prefix_table* t) { return t->hits; }
uint64_t orc_pt_tokens_saved(const orc_prefix_table* t) { return t->tokens_saved; }
int64_t orc_pt_ref_count(const orc_prefix_table* t, const uint32_t* tok, size_t n, const char* salt) {
    int64_t i = pt_find(t, tok, n, salt);
    return i < 0 ? -1 : (int64_t)t->e[i].ref_count;
}

/* ======================================================================= */
/* PageRunAllocator: engine/src/gpu_page_pool.rs:34-218                     */
/* ======================================================================= */
#define ORC_MAX_FREE_RUNS 128
struct orc_run_allocator {
    size_t start[ORC_MAX_FREE_RUNS], pages[ORC_MAX_FREE_RUNS];
    size_t free_len, total, allocated;
};
orc_run_allocator* orc_ra_new(size_t total) {
    orc_run_allocator* a = calloc(1, sizeof *a);
    a->pages[0] = total;
    a->free_len = total > 0;
    a->total = total;
    return a;
}
void orc_ra_delete(orc_run_allocator* a) { free(a); }
/* :95-128 best fit, earliest scanned on ties; swap-remove when consumed. */
int orc_ra_alloc(orc_run_allocator* a, size_t pages, size_t* start_out) {
    if (pages == 0) return 0;
    int64_t best = -1;
    for (size_t i = 0; i < a->free_len; i++)
        if (a->pages[i] >= pages && (best < 0 || a->pages[i] < a->pages[best])) best = (int64_t)i;
    if (best < 0) return 0;
    *start_out = a->start[best];
    size_t rem = a->pages[best] - pages;
    if (rem == 0) {
        a->start[best] = a->start[a->free_len - 1];
        a->pages[best] = a->pages[a->free_len - 1];
        a->free_len--;
    } else {
        a->start[best] += pages;
        a->pages[best] = rem;
    }
    a->allocated += pages;
    return 1;
}
/* :132-181 absorb adjacent runs until none is adjacent, then append once. */
void orc_ra_free(orc_run_allocator* a, size_t start, size_t pages) {
    if (pages == 0 || start + pages > a->total) return;
    a->allocated -= pages;
    for (;;) {
        int64_t hit = -1;
        for (size_t i = 0; i < a->free_len; i++) {
            if (a->start[i] + a->pages[i] == start) {
                start = a->start[i];
                pages += a->pages[i];
                hit = (int64_t)i;
                break;
            }
            if (a->start[i] == start + pages) {
                pages += a->pages[i];
                hit = (int64_t)i;
                break;
            }
        }
        if (hit < 0) break;
        a->start[hit] = a->start[a->free_len - 1];
        a->pages[hit] = a->pages[a->free_len - 1];
        a->free_len--;
    }
    if (a->free_len >= ORC_MAX_FREE_RUNS) abort(); /* reference panics (:172-176) */
    a->start[a->free_len] = start;
    a->pages[a->free_len++] = pages;
}
/* :192-217 */
int orc_ra_try_extend(orc_run_allocator* a, size_t start, size_t pages, size_t target) {
    if (target <= pages) return 1;
    size_t extra = target - pages, end = start + pages;
    for (size_t i = 0; i < a->free_len; i++)
        if (a->start[i] == end && a->pages[i] >= extra) {
            size_t rem = a->pages[i] - extra;
            if (rem == 0) {
                a->start[i] = a->start[a->free_len - 1];
                a->pages[i] = a->pages[a->free_len - 1];
                a->free_len--;
            } else {
                a->start[i] = end + extra;
                a->pages[i] = rem;
            }
            a->allocated += extra;
            return 1;
        }
    return 0;
}
size_t orc_ra_free_pages(const orc_run_allocator* a) {
    size_t s = 0;
    for (size_t i = 0; i < a->free_len; i++) s += a->pages[i];
    return s;
}
size_t orc_ra_allocated_pages(const orc_run_allocator* a) { return a->allocated; }
size_t orc_ra_free_runs(const orc_run_allocator* a, size_t* starts, size_t* pages, size_t cap) {
    for (size_t i = 0; i < a->free_len && i < cap; i++) {
        starts[i] = a->start[i];
        pages[i] = a->pages[i];
    }
    return a->free_len;
}

/* ======================================================================= */
/* synthetic inputs.  The reference has no benchmark for this path; these    */
/* generators define the seeded workloads (counter-based, order-free).       */
/* ======================================================================= */
uint64_t orc_mix64(uint64_t seed, uint64_t stream, uint64_t index) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + stream * 0xD1B54A32D192ED03ull + index;
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void orc_gen_normal_f16(uint16_t* out, size_t n, uint64_t seed, uint64_t stream, double sigma,
                        uint32_t head_dim, const uint32_t* outlier_channels, uint32_t n_outliers,
                        double outlier_gain, size_t first_index) {
    const double two_pi = 6.283185307179586476925286766559;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long i = 0; i < (long)n; i++) {
        size_t g = first_index + (size_t)i;
        uint64_t a = orc_mix64(seed, stream, 2 * g), b = orc_mix64(seed, stream, 2 * g + 1);
        double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0); /* (0, 1] */
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
        double z = sqrt(-2.0 * log(u1)) * cos(two_pi * u2) * sigma;
        if (n_outliers && head_dim) {
            uint32_t ch = (uint32_t)(g % head_dim);
            for (uint32_t k = 0; k < n_outliers; k++)
                if (outlier_channels[k] == ch) z *= outlier_gain;
        }
        out[i] = orc_f32_to_f16((float)z);
    }
}

/* Fisher-Yates, high index down, as tools/bench-gpu/src/bench_decode_ops.rs:2935-2947
 * does (the mixer differs: counter-based instead of an LCG).                */
void orc_gen_permutation(uint32_t* out, uint32_t n, uint64_t seed, uint64_t stream) {
    for (uint32_t i = 0; i < n; i++) out[i] = i;
    for (uint32_t i = n; i-- > 1;) {
        uint32_t j = (uint32_t)(orc_mix64(seed, stream, i) % (uint64_t)(i + 1));
        uint32_t t = out[i];
        out[i] = out[j];
        out[j] = t;
    }
}

void orc_gen_lengths(uint32_t* out, uint32_t n, uint32_t lo, uint32_t hi, uint64_t seed,
                     uint64_t stream) {
    for (uint32_t i = 0; i < n; i++)
        out[i] = lo + (uint32_t)(orc_mix64(seed, stream, i) % (uint64_t)(hi - lo + 1));
}
