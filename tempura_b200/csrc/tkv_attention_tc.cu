// Decode attention over the paged pool on the fifth-generation tensor cores (tcgen05, sm_100a).
//
// What is computed is what tkv_attention.cu computes (paged_flash_attention of
// kernels/src/attention.rs:486-590 over the widened pool values, one query token per sequence, grouped
// query heads, per-(layer, block, kv-head) scales of an E4M3 pool applied on the fly); what differs is
// where the two contractions run.  A 16-token block of an 8-kv-head pool is 128 rows of 128 elements,
// [token][kv head][dim]: exactly one M = 128 operand tile, in the order the pool stores it.  So per block
//
//     S^T[128 rows (token, kv head)][NQ columns (query head, term)] = K_block . Q^T        (tcgen05.mma, K from shared memory as it arrived)
//     O^T[128 rows (dim)][NP columns (query head, term)]           += V_block^T . P^T      (V read MN-major from the same kind of tile)
//
// with the accumulators in tensor memory.  The K and V bytes are never touched by a thread: a producer
// warp brings whole blocks in with 2-D tensor-map copies (128-byte swizzle, the layout the MMA's shared
// memory descriptors name), one thread issues the MMAs, and two groups of four softmax warps take
// alternate blocks (each group with its own accumulators, merged at the end).  A softmax thread owns one
// (token, kv head) row: it reads its row of S^T from tensor memory, keeps the columns of its own kv
// head, and writes the probabilities into P^T, whose entries for other kv heads stay zero.
// A row's columns of the other seven kv heads are computed and dropped: that is 7/8 of the tensor work
// and still a fifth of the time the block takes to arrive from HBM, which is the bound.
//
// Operand precision.  F16 pool: q and the probabilities are F16 (as the mma.sync kernel feeds them).
// E4M3 pool: both operands of an MMA must be 8-bit, so q is split into two E4M3 terms (per-head power
// of two scale, residual in the second term: 2^-8 relative) and a probability into three E5M2 terms
// (E5M2 for its range: weights down to 2^-31 of the running maximum survive; three 3-bit terms give
// 2^-9 relative).  The terms are separate columns of Q^T / P^T, summed after the MMA.
//
// The running maximum is kept per query head in shared memory and only raised when a block exceeds it
// by more than 2^6 (weights stay below 2^6 * 2^9 < the E5M2 maximum); raising it rescales O^T in tensor
// memory, which happens a few times per sequence at most.  Every wait is bounded; a CTA that gives up
// reports through `status`, drains its copies and frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <mutex>

#include "../../include/tkv.h"
#include "tkv_attention_tc.h"
#include "tkv_tc_common.cuh"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
}

namespace tkv_tc {

constexpr int D = 128, BS = 16, HKV = 8, ROWS = BS * HKV;   // one block = 128 operand rows
constexpr int TILE = ROWS * 128;                           // bytes of one [128 rows][128 B] swizzled tile
constexpr float RAISE = 6.0f;                              // the running maximum is raised when a block exceeds it by 2^RAISE
constexpr float SHIFT = 9.0f;                              // probabilities enter P^T as 2^(s - m + SHIFT): below the E5M2 / F16 maximum

// Control block at the head of shared memory.  Two softmax groups (warps 0-3 and 4-7) take alternate blocks of a token
// range; each has its own S^T buffers, P^T buffers, O^T accumulator, running maxima and row sums, and writes its own
// partial result (the split-merge kernel folds them together with the other ranges').
constexpr int MAX_ITEMS = 128;        // token ranges one CTA walks
constexpr int NG = (int)PARTS_PER_RANGE;   // softmax groups, taking the blocks of a range in turn
constexpr int SBUF = NG == 2 ? 2 : 1; // S^T buffers per group (tensor memory: NG * (O^T + SBUF * S^T) <= 512 columns)
constexpr int ATHREADS = (4 * NG + 3) * 32;
struct Group {
    uint64_t s_full[2], s_free[2];    // S^T buffers: QK done / every warp of the group has read it
    uint64_t p_full[2], p_free[2];    // P^T buffers: written / the PV MMA has read it
    int block_max[2][32];             // per block parity: ordered-int maxima of the query heads that asked for a raise
    uint32_t raise[2];
    float m_used[32], factor[32], l_sum[4][32];
};
struct Control {
    uint64_t k_full[8], k_empty[8];   // K ring: tile landed / the QK MMAs that read it are done (a K tile is held only that long)
    uint64_t v_full[8], v_empty[8];   // V ring (the block's scales travel with it): landed / the PV MMAs are done
    uint64_t q_full, q_free;          // Q^T: written for the next range / every QK MMA of the current range done
    uint64_t drained[2];              // teardown: every MMA an issuer has issued has completed
    uint32_t tmem_base, fail, n_items, pad;
    float q_inv[2][32];               // per range parity: what undoes the power-of-two scale of each query head
    float scales[8][16];              // per V slot: 8 K scales, 8 V scales
    Group g[NG];
    uint32_t item_id[MAX_ITEMS];      // sequence * ranges per sequence + range
    uint16_t item_blocks[MAX_ITEMS];
};
static_assert(sizeof(Control) <= 6144, "control block");
constexpr int ACTRL = 6144;

// Shared-memory shape of the kernel, known at compile time (so that ring positions are divisions by constants, not by kernel arguments):
// what is fixed, and how many K and V tiles the rest holds.  A K tile is held from its arrival to the end of its QK MMAs, a V tile
// through the softmax of its block as well: most slots go to V.
template <bool FP8, int G> struct Shape {
    static constexpr int ES = FP8 ? 1 : 2, QTERMS = FP8 ? 2 : 1, PT = FP8 ? 3 : 1, PBUF = 1;
    static constexpr int CQ = (G * QTERMS < 2) ? 2 : G * QTERMS, CP = (G * PT < 2) ? 2 : G * PT;
    // P^T of an E4M3 pool is kept MN-major, [128 block rows][128 B]: a thread's twelve bytes (three terms x four query heads) are three
    // words of its own row; an F16 pool's P^T stays K-major, [NP rows][128 B] per 64 block rows
    static constexpr size_t p_bytes = FP8 ? (size_t)ROWS * 128 : (size_t)HKV * CP * 128 * ES;
    static constexpr size_t fixed = ACTRL + (size_t)HKV * CQ * 128 * ES + NG * (size_t)PBUF * p_bytes;
    static constexpr size_t tile = (size_t)TILE * ES;              // K or V of one block
    static constexpr uint32_t tiles = (uint32_t)((227 * 1024 - fixed) / tile);
    static constexpr uint32_t n_k = FP8 ? 4u : 2u, n_v = tiles - n_k < 8u ? tiles - n_k : 8u;
    static_assert(tiles >= n_k + 2, "room for the rings");
    static constexpr size_t smem = fixed + (size_t)(n_k + n_v) * tile;
};

// A persistent CTA per SM walks token ranges (sequence, range) c, c + gridDim.x, ...: barriers, tensor memory and the ring
// are set up once, and the producer runs ahead across range boundaries, so the ring never drains between ranges.
template <bool FP8, int G>
__global__ void __launch_bounds__(ATHREADS, 1)
decode_attn_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a) {
    constexpr uint32_t n_k = Shape<FP8, G>::n_k, n_v = Shape<FP8, G>::n_v;      // K and V tiles in the rings
    constexpr int ES = FP8 ? 1 : 2;                    // bytes per pool element = 128-byte column groups per row
    constexpr int QTERMS = FP8 ? 2 : 1, PT = FP8 ? 3 : 1;   // terms a query element / a probability is split into
    constexpr int PBUF = 1;     // P^T buffers per group
    constexpr uint32_t GCOLS = NG == 2 ? 256u : 160u, S_OFF = NG == 2 ? 128u : 96u;   // a group's tensor-memory columns: O^T at 0, S^T behind it
    constexpr int CQ = (G * QTERMS < 2) ? 2 : G * QTERMS;   // columns per kv head in S^T and in O^T (N must be a multiple of 16)
    constexpr int CP = (G * PT < 2) ? 2 : G * PT;
    constexpr int NQ = HKV * CQ, NP = HKV * CP;
    static_assert(NQ % 16 == 0 && NP % 16 == 0 && NQ <= 64 && NP <= 128, "MMA N; a group owns 256 tensor-memory columns: O^T at 0, S^T at 128 and 192");
    static_assert(NQ == 64 || NQ == 32, "S^T is read as one 64- or 32-column load");
    constexpr int KV_TILE = TILE * ES;                 // K (or V) of one block in shared memory
    constexpr int Q_SUB = NQ * 128;                    // one [NQ rows][128 B] tile of Q^T (F16: one per 64-dim column group)
    constexpr int QT_BYTES = Q_SUB * ES, PT_BYTES = (int)Shape<FP8, G>::p_bytes;
    constexpr uint32_t FMT_P = FP8 ? 1u : 0u;          // kind::f8f6f4: E4M3 = 0, E5M2 = 1; kind::f16: F16 = 0
    constexpr uint32_t IDESC_QK = instr_desc(0u, 0u, 0u, NQ), IDESC_PV = FP8 ? instr_desc2(0u, FMT_P, 1u, 1u, NP) : instr_desc(0u, FMT_P, 1u, NP);
    constexpr int KSTEPS = 4 * ES;                     // 32 bytes of the contraction per MMA: 4 steps per 128-byte group
    // operand descriptors: everything but the start address is constant (stride between 8-row groups 1024 B, version 1, 128-byte swizzle)
    constexpr uint64_t DESC_HI = ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
    constexpr uint64_t DESC_K = DESC_HI | ((uint64_t)1u << 16);                       // leading offset unused by K-major operands
    constexpr uint64_t DESC_V = DESC_HI | ((uint64_t)(TILE >> 4) << 16);              // MN-major: the second 64-dim column group one tile further

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t ranges = a.n_splits;                // token ranges per sequence
    const uint32_t n_parts = (uint32_t)NG * a.n_splits;  // partial slots per (sequence, kv head): one per range and group

    extern __shared__ __align__(1024) unsigned char smem[];
    Control* c = reinterpret_cast<Control*>(smem);
    unsigned char* q_tile = smem + ACTRL;                          // Q^T of the current range
    unsigned char* p_tile = q_tile + QT_BYTES;                    // P^T: PBUF buffers per group
    unsigned char* k_ring = p_tile + NG * PBUF * PT_BYTES;         // n_k K tiles, then n_v V tiles
    unsigned char* v_ring = k_ring + (size_t)n_k * KV_TILE;
    const volatile uint32_t* fail_word = &c->fail;

    if (tid == 0) {
        for (uint32_t s = 0; s < 8; s++) {
            mbar_init(c->k_full + s, 1);
            mbar_init(c->k_empty + s, 1);
            mbar_init(c->v_full + s, 1);
            mbar_init(c->v_empty + s, 1);
        }
        for (int g = 0; g < NG; g++)
            for (int b = 0; b < 2; b++) {
                mbar_init(c->g[g].s_full + b, 1);
                mbar_init(c->g[g].s_free + b, 4);
                mbar_init(c->g[g].p_full + b, 4);
                mbar_init(c->g[g].p_free + b, 1);
                c->g[g].raise[b] = 0;
            }
        mbar_init(&c->q_full, 4);
        mbar_init(&c->q_free, 1);
        mbar_init(c->drained, 1);
        mbar_init(c->drained + 1, 1);
        // tiles are addressed through descriptors that assume 1024-byte alignment: refuse to run rather than compute garbage
        c->fail = (smem_u32(smem) & 1023u) ? 2u : 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 64 * NG) c->g[tid >> 6].block_max[(tid >> 5) & 1][tid & 31] = ordered(-INFINITY);
    if (warp == 4 * NG + 1) {                                      // tensor memory: 512 columns, this CTA alone on its SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&c->tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else if (warp == 4 * NG) {
        // this CTA's ranges: the non-empty (sequence, range) pairs are ranked in sequence order and CTA c takes ranks c, c + gridDim.x,
        // ..., so every CTA gets the same number of ranges (one more or less) however ragged the lengths are
        uint32_t count = 0, before = 0;
        for (uint32_t base = 0; base < a.n_seqs; base += 32) {
            const uint32_t seq = base + lane;
            const uint32_t kv_len = seq < a.n_seqs ? min(a.kv_lens[seq], a.max_kv_len) : 0u;
            const uint32_t cnt = (kv_len + a.split_tokens - 1) / a.split_tokens;
            uint32_t incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= (uint32_t)o) incl += v;
            }
            const uint32_t first_rank = before + incl - cnt;
            const uint32_t mine = first_rank + (blockIdx.x + gridDim.x - first_rank % gridDim.x) % gridDim.x;   // first rank >= first_rank that is this CTA's
            const uint32_t n_emit = mine < first_rank + cnt ? (first_rank + cnt - 1 - mine) / gridDim.x + 1 : 0u;
            uint32_t pos = n_emit;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, pos, o);
                if (lane >= (uint32_t)o) pos += v;
            }
            const uint32_t chunk_total = __shfl_sync(0xFFFFFFFFu, pos, 31);
            pos = count + pos - n_emit;
            for (uint32_t e = 0; e < n_emit && pos + e < MAX_ITEMS; e++) {
                const uint32_t split = mine - first_rank + e * gridDim.x, t_begin = split * a.split_tokens;
                c->item_id[pos + e] = seq * ranges + split;
                c->item_blocks[pos + e] = (uint16_t)((min(kv_len, t_begin + a.split_tokens) + BS - 1) / BS - t_begin / BS);
            }
            count = min(count + chunk_total, (uint32_t)MAX_ITEMS);
            before += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
        if (lane == 0) c->n_items = count;
    } else if (warp < 4 * NG) {
        // zero the P^T buffers once: entries of other kv heads stay zero for good
        for (uint32_t i = tid; i < (QT_BYTES + NG * PBUF * PT_BYTES) / 16; i += 128 * NG) reinterpret_cast<uint4*>(q_tile)[i] = make_uint4(0, 0, 0, 0);
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = c->tmem_base, n_items = c->n_items;

    if (warp == 4 * NG) {
        // ---- producer: every block of every range of this CTA, in order; lane 0 issues the copies ----
        uint32_t k = 0, issued = 0, why = 4u;
        bool ok = c->fail == 0;
        for (uint32_t n = 0; n < n_items && ok; n++) {
            const uint32_t id = c->item_id[n], seq = id / ranges, split = id - seq * ranges, n_blk = c->item_blocks[n];
            const uint32_t* table = a.tables + (size_t)seq * a.table_stride + split * (a.split_tokens / BS);
            uint32_t ids_next = lane < n_blk ? __ldg(table + lane) : 0u;
            for (uint32_t k0 = 0; k0 < n_blk && ok; k0 += 32) {
                const uint32_t ids = ids_next;
                ids_next = k0 + 32 + lane < n_blk ? __ldg(table + k0 + 32 + lane) : 0u;
                const uint32_t lim = min(32u, n_blk - k0);
                for (uint32_t i = 0; i < lim && ok; i++, k++) {
                    const uint32_t blk = __shfl_sync(0xFFFFFFFFu, ids, i), sk = k % n_k, sv = k % n_v;
                    if (lane == 0) {
                        if (blk >= a.total_blocks) {               // a stale or foreign id is never turned into an address
                            ok = false;
                            why = 2u;
                        }
                        if (ok && k >= n_k) ok = mbar_wait(c->k_empty + sk, ((k / n_k) - 1u) & 1u, fail_word);
                        if (ok) {
                            const uint32_t dst = smem_u32(k_ring + (size_t)sk * KV_TILE);
                            mbar_expect_tx(c->k_full + sk, KV_TILE);
#pragma unroll
                            for (int cg = 0; cg < ES; cg++) tma_box(dst + cg * TILE, &map_k, cg * 128, (int32_t)(blk * ROWS), c->k_full + sk);
                        }
                        if (ok && k >= n_v) ok = mbar_wait(c->v_empty + sv, ((k / n_v) - 1u) & 1u, fail_word);
                        if (ok) {
                            const uint32_t sc_bytes = a.k_scales ? HKV * 4u : 0u;
                            const uint32_t dst = smem_u32(v_ring + (size_t)sv * KV_TILE);
                            mbar_expect_tx(c->v_full + sv, KV_TILE + 2u * sc_bytes);
#pragma unroll
                            for (int cg = 0; cg < ES; cg++) tma_box(dst + cg * TILE, &map_v, cg * 128, (int32_t)(blk * ROWS), c->v_full + sv);
                            if (sc_bytes) {
                                bulk_copy(smem_u32(&c->scales[sv][0]), a.k_scales + (size_t)blk * HKV, sc_bytes, c->v_full + sv);
                                bulk_copy(smem_u32(&c->scales[sv][8]), a.v_scales + (size_t)blk * HKV, sc_bytes, c->v_full + sv);
                            }
                            issued = k + 1;
                        }
                    }
                    ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0u;
                }
            }
        }
        if (!ok && lane == 0) {
            atomicCAS(&c->fail, 0u, why);
            // give the copies still in flight a bounded chance to land before the CTA's shared memory is released
            for (uint32_t j = issued > n_v ? issued - n_v : 0u; j < issued; j++)
                for (uint32_t it = 0; it < (1u << 20); it++)
                    if (mbar_test(c->v_full + j % n_v, (j / n_v) & 1u) && (j + n_k < issued || mbar_test(c->k_full + j % n_k, (j / n_k) & 1u))) break;
        }
    } else if (warp == 4 * NG + 1) {
        // ---- QK issuer: S^T of block i of a range goes to group i & 1, into that group's next S^T buffer ----
        if (lane == 0) {
            const uint32_t q_lo = smem_u32(q_tile) >> 4, kr_lo = smem_u32(k_ring) >> 4;
            uint32_t k = 0, gq[NG] = {};
            bool ok = c->fail == 0;
            for (uint32_t n = 0; n < n_items && ok; n++) {
                const uint32_t n_blk = c->item_blocks[n];
                ok = mbar_wait(&c->q_full, n & 1u, fail_word);                    // this range's Q^T is in place
                for (uint32_t i = 0; i < n_blk && ok; i++, k++) {
                    const uint32_t g = i % NG, sb = gq[g] % SBUF, sk = k % n_k;
                    ok = mbar_wait(c->k_full + sk, (k / n_k) & 1u, fail_word);
                    if (ok && gq[g] >= (uint32_t)SBUF) ok = mbar_wait(c->g[g].s_free + sb, ((gq[g] / SBUF) - 1u) & 1u, fail_word);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem + g * GCOLS + S_OFF + sb * 64u, k_lo = kr_lo + sk * (KV_TILE >> 4);
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ks++)
                        mma<FP8>(d, DESC_K | (k_lo + (ks / 4) * (TILE >> 4) + (ks % 4) * 2),
                                 DESC_K | (q_lo + (ks / 4) * (Q_SUB >> 4) + (ks % 4) * 2), IDESC_QK, ks > 0 ? 1u : 0u);
                    tc_commit(c->g[g].s_full + sb);
                    tc_commit(c->k_empty + sk);                                    // the K tile goes back to the producer as soon as its scores exist
                    gq[g]++;
                }
                tc_commit(&c->q_free);                                            // Q^T may be rewritten once these MMAs are done
            }
            if (!ok) atomicCAS(&c->fail, 0u, 4u);
            tc_commit(c->drained);
            for (uint32_t it = 0; it < (1u << 22); it++)
                if (mbar_test(c->drained, 0u)) break;
        }
        __syncwarp();
    } else if (warp == 4 * NG + 2) {
        // ---- PV issuer: O^T of the block's group += V^T P^T as soon as the group has written P^T ----
        if (lane == 0) {
            const uint32_t vr_lo = smem_u32(v_ring) >> 4, p_lo = smem_u32(p_tile) >> 4;
            uint32_t k = 0, gp[NG] = {};
            bool ok = c->fail == 0;
            for (uint32_t n = 0; n < n_items && ok; n++) {
                const uint32_t n_blk = c->item_blocks[n];
                for (uint32_t i = 0; i < n_blk && ok; i++, k++) {
                    const uint32_t g = i % NG, pb = gp[g] % PBUF, sv = k % n_v;
                    ok = mbar_wait(c->g[g].p_full + pb, (gp[g] / PBUF) & 1u, fail_word) && mbar_wait(c->v_full + sv, (k / n_v) & 1u, fail_word);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t v_lo = vr_lo + sv * (KV_TILE >> 4), pg_lo = p_lo + (g * PBUF + pb) * (PT_BYTES >> 4);
#pragma unroll
                    for (int ks = 0; ks < KSTEPS; ks++)         // V^T MN-major: 32 / ES block rows of 128 B per step; P^T K-major: 32 bytes of the row per step
                        mma<FP8>(tmem + g * GCOLS, DESC_V | (v_lo + ks * ((32 / ES) * 128 >> 4)),
                                 FP8 ? (DESC_V | (pg_lo + ks * (32 * 128 >> 4))) : (DESC_K | (pg_lo + (ks / 4) * (NP * 128 >> 4) + (ks % 4) * 2)),
                                 IDESC_PV, (i >= (uint32_t)NG || ks > 0) ? 1u : 0u);            // a group's first block of a range starts its accumulator afresh
                    tc_commit(c->v_empty + sv);
                    tc_commit(c->g[g].p_free + pb);
                    gp[g]++;
                }
            }
            if (!ok) atomicCAS(&c->fail, 0u, 4u);
            tc_commit(c->drained + 1);
            for (uint32_t it = 0; it < (1u << 22); it++)
                if (mbar_test(c->drained + 1, 0u)) break;
        }
        __syncwarp();
    } else {
        // ---- softmax: group grp = warp / 4 takes blocks grp, grp + 2, ... of every range; thread t of the group owns block
        // row t = (token t / 8, kv head t % 8) and tensor-memory lane t ----
        const uint32_t grp = warp >> 2, t = tid & 127u, kvh = t & 7u, tok = t >> 3;
        Group* gs = &c->g[grp];
        const uint32_t lane_base = ((warp & 3u) * 32u) << 16;
        const uint32_t tmem_o = tmem + grp * GCOLS, tmem_s = tmem_o + S_OFF;
        uint32_t p_off[G][PT];                                      // F16 pool: where this row's probabilities go in P^T (row = kv head, query head; column = this row)
        uint32_t p_word[PT];                                        // E4M3 pool: the word of each term in this row of the MN-major P^T (columns kv head, term, query head)
#pragma unroll
        for (int term = 0; term < PT; term++) {
            const uint32_t off = kvh * CP + term * G;               // a multiple of 4: a word never straddles a 16-byte chunk
            p_word[term] = (t >> 3) * 1024u + (t & 7u) * 128u + (((off >> 4) ^ (t & 7u)) << 4) + (off & 15u);
        }
#pragma unroll
        for (int g = 0; g < G; g++)
#pragma unroll
            for (int term = 0; term < PT; term++)
                p_off[g][term] = (t >> 6) * (NP * 128) + swz(kvh * CP + g, (t & 63u) >> 3) + (t & 7u) * 2;
        // Q^T of a range: group 0, thread (query head qh = t / 4, dims [32 * (t % 4), +32)); the values wait in registers
        // from the start of the previous range
        float qx[32];
        auto q_fetch = [&](uint32_t n) {
            const uint32_t seq = c->item_id[n] / ranges, qh = t >> 2;
            const float* qrow = a.q + ((size_t)seq * a.n_q_heads + (qh < a.n_q_heads ? qh : 0)) * D + (t & 3u) * 32;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 f = qh < a.n_q_heads ? __ldg(reinterpret_cast<const float4*>(qrow) + i) : make_float4(0, 0, 0, 0);
                qx[4 * i] = f.x;
                qx[4 * i + 1] = f.y;
                qx[4 * i + 2] = f.z;
                qx[4 * i + 3] = f.w;
            }
        };
        auto q_write = [&](uint32_t n) {
            const uint32_t qh = t >> 2, part = t & 3u, qkvh = qh / G, g = qh % G;
            if (FP8) {
                float amax = 0.0f;
#pragma unroll
                for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(qx[i] * a.q_scale));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
                // power of two that brings the head's largest element into [128, 256): exact to apply and to undo
                int e = 0;
                if (amax > 0.0f && amax < INFINITY) e = 7 - (int)((__float_as_uint(amax) >> 23) & 0xFFu) + 127;
                e = max(-60, min(60, e));
                const float up = a.q_scale * __uint_as_float((uint32_t)(127 + e) << 23);
                if (part == 0) c->q_inv[n & 1u][qh] = __uint_as_float((uint32_t)(127 - e) << 23);
#pragma unroll
                for (int ch = 0; ch < 2; ch++) {                    // two 16-byte chunks of the row per term
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        hi[wd] = lo[wd] = 0;
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            const float v = qx[ch * 16 + wd * 4 + b] * up;
                            const uint32_t h = e4m3_of(v);
                            const uint32_t l = e4m3_of(v - e4m3_to_f32(h));
                            hi[wd] |= h << (8 * b);
                            lo[wd] |= l << (8 * b);
                        }
                    }
                    const uint32_t chunk = part * 2 + ch;
                    *reinterpret_cast<uint4*>(q_tile + swz(qkvh * CQ + g, chunk)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(q_tile + swz(qkvh * CQ + G + g, chunk)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            } else {
                if (part == 0) c->q_inv[n & 1u][qh] = 1.0f;
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {                    // 32 dims * 2 B = four 16-byte chunks; dims [64, 128) live in the second column group
                    uint32_t wv[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        __half2 h = __floats2half2_rn(qx[ch * 8 + wd * 2] * a.q_scale, qx[ch * 8 + wd * 2 + 1] * a.q_scale);
                        wv[wd] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    const uint32_t cgp = part >> 1, chunk = (part & 1u) * 4 + ch;
                    *reinterpret_cast<uint4*>(q_tile + cgp * Q_SUB + swz(qkvh * CQ + g, chunk)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->q_full);
        };
        bool ok = c->fail == 0;
        if (grp == 0 && n_items) {
            q_fetch(0);
            q_write(0);
        }
        uint32_t gj = 0, base_k = 0;                                // blocks this group has taken so far; ring index of the range's first block
        for (uint32_t n = 0; n < n_items; n++) {
            const uint32_t id = c->item_id[n], seq = id / ranges, split = id - seq * ranges, n_blk = c->item_blocks[n];
            const uint32_t kv_len = min(a.kv_lens[seq], a.max_kv_len), b_begin = split * (a.split_tokens / BS);
            const uint32_t n_mine = n_blk > grp ? (n_blk - grp + (uint32_t)NG - 1u) / (uint32_t)NG : 0u;
            if (grp == 0 && n + 1 < n_items) q_fetch(n + 1);        // the next range's query rows, on their way while this one is worked
            float m_used[G], l[G], q_inv[G];
#pragma unroll
            for (int g = 0; g < G; g++) {
                m_used[g] = -INFINITY;
                l[g] = 0.0f;
            }
            if (t < 32) gs->m_used[t] = -INFINITY;
            asm volatile("bar.sync %0, 128;" ::"r"(1u + grp) : "memory");
            for (uint32_t j = 0; j < n_mine; j++, gj++) {
                const uint32_t i = (uint32_t)NG * j + grp, k = base_k + i, s = k % n_v, b = gj & 1u, sbuf = gj % SBUF, pb = gj % PBUF;
                const uint32_t n_valid = min((uint32_t)BS, kv_len - (b_begin + i) * BS);
                const bool valid = tok < n_valid;
                float sc[G];                                        // this row's scores against its own kv head's query heads (log2 domain)
                float inv_vs = 1.0f;
                if (ok) {
                    ok = mbar_wait(gs->s_full + sbuf, (gj / SBUF) & 1u, fail_word) && mbar_wait(c->v_full + s, (k / n_v) & 1u, fail_word);
                    if (!ok) atomicCAS(&c->fail, 0u, 4u);
                }
                if (ok) {
                    tc_fence_after();
                    if (j == 0) {
#pragma unroll
                        for (int g = 0; g < G; g++) q_inv[g] = c->q_inv[n & 1u][kvh * G + g];
                    }
                    float part[CQ];
                    // the whole row of S^T in one load (two 32-column loads with their waits cost the E4M3 path 4 us per layer at 16 prompts);
                    // a thread keeps the CQ columns of its own kv head
                    uint32_t r[NQ];
                    if (NQ == 64) tmem_ld64(tmem_s + sbuf * 64u + lane_base, reinterpret_cast<uint32_t(&)[64]>(r));
                    else tmem_ld32(tmem_s + sbuf * 64u + lane_base, reinterpret_cast<uint32_t(&)[32]>(r));
                    tmem_wait_ld();
                    // the CQ columns of this row's kv head, picked by halving on the bits of the head number (56 selects instead of 64 moves
                    // under eight predicates)
                    {
                        static_assert(HKV == 8, "three halvings");
                        uint32_t h4[4 * CQ], h2[2 * CQ];
#pragma unroll
                        for (int q = 0; q < 4 * CQ; q++) h4[q] = (kvh & 4u) ? r[4 * CQ + q] : r[q];
#pragma unroll
                        for (int q = 0; q < 2 * CQ; q++) h2[q] = (kvh & 2u) ? h4[2 * CQ + q] : h4[q];
#pragma unroll
                        for (int q = 0; q < CQ; q++) part[q] = __uint_as_float((kvh & 1u) ? h2[CQ + q] : h2[q]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(gs->s_free + sbuf);
                    float ks = 1.0f, lv = 0.0f;
                    if (a.k_scales) {
                        ks = c->scales[s][kvh];
                        const float vs = c->scales[s][8 + kvh];
                        lv = fast_log2(vs);
                        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_vs) : "f"(vs));   // scales the row sum only
                    }
#pragma unroll
                    for (int g = 0; g < G; g++) {                   // the V scale rides in the exponent
                        const float raw = FP8 ? part[g] + part[G + g] : part[g];
                        sc[g] = valid ? raw * (ks * q_inv[g]) + lv : -INFINITY;
                    }
                } else {
#pragma unroll
                    for (int g = 0; g < G; g++) sc[g] = -INFINITY;
                }
                // does any query head of this kv head exceed its running maximum by more than 2^RAISE in this block?
                bool want = false;
#pragma unroll
                for (int g = 0; g < G; g++) want = want || sc[g] > m_used[g] + RAISE;
                if (__any_sync(0xFFFFFFFFu, want)) {                // rare: post this warp's maxima
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        float bm = sc[g];
                        bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 8));
                        bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 16));
                        if (lane < 8 && bm > m_used[g] + RAISE) {
                            atomicMax(&gs->block_max[b][kvh * G + g], ordered(bm));
                            gs->raise[b] = 1u;
                        }
                    }
                }
                asm volatile("bar.sync %0, 128;" ::"r"(1u + grp) : "memory");
                if (gs->raise[b]) {
                    // ---- raise the maxima: rescale O^T in tensor memory and the row sums; a few times per range at most ----
                    if (t < 32) {
                        const float bm = unordered(gs->block_max[b][t]), mo = gs->m_used[t];
                        const float mn = fmaxf(mo, bm);
                        gs->factor[t] = (mn == mo) ? 1.0f : (mo == -INFINITY ? 0.0f : fast_exp2(mo - mn));
                        gs->m_used[t] = mn;
                        gs->block_max[b][t] = ordered(-INFINITY);
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1u + grp) : "memory");
                    if (t == 0) gs->raise[b] = 0u;
                    if (j > 0) {
                        // the PV MMA of the group's previous block must have finished with O^T; none follows until this block's P^T is published
                        if (ok) ok = mbar_wait(gs->p_free + (gj - 1u) % PBUF, ((gj - 1u) / PBUF) & 1u, fail_word);
                        if (ok) {
                            tc_fence_after();
#pragma unroll
                            for (int c0 = 0; c0 < NP; c0 += 32) {
                                uint32_t r[32];
                                tmem_ld32(tmem_o + lane_base + c0, r);
                                tmem_wait_ld();
#pragma unroll
                                for (int q = 0; q < 32; q++) {
                                    const int col = c0 + q, head = (col / CP) * G + (col % CP) % G;
                                    r[q] = __float_as_uint(__uint_as_float(r[q]) * gs->factor[head]);
                                }
                                tmem_st32(tmem_o + lane_base + c0, r);
                            }
                            tmem_wait_st();
                            tc_fence_before();
                        }
                    }
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        l[g] *= gs->factor[kvh * G + g];
                        m_used[g] = gs->m_used[kvh * G + g];
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1u + grp) : "memory");   // factor[] and m_used[] are read before the next raise rewrites them
                }
                if (ok && gj >= (uint32_t)PBUF) ok = mbar_wait(gs->p_free + pb, ((gj / PBUF) - 1u) & 1u, fail_word);
                if (ok) {
                    // weights 2^(score - maximum + SHIFT), two query heads at a time in half2.  E4M3 pool: an E5M2 byte is the top
                    // byte of an F16, so the three terms are peeled off by masking the low byte and subtracting (exact in F16: the
                    // weights are non-negative and every residual fits); the row sum takes the value the three terms add up to.
                    unsigned char* pt = p_tile + (grp * PBUF + pb) * PT_BYTES;
                    const float l_scale = inv_vs * __uint_as_float((uint32_t)(127 - (int)SHIFT) << 23);
                    uint32_t terms[PT][(G + 1) / 2];                  // E4M3 pool: per term, the half2 pairs with their low bytes cleared
#pragma unroll
                    for (int g = 0; g < G; g += 2) {
                        const int g1 = g + 1 < G ? g + 1 : g;
                        const float x0 = fast_exp2(sc[g] - m_used[g] + SHIFT);                     // <= 2^(RAISE + SHIFT); 0 for a row past the sequence end
                        const float x1 = (g + 1 < G) ? fast_exp2(sc[g1] - m_used[g1] + SHIFT) : 0.0f;
                        __half2 h = __floats2half2_rn(x0, x1);
                        if (FP8) {
                            const uint32_t t1 = *reinterpret_cast<uint32_t*>(&h) & 0xFF00FF00u;
                            const __half2 r1 = __hsub2(h, *reinterpret_cast<const __half2*>(&t1));
                            const uint32_t t2 = *reinterpret_cast<const uint32_t*>(&r1) & 0xFF00FF00u;
                            const __half2 r2 = __hsub2(r1, *reinterpret_cast<const __half2*>(&t2));
                            const uint32_t t3 = *reinterpret_cast<const uint32_t*>(&r2) & 0xFF00FF00u;
                            h = __hsub2(h, __hsub2(r2, *reinterpret_cast<const __half2*>(&t3)));     // = t1 + t2 + t3
                            terms[0][g >> 1] = t1;
                            terms[1 < PT ? 1 : 0][g >> 1] = t2;
                            terms[2 < PT ? 2 : 0][g >> 1] = t3;
                        } else {
                            *reinterpret_cast<__half*>(pt + p_off[g][0]) = __low2half(h);
                            if (g + 1 < G) *reinterpret_cast<__half*>(pt + p_off[g1][0]) = __high2half(h);
                        }
                        const float2 q = __half22float2(h);
                        l[g] += q.x * l_scale;
                        if (g + 1 < G) l[g1] += q.y * l_scale;
                    }
                    if (FP8) {
                        static_assert(!FP8 || G == 4, "a term's four query heads are one word");
#pragma unroll
                        for (int term = 0; term < PT; term++)      // the top bytes of the two pairs, in query-head order
                            *reinterpret_cast<uint32_t*>(pt + p_word[term]) = __byte_perm(terms[term][0], terms[term][(G + 1) / 2 - 1], 0x7531);
                    }
                    if (!valid) {
                        // a row past the sequence end holds whatever the pool held there: 0 * NaN must not reach O^T
                        unsigned char* vt = v_ring + (size_t)s * KV_TILE;
#pragma unroll
                        for (int cg = 0; cg < ES; cg++)
#pragma unroll
                            for (int ch = 0; ch < 8; ch++) *reinterpret_cast<uint4*>(vt + cg * TILE + swz(t, ch)) = make_uint4(0, 0, 0, 0);
                    }
                    fence_async_smem();
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(gs->p_full + pb);        // also after a failure: the issuer then ends through the fail word
            }
            // ---- the next range's Q^T goes in as soon as this range's QK MMAs are done, ahead of this range's epilogue ----
            if (grp == 0 && n + 1 < n_items) {
                if (ok) ok = mbar_wait(&c->q_free, n & 1u, fail_word);
                q_write(n + 1);
            }
            // ---- this group's partial of the range: its last PV MMA done, row sums over the group, O^T rows out of tensor memory ----
            if (ok && n_mine) {
                ok = mbar_wait(gs->p_free + (gj - 1u) % PBUF, ((gj - 1u) / PBUF) & 1u, fail_word);
                if (!ok) atomicCAS(&c->fail, 0u, 4u);
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                float x = l[g];
                x += __shfl_xor_sync(0xFFFFFFFFu, x, 8);
                x += __shfl_xor_sync(0xFFFFFFFFu, x, 16);
                if (lane < 8) gs->l_sum[warp & 3u][kvh * G + g] = x;
            }
            asm volatile("bar.sync %0, 128;" ::"r"(1u + grp) : "memory");
            if (ok) {
                const float down = __uint_as_float((uint32_t)(127 - (int)SHIFT) << 23);
                const uint32_t part_slot = split * (uint32_t)NG + grp;
                float* pr0 = a.partial + (((size_t)seq * HKV * n_parts + part_slot) * G) * (D + 2);
                const size_t head_stride = (size_t)n_parts * G * (D + 2);
                if (t < HKV * G && t < a.n_q_heads) {               // one thread per query head: its maximum and row sum (-inf and 0 for a group without blocks)
                    float* pr = pr0 + (size_t)(t / G) * head_stride + (size_t)(t % G) * (D + 2);
                    pr[0] = n_mine ? gs->m_used[t] : -INFINITY;
                    pr[1] = n_mine ? gs->l_sum[0][t] + gs->l_sum[1][t] + gs->l_sum[2][t] + gs->l_sum[3][t] : 0.0f;
                }
                float acc[HKV * G];                                 // this thread's output dim t, every query head: the terms' columns folded
#pragma unroll
                for (int q = 0; q < HKV * G; q++) acc[q] = 0.0f;
                if (n_mine) {
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < NP; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(tmem_o + lane_base + c0, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int q = 0; q < 32; q++) {
                            const int col = c0 + q;
                            if (col < NP) acc[(col / CP) * G + (col % CP) % G] += __uint_as_float(r[q]);
                        }
                    }
                }
#pragma unroll
                for (int q = 0; q < HKV * G; q++)
                    if ((uint32_t)q < a.n_q_heads) pr0[(size_t)(q / G) * head_stride + (size_t)(q % G) * (D + 2) + 2 + t] = acc[q] * down;
                if (n_mine) tc_fence_before();
            }
            base_k += n_blk;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4 * NG + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
    if (tid == 0 && c->fail && a.status) atomicCAS(a.status, 0u, c->fail);
}

// ---- self-check of the operand plumbing ---------------------------------------------------------------
// One CTA, one MMA shape at a time, operands of small dyadic values (every product and sum exact in FP32):
//   form 0:  D[128 rows][64]  = A . B^T, A a [128][128 * ES B] tile brought in by the tensor-map copy and read K-major (the K block),
//            B [64 rows] written by threads with the swizzle (Q^T);
//   form 1:  D[128 dims][128] = A^T . B^T, A the same kind of tile read MN-major (the V block), B [128 rows] written by threads (P^T).
// Thread r compares row r of D from tensor memory with the same sums computed from the plain global copies.
template <bool FP8>
__global__ void __launch_bounds__(128, 1) selfcheck_kernel(const __grid_constant__ CUtensorMap map, const unsigned char* a_plain,
                                                           const unsigned char* b_plain, uint32_t form, uint32_t b_e5m2, unsigned long long* bad) {
    constexpr int ES = FP8 ? 1 : 2;
    constexpr int KSTEPS = 4 * ES;
    const uint32_t n = form == 0 ? 64u : 128u;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);          // [0] copy landed, [1] MMA done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 64);
    unsigned char* a_tile = smem + 1024;                          // ES column groups of [128][128 B]
    unsigned char* b_tile = a_tile + TILE * ES;                   // ES column groups of [n][128 B]
    const uint32_t tid = threadIdx.x, warp = tid >> 5;
    volatile uint32_t never = 0;
    if (tid == 0) {
        mbar_init(bars, 1);
        mbar_init(bars + 1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // B: row j of b_plain ([n][128 elements]) into the swizzled tile(s)
    for (uint32_t i = tid; i < n * 8 * ES; i += 128) {
        const uint32_t row = i / (8 * ES), c16 = i % (8 * ES);       // 16-byte chunk c16 of the row
        const uint4 v = *reinterpret_cast<const uint4*>(b_plain + (size_t)row * 128 * ES + c16 * 16);
        *reinterpret_cast<uint4*>(b_tile + (c16 / 8) * (n * 128) + swz(row, c16 % 8)) = v;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;
    if (tid == 0) {
        mbar_expect_tx(bars, TILE * ES);
        for (int grp = 0; grp < ES; grp++) tma_box(smem_u32(a_tile) + grp * TILE, &map, grp * 128, 0, bars);
        ok = mbar_wait(bars, 0, &never);
        if (ok) {
            tc_fence_after();
            const uint32_t fmt_b = FP8 ? b_e5m2 : 0u;
            const uint32_t idesc = instr_desc(0u, fmt_b, form, n);
            for (int ks = 0; ks < KSTEPS; ks++) {
                uint64_t da, db;
                if (form == 0) {
                    da = smem_desc(smem_u32(a_tile) + (ks / 4) * TILE + (ks % 4) * 32, 16, 1024);
                } else {
                    da = smem_desc(smem_u32(a_tile) + ks * (32 / ES) * 128, TILE, 1024);
                }
                db = smem_desc(smem_u32(b_tile) + (ks / 4) * (n * 128) + (ks % 4) * 32, 16, 1024);
                mma<FP8>(tmem, da, db, idesc, ks > 0 ? 1u : 0u);
            }
            tc_commit(bars + 1);
        }
    }
    ok = mbar_wait(bars + 1, 0, &never);
    unsigned long long wrong = 0;
    if (ok) {
        tc_fence_after();
        auto val = [&](const unsigned char* base, size_t idx, bool e5) -> float {
            if (!FP8) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
            return e5 ? e5m2_to_f32(base[idx]) : e4m3_to_f32(base[idx]);
        };
        for (uint32_t c0 = 0; c0 < n; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem + ((warp * 32u) << 16) + c0, r);
            tmem_wait_ld();
            for (uint32_t j = 0; j < 32; j++) {
                float want = 0.0f;
                for (uint32_t k = 0; k < 128; k++) {
                    // form 0: D[row tid][col] = sum_k A[tid][k] B[col][k];  form 1: D[dim tid][col] = sum_k A[k][tid] B[col][k]
                    const float av = form == 0 ? val(a_plain, (size_t)tid * 128 + k, false) : val(a_plain, (size_t)k * 128 + tid, false);
                    want += av * val(b_plain, (size_t)(c0 + j) * 128 + k, b_e5m2 != 0);
                }
                if (__uint_as_float(r[j]) != want) wrong++;
            }
        }
        tc_fence_before();
    } else {
        wrong = 1ull << 40;                                        // the copy or the MMA never completed
    }
    if (wrong) atomicAdd(bad, wrong);
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------
// A layer tensor as a 2-D byte array [rows = blocks * 16 * 8][128 * ES bytes], boxes of [128 rows][128 B], 128-byte swizzle.
static bool make_map(CUtensorMap* map, uint64_t base, uint32_t total_blocks, uint32_t es) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {128ull * es, (cuuint64_t)total_blocks * ROWS};
    const cuuint64_t strides[1] = {128ull * es};
    const cuuint32_t box[2] = {128u, (cuuint32_t)ROWS};
    const cuuint32_t elem[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, reinterpret_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool eligible(uint32_t n_kv_heads, uint32_t group, bool has_scales, uint32_t total_blocks) {
    (void)has_scales;
    return n_kv_heads == HKV && group == 4 && (uint64_t)total_blocks * ROWS < (1ull << 31);
}

template <bool FP8, int G> static cudaError_t launch_one(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, cudaStream_t st) {
    constexpr size_t smem = Shape<FP8, G>::smem;
    auto kernel = decode_attn_tc<FP8, G>;
    static std::mutex mu;
    static bool granted[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!granted[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return e;
            granted[dev] = true;
        }
    }
    // one persistent CTA per SM walks its share of the (sequence, range) list; more CTAs only when a share would not fit its list
    const uint64_t total = (uint64_t)a.n_seqs * a.n_splits;
    const uint64_t grid = std::max<uint64_t>(std::min<uint64_t>(total, (uint64_t)sms[dev]), (total + (MAX_ITEMS - 32) - 1) / (MAX_ITEMS - 32));
    kernel<<<(uint32_t)grid, ATHREADS, smem, st>>>(mk, mv, a);
    return cudaGetLastError();
}

cudaError_t launch(bool fp8, uint32_t group, uint64_t k_layer, uint64_t v_layer, const Args& a, cudaStream_t st) {
    CUtensorMap mk, mv;
    const uint32_t es = fp8 ? 1u : 2u;
    if (!make_map(&mk, k_layer, a.total_blocks, es) || !make_map(&mv, v_layer, a.total_blocks, es)) return cudaErrorInvalidValue;
    if (group != 4) return cudaErrorInvalidConfiguration;
    return fp8 ? launch_one<true, 4>(mk, mv, a, st) : launch_one<false, 4>(mk, mv, a, st);
}

// Fills the two operands with small dyadic values, runs the four combinations, returns the mismatch counts.
cudaError_t selfcheck(uint64_t out[4]) {
    const size_t a_bytes = (size_t)TILE * 2, b_bytes = 128 * 128 * 2;
    unsigned char *d_a = nullptr, *d_b = nullptr;
    unsigned long long* d_bad = nullptr;
    cudaError_t e = cudaMalloc((void**)&d_a, a_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&d_b, b_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&d_bad, 4 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(d_bad, 0, 4 * sizeof(unsigned long long));
    // values k / 4, k in [-8, 8]: exact in E4M3, E5M2 (multiples of 1/4 up to 2 need 3 significant bits at most) and F16
    static const float pick[8] = {0.0f, 0.25f, -0.5f, 1.0f, -1.5f, 2.0f, -0.25f, 0.5f};
    static const unsigned char e4[8] = {0x00, 0x28, 0xB0, 0x38, 0xBC, 0x40, 0xA8, 0x30};   // E4M3 encodings of pick[]
    static const unsigned char e5[8] = {0x00, 0x34, 0xB8, 0x3C, 0xBE, 0x40, 0xB4, 0x38};   // E5M2 encodings of pick[]
    unsigned char* h = (unsigned char*)malloc(a_bytes);
    for (int t = 0; t < 4 && e == cudaSuccess; t++) {
        const bool fp8 = t < 2;
        const uint32_t form = t & 1u, es = fp8 ? 1u : 2u, n = form == 0 ? 64u : 128u;
        uint32_t x = 12345u + t;
        auto next = [&]() { x = x * 1664525u + 1013904223u; return (x >> 13) & 7u; };
        for (size_t i = 0; i < 128 * 128; i++) {
            const uint32_t k = next();
            if (fp8) h[i] = e4[k];
            else reinterpret_cast<__half*>(h)[i] = __float2half(pick[k]);
        }
        e = cudaMemcpy(d_a, h, 128 * 128 * es, cudaMemcpyHostToDevice);
        for (size_t i = 0; i < (size_t)n * 128; i++) {
            const uint32_t k = next();
            if (fp8) h[i] = form == 1 ? e5[k] : e4[k];
            else reinterpret_cast<__half*>(h)[i] = __float2half(pick[k]);
        }
        if (e == cudaSuccess) e = cudaMemcpy(d_b, h, (size_t)n * 128 * es, cudaMemcpyHostToDevice);
        CUtensorMap map;
        if (e == cudaSuccess && !make_map(&map, reinterpret_cast<uint64_t>(d_a), 1, es)) e = cudaErrorInvalidValue;
        const size_t smem = 1024 + 1024 + (size_t)TILE * es + (size_t)n * 128 * es;
        if (e == cudaSuccess) {
            if (fp8) {
                e = cudaFuncSetAttribute(selfcheck_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
                if (e == cudaSuccess) selfcheck_kernel<true><<<1, 128, smem>>>(map, d_a, d_b, form, form, d_bad + t);
            } else {
                e = cudaFuncSetAttribute(selfcheck_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
                if (e == cudaSuccess) selfcheck_kernel<false><<<1, 128, smem>>>(map, d_a, d_b, form, 0u, d_bad + t);
            }
            if (e == cudaSuccess) e = cudaGetLastError();
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
        }
    }
    free(h);
    unsigned long long host_bad[4] = {0, 0, 0, 0};
    if (e == cudaSuccess) e = cudaMemcpy(host_bad, d_bad, sizeof host_bad, cudaMemcpyDeviceToHost);
    for (int t = 0; t < 4; t++) out[t] = host_bad[t];
    cudaFree(d_a);
    cudaFree(d_b);
    cudaFree(d_bad);
    return e;
}


}  // namespace tkv_tc
