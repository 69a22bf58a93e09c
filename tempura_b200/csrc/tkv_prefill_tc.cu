// Causal attention of a chunk of new tokens of one sequence over the paged pool, on the fifth-generation tensor
// cores (tcgen05, sm_100a): the prefill-side twin of the decode kernel, scale-aware for an E4M3 pool.
//
// What is computed is paged_flash_attention (kernels/src/attention.rs:486-590) for query tokens at positions
// start_pos .. start_pos + T - 1, token t attending to positions 0 .. start_pos + t, over the widened pool values
// (the reference's paged prefill kernel for the FP8 pool, cutile_flash_attn_heads_paged_e4m3,
// kernels/src/cutile_flash_attention.rs:868, reads unscaled bytes; here every (block, kv head) carries its scale).
//
// A query tile is one kv head and 32 consecutive query tokens: with four query heads per kv head that is 128 rows, row
// r = (query head r / 32, token r % 32).  A CTA owns one query tile, or two that take turns (E4M3 pool: the MMAs of one tile run
// under the softmax of the other, and each K/V tile is fetched once for both).  It walks the cached tokens 128 at a time (eight
// pool blocks).  Per query tile and cached tile
//
//     S[128 rows][128 tokens] = Q . K_tile^T     (tcgen05.mma, M = N = 128; K_tile = eight [16 tokens][128 B] tensor-map boxes of this kv head)
//     O[128 rows][128 dims]  += P . V_tile       (P written by the softmax threads, V read MN-major from the same kind of tile)
//
// with S and O in tensor memory.  Four softmax threads share a row (32 of the tile's 128 columns each, the same tensor-memory
// lane): the row's maximum is exchanged through shared memory, the rescale of O on a raised maximum is taken lazily (when a tile
// exceeds the maximum in use by 2^6) and each thread rescales its own 32 columns.  Operand precision as in the decode kernel: an F16 pool
// takes F16 q and probabilities; an E4M3 pool takes q as two E4M3 terms under a per-row power-of-two scale and the
// probabilities as three E5M2 terms (all terms accumulate into the same accumulator here, since they differ in the A
// operand only).  The block scales: K's multiplies the scores of its 16 columns; V's multiplies the probabilities of
// its 16 columns, normalised by a power of two that bounds every V scale of the sequence (found by a pass over the
// scales before the first tile) so that the scaled probabilities stay inside the E5M2 range whatever the scales are.
//
// Every wait is bounded; a CTA that gives up reports through `status`, waits for its copies and frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <mutex>

#include <cstdarg>
#include <cstdio>

#include "../../include/tkv.h"
#include "tkv_attention_tc.h"
#include "tkv_tc_common.cuh"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
}

namespace tkv_tc {

namespace {

constexpr int PD = 128, PBS = 16, PHKV = 8, PG = 4;
constexpr int QT = 32;                         // query tokens per CTA: QT * PG = 128 rows
constexpr int KT = 128;                        // cached tokens per tile = 8 blocks
constexpr int PTILE = 128 * 128;               // bytes of one [128 rows][128 B] swizzled tile
constexpr float P_RAISE = 6.0f, P_SHIFT = 9.0f;
constexpr int NSPLIT = 4;                      // softmax threads per row, 32 of the tile's 128 columns each
constexpr int SM_WARPS = 4 * NSPLIT, PTHREADS = (SM_WARPS + 2) * 32;   // + producer warp + issuer warp

struct PControl {
    uint64_t k_full[2], k_empty[2];            // K of a tile landed / the QK MMAs of every query tile that reads it are done
    uint64_t v_full[2], v_empty[2];            // V of a tile landed / the PV MMAs of every query tile that reads it are done
    uint64_t s_full[2], s_free[2];             // S buffers: QK done / all softmax warps have read it
    uint64_t p_full[2], pv_done[2];            // P buffers: written by all softmax warps / its PV MMAs are done
    uint64_t q_ready, drained;
    uint32_t tmem_base, fail, pad[2];
    float scales[4][16];                       // per cached tile (mod 4): 8 K scales, 8 V scales (normalised) of the tile's blocks
    float vmax_part[SM_WARPS];
    // Exchange area, one use at a time: q_inv[query tile][row] before the first tile; then per step the splits' row maxima
    // [split][row]; then the splits' row sums [split][row] in the epilogue.
    float exch[NSPLIT * 128];
};
static_assert(sizeof(PControl) <= 3072, "control block");
constexpr int CTRL = 3072;

// Sixteen scores of one row (one block of the pool: one K scale, one V scale) -> sixteen probabilities in P.
//   x = 2^(raw * ks + lv)   with lv = log2(v scale) + SHIFT - maximum in use, 0 for a column past the row's causal bound;
// F16 pool: x as F16.  E4M3 pool: x as three E5M2 terms, peeled off an F16 two columns at a time (an E5M2 byte is the top byte of
// an F16, so a term is the F16 with its low byte cleared, and the residual is exact).  Returns the sum of the sixteen x.
template <bool FP8, bool MASKED>
__device__ __forceinline__ float probabilities16(const uint32_t* raw, float ks, float lv, uint32_t first_pos, uint32_t q_pos, unsigned char* p_tile,
                                                 uint32_t r, uint32_t blk) {
    float sum = 0.0f;
    __half2 dropped = __floats2half2_rn(0.0f, 0.0f);            // what the three terms leave out: the row sum must be the sum of what the MMA sees
    uint32_t w1[4], w2[4], w3[4], hw[8];
#pragma unroll
    for (int q = 0; q < 16; q += 4) {
        float x[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            x[i] = fast_exp2(__fmaf_rn(__uint_as_float(raw[q + i]), ks, lv));
            if (MASKED && first_pos + q + i > q_pos) x[i] = 0.0f;
        }
        sum += (x[0] + x[1]) + (x[2] + x[3]);
        const __half2 ha = __floats2half2_rn(x[0], x[1]), hb = __floats2half2_rn(x[2], x[3]);
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&ha), b0 = *reinterpret_cast<const uint32_t*>(&hb);
        if (FP8) {
            const uint32_t a1 = a0 & 0xFF00FF00u, b1 = b0 & 0xFF00FF00u;
            const __half2 ra = __hsub2(ha, *reinterpret_cast<const __half2*>(&a1)), rb = __hsub2(hb, *reinterpret_cast<const __half2*>(&b1));
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&ra) & 0xFF00FF00u, b2 = *reinterpret_cast<const uint32_t*>(&rb) & 0xFF00FF00u;
            const __half2 sa = __hsub2(ra, *reinterpret_cast<const __half2*>(&a2)), sb = __hsub2(rb, *reinterpret_cast<const __half2*>(&b2));
            const uint32_t a3 = *reinterpret_cast<const uint32_t*>(&sa) & 0xFF00FF00u, b3 = *reinterpret_cast<const uint32_t*>(&sb) & 0xFF00FF00u;
            dropped = __hadd2(dropped, __hadd2(__hsub2(sa, *reinterpret_cast<const __half2*>(&a3)), __hsub2(sb, *reinterpret_cast<const __half2*>(&b3))));
            w1[q >> 2] = __byte_perm(a1, b1, 0x7531);           // the four top bytes, in column order
            w2[q >> 2] = __byte_perm(a2, b2, 0x7531);
            w3[q >> 2] = __byte_perm(a3, b3, 0x7531);
        } else {
            hw[q >> 1] = a0;
            hw[(q >> 1) + 1] = b0;
        }
    }
    if (FP8) {
        const uint32_t off = swz(r, blk);                       // 16 columns = one 16-byte chunk of the row
        *reinterpret_cast<uint4*>(p_tile + off) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        *reinterpret_cast<uint4*>(p_tile + PTILE + off) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
        *reinterpret_cast<uint4*>(p_tile + 2 * PTILE + off) = make_uint4(w3[0], w3[1], w3[2], w3[3]);
        const float2 d = __half22float2(dropped);
        sum -= d.x + d.y;
    } else {
        unsigned char* base = p_tile + (blk >> 2) * PTILE;      // columns [64, 128) live in the second column group
        *reinterpret_cast<uint4*>(base + swz(r, (blk & 3u) * 2)) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4*>(base + swz(r, (blk & 3u) * 2 + 1)) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
    }
    return sum;
}

// NQT query tiles of 32 tokens per CTA.  With two, the softmax warps take the tiles in turns and the MMAs of one tile run under the
// softmax of the other; each K/V tile is fetched once for both.  (Two tiles of E4M3 operand terms fill shared memory to the byte;
// an F16 pool's tiles leave room for one.)
template <bool FP8, int NQT>
__global__ void __launch_bounds__(PTHREADS, 1)
prefill_attn_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
    constexpr int ES = FP8 ? 1 : 2;
    constexpr int QTERMS = FP8 ? 2 : 1, PT = FP8 ? 3 : 1;
    constexpr int KV_TILE = PTILE * ES;                     // K (or V) of one tile of 128 tokens
    constexpr int Q_BYTES = 2 * PTILE, P_BYTES = FP8 ? PT * PTILE : 2 * PTILE;     // per query tile
    constexpr int KSTEPS = 4 * ES;
    // K and V tiles in flight (separate rings: a K tile is free again after its QK MMAs, a V tile after its PV MMAs).  Two query tiles of
    // F16 operands leave room for one of each.
    constexpr int NSK = 2, NSV = (!FP8 && NQT == 2) ? 1 : 2;       // an F16 pool's two query tiles leave room for two K tiles and one V tile
    constexpr uint32_t IDESC_QK = instr_desc2(0u, 0u, 0u, 0u, 128u);
    constexpr uint32_t IDESC_PV = instr_desc2(FP8 ? 1u : 0u, 0u, 0u, 1u, 128u);      // A = P (E5M2 / F16, K-major), B = V (MN-major)
    constexpr uint64_t DESC_HI = ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
    constexpr uint64_t DESC_K = DESC_HI | ((uint64_t)1u << 16);
    constexpr uint64_t DESC_V = DESC_HI | ((uint64_t)(PTILE >> 4) << 16);              // MN-major: the second 64-dim column group one tile further

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    // CTAs start in index order and a CTA's length grows with its query position (causal): all kv heads of the last query rows
    // first, then the rows before them, so the SMs end together (with the kv heads outermost a 4 096-token launch ended 17 % later).
    const uint32_t kvh = blockIdx.x % PHKV;
    const uint32_t q0 = (gridDim.x / PHKV - 1u - blockIdx.x / PHKV) * (QT * NQT);
    uint32_t rows_tokens[NQT], n_tiles_x[NQT], n_tiles = 0, kv_limit = 0;
#pragma unroll
    for (int x = 0; x < NQT; x++) {
        const uint32_t first = q0 + x * QT;
        rows_tokens[x] = first < a.n_tokens ? min((uint32_t)QT, a.n_tokens - first) : 0u;
        const uint32_t lim = rows_tokens[x] ? a.start_pos + first + rows_tokens[x] : 0u;   // tokens the tile's last row attends to
        n_tiles_x[x] = (lim + KT - 1) / KT;
        n_tiles = max(n_tiles, n_tiles_x[x]);
        kv_limit = max(kv_limit, lim);
    }
    const uint32_t n_blocks = (kv_limit + PBS - 1) / PBS;
    // S of query tile x for cached tile j: one buffer per query tile when there are two, two alternating buffers when there is one
    auto s_index = [&](uint32_t x, uint32_t j) { return NQT == 2 ? x : (j & 1u); };
    auto s_phase = [&](uint32_t j) { return NQT == 2 ? j : (j >> 1); };

    extern __shared__ __align__(1024) unsigned char smem[];
    PControl* c = reinterpret_cast<PControl*>(smem);
    unsigned char* q_tile = smem + CTRL;                    // NQT tiles
    unsigned char* p_tile = q_tile + NQT * Q_BYTES;         // NQT buffers
    unsigned char* k_ring = p_tile + NQT * P_BYTES;         // NSK stages of K, then NSV stages of V
    unsigned char* v_ring = k_ring + NSK * KV_TILE;
    const volatile uint32_t* fail_word = &c->fail;

    if (tid == 0) {
        for (int s = 0; s < 2; s++) {
            mbar_init(c->k_full + s, 1);
            mbar_init(c->k_empty + s, 1);
            mbar_init(c->v_full + s, 1);
            mbar_init(c->v_empty + s, 1);
            mbar_init(c->s_full + s, 1);
            mbar_init(c->s_free + s, SM_WARPS / NQT);
            mbar_init(c->p_full + s, SM_WARPS / NQT);
            mbar_init(c->pv_done + s, 1);
        }
        mbar_init(&c->q_ready, 4 * NQT);
        mbar_init(&c->drained, 1);
        c->fail = (smem_u32(smem) & 1023u) ? 2u : 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == SM_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&c->tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the largest V scale among the blocks this CTA will read, as a power of two (1 for an unscaled pool)
    float vmax = 0.0f;
    if (warp < SM_WARPS && a.v_scales) {
        for (uint32_t b = tid; b < n_blocks; b += SM_WARPS * 32) {
            const uint32_t blk = a.table[b];
            if (blk < a.total_blocks) vmax = fmaxf(vmax, a.v_scales[(size_t)blk * PHKV + kvh]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xFFFFFFFFu, vmax, o));
        if (lane == 0) c->vmax_part[warp] = vmax;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = c->tmem_base;
    int v_exp = 0;                                                         // V scales are used as vs * 2^-v_exp <= 1
    if (a.v_scales) {
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < SM_WARPS; i++) m = fmaxf(m, c->vmax_part[i]);
        if (m > 0.0f && m < INFINITY) v_exp = (int)((__float_as_uint(m) >> 23) & 0xFFu) - 126;   // 2^(v_exp - 1) <= m < 2^v_exp
        v_exp = max(-100, min(100, v_exp));
    }
    const float v_down = __uint_as_float((uint32_t)(127 - v_exp) << 23);

    if (warp == SM_WARPS) {
        // ---- producer: the tile's blocks, one lane per block: K and V boxes of this kv head, the block's two scales ----
        bool ok = c->fail == 0;
        uint32_t why = 4u, issued = 0, issued_k = 0;
        // K runs NSK - NSV tiles ahead of V (a K stage frees after its QK MMAs, long before the V stage of the same tile): the wait for
        // a V stage never holds back a K tile whose stage is free.
        auto tile_blocks = [&](uint32_t j, uint32_t& nb) -> uint32_t {     // lane's block of tile j; a stale or foreign id is never turned into an address
            nb = min(8u, n_blocks - j * 8u);
            uint32_t blk = 0;
            if (lane < nb) {
                blk = a.table[j * 8u + lane];
                if (blk >= a.total_blocks) {
                    ok = false;
                    why = 2u;
                }
            }
            if (__any_sync(0xFFFFFFFFu, why == 2u)) why = 2u;      // whichever lane met the bad id, lane 0 reports it
            ok = __all_sync(0xFFFFFFFFu, ok);
            return blk;
        };
        for (uint32_t j = 0; j < n_tiles && ok; j++) {
            while (ok && issued_k < n_tiles && issued_k <= j + (uint32_t)(NSK - NSV)) {
                const uint32_t jk = issued_k, sk = jk % NSK;
                uint32_t nb;
                const uint32_t blk = tile_blocks(jk, nb);
                // its stage frees as soon as the QK MMAs of the tile that held it are done
                if (ok && lane == 0 && jk >= (uint32_t)NSK) ok = mbar_wait(c->k_empty + sk, ((jk / NSK) - 1u) & 1u, fail_word);
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0u;
                if (!ok) break;
                if (lane < 8) {                              // the scales of a tile are read until its softmax ends: four slots outlast any stage
                    float ks = 1.0f, vs = 1.0f;
                    if (lane < nb && a.k_scales) {
                        ks = a.k_scales[(size_t)blk * PHKV + kvh];
                        vs = a.v_scales[(size_t)blk * PHKV + kvh] * v_down;
                    }
                    c->scales[jk & 3u][lane] = ks;
                    c->scales[jk & 3u][8 + lane] = vs;
                }
                __syncwarp();
                if (lane == 0) mbar_expect_tx(c->k_full + sk, nb * (PBS * 128u) * ES);
                __syncwarp();
                if (lane < nb) {
                    const uint32_t kd = smem_u32(k_ring + (size_t)sk * KV_TILE) + lane * (PBS * 128u);
#pragma unroll
                    for (int cg = 0; cg < ES; cg++) tma_head_rows(kd + cg * PTILE, &map_k, cg * 128, (int32_t)kvh, (int32_t)(blk * PBS), c->k_full + sk);
                }
                issued_k = jk + 1;
            }
            if (!ok) break;
            const uint32_t sv = j % NSV;
            uint32_t nb;
            const uint32_t blk = tile_blocks(j, nb);
            if (ok && lane == 0 && j >= (uint32_t)NSV) ok = mbar_wait(c->v_empty + sv, ((j / NSV) - 1u) & 1u, fail_word);
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0u;
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(c->v_full + sv, nb * (PBS * 128u) * ES);
            __syncwarp();
            if (lane < nb) {
                const uint32_t vd = smem_u32(v_ring + (size_t)sv * KV_TILE) + lane * (PBS * 128u);
#pragma unroll
                for (int cg = 0; cg < ES; cg++) tma_head_rows(vd + cg * PTILE, &map_v, cg * 128, (int32_t)kvh, (int32_t)(blk * PBS), c->v_full + sv);
            }
            issued = j + 1;
        }
        if (!ok && lane == 0) {
            atomicCAS(&c->fail, 0u, why);
            for (uint32_t j = issued_k > (uint32_t)NSK ? issued_k - NSK : 0u; j < issued_k; j++)   // copies still in flight get a bounded chance to land
                for (uint32_t it = 0; it < (1u << 20); it++)
                    if (mbar_test(c->k_full + j % NSK, (j / NSK) & 1u)) break;
            for (uint32_t j = issued > (uint32_t)NSV ? issued - NSV : 0u; j < issued; j++)
                for (uint32_t it = 0; it < (1u << 20); it++)
                    if (mbar_test(c->v_full + j % NSV, (j / NSV) & 1u)) break;
        }
    } else if (warp == SM_WARPS + 1) {
        // ---- MMA issuer.  Whichever is ready goes next, per query tile: the scores of its next cached tile (K has landed, its S buffer has
        // been read) or the PV product of its oldest tile whose probabilities are written.  Nothing waits behind anything else, so a stage's
        // copies are asked for as soon as its last PV is done and land while the softmax of other tiles runs. ----
        if (lane == 0) {
            const uint32_t q_lo = smem_u32(q_tile) >> 4, p_lo = smem_u32(p_tile) >> 4;
            const uint32_t kr_lo = smem_u32(k_ring) >> 4, vr_lo = smem_u32(v_ring) >> 4;
            bool ok = c->fail == 0 && mbar_wait(&c->q_ready, 0u, fail_word);
            uint32_t jq[NQT], jp[NQT], qk_left[2] = {0, 0}, pv_left[2] = {0, 0}, idle = 0, todo = 0;
#pragma unroll
            for (int x = 0; x < NQT; x++) {
                jq[x] = jp[x] = 0;
                todo += n_tiles_x[x];
            }
            while (ok && todo) {
                bool did = false;
#pragma unroll
                for (int x = 0; x < NQT; x++) {
                    if (jq[x] < n_tiles_x[x]) {
                        const uint32_t j = jq[x], st = j % NSK, sb = s_index(x, j);
                        const bool s_ok = NQT == 2 ? (j < 1 || mbar_test(c->s_free + sb, (j - 1u) & 1u)) : (j < 2 || mbar_test(c->s_free + sb, ((j >> 1) - 1u) & 1u));
                        if (s_ok && mbar_test(c->k_full + st, (j / NSK) & 1u)) {
                            tc_fence_after();
                            const uint32_t k_lo = kr_lo + st * (KV_TILE >> 4), qx_lo = q_lo + x * (Q_BYTES >> 4);
#pragma unroll
                            for (int term = 0; term < QTERMS; term++)
#pragma unroll
                                for (int ks = 0; ks < KSTEPS; ks++) {
                                    const uint32_t a_off = FP8 ? term * (PTILE >> 4) + ks * 2 : (ks / 4) * (PTILE >> 4) + (ks % 4) * 2;
                                    const uint32_t b_off = (ks / 4) * (PTILE >> 4) + (ks % 4) * 2;
                                    mma<FP8>(tmem + sb * 128u, DESC_K | (qx_lo + a_off), DESC_K | (k_lo + b_off), IDESC_QK, (term > 0 || ks > 0) ? 1u : 0u);
                                }
                            tc_commit(c->s_full + sb);
                            // the K stage goes back to the producer behind the QK of the last query tile that reads this cached tile
                            uint32_t k_readers = 0;
#pragma unroll
                            for (int y = 0; y < NQT; y++) k_readers += j < n_tiles_x[y] ? 1u : 0u;
                            if (++qk_left[st] == k_readers) {
                                tc_commit(c->k_empty + st);
                                qk_left[st] = 0;
                            }
                            jq[x]++;
                            did = true;
                        }
                    }
                    if (jp[x] < jq[x]) {
                        const uint32_t j = jp[x], st = j % NSV;
                        if (mbar_test(c->p_full + x, j & 1u) && mbar_test(c->v_full + st, (j / NSV) & 1u)) {
                            tc_fence_after();
                            const uint32_t v_lo = vr_lo + st * (KV_TILE >> 4), pj_lo = p_lo + x * (P_BYTES >> 4);
#pragma unroll
                            for (int term = 0; term < PT; term++)
#pragma unroll
                                for (int ks = 0; ks < KSTEPS; ks++)
                                    mma<FP8>(tmem + 256u + x * 128u,
                                             DESC_K | (pj_lo + (FP8 ? term * (PTILE >> 4) + ks * 2 : (ks / 4) * (PTILE >> 4) + (ks % 4) * 2)),
                                             DESC_V | (v_lo + ks * ((32 / ES) * 128 >> 4)), IDESC_PV, (j > 0 || term > 0 || ks > 0) ? 1u : 0u);
                            tc_commit(c->pv_done + x);
                            // the stage goes back to the producer behind the PV of the last query tile that reads this cached tile
                            uint32_t readers = 0;
#pragma unroll
                            for (int y = 0; y < NQT; y++) readers += j < n_tiles_x[y] ? 1u : 0u;
                            if (++pv_left[st] == readers) {
                                tc_commit(c->v_empty + st);
                                pv_left[st] = 0;
                            }
                            jp[x]++;
                            todo--;
                            did = true;
                        }
                    }
                }
                if (did) {
                    idle = 0;
                } else {
                    if (++idle > (1u << 22) || ((idle & 63u) == 0 && *fail_word)) ok = false;       // bounded: a stuck barrier ends the CTA, not the GPU
                    __nanosleep(40);                              // leave the issue slots to the softmax warps on this scheduler
                }
            }
            if (!ok) atomicCAS(&c->fail, 0u, 4u);
            tc_commit(&c->drained);
            for (uint32_t it = 0; it < (1u << 22); it++)
                if (mbar_test(&c->drained, 0u)) break;
        }
        __syncwarp();
    } else {
        // ---- softmax.  One query tile: all sixteen warps work on it, four threads per row (32 columns each).  Two query tiles: eight
        // warps each, two threads per row (64 columns each), and the two groups run out of step, so one group's waits (for S, for the
        // tensor-memory load, for its partner's maximum) are filled by the other group's arithmetic.  Thread (split, r) owns columns
        // [CPT * split, +CPT) of row r = (query head r / 32, token r % 32) of every S tile and the same columns of the row in O. ----
        constexpr int NSP = NQT == 2 ? 2 : 4, CPT = 128 / NSP, GW = NSP * 4;            // splits per row, columns per thread, warps per group
        const uint32_t x = NQT == 2 ? warp / GW : 0u, gw = warp % GW;                   // this thread's query tile; warp within the group
        const uint32_t split = gw >> 2, r = (gw & 3u) * 32u + lane, g = r >> 5, tq = r & 31u;
        const uint32_t lane_base = ((gw & 3u) * 32u) << 16, col0 = split * CPT;
        const uint32_t bar_rows = 2u + (gw & 3u) + 4u * x, bar_group = 10u + x;        // named barriers: the warps sharing 32 rows; the whole group
        float* exch = c->exch + x * (NSP * 128);
        const uint32_t my_rows = rows_tokens[x], my_tiles = n_tiles_x[x];
        const bool row_live = tq < my_rows;
        const uint32_t q_pos = a.start_pos + q0 + x * QT + (row_live ? tq : 0u);
        if (split == 0) {
            // Q row: scaled into the log2 domain; E4M3 pool: two E4M3 terms under a power-of-two scale that brings the row's largest
            // element into [128, 256)
            const float* qrow = a.q + ((size_t)(q0 + x * QT + (row_live ? tq : 0u)) * a.n_q_heads + kvh * PG + g) * PD;
            unsigned char* qt = q_tile + x * Q_BYTES;
            float up = a.q_scale, qi = 1.0f;
            if (FP8 && row_live) {
                float amax = 0.0f;
                for (int i = 0; i < PD / 4; i++) {
                    const float4 f = __ldg(reinterpret_cast<const float4*>(qrow) + i);
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
                }
                amax *= fabsf(a.q_scale);
                int e = 0;
                if (amax > 0.0f && amax < INFINITY) e = 7 - (int)((__float_as_uint(amax) >> 23) & 0xFFu) + 127;
                e = max(-60, min(60, e));
                up = a.q_scale * __uint_as_float((uint32_t)(127 + e) << 23);
                qi = __uint_as_float((uint32_t)(127 - e) << 23);
            }
            if (!row_live) up = 0.0f;
#pragma unroll 1
            for (int ch = 0; ch < PD / 16; ch++) {                  // 16 dims at a time
                float xv[16];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 f = row_live ? __ldg(reinterpret_cast<const float4*>(qrow) + ch * 4 + i) : make_float4(0, 0, 0, 0);
                    xv[4 * i] = f.x * up;
                    xv[4 * i + 1] = f.y * up;
                    xv[4 * i + 2] = f.z * up;
                    xv[4 * i + 3] = f.w * up;
                }
                if (FP8) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        hi[wd] = lo[wd] = 0;
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            const float v = xv[wd * 4 + b];
                            const uint32_t h = e4m3_of(v);
                            const uint32_t l = e4m3_of(v - e4m3_to_f32(h));
                            hi[wd] |= h << (8 * b);
                            lo[wd] |= l << (8 * b);
                        }
                    }
                    *reinterpret_cast<uint4*>(qt + swz(r, ch)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(qt + PTILE + swz(r, ch)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                } else {
                    uint32_t wv[8];
#pragma unroll
                    for (int wd = 0; wd < 8; wd++) {
                        __half2 h = __floats2half2_rn(xv[2 * wd], xv[2 * wd + 1]);
                        wv[wd] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    // 16 dims = 32 B = two 16-byte chunks; dims [64, 128) live in the second column group
                    unsigned char* base = qt + (ch / 4) * PTILE;
                    *reinterpret_cast<uint4*>(base + swz(r, (ch % 4) * 2)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                    *reinterpret_cast<uint4*>(base + swz(r, (ch % 4) * 2 + 1)) = make_uint4(wv[4], wv[5], wv[6], wv[7]);
                }
            }
            exch[r] = qi;
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->q_ready);
        }
        asm volatile("bar.sync %0, %1;" ::"r"(bar_group), "n"(GW * 32) : "memory");        // q_inv is in place
        const float q_inv = exch[r];
        asm volatile("bar.sync %0, %1;" ::"r"(bar_group), "n"(GW * 32) : "memory");        // the exchange area now holds row maxima
        bool ok = c->fail == 0;
        float m_used = -INFINITY, l = 0.0f;
        unsigned char* pj = p_tile + x * P_BYTES;
        const uint32_t tmem_o = tmem + 256u + x * 128u + lane_base + col0;
        for (uint32_t j = 0; j < my_tiles; j++) {
            const uint32_t sb = s_index(x, j), st = j & 3u, sv = j % NSV, t0 = j * KT;
            if (ok) {
                ok = mbar_wait(c->s_full + sb, s_phase(j) & 1u, fail_word);
                if (!ok) atomicCAS(&c->fail, 0u, 4u);
            }
            const uint32_t tmem_s = tmem + sb * 128u + lane_base + col0;
            const bool masked = t0 + KT > a.start_pos + q0 + x * QT + 1u;          // some row of this query tile stops inside the cached tile (or before it)
            // ---- pass 1: this thread's maximum over its allowed columns (16 columns = one block of the pool = one K scale) ----
            float m_part = -INFINITY;
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_s + c0, v);
                    tmem_wait_ld();
                    float mx0 = -INFINITY, mx1 = -INFINITY;                   // the scales are positive: the maximum commutes with them
                    if (masked) {
#pragma unroll
                        for (int q = 0; q < 16; q++) {
                            if (t0 + col0 + c0 + q <= q_pos) mx0 = fmaxf(mx0, __uint_as_float(v[q]));
                            if (t0 + col0 + c0 + 16 + q <= q_pos) mx1 = fmaxf(mx1, __uint_as_float(v[16 + q]));
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 16; q++) {
                            mx0 = fmaxf(mx0, __uint_as_float(v[q]));
                            mx1 = fmaxf(mx1, __uint_as_float(v[16 + q]));
                        }
                    }
                    const uint32_t blk = (col0 + c0) >> 4;
                    m_part = fmaxf(m_part, fmaxf(mx0 * (c->scales[st][blk] * q_inv), mx1 * (c->scales[st][blk + 1u] * q_inv)));
                }
            }
            // the splits of a row exchange their maxima: wait until the previous tile's values have been read, write, wait, read
            asm volatile("bar.sync %0, %1;" ::"r"(bar_rows), "n"(NSP * 32) : "memory");
            exch[split * 128 + r] = m_part;
            asm volatile("bar.sync %0, %1;" ::"r"(bar_rows), "n"(NSP * 32) : "memory");
            float m_tile = exch[r];
#pragma unroll
            for (int i = 1; i < NSP; i++) m_tile = fmaxf(m_tile, exch[i * 128 + r]);
            // ---- a raised maximum rescales the row sum and this thread's columns of the row of O (after the previous tile's PV MMAs) ----
            const bool raise = m_tile > m_used + P_RAISE;
            float factor = 1.0f;
            if (raise) {
                factor = m_used == -INFINITY ? 0.0f : fast_exp2(m_used - m_tile);
                m_used = m_tile;
                l *= factor;
            }
            if (ok && j > 0) {
                ok = mbar_wait(c->pv_done + x, (j - 1u) & 1u, fail_word);            // P may be rewritten, O may be touched
                if (!ok) atomicCAS(&c->fail, 0u, 4u);
            }
            if (j > 0 && __any_sync(0xFFFFFFFFu, raise) && ok) {
                tc_fence_after();
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < (uint32_t)CPT; c0 += 16) {
                    uint32_t o[16];
                    tmem_ld16(tmem_o + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 16; q++) o[q] = __float_as_uint(__uint_as_float(o[q]) * factor);
                    tmem_st16(tmem_o + c0, o);
                }
                tmem_wait_st();
                tc_fence_before();
            }
            // ---- pass 2: probabilities 2^(s - m + SHIFT) * v scale into P (three E5M2 terms for an E4M3 pool), S read again ----
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tmem_s + c0, v);
                    tmem_wait_ld();
                    if (c0 == CPT - 32) {                            // S has been read for the last time
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(c->s_free + sb);
                    }
#pragma unroll
                    for (int half = 0; half < 2; half++) {           // 16 columns = one block of the pool = one pair of scales
                        const uint32_t blk = ((col0 + c0) >> 4) + half;
                        const float ks = c->scales[st][blk] * q_inv, vs = c->scales[st][8 + blk];
                        float inv_vs;
                        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_vs) : "f"(vs));
                        const float lv = fast_log2(vs) + P_SHIFT - m_used;
                        const float sum = masked ? probabilities16<FP8, true>(v + half * 16, ks, lv, t0 + blk * 16u, q_pos, pj, r, blk)
                                                 : probabilities16<FP8, false>(v + half * 16, ks, lv, 0u, 0u, pj, r, blk);
                        l += sum * (inv_vs * __uint_as_float((uint32_t)(127 - (int)P_SHIFT) << 23));
                    }
                }
                // rows of the V tile past the last attended token hold whatever the pool (or an earlier tile) left there: 0 * NaN must not
                // reach O.  Each group clears them before its own PV (the same zeros, whoever comes first).
                if (split == 0 && t0 + KT > kv_limit) {               // uniform over the warp; the copies of V must have landed first
                    ok = mbar_wait(c->v_full + sv, (j / NSV) & 1u, fail_word);
                    if (!ok) atomicCAS(&c->fail, 0u, 4u);
                }
                if (ok && split == 0 && t0 + KT > kv_limit && t0 + r >= kv_limit) {
                    unsigned char* vt = v_ring + (size_t)sv * KV_TILE;
#pragma unroll
                    for (int cg = 0; cg < ES; cg++)
#pragma unroll
                        for (int ch = 0; ch < 8; ch++) *reinterpret_cast<uint4*>(vt + cg * PTILE + swz(r, ch)) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c->p_full + x);            // also after a failure: the issuer then ends through the fail word
        }
        // ---- epilogue: this thread's columns of the O row / the row sum of all splits, undoing the shift and the V-scale normalisation ----
        asm volatile("bar.sync %0, %1;" ::"r"(bar_group), "n"(GW * 32) : "memory");        // the last maxima have been read
        exch[split * 128 + r] = l;
        asm volatile("bar.sync %0, %1;" ::"r"(bar_group), "n"(GW * 32) : "memory");
        float l_row = 0.0f;
#pragma unroll
        for (int i = 0; i < NSP; i++) l_row += exch[i * 128 + r];
        if (ok && my_tiles) {
            ok = mbar_wait(c->pv_done + x, (my_tiles - 1u) & 1u, fail_word);
            if (!ok) atomicCAS(&c->fail, 0u, 4u);
        }
        if (ok && my_tiles) {
            tc_fence_after();
            const float norm = __uint_as_float((uint32_t)(127 - (int)P_SHIFT + v_exp) << 23) / l_row;
            float* orow = a.out + ((size_t)(q0 + x * QT + tq) * a.n_q_heads + kvh * PG + g) * PD + col0;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)CPT; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem_o + c0, o);
                tmem_wait_ld();
                if (row_live) {
#pragma unroll
                    for (int q = 0; q < 32; q += 4)
                        *reinterpret_cast<float4*>(orow + c0 + q) = make_float4(__uint_as_float(o[q]) * norm, __uint_as_float(o[q + 1]) * norm,
                                                                                 __uint_as_float(o[q + 2]) * norm, __uint_as_float(o[q + 3]) * norm);
                }
            }
            tc_fence_before();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == SM_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
    if (tid == 0 && c->fail && a.status) atomicCAS(a.status, 0u, c->fail);
}

// A layer tensor as a 3-D byte array [token = blocks * 16][kv head = 8][128 * ES bytes], boxes of [16 tokens][1 kv head][128 B]:
// one kv head's rows of one block.
bool make_head_map(CUtensorMap* map, uint64_t base, uint32_t total_blocks, uint32_t es) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[3] = {128ull * es, (cuuint64_t)PHKV, (cuuint64_t)total_blocks * PBS};
    const cuuint64_t strides[2] = {128ull * es, 128ull * es * PHKV};
    const cuuint32_t box[3] = {128u, 1u, (cuuint32_t)PBS};
    const cuuint32_t elem[3] = {1u, 1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, reinterpret_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool FP8, int NQT> cudaError_t launch_prefill(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillArgs& a, cudaStream_t st) {
    constexpr int ES = FP8 ? 1 : 2;
    constexpr size_t stages = (!FP8 && NQT == 2) ? 3 : 4;          // K and V stages together (an F16 pool's two query tiles: two of K, one of V)
    constexpr size_t smem = CTRL + NQT * (2 * (size_t)PTILE + (FP8 ? 3 : 2) * (size_t)PTILE) + stages * (size_t)PTILE * ES;
    static_assert(smem <= 227 * 1024, "shared memory of one CTA");
    auto kernel = prefill_attn_tc<FP8, NQT>;
    static std::mutex mu;
    static bool granted[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!granted[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
            granted[dev] = true;
        }
    }
    const dim3 grid((a.n_tokens + QT * NQT - 1) / (QT * NQT) * PHKV);
    kernel<<<grid, PTHREADS, smem, st>>>(mk, mv, a);
    return cudaGetLastError();
}

}  // namespace

bool prefill_eligible(uint32_t n_kv_heads, uint32_t n_q_heads, uint32_t head_dim, uint32_t block_size, uint32_t total_blocks) {
    return n_kv_heads == PHKV && n_q_heads == PHKV * PG && head_dim == PD && block_size == PBS && (uint64_t)total_blocks * PBS < (1ull << 31);
}

cudaError_t launch_prefill(bool fp8, uint64_t k_layer, uint64_t v_layer, const PrefillArgs& a, cudaStream_t st) {
    CUtensorMap mk, mv;
    const uint32_t es = fp8 ? 1u : 2u;
    if (!make_head_map(&mk, k_layer, a.total_blocks, es) || !make_head_map(&mv, v_layer, a.total_blocks, es)) return cudaErrorInvalidValue;
    // Two query tiles per CTA, their softmax groups out of step, unless a.single_tile asks for one.  Measured on B200 (useful TFLOP/s,
    // one tile / two tiles): E4M3 pool 69 / 59 at 512 new tokens, 192 / 177 at 1 024, 245 / 288 at 1 536, 295 / 373 at 2 048, 398 / 520 at
    // 4 096; F16 pool 71 / 66, 249 / 198, 315 / 337, 364 / 468, 489 / 619, 578 / 786 at 8 192: below 1 536 tokens two tiles leave SMs
    // without a CTA, from there on they win.
    const bool two = a.single_tile == 2u || (a.single_tile == 0u && a.n_tokens >= 1536u);
    if (fp8) return two ? launch_prefill<true, 2>(mk, mv, a, st) : launch_prefill<true, 1>(mk, mv, a, st);
    return two ? launch_prefill<false, 2>(mk, mv, a, st) : launch_prefill<false, 1>(mk, mv, a, st);
}

}  // namespace tkv_tc

namespace {
int32_t pfail(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return tkv_internal::set_error(code, 0, buf);
}
}  // namespace

extern "C" int32_t tkv_prefill_attn_enqueue(const TkvPool* pool, const TkvPrefillAttn* p, void* stream) {
    if (!pool || !p) return pfail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (pool->dtype != TKV_DTYPE_F16 && pool->dtype != TKV_DTYPE_E4M3)
        return pfail(TKV_ERR_INVALID_CONFIG, "prefill attention reads F16 or E4M3 pools (dtype %d)", (int)pool->dtype);
    if (!tkv_tc::prefill_eligible(pool->n_kv_heads, p->n_q_heads, pool->head_dim, pool->block_size, pool->total_blocks))
        return pfail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (prefill attention is built for 8 kv heads of 128 dims, 32 query heads, 16-token blocks)",
                     8u, pool->n_kv_heads);
    if (p->layer >= pool->n_layers) return pfail(TKV_ERR_INVALID_CONFIG, "layer %u outside the pool (%u layers)", p->layer, pool->n_layers);
    if ((pool->k_scales == 0) != (pool->v_scales == 0)) return pfail(TKV_ERR_INVALID_CONFIG, "k_scales and v_scales must both be set or both be 0");
    if (pool->k_scales && pool->dtype != TKV_DTYPE_E4M3) return pfail(TKV_ERR_INVALID_CONFIG, "only an E4M3 pool carries scales");
    if (p->n_tokens == 0) return TKV_OK;
    if (!p->q || !p->out || !p->table || !pool->k_layer_ptrs || !pool->v_layer_ptrs) return pfail(TKV_ERR_INVALID_CONFIG, "NULL buffer");
    const uint64_t kv_len = (uint64_t)p->start_pos + p->n_tokens;
    if (kv_len > (uint64_t)p->table_len * 16u)
        return pfail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (table entries for start_pos + n_tokens)",
                     (unsigned long long)((kv_len + 15) / 16), (unsigned long long)p->table_len);
    const uint64_t kp = pool->k_layer_ptrs[p->layer], vp = pool->v_layer_ptrs[p->layer];
    if ((kp | vp | p->q | p->out) % 16) return pfail(TKV_ERR_INVALID_CONFIG, "layer tensors, q and out must be 16-byte aligned");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return pfail(TKV_ERR_CUDA, "cudaGetDevice failed");
    if (dev != pool->device && cudaSetDevice(pool->device) != cudaSuccess) return pfail(TKV_ERR_CUDA, "cannot select device %d", pool->device);
    tkv_tc::PrefillArgs a{};
    const size_t layer_scales = (size_t)pool->total_blocks * pool->n_kv_heads;
    a.k_scales = pool->k_scales ? reinterpret_cast<const float*>(pool->k_scales) + (size_t)p->layer * layer_scales : nullptr;
    a.v_scales = pool->v_scales ? reinterpret_cast<const float*>(pool->v_scales) + (size_t)p->layer * layer_scales : nullptr;
    a.q = reinterpret_cast<const float*>(p->q);
    a.out = reinterpret_cast<float*>(p->out);
    a.table = reinterpret_cast<const uint32_t*>(p->table);
    a.n_tokens = p->n_tokens;
    a.start_pos = p->start_pos;
    a.n_q_heads = p->n_q_heads;
    a.total_blocks = pool->total_blocks;
    a.q_scale = p->sm_scale * 1.4426950408889634f;
    a.status = reinterpret_cast<uint32_t*>(p->status);
    a.single_tile = (p->flags & TKV_PREFILL_SINGLE_TILE) ? 1u : (p->flags & TKV_PREFILL_TWO_TILES) ? 2u : 0u;
    const cudaError_t e = tkv_tc::launch_prefill(pool->dtype == TKV_DTYPE_E4M3, kp, vp, a, static_cast<cudaStream_t>(stream));
    if (dev != pool->device) cudaSetDevice(dev);
    if (e != cudaSuccess) return tkv_internal::set_error(TKV_ERR_CUDA, (int32_t)e, cudaGetErrorString(e));
    return TKV_OK;
}
