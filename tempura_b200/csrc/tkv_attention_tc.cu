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
// memory descriptors name), one thread issues the MMAs, and the four softmax warps own one
// (token, kv head) row each: they read their row of S^T from tensor memory, keep the columns of their
// own kv head, and write the probabilities into P^T, whose entries for other kv heads stay zero.
// A row's columns of the other seven kv heads are computed and dropped: that is 7/8 of the tensor work
// and still a fifth of the time the block takes to arrive from HBM, which is the bound.
//
// Operand precision.  F16 pool: q and the probabilities are F16 (as the mma.sync kernel feeds them).
// E4M3 pool: both operands of an MMA must be 8-bit, so q is split into two E4M3 terms (per-head power
// of two scale, residual in the second term: 2^-8 relative) and a probability into four E5M2 terms
// (E5M2 for its range: weights down to 2^-31 of the running maximum survive; four 3-bit terms give
// 2^-12 relative).  The terms are separate columns of Q^T / P^T, summed after the MMA.
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

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
}

namespace tkv_tc {

constexpr int D = 128, BS = 16, HKV = 8, ROWS = BS * HKV;   // one block = 128 operand rows
constexpr int TILE = ROWS * 128;                           // bytes of one [128 rows][128 B] swizzled tile
constexpr float RAISE = 6.0f;                              // the running maximum is raised when a block exceeds it by 2^RAISE
constexpr float SHIFT = 9.0f;                              // probabilities enter P^T as 2^(s - m + SHIFT): below the E5M2 / F16 maximum

// ---- small PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded: gives up after 2^22 polls, or as soon as another role of the CTA has recorded a failure
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile uint32_t* fail_word) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < (1u << 22); it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 15u) == 15u && *fail_word) return false;
    }
    return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_barrier_softmax() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// 2-D tensor-map copy of one [128 rows][128 B] box (no multicast), completing on an mbarrier
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory operand descriptor, 128-byte swizzle: start address, leading and stride byte offsets in
// 16-byte units, descriptor version 1 (bit 46), swizzle mode 2 (bits 61-63).  Tiles are 1024-byte aligned.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: F32 accumulate, operand formats, A / B major-ness, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
template <bool FP8>
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if (FP8)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 columns of 32-bit cells: thread t of warp w reads lane 32 * (w % 4) + t
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
          "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fast_log2(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// byte offset of (row, 16-byte chunk) inside a [rows][128 B] tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) { return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4); }

__device__ __forceinline__ uint32_t e4m3_of(float x) {          // round to nearest even, saturating; one byte
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xFFu;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((unsigned short)b));
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}
__device__ __forceinline__ uint32_t e5m2_of(float x) {
    uint16_t r;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xFFu;
}
__device__ __forceinline__ float e5m2_to_f32(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)(b << 8))); }   // E5M2 = the top byte of an F16

// order-preserving map float -> int for atomicMax on shared memory
__device__ __forceinline__ int ordered(float f) {
    const int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7FFFFFFF;
}
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i >= 0 ? i : i ^ 0x7FFFFFFF); }

// Control block at the head of shared memory.
struct Control {
    uint64_t full[8], empty[8];       // ring stages: copies landed / both MMAs of the block done
    uint64_t s_full[2], s_free[2];    // S^T buffers: QK done / every softmax warp has read it
    uint64_t p_full[2], p_free[2];    // P^T buffers: written / the PV MMA has read it
    uint64_t drained;                 // teardown: every MMA issued so far has completed
    uint32_t tmem_base, fail;
    int block_max[2][32];             // per block parity: ordered-int maxima of the query heads that asked for a raise
    uint32_t raise[2];
    float m_used[32], factor[32], q_inv[32], l_sum[4][32];
};

template <bool FP8, int G>
__global__ void __launch_bounds__(192, 1)
decode_attn_tc(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const Args a, const uint32_t n_stages) {
    constexpr int ES = FP8 ? 1 : 2;                    // bytes per pool element = 128-byte column groups per row
    constexpr int QT = FP8 ? 2 : 1, PT = FP8 ? 4 : 1;  // terms a query element / a probability is split into
    constexpr int CQ = (G * QT < 2) ? 2 : G * QT;      // columns per kv head in S^T and in O^T (N must be a multiple of 16)
    constexpr int CP = (G * PT < 2) ? 2 : G * PT;
    constexpr int NQ = HKV * CQ, NP = HKV * CP;
    static_assert(NQ % 16 == 0 && NP % 16 == 0 && NQ <= 256 && NP <= 256 && NP + 2 * NQ <= 512, "MMA N and tensor memory columns");
    static_assert(NQ % 32 == 0 || NQ == 16, "S^T is read 32 columns at a time");
    constexpr int KV_TILE = TILE * ES;                 // K (or V) of one block in shared memory
    constexpr int QT_BYTES = NQ * 128 * ES, PT_BYTES = NP * 128 * ES;
    constexpr uint32_t FMT_KV = 0u, FMT_P = FP8 ? 1u : 0u;          // kind::f8f6f4: E4M3 = 0, E5M2 = 1; kind::f16: F16 = 0
    constexpr uint32_t IDESC_QK = instr_desc(FMT_KV, 0u, 0u, NQ), IDESC_PV = instr_desc(FMT_KV, FMT_P, 1u, NP);
    constexpr int KSTEPS = 4 * ES;                     // 32 bytes of the contraction per MMA: 4 steps per 128-byte group

    const uint32_t split = blockIdx.x, seq = blockIdx.y;
    const uint32_t kv_len = min(a.kv_lens[seq], a.max_kv_len);
    const uint32_t t_begin = split * a.split_tokens;
    if (t_begin >= kv_len) return;
    const uint32_t t_end = min(kv_len, t_begin + a.split_tokens);
    const uint32_t b_begin = t_begin / BS, n_blk = (t_end + BS - 1) / BS - b_begin;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t* table = a.tables + (size_t)seq * a.table_stride + b_begin;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    Control* c = reinterpret_cast<Control*>(smem);
    unsigned char* q_tile = smem + 2048;                          // Q^T: [NQ rows][128 B] per column group
    unsigned char* p_tile = q_tile + QT_BYTES;                    // P^T: two buffers
    float* scales = reinterpret_cast<float*>(p_tile + 2 * PT_BYTES);   // per stage: 8 K scales, 8 V scales
    unsigned char* stages = reinterpret_cast<unsigned char*>(scales) + 1024;   // per stage: K tile(s), V tile(s)
    const volatile uint32_t* fail_word = &c->fail;
    const uint32_t stage_bytes = 2 * KV_TILE;

    if (tid == 0) {
        for (uint32_t s = 0; s < n_stages; s++) {
            mbar_init(c->full + s, 1);
            mbar_init(c->empty + s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(c->s_full + b, 1);
            mbar_init(c->s_free + b, 4);
            mbar_init(c->p_full + b, 4);
            mbar_init(c->p_free + b, 1);
            c->raise[b] = 0;
        }
        mbar_init(&c->drained, 1);
        c->fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 64) c->block_max[tid >> 5][tid & 31] = ordered(-INFINITY);
    if (tid < 32) c->m_used[tid] = -INFINITY;
    if (warp == 5) {                                               // tensor memory: 512 columns, this CTA alone on its SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&c->tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < 4) {
        // ---- Q^T: thread (query head qh = tid / 4, dims [32 * (tid % 4), +32)) ----
        const uint32_t qh = tid >> 2, part = tid & 3u, kvh = qh / G, g = qh % G;
        float x[32];
        const bool live = qh < a.n_q_heads;
        const float* qrow = a.q + ((size_t)seq * a.n_q_heads + (live ? qh : 0)) * D + part * 32;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 f = live ? *reinterpret_cast<const float4*>(qrow + 4 * i) : make_float4(0, 0, 0, 0);
            x[4 * i] = f.x * a.q_scale;
            x[4 * i + 1] = f.y * a.q_scale;
            x[4 * i + 2] = f.z * a.q_scale;
            x[4 * i + 3] = f.w * a.q_scale;
        }
        // zero both P^T buffers and the unused rows of Q^T first (entries of other kv heads stay zero for good)
        for (uint32_t i = tid; i < (2 * PT_BYTES + QT_BYTES) / 16; i += 128) reinterpret_cast<uint4*>(q_tile)[i] = make_uint4(0, 0, 0, 0);
        named_barrier_softmax();
        if (FP8) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
            // power of two that brings the head's largest element into [128, 256): exact to apply and to undo
            int e = 0;
            if (amax > 0.0f && amax < INFINITY) e = 7 - (int)((__float_as_uint(amax) >> 23) & 0xFFu) + 127;
            e = max(-60, min(60, e));
            const float up = __uint_as_float((uint32_t)(127 + e) << 23);
            if (part == 0 && live) c->q_inv[qh] = __uint_as_float((uint32_t)(127 - e) << 23);
            if (live) {
#pragma unroll
                for (int ch = 0; ch < 2; ch++) {                    // two 16-byte chunks of the row per term
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        hi[wd] = lo[wd] = 0;
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            const float v = x[ch * 16 + wd * 4 + b] * up;
                            const uint32_t h = e4m3_of(v);
                            const uint32_t l = e4m3_of(v - e4m3_to_f32(h));
                            hi[wd] |= h << (8 * b);
                            lo[wd] |= l << (8 * b);
                        }
                    }
                    const uint32_t chunk = part * 2 + ch;
                    *reinterpret_cast<uint4*>(q_tile + swz(kvh * CQ + g, chunk)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(q_tile + swz(kvh * CQ + G + g, chunk)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
        } else {
            if (part == 0 && live) c->q_inv[qh] = 1.0f;
            if (live) {
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {                    // 32 dims * 2 B = four 16-byte chunks; dims [64, 128) live in the second column group
                    uint32_t wv[4];
#pragma unroll
                    for (int wd = 0; wd < 4; wd++) {
                        __half2 h = __floats2half2_rn(x[ch * 8 + wd * 2], x[ch * 8 + wd * 2 + 1]);
                        wv[wd] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    const uint32_t group = part >> 1, chunk = (part & 1u) * 4 + ch;
                    *reinterpret_cast<uint4*>(q_tile + group * (NQ * 128) + swz(kvh * CQ + g, chunk)) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                }
            }
        }
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = c->tmem_base;
    const uint32_t tmem_o = tmem, tmem_s0 = tmem + NP;            // O^T at column 0, the two S^T buffers behind it

    if (warp == 4) {
        // ---- producer: the block table 32 entries at a time; lane 0 issues the copies ----
        uint32_t issued = 0, why = 4u;
        bool ok = true;
        uint32_t ids_next = lane < n_blk ? __ldg(table + lane) : 0u;
        for (uint32_t k0 = 0; k0 < n_blk && ok; k0 += 32) {
            const uint32_t ids = ids_next;
            ids_next = k0 + 32 + lane < n_blk ? __ldg(table + k0 + 32 + lane) : 0u;
            const uint32_t lim = min(32u, n_blk - k0);
            for (uint32_t i = 0; i < lim && ok; i++) {
                const uint32_t id = __shfl_sync(0xFFFFFFFFu, ids, i);
                const uint32_t k = k0 + i, s = k % n_stages;
                if (lane == 0) {
                    if (id >= a.total_blocks) {                   // a stale or foreign id is never turned into an address
                        ok = false;
                        why = 2u;
                    }
                    if (ok && k >= n_stages) ok = mbar_wait(c->empty + s, ((k / n_stages) - 1u) & 1u, fail_word);
                    if (ok) {
                        const uint32_t sc_bytes = a.k_scales ? HKV * 4u : 0u;
                        const uint32_t dst = smem_u32(stages + (size_t)s * stage_bytes);
                        mbar_expect_tx(c->full + s, 2u * KV_TILE + 2u * sc_bytes);
#pragma unroll
                        for (int grp = 0; grp < ES; grp++) {
                            tma_box(dst + grp * TILE, &map_k, grp * 128, (int32_t)(id * ROWS), c->full + s);
                            tma_box(dst + KV_TILE + grp * TILE, &map_v, grp * 128, (int32_t)(id * ROWS), c->full + s);
                        }
                        if (sc_bytes) {
                            bulk_copy(smem_u32(scales + s * 16), a.k_scales + (size_t)id * HKV, sc_bytes, c->full + s);
                            bulk_copy(smem_u32(scales + s * 16 + 8), a.v_scales + (size_t)id * HKV, sc_bytes, c->full + s);
                        }
                        issued = k + 1;
                    }
                }
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0u;
            }
        }
        if (!ok && lane == 0) {
            atomicCAS(&c->fail, 0u, why);
            // give the copies still in flight a bounded chance to land before the CTA's shared memory is released
            for (uint32_t k = issued > n_stages ? issued - n_stages : 0u; k < issued; k++) {
                const uint32_t addr = smem_u32(c->full + k % n_stages), parity = (k / n_stages) & 1u;
                for (uint32_t it = 0; it < (1u << 20); it++) {
                    uint32_t done;
                    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
                    if (done) break;
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer: one thread ----
        if (lane == 0) {
            bool ok = true;
            auto issue_pv = [&](uint32_t j) {
                const uint32_t s = j % n_stages, b = j & 1u;
                if (!mbar_wait(c->p_full + b, (j >> 1) & 1u, fail_word)) return false;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(stages + (size_t)s * stage_bytes + KV_TILE), p_addr = smem_u32(p_tile + b * PT_BYTES);
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
                    // V^T (A, MN-major): 32 / ES block rows per step, 128 B each; dims beyond 64 (F16) in the second column group
                    const uint64_t da = smem_desc(v_addr + ks * (32 / ES) * 128, TILE, 1024);
                    // P^T (B, K-major): 32 bytes of the row per step
                    const uint64_t db = smem_desc(p_addr + (ks / 4) * (NP * 128) + (ks % 4) * 32, 16, 1024);
                    mma<FP8>(tmem_o, da, db, IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(c->empty + s);
                tc_commit(c->p_free + b);
                return true;
            };
            const uint32_t q_addr = smem_u32(q_tile);
            for (uint32_t i = 0; i < n_blk && ok; i++) {
                const uint32_t s = i % n_stages, b = i & 1u;
                ok = mbar_wait(c->full + s, (i / n_stages) & 1u, fail_word);
                if (ok && i >= 2) ok = mbar_wait(c->s_free + b, ((i >> 1) - 1u) & 1u, fail_word);
                if (!ok) break;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(stages + (size_t)s * stage_bytes);
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
                    const uint64_t da = smem_desc(k_addr + (ks / 4) * TILE + (ks % 4) * 32, 16, 1024);
                    const uint64_t db = smem_desc(q_addr + (ks / 4) * (NQ * 128) + (ks % 4) * 32, 16, 1024);
                    mma<FP8>(tmem_s0 + b * NQ, da, db, IDESC_QK, ks > 0 ? 1u : 0u);
                }
                tc_commit(c->s_full + b);
                if (i >= 1) ok = issue_pv(i - 1);
            }
            if (ok) ok = issue_pv(n_blk - 1);
            if (!ok) atomicCAS(&c->fail, 0u, 4u);
            // nothing of this CTA may still be writing tensor memory when it is freed
            tc_commit(&c->drained);
            const uint32_t addr = smem_u32(&c->drained);
            for (uint32_t it = 0; it < (1u << 22); it++) {
                uint32_t done;
                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(done) : "r"(addr), "r"(0u) : "memory");
                if (done) break;
            }
        }
        __syncwarp();
    } else {
        // ---- softmax: thread tid owns block row tid = (token tid / 8, kv head tid % 8) and tensor-memory lane tid ----
        const uint32_t kvh = tid & 7u, tok = tid >> 3;
        const uint32_t lane_base = (warp * 32u) << 16;
        float m_used[G], l[G], q_inv[G];
#pragma unroll
        for (int g = 0; g < G; g++) {
            m_used[g] = -INFINITY;
            l[g] = 0.0f;
            q_inv[g] = c->q_inv[kvh * G + g];
        }
        bool ok = true;
        for (uint32_t i = 0; i < n_blk; i++) {
            const uint32_t s = i % n_stages, b = i & 1u;
            const uint32_t n_valid = min((uint32_t)BS, kv_len - (b_begin + i) * BS);
            const bool valid = tok < n_valid;
            float sc[G];                                            // this row's scores against its own kv head's query heads (log2 domain)
            float lv = 0.0f, inv_vs = 1.0f;
            if (ok) {
                ok = mbar_wait(c->s_full + b, (i >> 1) & 1u, fail_word) && mbar_wait(c->full + s, (i / n_stages) & 1u, fail_word);
                if (!ok) atomicCAS(&c->fail, 0u, 4u);
            }
            if (ok) {
                tc_fence_after();
                float part[CQ];
                // the row's NQ columns, 32 at a time (16 when that is all there is); keep the CQ columns of this row's kv head
                if (NQ >= 32) {
#pragma unroll
                    for (int c0 = 0; c0 < NQ; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32(tmem_s0 + b * NQ + lane_base + c0, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int h = 0; h < 32 / CQ; h++)
                            if ((uint32_t)(c0 / CQ + h) == kvh) {
#pragma unroll
                                for (int j = 0; j < CQ; j++) part[j] = __uint_as_float(r[h * CQ + j]);
                            }
                    }
                } else {
                    uint32_t r[32];
                    tmem_ld32(tmem_s0 + b * NQ + lane_base, r);     // NQ = 16: the upper 16 columns read belong to the next buffer and are ignored
                    tmem_wait_ld();
#pragma unroll
                    for (int h = 0; h < 16 / CQ; h++)
                        if ((uint32_t)h == kvh) {
#pragma unroll
                            for (int j = 0; j < CQ; j++) part[j] = __uint_as_float(r[h * CQ + j]);
                        }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(c->s_free + b);
                float ks = 1.0f, vs = 1.0f;
                if (a.k_scales) {
                    ks = scales[s * 16 + kvh];
                    vs = scales[s * 16 + 8 + kvh];
                    lv = fast_log2(vs);
                    inv_vs = __frcp_rn(vs);
                }
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float raw = FP8 ? part[g] + part[G + g] : part[g];
                    sc[g] = valid ? raw * (ks * q_inv[g]) : -INFINITY;
                }
            } else {
#pragma unroll
                for (int g = 0; g < G; g++) sc[g] = -INFINITY;
            }
            // does any query head of this kv head exceed its running maximum by more than 2^RAISE in this block?
            bool want = false;
#pragma unroll
            for (int g = 0; g < G; g++) {
                float bm = sc[g] + lv;                              // the weight's exponent carries the V scale
                bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 8));
                bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 16));
                if (bm > m_used[g] + RAISE) {
                    want = true;
                    if (lane < 8) atomicMax(&c->block_max[b][kvh * G + g], ordered(bm));
                }
            }
            if (want && lane < 8) c->raise[b] = 1u;
            named_barrier_softmax();
            if (c->raise[b]) {
                // ---- raise the maxima: rescale O^T in tensor memory and the row sums; rare ----
                if (tid < 32) {
                    const float bm = unordered(c->block_max[b][tid]), mo = c->m_used[tid];
                    const float mn = fmaxf(mo, bm);
                    c->factor[tid] = (mn == mo) ? 1.0f : (mo == -INFINITY ? 0.0f : fast_exp2(mo - mn));
                    c->m_used[tid] = mn;
                    c->block_max[b][tid] = ordered(-INFINITY);
                }
                named_barrier_softmax();
                if (tid == 0) c->raise[b] = 0u;
                if (i > 0) {
                    // the PV MMA of the previous block must have finished with O^T; none follows until this block's P^T is published
                    if (ok) ok = mbar_wait(c->p_free + ((i - 1) & 1u), ((i - 1) >> 1) & 1u, fail_word);
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < NP; c0 += 32) {
                            uint32_t r[32];
                            tmem_ld32(tmem_o + lane_base + c0, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const int col = c0 + j, head = (col / CP) * G + (col % CP) % G;
                                r[j] = __float_as_uint(__uint_as_float(r[j]) * c->factor[head]);
                            }
                            tmem_st32(tmem_o + lane_base + c0, r);
                        }
                        tmem_wait_st();
                        tc_fence_before();
                    }
                }
#pragma unroll
                for (int g = 0; g < G; g++) {
                    l[g] *= c->factor[kvh * G + g];
                    m_used[g] = c->m_used[kvh * G + g];
                }
                named_barrier_softmax();                            // factor[] and m_used[] are read before the next raise rewrites them
            }
            if (ok && i >= 2) ok = mbar_wait(c->p_free + b, ((i >> 1) - 1u) & 1u, fail_word);
            if (ok) {
                unsigned char* pt = p_tile + b * PT_BYTES;
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float e = sc[g] + lv - m_used[g];          // <= RAISE; -inf for a row past the sequence end
                    const float w = fast_exp2(e);
                    l[g] += w * inv_vs;
                    float x = fast_exp2(e + SHIFT);
                    if (FP8) {
#pragma unroll
                        for (int t = 0; t < PT; t++) {
                            const uint32_t byte = e5m2_of(x);
                            x -= e5m2_to_f32(byte);
                            const uint32_t row = kvh * CP + t * G + g;
                            pt[swz(row, tid >> 4) + (tid & 15u)] = (unsigned char)byte;
                        }
                    } else {
                        const uint32_t row = kvh * CP + g, el = tid & 63u;        // element tid of the row: column group tid / 64
                        *reinterpret_cast<__half*>(pt + (tid >> 6) * (NP * 128) + swz(row, el >> 3) + (el & 7u) * 2) = __float2half_rn(x);
                    }
                }
                if (!valid) {
                    // a row past the sequence end holds whatever the pool held there: 0 * NaN must not reach O^T
                    unsigned char* vt = stages + (size_t)s * stage_bytes + KV_TILE;
#pragma unroll
                    for (int grp = 0; grp < ES; grp++)
#pragma unroll
                        for (int ch = 0; ch < 8; ch++) *reinterpret_cast<uint4*>(vt + grp * TILE + swz(tid, ch)) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c->p_full + b);              // also after a failure: the issuer's wait then ends through the fail word
        }
        // ---- the partial of this (sequence, token range): wait for the last PV MMA, then O^T rows back out ----
        if (ok) ok = mbar_wait(c->p_free + ((n_blk - 1) & 1u), ((n_blk - 1) >> 1) & 1u, fail_word);
#pragma unroll
        for (int g = 0; g < G; g++) {
            float x = l[g];
            x += __shfl_xor_sync(0xFFFFFFFFu, x, 8);
            x += __shfl_xor_sync(0xFFFFFFFFu, x, 16);
            if (lane < 8) c->l_sum[warp][kvh * G + g] = x;
        }
        named_barrier_softmax();
        if (ok) {
            tc_fence_after();
            const float down = __uint_as_float((uint32_t)(127 - (int)SHIFT) << 23);
            const uint32_t d = tid;                                  // this thread's tensor-memory lane is output dim d
#pragma unroll
            for (int c0 = 0; c0 < NP; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_o + lane_base + c0, r);
                tmem_wait_ld();
#pragma unroll
                for (int h = 0; h < 32 / CP; h++) {
                    const uint32_t head_kv = c0 / CP + h;
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        float acc = 0.0f;
#pragma unroll
                        for (int t = 0; t < PT; t++) acc += __uint_as_float(r[h * CP + t * G + g]);
                        const uint32_t qh = head_kv * G + g;
                        if (qh < a.n_q_heads) {
                            float* pr = a.partial + ((((size_t)seq * HKV + head_kv) * a.n_splits + split) * G + g) * (D + 2);
                            pr[2 + d] = acc * down;
                        }
                    }
                }
            }
            tc_fence_before();
            if (tid < 32 && tid < a.n_q_heads) {
                const uint32_t head_kv = tid / G, g = tid % G;
                float* pr = a.partial + ((((size_t)seq * HKV + head_kv) * a.n_splits + split) * G + g) * (D + 2);
                pr[0] = c->m_used[tid];
                pr[1] = c->l_sum[0][tid] + c->l_sum[1][tid] + c->l_sum[2][tid] + c->l_sum[3][tid];
            }
        } else if (tid == 0) {
            atomicCAS(&c->fail, 0u, 4u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

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

template <bool FP8, int G> static cudaError_t launch_one(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, dim3 grid, cudaStream_t st) {
    constexpr int ES = FP8 ? 1 : 2, QT = FP8 ? 2 : 1, PT = FP8 ? 4 : 1;
    constexpr int CQ = (G * QT < 2) ? 2 : G * QT, CP = (G * PT < 2) ? 2 : G * PT;
    constexpr size_t fixed = 1024 /* alignment slack */ + 2048 + (size_t)HKV * CQ * 128 * ES + 2 * (size_t)HKV * CP * 128 * ES + 1024;
    constexpr size_t stage = 2 * (size_t)TILE * ES;
    const uint32_t n_stages = (uint32_t)std::min<size_t>(8, (227 * 1024 - fixed) / stage);
    if (n_stages < 2) return cudaErrorInvalidConfiguration;
    const size_t smem = fixed + n_stages * stage;
    auto kernel = decode_attn_tc<FP8, G>;
    static std::mutex mu;
    static bool granted[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (dev >= 0 && dev < 64 && !granted[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
            granted[dev] = true;
        }
    }
    kernel<<<grid, 192, smem, st>>>(mk, mv, a, n_stages);
    return cudaGetLastError();
}

cudaError_t launch(bool fp8, uint32_t group, uint64_t k_layer, uint64_t v_layer, const Args& a, uint32_t n_splits, uint32_t n_seqs, cudaStream_t st) {
    CUtensorMap mk, mv;
    const uint32_t es = fp8 ? 1u : 2u;
    if (!make_map(&mk, k_layer, a.total_blocks, es) || !make_map(&mv, v_layer, a.total_blocks, es)) return cudaErrorInvalidValue;
    const dim3 grid(n_splits, n_seqs);
    if (group != 4) return cudaErrorInvalidConfiguration;
    return fp8 ? launch_one<true, 4>(mk, mv, a, grid, st) : launch_one<false, 4>(mk, mv, a, grid, st);
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
