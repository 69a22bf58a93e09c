// Decode attention over the paged KV pool: the consumer of the FP8 cache the handoff fills.
// One query token per sequence, grouped-query heads, K/V rows found through the block table,
// an E4M3 pool read as decode(byte) * per-(layer, block, kv-head) scale.  It replaces the
// reference's per-dtype decode twins (kernels/src/oxide_decode_attn_host.rs:198-260,682-760:
// forward_d2d_ptrs_{f16,e4m3}, forward_batch_d2d_ptrs_{f16,e4m3}), which read a contiguous
// run and assume unscaled E4M3 bytes; the arithmetic it must match is paged_flash_attention
// (kernels/src/attention.rs:486-590) over the widened pool values.
//
// Shape of the work: HBM-bound (every K and V byte of the layer is read once, 1 B per element
// for E4M3).  A CTA of 4 warps owns one (sequence, kv head, split of the cached tokens); each
// warp walks 16-token blocks with its own online softmax and the partials are merged in shared
// memory, then across splits by a second kernel.  Both contractions run on mma.sync
// m16n8k16 (f16 in, f32 accumulate) with the group's query heads as the M rows: per token and
// kv head that is ~13 warp instructions instead of ~45 on the FP32 pipes, which keeps the
// kernel under the memory time.  Lanes load whole 16-byte pieces of a row; the head_dim
// order inside a contraction is free, so each lane's piece is used where the fragment layout
// wants it and the permutation is undone once, at the output.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <stdint.h>

#include <algorithm>
#include <cstdio>

#include "../../include/tkv.h"
#include "tkv_attention_tc.h"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
}

namespace {

constexpr int D = 128;            // head_dim of the fast path
constexpr int BS = 16;            // tokens per block
constexpr int WARPS = 4;
constexpr uint32_t DEFAULT_SPLIT_TOKENS = 1024;   // cached tokens per CTA (a multiple of WARPS * BS)

struct AttnArgs {
    const char* k_base;           // layer tensor
    const char* v_base;
    const float* k_scales;        // [total_blocks][n_kv_heads] of this layer, or null
    const float* v_scales;
    const float* q;               // [n_seqs][n_q_heads][D]
    float* out;
    const uint32_t* tables;       // [n_seqs][table_stride]
    const uint32_t* kv_lens;
    float* partial;               // [n_seqs][n_kv_heads][n_splits][group][D + 2]
    uint64_t block_stride;        // bytes
    uint32_t row_stride;          // bytes between token rows
    uint32_t n_q_heads, n_kv_heads, group, table_stride, n_splits, split_tokens;   // n_splits counts partial slots
    uint32_t parts_per_split;     // partial slots one token range writes (one per softmax group in the tcgen05 form)
    float q_scale;                // softmax scale * log2(e), folded into q
    uint32_t max_kv_len;          // the host's bound: sized the grid, the table rows and the scratch; device lengths are clamped to it
    uint32_t total_blocks;        // blocks in the pool: a table entry at or above it is never dereferenced
    uint32_t* status;             // optional: first failure wins -- TKV_ERR_TIMEOUT (a bounded wait gave up) or
                                  // TKV_ERR_INVALID_CONFIG (a length above max_kv_len, a block id outside the pool)
};

// first failure wins; the output of a launch that reports one is not valid
__device__ __forceinline__ void report(const AttnArgs& a, uint32_t code) {
    if (a.status) atomicCAS(a.status, 0u, code);
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// two e4m3 bytes (low 16 bits) -> two f16; every byte the handoff's writer emits (normals,
// signed zero) converts exactly as kernels/src/e4m3.rs:27-41 reads it
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint32_t two_bytes) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((unsigned short)two_bytes));
    return r;
}

// 2^x on the special-function unit (relative error 2^-22, -inf -> 0): the softmax runs in the exp2 domain
__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// FP8: pool elements are e4m3 bytes; else f16.
template <bool FP8> struct Tile {
    // K: the lane's two tokens (n-tiles 0 and 1), each as two pieces: dims [16j, 16j+16) and [64+16j, 64+16j+16)
    // V: the lane's four tokens {2j, 2j+1, 2j+8, 2j+9}, each dims [16g, 16g+16)
    static constexpr int KW = FP8 ? 1 : 2;   // uint4 per piece
    uint4 k[2][2][KW];
    uint4 v[4][KW];
    float ks, vs;
};

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, bool valid) {
    // src-size 0 zero-fills the 16 bytes (rows past the sequence end)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(valid ? 16u : 0u) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}

// Per warp and ring stage: PIECES 16-byte pieces per lane ([piece][lane], so a warp's reads of one piece
// are 512 contiguous bytes), then 8 bytes per lane for the block's two scales.  Every lane copies and
// later reads only its own slots, so the ring needs no cross-lane synchronisation.
template <bool FP8> struct Ring {
    static constexpr int KW = Tile<FP8>::KW;
    static constexpr int PIECES = 8 * KW;                       // 4 K pieces + 4 V pieces, KW uint4 each
    static constexpr int STAGE_BYTES = PIECES * 32 * 16 + 32 * 8;
    static constexpr int STAGES = FP8 ? 4 : 2;                  // 68 KB per CTA either way: three CTAs per SM
};

template <bool FP8>
__device__ __forceinline__ void issue_tile(uint32_t stage_smem, const AttnArgs& a, uint32_t block_id, uint32_t kvh, uint32_t grp, uint32_t j,
                                           uint32_t lane, uint32_t n_valid) {
    constexpr int ES = FP8 ? 1 : 2;
    constexpr int KW = Tile<FP8>::KW;
    const char* kb = a.k_base + (uint64_t)block_id * a.block_stride + (size_t)kvh * D * ES;
    const char* vb = a.v_base + (uint64_t)block_id * a.block_stride + (size_t)kvh * D * ES;
    int piece_no = 0;
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const uint32_t tok = grp + 8 * nt;
        const bool ok = tok < n_valid;
        const char* row = kb + (size_t)(ok ? tok : 0) * a.row_stride;
#pragma unroll
        for (int piece = 0; piece < 2; piece++)
#pragma unroll
            for (int w = 0; w < KW; w++, piece_no++)
                cp_async16(stage_smem + (piece_no * 32 + lane) * 16, row + (piece * 64 + 16 * j) * ES + 16 * w, ok);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t tok = 2 * j + (i & 1) + 8 * (i >> 1);
        const bool ok = tok < n_valid;
        const char* row = vb + (size_t)(ok ? tok : 0) * a.row_stride + 16 * grp * ES;
#pragma unroll
        for (int w = 0; w < KW; w++, piece_no++) cp_async16(stage_smem + (piece_no * 32 + lane) * 16, row + 16 * w, ok);
    }
    if (a.k_scales) {
        const uint32_t sc = stage_smem + Ring<FP8>::PIECES * 32 * 16 + lane * 8;
        cp_async4(sc, a.k_scales + (size_t)block_id * a.n_kv_heads + kvh);
        cp_async4(sc + 4, a.v_scales + (size_t)block_id * a.n_kv_heads + kvh);
    }
}

template <bool FP8>
__device__ __forceinline__ void read_tile(Tile<FP8>& t, const unsigned char* stage, const AttnArgs& a, uint32_t lane) {
    constexpr int KW = Tile<FP8>::KW;
    const uint4* p = reinterpret_cast<const uint4*>(stage);
    int piece_no = 0;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int piece = 0; piece < 2; piece++)
#pragma unroll
            for (int w = 0; w < KW; w++, piece_no++) t.k[nt][piece][w] = p[piece_no * 32 + lane];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int w = 0; w < KW; w++, piece_no++) t.v[i][w] = p[piece_no * 32 + lane];
    if (a.k_scales) {
        const float2 sc = *reinterpret_cast<const float2*>(stage + Ring<FP8>::PIECES * 32 * 16 + lane * 8);
        t.ks = sc.x;
        t.vs = sc.y;
    } else {
        t.ks = t.vs = 1.0f;
    }
}

// One 16-token block of one kv head: scores, online softmax on this lane's row, O += P V.
template <bool FP8>
__device__ __forceinline__ void attend_block(const Tile<FP8>& cur, uint32_t n_valid, uint32_t j, const uint32_t (&qa)[8][2], float (&o)[16][4],
                                             float& m, float& l) {
    // scores[16 rows][16 tokens] = Q K^T, two n-tiles of 8 tokens
    float sc[2][4], sc_odd[2][4];                                  // even and odd k-steps accumulate apart: shorter chains
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.0f;
        sc_odd[nt][0] = sc_odd[nt][1] = sc_odd[nt][2] = sc_odd[nt][3] = 0.0f;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            uint32_t b0, b1;
            if (FP8) {
                const uint32_t w = word_of(cur.k[nt][s >> 2][0], s & 3);
                b0 = e4m3x2_to_h2(w & 0xFFFFu);
                b1 = e4m3x2_to_h2(w >> 16);
            } else {
                const int e = (s & 3) * 2;                       // f16 words 2e', 2e'+1 of the 32-byte piece
                b0 = word_of(cur.k[nt][s >> 2][e >> 2], e & 3);
                b1 = word_of(cur.k[nt][s >> 2][(e + 1) >> 2], (e + 1) & 3);
            }
            mma_16816((s & 1) ? sc_odd[nt] : sc[nt], qa[s][0], 0u, qa[s][1], 0u, b0, b1);
        }
        sc[nt][0] += sc_odd[nt][0];
        sc[nt][1] += sc_odd[nt][1];
    }
    // block scale, mask past the sequence end, online softmax on this lane's row
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t tok = 8 * nt + 2 * j + i;
            sc[nt][i] = tok < n_valid ? sc[nt][i] * cur.ks : -INFINITY;
            mx = fmaxf(mx, sc[nt][i]);
        }
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float corr = m == -INFINITY ? 0.0f : exp2f(m - m_new);
    float p[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int i = 0; i < 2; i++) p[nt][i] = exp2f(sc[nt][i] - m_new);     // exp2f(-inf) == 0
    l = l * corr + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
    m = m_new;
#pragma unroll
    for (int t = 0; t < 16; t++) {
        o[t][0] *= corr;
        o[t][1] *= corr;
    }
    // O += (P * v_scale) V : P as the A fragment (tokens 2j, 2j+1 | 2j+8, 2j+9), V bytes paired per dim
    const uint32_t pa0 = pack_h2(p[0][0] * cur.vs, p[0][1] * cur.vs), pa2 = pack_h2(p[1][0] * cur.vs, p[1][1] * cur.vs);
#pragma unroll
    for (int t = 0; t < 16; t++) {
        uint32_t b0, b1;
        if (FP8) {
            const uint32_t sel = (uint32_t)(t & 3) | ((4u + (uint32_t)(t & 3)) << 4);
            b0 = e4m3x2_to_h2(__byte_perm(word_of(cur.v[0][0], t >> 2), word_of(cur.v[1][0], t >> 2), sel));
            b1 = e4m3x2_to_h2(__byte_perm(word_of(cur.v[2][0], t >> 2), word_of(cur.v[3][0], t >> 2), sel));
        } else {
            const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;                 // halves t of two tokens -> one f16x2
            b0 = __byte_perm(word_of(cur.v[0][t >> 3], (t >> 1) & 3), word_of(cur.v[1][t >> 3], (t >> 1) & 3), sel);
            b1 = __byte_perm(word_of(cur.v[2][t >> 3], (t >> 1) & 3), word_of(cur.v[3][t >> 3], (t >> 1) & 3), sel);
        }
        mma_16816(o[t], pa0, 0u, pa2, 0u, b0, b1);
    }
}

template <bool FP8>
__global__ void __launch_bounds__(WARPS * 32) decode_attn_paged(const AttnArgs a) {
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const uint32_t kv_len = min(a.kv_lens[seq], a.max_kv_len);
    if (split == 0 && kvh == 0 && threadIdx.x == 0 && a.kv_lens[seq] > a.max_kv_len) report(a, 2u);
    const uint32_t t_begin = split * a.split_tokens;
    if (t_begin >= kv_len) return;
    const uint32_t t_end = min(kv_len, t_begin + a.split_tokens);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, grp = lane >> 2, j = lane & 3u;
    const uint32_t* table = a.tables + (size_t)seq * a.table_stride;

    // query fragments of this lane's row (query head kvh * group + grp), scaled and in the dim order the K pieces use
    uint32_t qa[8][2];
    {
        const bool live = grp < a.group;
        const float* qrow = a.q + ((size_t)seq * a.n_q_heads + kvh * a.group + (live ? grp : 0)) * D;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            const int base = (s < 4 ? 16 * (int)j + 4 * s : 64 + 16 * (int)j + 4 * (s - 4));
            float4 f = live ? *reinterpret_cast<const float4*>(qrow + base) : make_float4(0, 0, 0, 0);
            qa[s][0] = pack_h2(f.x * a.q_scale, f.y * a.q_scale);
            qa[s][1] = pack_h2(f.z * a.q_scale, f.w * a.q_scale);
        }
    }

    float o[16][4];
#pragma unroll
    for (int t = 0; t < 16; t++) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    const uint32_t b_begin = t_begin / BS, b_end = (t_end + BS - 1) / BS;
    extern __shared__ __align__(128) unsigned char ring[];
    constexpr int STAGES = Ring<FP8>::STAGES, STAGE_BYTES = Ring<FP8>::STAGE_BYTES;
    unsigned char* my_ring = ring + (size_t)warp * STAGES * STAGE_BYTES;
    const uint32_t my_ring_smem = (uint32_t)__cvta_generic_to_shared(my_ring);
    // this warp's blocks are b_begin + warp + WARPS * k; keep STAGES - 1 of them in flight
    const uint32_t n_mine = b_begin + warp < b_end ? (b_end - b_begin - warp + WARPS - 1) / WARPS : 0u;
    auto issue = [&](uint32_t k, uint32_t block_id) {
        if (k < n_mine) {
            const uint32_t bb = b_begin + warp + WARPS * k;
            issue_tile<FP8>(my_ring_smem + (k % STAGES) * STAGE_BYTES, a, block_id, kvh, grp, j, lane, min((uint32_t)BS, kv_len - bb * BS));
        }
        asm volatile("cp.async.commit_group;" ::: "memory");          // one group per k, empty past the end
    };
    auto table_entry = [&](uint32_t k) {
        const uint32_t id = k < n_mine ? __ldg(table + b_begin + warp + WARPS * k) : 0u;
        if (id >= a.total_blocks) {                                    // never dereferenced: block 0 is read instead and the launch reports it
            report(a, 2u);
            return 0u;
        }
        return id;
    };
    for (uint32_t k = 0; k + 1 < (uint32_t)STAGES; k++) issue(k, table_entry(k));
    uint32_t id_ahead = table_entry(STAGES - 1);                       // block ids are fetched one iteration before they are needed
    Tile<FP8> cur;
    for (uint32_t k = 0; k < n_mine; k++) {
        const uint32_t b = b_begin + warp + WARPS * k;
        const uint32_t id_now = id_ahead;
        id_ahead = table_entry(k + STAGES);
        issue(k + STAGES - 1, id_now);                                 // refills the stage read one iteration ago
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
        read_tile<FP8>(cur, my_ring + (k % STAGES) * STAGE_BYTES, a, lane);
        const uint32_t n_valid = min((uint32_t)BS, kv_len - b * BS);

        attend_block<FP8>(cur, n_valid, j, qa, o, m, l);
    }
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);

    // merge the warps' partials: [warp][row][D + 2] (m, l, then D values), laid over the ring once every warp has left it
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float(*sh)[8][D + 2] = reinterpret_cast<float(*)[8][D + 2]>(ring);
    if (j == 0) {
        sh[warp][grp][0] = m;
        sh[warp][grp][1] = l;
    }
#pragma unroll
    for (int t = 0; t < 16; t++) {
        sh[warp][grp][2 + 32 * j + t] = o[t][0];          // column 2j of n-tile t  <->  dim 16 * (2j) + t
        sh[warp][grp][2 + 32 * j + 16 + t] = o[t][1];     // column 2j + 1          <->  dim 16 * (2j + 1) + t
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < a.group * D; i += WARPS * 32) {
        const uint32_t g = i / D, d = i % D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) mm = fmaxf(mm, sh[w][g][0]);
        float ll = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            const float f = sh[w][g][0] == -INFINITY ? 0.0f : exp2f(sh[w][g][0] - mm);
            ll += sh[w][g][1] * f;
            acc += sh[w][g][2 + d] * f;
        }
        if (a.n_splits == 1) {
            a.out[((size_t)seq * a.n_q_heads + kvh * a.group + g) * D + d] = ll > 0.0f ? acc / ll : 0.0f;
        } else {
            float* pr = a.partial + ((((size_t)seq * a.n_kv_heads + kvh) * a.n_splits + split) * a.group + g) * (D + 2);
            if (d == 0) {
                pr[0] = mm;
                pr[1] = ll;
            }
            pr[2 + d] = acc;
        }
    }
}

// The same block, transposed: S^T = K Q^T with the 16 tokens as the M rows and the group's query heads
// as the 8 columns, then O^T += V^T P^T with head_dim as the M rows.  Every accumulator register is a
// live (dim, head) pair, half as many MMAs are issued, and the 8x8 transposes of the probabilities that
// turn an accumulator fragment into a B fragment are one movmatrix each.  State per lane: the two heads
// 2j and 2j + 1 (running max m2, partial sum l2) and o[t] = dims 16 * grp + 2t (+1) of those two heads.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

template <bool FP8>
__device__ __forceinline__ void attend_block_t(const Tile<FP8>& cur, uint32_t n_valid, uint32_t grp, const uint32_t (&qa)[8][2],
                                               float (&o)[8][4], float (&m2)[2], float (&l2)[2]) {
    float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sc_odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int s = 0; s < 8; s++) {
        uint32_t a0, a1, a2, a3;
        if (FP8) {
            const uint32_t w0 = word_of(cur.k[0][s >> 2][0], s & 3), w1 = word_of(cur.k[1][s >> 2][0], s & 3);
            a0 = e4m3x2_to_h2(w0 & 0xFFFFu);
            a2 = e4m3x2_to_h2(w0 >> 16);
            a1 = e4m3x2_to_h2(w1 & 0xFFFFu);
            a3 = e4m3x2_to_h2(w1 >> 16);
        } else {
            const int e = (s & 3) * 2;
            a0 = word_of(cur.k[0][s >> 2][e >> 2], e & 3);
            a2 = word_of(cur.k[0][s >> 2][(e + 1) >> 2], (e + 1) & 3);
            a1 = word_of(cur.k[1][s >> 2][e >> 2], e & 3);
            a3 = word_of(cur.k[1][s >> 2][(e + 1) >> 2], (e + 1) & 3);
        }
        mma_16816((s & 1) ? sc_odd : sc, a0, a1, a2, a3, qa[s][0], qa[s][1]);
    }
    // sc[0..1]: token grp, heads 2j, 2j+1; sc[2..3]: token grp + 8
    float p[4];
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float s_lo = grp < n_valid ? (sc[h] + sc_odd[h]) * cur.ks : -INFINITY;
        const float s_hi = grp + 8 < n_valid ? (sc[2 + h] + sc_odd[2 + h]) * cur.ks : -INFINITY;
        float mx = fmaxf(s_lo, s_hi);
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
        const float m_new = fmaxf(m2[h], mx);
        corr[h] = m2[h] == -INFINITY ? 0.0f : fast_exp2(m2[h] - m_new);
        p[h] = fast_exp2(s_lo - m_new);
        p[2 + h] = fast_exp2(s_hi - m_new);
        l2[h] = l2[h] * corr[h] + p[h] + p[2 + h];
        m2[h] = m_new;
    }
    // probabilities (times the V scale) as the B fragment: rows = tokens 2j, 2j+1 (+8), column = head grp
    const uint32_t b0 = movmatrix_trans(pack_h2(p[0] * cur.vs, p[1] * cur.vs));
    const uint32_t b1 = movmatrix_trans(pack_h2(p[2] * cur.vs, p[3] * cur.vs));
#pragma unroll
    for (int t = 0; t < 8; t++) {
        o[t][0] *= corr[0];
        o[t][1] *= corr[1];
        o[t][2] *= corr[0];
        o[t][3] *= corr[1];
        uint32_t a0, a1, a2, a3;
        if (FP8) {
            const uint32_t lo = 2u * (t & 1), sel0 = lo | ((4u + lo) << 4), sel1 = (lo + 1u) | ((5u + lo) << 4);
            const uint32_t v0 = word_of(cur.v[0][0], t >> 1), v1 = word_of(cur.v[1][0], t >> 1);
            const uint32_t v2 = word_of(cur.v[2][0], t >> 1), v3 = word_of(cur.v[3][0], t >> 1);
            a0 = e4m3x2_to_h2(__byte_perm(v0, v1, sel0));      // dim 16 grp + 2t,     tokens 2j, 2j+1
            a1 = e4m3x2_to_h2(__byte_perm(v0, v1, sel1));      // dim 16 grp + 2t + 1
            a2 = e4m3x2_to_h2(__byte_perm(v2, v3, sel0));      // tokens 2j+8, 2j+9
            a3 = e4m3x2_to_h2(__byte_perm(v2, v3, sel1));
        } else {
            const uint32_t v0 = word_of(cur.v[0][t >> 2], t & 3), v1 = word_of(cur.v[1][t >> 2], t & 3);
            const uint32_t v2 = word_of(cur.v[2][t >> 2], t & 3), v3 = word_of(cur.v[3][t >> 2], t & 3);
            a0 = __byte_perm(v0, v1, 0x5410u);
            a1 = __byte_perm(v0, v1, 0x7632u);
            a2 = __byte_perm(v2, v3, 0x5410u);
            a3 = __byte_perm(v2, v3, 0x7632u);
        }
        mma_16816(o[t], a0, a1, a2, a3, b0, b1);
    }
}

// Two blocks (32 tokens) in one step: twice the independent MMA chains per softmax, one max / rescale per 32 tokens.
// n_valid1 == 0 when the range ends on an odd block (the second tile is then all zeros and fully masked).
template <bool FP8>
__device__ __forceinline__ void kq_tile(const Tile<FP8>& t, const uint32_t (&qa)[8][2], float (&sc)[4]) {
    float odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    sc[0] = sc[1] = sc[2] = sc[3] = 0.0f;
#pragma unroll
    for (int s = 0; s < 8; s++) {
        uint32_t a0, a1, a2, a3;
        if (FP8) {
            const uint32_t w0 = word_of(t.k[0][s >> 2][0], s & 3), w1 = word_of(t.k[1][s >> 2][0], s & 3);
            a0 = e4m3x2_to_h2(w0 & 0xFFFFu);
            a2 = e4m3x2_to_h2(w0 >> 16);
            a1 = e4m3x2_to_h2(w1 & 0xFFFFu);
            a3 = e4m3x2_to_h2(w1 >> 16);
        } else {
            const int e = (s & 3) * 2;
            a0 = word_of(t.k[0][s >> 2][e >> 2], e & 3);
            a2 = word_of(t.k[0][s >> 2][(e + 1) >> 2], (e + 1) & 3);
            a1 = word_of(t.k[1][s >> 2][e >> 2], e & 3);
            a3 = word_of(t.k[1][s >> 2][(e + 1) >> 2], (e + 1) & 3);
        }
        mma_16816((s & 1) ? odd : sc, a0, a1, a2, a3, qa[s][0], qa[s][1]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) sc[i] += odd[i];
}

template <bool FP8>
__device__ __forceinline__ void pv_tile(const Tile<FP8>& cur, uint32_t b0, uint32_t b1, float (&o)[8][4]) {
#pragma unroll
    for (int t = 0; t < 8; t++) {
        uint32_t a0, a1, a2, a3;
        if (FP8) {
            const uint32_t lo = 2u * (t & 1), sel0 = lo | ((4u + lo) << 4), sel1 = (lo + 1u) | ((5u + lo) << 4);
            const uint32_t v0 = word_of(cur.v[0][0], t >> 1), v1 = word_of(cur.v[1][0], t >> 1);
            const uint32_t v2 = word_of(cur.v[2][0], t >> 1), v3 = word_of(cur.v[3][0], t >> 1);
            a0 = e4m3x2_to_h2(__byte_perm(v0, v1, sel0));
            a1 = e4m3x2_to_h2(__byte_perm(v0, v1, sel1));
            a2 = e4m3x2_to_h2(__byte_perm(v2, v3, sel0));
            a3 = e4m3x2_to_h2(__byte_perm(v2, v3, sel1));
        } else {
            const uint32_t v0 = word_of(cur.v[0][t >> 2], t & 3), v1 = word_of(cur.v[1][t >> 2], t & 3);
            const uint32_t v2 = word_of(cur.v[2][t >> 2], t & 3), v3 = word_of(cur.v[3][t >> 2], t & 3);
            a0 = __byte_perm(v0, v1, 0x5410u);
            a1 = __byte_perm(v0, v1, 0x7632u);
            a2 = __byte_perm(v2, v3, 0x5410u);
            a3 = __byte_perm(v2, v3, 0x7632u);
        }
        mma_16816(o[t], a0, a1, a2, a3, b0, b1);
    }
}

template <bool FP8>
__device__ __forceinline__ void attend_two_blocks_t(const Tile<FP8>& t0, const Tile<FP8>& t1, uint32_t n_valid0, uint32_t n_valid1, uint32_t grp,
                                                    const uint32_t (&qa)[8][2], float (&o)[8][4], float (&m2)[2], float (&l2)[2]) {
    float sc0[4], sc1[4];
    kq_tile<FP8>(t0, qa, sc0);
    kq_tile<FP8>(t1, qa, sc1);
    float p0[4], p1[4], corr[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const float s00 = grp < n_valid0 ? sc0[h] * t0.ks : -INFINITY, s01 = grp + 8 < n_valid0 ? sc0[2 + h] * t0.ks : -INFINITY;
        const float s10 = grp < n_valid1 ? sc1[h] * t1.ks : -INFINITY, s11 = grp + 8 < n_valid1 ? sc1[2 + h] * t1.ks : -INFINITY;
        float mx = fmaxf(fmaxf(s00, s01), fmaxf(s10, s11));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
        const float m_new = fmaxf(m2[h], mx);
        corr[h] = m2[h] == -INFINITY ? 0.0f : fast_exp2(m2[h] - m_new);
        p0[h] = fast_exp2(s00 - m_new);
        p0[2 + h] = fast_exp2(s01 - m_new);
        p1[h] = fast_exp2(s10 - m_new);
        p1[2 + h] = fast_exp2(s11 - m_new);
        l2[h] = l2[h] * corr[h] + (p0[h] + p0[2 + h]) + (p1[h] + p1[2 + h]);
        m2[h] = m_new;
    }
    const uint32_t b00 = movmatrix_trans(pack_h2(p0[0] * t0.vs, p0[1] * t0.vs)), b01 = movmatrix_trans(pack_h2(p0[2] * t0.vs, p0[3] * t0.vs));
    const uint32_t b10 = movmatrix_trans(pack_h2(p1[0] * t1.vs, p1[1] * t1.vs)), b11 = movmatrix_trans(pack_h2(p1[2] * t1.vs, p1[3] * t1.vs));
    if (__any_sync(0xFFFFFFFFu, corr[0] != 1.0f || corr[1] != 1.0f)) {   // exactly 1 once the running maxima have settled
#pragma unroll
        for (int t = 0; t < 8; t++) {
            o[t][0] *= corr[0];
            o[t][1] *= corr[1];
            o[t][2] *= corr[0];
            o[t][3] *= corr[1];
        }
    }
    pv_tile<FP8>(t0, b00, b01, o);
    pv_tile<FP8>(t1, b10, b11, o);
}

// ---------------------------------------------------------------------------------------------
// Whole-block form (at most 8 kv heads): a CTA owns a token range of one sequence for ALL kv
// heads, so what it reads is whole 16-token blocks, each one contiguous run per K and per V.  A
// producer warp keeps a ring of blocks in flight with the bulk async-copy engine (cp.async.bulk
// completing on an mbarrier, as the handoff's staged kernel does); consumer warp h computes kv
// head h out of shared memory and hands the stage back through a second mbarrier as soon as
// its fragments are in registers.  No warp merges with another: each writes its own partial.
// Every wait is bounded; a CTA that gives up reports through `status` and drains its copies.
// ---------------------------------------------------------------------------------------------
constexpr int MAX_KV_HEADS_PER_CTA = 8;   // consumer warps, one per kv head (two per head, on alternate blocks, measured no faster)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A stage is handed back to the producer as soon as its fragments are in registers, so these loads must
// never be re-issued later by the compiler (a reload in place of a spill would read the refilled stage).
__device__ __forceinline__ uint4 lds_once(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr(p)) : "memory");
    return v;
}
__device__ __forceinline__ float lds_once_f32(const void* p) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(smem_addr(p)) : "memory");
    return v;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 22); it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// the same wait, given up early once another warp of the CTA has recorded a failure
__device__ __forceinline__ bool mbar_wait_unless(uint32_t bar, uint32_t parity, const uint32_t* fail_word) {
    for (uint32_t it = 0; it < (1u << 22); it++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 15u) == 15u && *reinterpret_cast<const volatile uint32_t*>(fail_word)) return false;
    }
    return false;
}

template <bool FP8>
__global__ void __launch_bounds__((MAX_KV_HEADS_PER_CTA + 1) * 32, 1)
decode_attn_blocks(const AttnArgs a, uint32_t n_stages, uint32_t stage_bytes) {
    constexpr int CW = MAX_KV_HEADS_PER_CTA;
    constexpr int ES = FP8 ? 1 : 2;
    constexpr int KW = Tile<FP8>::KW;
    const uint32_t split = blockIdx.x, seq = blockIdx.y;
    const uint32_t kv_len = min(a.kv_lens[seq], a.max_kv_len);
    const uint32_t t_begin = split * a.split_tokens;
    if (t_begin >= kv_len) return;
    const uint32_t t_end = min(kv_len, t_begin + a.split_tokens);
    const uint32_t b_begin = t_begin / BS, n_blk = (t_end + BS - 1) / BS - b_begin;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, grp = lane >> 2, j = lane & 3u;
    const uint32_t* table = a.tables + (size_t)seq * a.table_stride + b_begin;
    const uint32_t block_bytes = BS * a.row_stride;

    extern __shared__ __align__(128) unsigned char ring[];
    uint64_t* full = reinterpret_cast<uint64_t*>(ring);            // [8]
    uint64_t* empty = full + 8;                                    // [8]
    uint32_t* fail_word = reinterpret_cast<uint32_t*>(ring + 128);
    unsigned char* stages = ring + 256;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < n_stages; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(full + s)));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(empty + s)), "r"(a.n_kv_heads));   // one arrival per head
        }
        *fail_word = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CW) {
        // ---- producer: lane 0 drives the ring; the warp reads the block table 32 entries at a time (one
        // coalesced load, the next one already in flight), so no copy waits for a table entry of its own ----
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
                    if (id >= a.total_blocks) {                      // a stale or foreign id is never turned into an address
                        ok = false;
                        why = 2u;
                    }
                    if (ok && k >= n_stages) ok = mbar_wait(smem_addr(empty + s), ((k / n_stages) - 1u) & 1u);   // every head has read the old block
                    if (ok) {
                        const uint32_t n_valid = min((uint32_t)BS, kv_len - (b_begin + k) * BS);
                        const uint32_t bytes = n_valid * a.row_stride, sc_bytes = a.k_scales ? a.n_kv_heads * 4u : 0u;
                        const uint32_t bar = smem_addr(full + s), dst = smem_addr(stages + (size_t)s * stage_bytes);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * bytes + 2u * sc_bytes) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst), "l"(a.k_base + (uint64_t)id * a.block_stride), "r"(bytes), "r"(bar) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dst + block_bytes), "l"(a.v_base + (uint64_t)id * a.block_stride), "r"(bytes), "r"(bar) : "memory");
                        if (sc_bytes) {
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(dst + 2u * block_bytes), "l"(a.k_scales + (size_t)id * a.n_kv_heads), "r"(sc_bytes), "r"(bar) : "memory");
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(dst + 2u * block_bytes + 32u), "l"(a.v_scales + (size_t)id * a.n_kv_heads), "r"(sc_bytes), "r"(bar) : "memory");
                        }
                        issued = k + 1;
                    }
                }
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0u;
            }
        }
        if (!ok && lane == 0) {
            atomicExch(fail_word, why);
            // give the copies still in flight a bounded chance to land before the CTA's shared memory is released
            for (uint32_t k = issued > n_stages ? issued - n_stages : 0u; k < issued; k++)
                mbar_wait(smem_addr(full + k % n_stages), (k / n_stages) & 1u);
            report(a, why);
        }
    } else if (warp < a.n_kv_heads) {
        // ---- consumer: kv head `warp`, every block of this CTA's range ----
        const uint32_t kvh = warp;
        uint32_t qa[8][2];
        {
            const bool live = grp < a.group;
            const float* qrow = a.q + ((size_t)seq * a.n_q_heads + kvh * a.group + (live ? grp : 0)) * D;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const int base = (s < 4 ? 16 * (int)j + 4 * s : 64 + 16 * (int)j + 4 * (s - 4));
                float4 f = live ? *reinterpret_cast<const float4*>(qrow + base) : make_float4(0, 0, 0, 0);
                qa[s][0] = pack_h2(f.x * a.q_scale, f.y * a.q_scale);
                qa[s][1] = pack_h2(f.z * a.q_scale, f.w * a.q_scale);
            }
        }
        float o[8][4];
#pragma unroll
        for (int t = 0; t < 8; t++) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
        float m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.0f, 0.0f};
        // fragments of block k out of its ring stage, which goes back to the producer as soon as they are in registers
        auto fetch = [&](uint32_t k, Tile<FP8>& t, uint32_t n_valid) -> bool {
            const uint32_t s = k % n_stages;
            if (!mbar_wait_unless(smem_addr(full + s), (k / n_stages) & 1u, fail_word) || *reinterpret_cast<volatile uint32_t*>(fail_word)) return false;
            const unsigned char* kb = stages + (size_t)s * stage_bytes + (size_t)kvh * D * ES;
            const unsigned char* vb = kb + block_bytes;
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const unsigned char* row = kb + (size_t)(grp + 8 * nt) * a.row_stride;
#pragma unroll
                for (int piece = 0; piece < 2; piece++)
#pragma unroll
                    for (int w = 0; w < KW; w++) t.k[nt][piece][w] = lds_once(row + (piece * 64 + 16 * j) * ES + 16 * w);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t tok = 2 * j + (i & 1) + 8 * (i >> 1);
                const unsigned char* row = vb + (size_t)tok * a.row_stride + 16 * grp * ES;
#pragma unroll
                for (int w = 0; w < KW; w++) t.v[i][w] = lds_once(row + 16 * w);
            }
            if (n_valid < (uint32_t)BS) {                            // rows the copy did not bring hold stale bytes: read them as zero
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int w = 0; w < KW; w++)
                        if (2 * j + (i & 1) + 8 * (i >> 1) >= n_valid) t.v[i][w] = make_uint4(0, 0, 0, 0);
            }
            if (a.k_scales) {
                const float* sc = reinterpret_cast<const float*>(stages + (size_t)s * stage_bytes + 2u * block_bytes);
                t.ks = lds_once_f32(sc + kvh);
                t.vs = lds_once_f32(sc + 8 + kvh);
            } else {
                t.ks = t.vs = 1.0f;
            }
            // The stage goes back only once every fragment load of this warp has returned: the arrive takes a value
            // folded from all of them as an (unused) operand, so it cannot issue while a load is still in flight.
            uint32_t landed = __float_as_uint(t.ks) ^ __float_as_uint(t.vs);
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int piece = 0; piece < 2; piece++)
#pragma unroll
                    for (int w = 0; w < KW; w++) landed ^= t.k[nt][piece][w].x ^ t.k[nt][piece][w].w;
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int w = 0; w < KW; w++) landed ^= t.v[i][w].x ^ t.v[i][w].w;
            __syncwarp();
            if (lane == 0)
                asm volatile("{\n\t.reg .b32 dep;\n\tmov.b32 dep, %1;\n\tmbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
                             ::"r"(smem_addr(empty + s)), "r"(landed) : "memory");
            return true;
        };
        bool ok = true;
        if (FP8) {
            Tile<FP8> t0, t1;
            for (uint32_t k = 0; k < n_blk && ok; k += 2) {           // two blocks (32 tokens) per step
                const uint32_t n_valid0 = min((uint32_t)BS, kv_len - (b_begin + k) * BS);
                const uint32_t n_valid1 = k + 1 < n_blk ? min((uint32_t)BS, kv_len - (b_begin + k + 1) * BS) : 0u;
                ok = fetch(k, t0, n_valid0);
                if (ok && n_valid1) {
                    ok = fetch(k + 1, t1, n_valid1);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++)
#pragma unroll
                        for (int w = 0; w < KW; w++) t1.v[i][w] = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int nt = 0; nt < 2; nt++)
#pragma unroll
                        for (int piece = 0; piece < 2; piece++)
#pragma unroll
                            for (int w = 0; w < KW; w++) t1.k[nt][piece][w] = make_uint4(0, 0, 0, 0);
                    t1.ks = t1.vs = 1.0f;
                }
                if (ok) attend_two_blocks_t<FP8>(t0, t1, n_valid0, n_valid1, grp, qa, o, m2, l2);
            }
        } else {
            Tile<FP8> cur;                                            // F16 fragments are twice the registers: one block per step
            for (uint32_t k = 0; k < n_blk && ok; k++) {
                const uint32_t n_valid = min((uint32_t)BS, kv_len - (b_begin + k) * BS);
                ok = fetch(k, cur, n_valid);
                if (ok) attend_block_t<FP8>(cur, n_valid, grp, qa, o, m2, l2);
            }
        }
        if (ok) {
            // partial of (kv head, split): this lane holds heads 2j, 2j+1, dims [16 grp, 16 grp + 16)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                l2[h] += __shfl_xor_sync(0xFFFFFFFFu, l2[h], 4);
                l2[h] += __shfl_xor_sync(0xFFFFFFFFu, l2[h], 8);
                l2[h] += __shfl_xor_sync(0xFFFFFFFFu, l2[h], 16);
                const uint32_t g = 2 * j + h;
                if (g < a.group) {
                    float* pr = a.partial + ((((size_t)seq * a.n_kv_heads + kvh) * a.n_splits + split) * a.group + g) * (D + 2);
                    if (grp == 0) {
                        pr[0] = m2[h];
                        pr[1] = l2[h];
                    }
#pragma unroll
                    for (int t = 0; t < 8; t++)          // a partial row is 8-byte aligned (130 floats per row, 2 ahead of the dims)
                        *reinterpret_cast<float2*>(pr + 2 + 16 * grp + 2 * t) = make_float2(o[t][h], o[t][2 + h]);
                }
            }
        } else if (lane == 0) {
            const uint32_t why = *reinterpret_cast<volatile uint32_t*>(fail_word);
            report(a, why ? why : 4u);
        }
    }
}

// merges the splits of one (sequence, query head): sixteen splits per round, every load of a round issued before any
// is used (one memory round trip for up to sixteen splits), the running maximum carried from round to round
__global__ void __launch_bounds__(D) decode_attn_combine(const AttnArgs a) {
    const uint32_t head = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    const uint32_t kvh = head / a.group, g = head % a.group;
    const uint32_t kv_len = min(a.kv_lens[seq], a.max_kv_len);
    if (head == 0 && d == 0 && a.kv_lens[seq] > a.max_kv_len) report(a, 2u);   // the tokens past max_kv_len were not attended to
    const uint32_t live = ((kv_len + a.split_tokens - 1) / a.split_tokens) * a.parts_per_split;
    const float* base = a.partial + (((size_t)seq * a.n_kv_heads + kvh) * a.n_splits * a.group + g) * (D + 2);
    const size_t stride = (size_t)a.group * (D + 2);
    constexpr int R = 16;
    float mm = -INFINITY, ll = 0.0f, acc = 0.0f;
    for (uint32_t s0 = 0; s0 < live; s0 += R) {
        float pm[R], pl[R], pa[R];
#pragma unroll
        for (int i = 0; i < R; i++) {
            const bool in = s0 + i < live;
            const float* p = base + (size_t)(in ? s0 + i : 0) * stride;
            pm[i] = in ? __ldg(p) : -INFINITY;       // a part that saw no block also reports -inf
            pl[i] = __ldg(p + 1);
            pa[i] = __ldg(p + 2 + d);
        }
        float m_new = mm;
#pragma unroll
        for (int i = 0; i < R; i++) m_new = fmaxf(m_new, pm[i]);
        if (m_new == -INFINITY) continue;
        const float keep = mm == -INFINITY ? 0.0f : fast_exp2(mm - m_new);
        ll *= keep;
        acc *= keep;
#pragma unroll
        for (int i = 0; i < R; i++) {
            const float f = fast_exp2(pm[i] - m_new);     // 2^-inf = 0
            ll += pl[i] * f;
            acc += pa[i] * f;
        }
        mm = m_new;
    }
    a.out[((size_t)seq * a.n_q_heads + head) * D + d] = ll > 0.0f ? acc / ll : 0.0f;
}

int32_t fail(int32_t code, const char* fmt, unsigned long long x = 0, unsigned long long y = 0) {
    char buf[256];
    snprintf(buf, sizeof buf, fmt, x, y);
    return tkv_internal::set_error(code, 0, buf);
}

uint32_t splits_for(uint32_t max_kv_len, uint32_t split_tokens) { return std::max(1u, (max_kv_len + split_tokens - 1) / split_tokens); }

}  // namespace

extern "C" {

uint64_t tkv_decode_attn_scratch_bytes(uint32_t n_seqs, uint32_t n_q_heads, uint32_t head_dim, uint32_t max_kv_len,
                                       uint32_t split_tokens) {
    // sized for the smallest token range the library may choose (64) unless the caller fixes one; one partial result per range and
    // softmax group of the tcgen05 kernel
    if (split_tokens == 0) split_tokens = 64;
    return (uint64_t)tkv_tc::PARTS_PER_RANGE * n_seqs * n_q_heads * splits_for(max_kv_len, split_tokens) * (head_dim + 2) * sizeof(float);
}

int32_t tkv_selfcheck_tensor_cores(uint64_t mismatches[4]) {
    if (!mismatches) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    const cudaError_t e = tkv_tc::selfcheck(mismatches);
    if (e != cudaSuccess) {
        char buf[256];
        snprintf(buf, sizeof buf, "tensor-core self-check: %s (cuda error %d)", cudaGetErrorString(e), (int)e);
        return tkv_internal::set_error(TKV_ERR_CUDA, (int32_t)e, buf);
    }
    return TKV_OK;
}

int32_t tkv_decode_attn_enqueue(const TkvPool* pool, const TkvDecodeAttn* d, void* stream) {
    if (!pool || !d) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (pool->dtype != TKV_DTYPE_F16 && pool->dtype != TKV_DTYPE_E4M3)
        return fail(TKV_ERR_INVALID_CONFIG, "decode attention reads F16 or E4M3 pools (dtype %llu)", (unsigned long long)pool->dtype);
    if (pool->head_dim != D || pool->block_size != BS)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (decode attention is built for head_dim 128, 16-token blocks)",
                    (unsigned long long)D, (unsigned long long)pool->head_dim);
    if (d->layer >= pool->n_layers) return fail(TKV_ERR_INVALID_CONFIG, "layer %llu outside the pool (%llu layers)", d->layer, pool->n_layers);
    if (!pool->n_kv_heads || !d->n_q_heads || d->n_q_heads % pool->n_kv_heads || d->n_q_heads / pool->n_kv_heads > 8)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (query heads must be 1..8 times the kv heads)",
                    (unsigned long long)pool->n_kv_heads, (unsigned long long)d->n_q_heads);
    if ((pool->k_scales == 0) != (pool->v_scales == 0)) return fail(TKV_ERR_INVALID_CONFIG, "k_scales and v_scales must both be set or both be 0");
    if (pool->k_scales && pool->dtype != TKV_DTYPE_E4M3) return fail(TKV_ERR_INVALID_CONFIG, "only an E4M3 pool carries scales");
    if (d->n_seqs == 0) return TKV_OK;
    if (!d->q || !d->out || !d->tables || !d->kv_lens || !pool->k_layer_ptrs || !pool->v_layer_ptrs)
        return fail(TKV_ERR_INVALID_CONFIG, "NULL buffer");
    if ((d->max_kv_len + BS - 1) / BS > d->table_stride)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (table_stride below the blocks of max_kv_len)",
                    (unsigned long long)((d->max_kv_len + BS - 1) / BS), (unsigned long long)d->table_stride);
    const uint32_t es = pool->dtype == TKV_DTYPE_E4M3 ? 1u : 2u;
    const uint64_t kp = pool->k_layer_ptrs[d->layer], vp = pool->v_layer_ptrs[d->layer];
    if ((kp | vp | d->q | d->scratch) % 16) return fail(TKV_ERR_INVALID_CONFIG, "layer tensors, q and scratch must be 16-byte aligned");
    // the scale rows of a block are bulk-copy sources too
    if (pool->k_scales && ((pool->k_scales | pool->v_scales) % 16 || ((uint64_t)pool->total_blocks * pool->n_kv_heads * 4u) % 16))
        return fail(TKV_ERR_INVALID_CONFIG, "scale arrays (and each layer's slice of them) must be 16-byte aligned");
    // whole-block form when a CTA can hold every kv head of a block (and the scale rows are bulk-copy sized)
    const uint32_t row_bytes = pool->n_kv_heads * D * es, stage_bytes = 2u * BS * row_bytes + 128u;
    const bool whole_blocks = pool->n_kv_heads <= (uint32_t)MAX_KV_HEADS_PER_CTA && (!pool->k_scales || pool->n_kv_heads % 4 == 0) &&
                              !(d->flags & TKV_ATTN_PER_HEAD_CTAS) && 256u + 2u * stage_bytes <= 200u * 1024u;
    uint32_t split_tokens = d->split_tokens ? d->split_tokens : DEFAULT_SPLIT_TOKENS;
    if (!d->split_tokens && d->total_kv_tokens) {
        // Two candidates, the cheaper by a simple makespan estimate (in tokens of work per SM, a CTA's start-up counted as
        // START tokens, the ragged end of the last wave as TAIL ranges): ONE wave of CTAs (sum over sequences of ceil(len / split) <= total / split + n_seqs <= SM count),
        // good while the sequences are few; or several waves of short ranges, whose tail is one short CTA instead of the
        // slack of n_seqs reserved slots, better when the batch has many sequences.
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, pool->device) == cudaSuccess && sms > 0) {
            const uint64_t step = whole_blocks ? 2u * BS : WARPS * BS;    // a range is walked two blocks (per-head form: four warps' blocks) at a time
            // START and TAIL are fitted to measurements on B200 (64 and 128 prompts of 512-4096 tokens, ranges of 128-416 tokens)
            const double START = 96.0, TAIL = 0.7, total = (double)d->total_kv_tokens, per_sm = total / sms;
            auto round_up = [&](double x) { return std::min<uint64_t>(std::max<uint64_t>(((uint64_t)x + step - 1) / step * step, 64), 1u << 20); };
            const uint64_t many = std::max<uint64_t>(round_up(std::sqrt(per_sm * START / TAIL)), 128);
            const double t_many = per_sm * (1.0 + START / (double)many) + TAIL * (double)many;
            uint64_t pick = many;
            if (sms > (int)d->n_seqs) {
                const uint64_t one = round_up(total / (sms - (int)d->n_seqs) + 0.999);
                if ((double)one + START <= t_many) pick = one;
            }
            split_tokens = (uint32_t)pick;
        }
    }
    if (split_tokens % (whole_blocks ? 2u * BS : WARPS * BS))
        return fail(TKV_ERR_INVALID_CONFIG, "split_tokens must be a multiple of %llu", (unsigned long long)(whole_blocks ? 2u * BS : WARPS * BS));
    const uint32_t n_splits = splits_for(d->max_kv_len, split_tokens);
    const uint64_t need = tkv_decode_attn_scratch_bytes(d->n_seqs, d->n_q_heads, D, d->max_kv_len, split_tokens);
    if (need > d->scratch_bytes || (need && !d->scratch))
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (scratch bytes)", need, d->scratch_bytes);

    AttnArgs a{};
    a.k_base = reinterpret_cast<const char*>(kp);
    a.v_base = reinterpret_cast<const char*>(vp);
    const size_t layer_scales = (size_t)d->layer * pool->total_blocks * pool->n_kv_heads;
    a.k_scales = pool->k_scales ? reinterpret_cast<const float*>(pool->k_scales) + layer_scales : nullptr;
    a.v_scales = pool->v_scales ? reinterpret_cast<const float*>(pool->v_scales) + layer_scales : nullptr;
    a.q = reinterpret_cast<const float*>(d->q);
    a.out = reinterpret_cast<float*>(d->out);
    a.tables = reinterpret_cast<const uint32_t*>(d->tables);
    a.kv_lens = reinterpret_cast<const uint32_t*>(d->kv_lens);
    a.partial = reinterpret_cast<float*>(d->scratch);
    a.row_stride = pool->n_kv_heads * D * es;
    a.block_stride = (uint64_t)BS * a.row_stride;
    a.n_q_heads = d->n_q_heads;
    a.n_kv_heads = pool->n_kv_heads;
    a.group = d->n_q_heads / pool->n_kv_heads;
    a.table_stride = d->table_stride;
    a.n_splits = n_splits;
    a.parts_per_split = 1;
    a.split_tokens = split_tokens;
    a.q_scale = d->sm_scale * 1.4426950408889634f;
    a.max_kv_len = d->max_kv_len;
    a.total_blocks = pool->total_blocks;
    a.status = reinterpret_cast<uint32_t*>(d->status);

    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != pool->device) e = cudaSetDevice(pool->device);
    if (e == cudaSuccess) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        dim3 grid(n_splits, pool->n_kv_heads, d->n_seqs);
        const bool tensor_memory = whole_blocks && !(d->flags & TKV_ATTN_MMA_SYNC) &&
                                   tkv_tc::eligible(pool->n_kv_heads, a.group, pool->k_scales != 0, pool->total_blocks);
        if (tensor_memory) {
            // the tcgen05 kernel: K and V tiles straight from shared memory into the tensor cores, accumulators in tensor memory
            tkv_tc::Args t{};
            t.k_scales = a.k_scales;
            t.v_scales = a.v_scales;
            t.q = a.q;
            t.tables = a.tables;
            t.kv_lens = a.kv_lens;
            t.partial = a.partial;
            t.n_seqs = d->n_seqs;
            t.n_q_heads = a.n_q_heads;
            t.table_stride = a.table_stride;
            t.n_splits = n_splits;
            t.split_tokens = split_tokens;
            t.max_kv_len = a.max_kv_len;
            t.total_blocks = a.total_blocks;
            t.q_scale = a.q_scale;
            t.status = a.status;
            e = tkv_tc::launch(pool->dtype == TKV_DTYPE_E4M3, a.group, kp, vp, t, st);
            a.n_splits = tkv_tc::PARTS_PER_RANGE * n_splits;   // partial slots per (sequence, kv head): one per token range and softmax group
            a.parts_per_split = tkv_tc::PARTS_PER_RANGE;
            if (e == cudaSuccess) {
                decode_attn_combine<<<dim3(d->n_q_heads, d->n_seqs), D, 0, st>>>(a);
                e = cudaGetLastError();
            }
        } else if (whole_blocks) {
            const uint32_t n_stages = std::min<uint32_t>(6u, (200u * 1024u - 256u) / stage_bytes);
            const size_t smem = 256 + (size_t)n_stages * stage_bytes;
            dim3 grid2(n_splits, d->n_seqs);
            a.parts_per_split = 1;
            a.n_splits = n_splits;
            const uint32_t threads = (MAX_KV_HEADS_PER_CTA + 1) * 32;
            if (pool->dtype == TKV_DTYPE_E4M3) {
                e = cudaFuncSetAttribute(decode_attn_blocks<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e == cudaSuccess) decode_attn_blocks<true><<<grid2, threads, smem, st>>>(a, n_stages, stage_bytes);
            } else {
                e = cudaFuncSetAttribute(decode_attn_blocks<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e == cudaSuccess) decode_attn_blocks<false><<<grid2, threads, smem, st>>>(a, n_stages, stage_bytes);
            }
            if (e == cudaSuccess) e = cudaGetLastError();
            if (e == cudaSuccess) {
                decode_attn_combine<<<dim3(d->n_q_heads, d->n_seqs), D, 0, st>>>(a);
                e = cudaGetLastError();
            }
        } else {
        constexpr size_t smem8 = (size_t)WARPS * Ring<true>::STAGES * Ring<true>::STAGE_BYTES;
        constexpr size_t smem16 = (size_t)WARPS * Ring<false>::STAGES * Ring<false>::STAGE_BYTES;
        static_assert(smem8 >= sizeof(float) * WARPS * 8 * (D + 2) && smem16 >= sizeof(float) * WARPS * 8 * (D + 2), "merge buffer fits the ring");
        if (pool->dtype == TKV_DTYPE_E4M3) {
            e = cudaFuncSetAttribute(decode_attn_paged<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem8);
            if (e == cudaSuccess) decode_attn_paged<true><<<grid, WARPS * 32, smem8, st>>>(a);
        } else {
            e = cudaFuncSetAttribute(decode_attn_paged<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem16);
            if (e == cudaSuccess) decode_attn_paged<false><<<grid, WARPS * 32, smem16, st>>>(a);
        }
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e == cudaSuccess && n_splits > 1) {
            decode_attn_combine<<<dim3(d->n_q_heads, d->n_seqs), D, 0, st>>>(a);
            e = cudaGetLastError();
        }
        }
    }
    if (prev >= 0 && prev != pool->device) cudaSetDevice(prev);
    if (e != cudaSuccess) {
        char buf[256];
        snprintf(buf, sizeof buf, "decode attention launch: %s (cuda error %d)", cudaGetErrorString(e), (int)e);
        return tkv_internal::set_error(TKV_ERR_CUDA, (int32_t)e, buf);
    }
    return TKV_OK;
}

}  // extern "C"
