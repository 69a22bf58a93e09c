// Device code of the KV handoff for sm_100a.
//
// Unit of work ("chunk"): one (block pair, layer, K|V).  At source and at
// destination a chunk is `n_valid` token rows of `row_bytes`, `row_stride`
// apart; when a pair moves every kv head of both pools the rows abut and the
// chunk is one contiguous run (32 KiB for 16 tokens x 8 heads x 128 dims of F16).
// The work list holds one uint4 {src_block, dst_block, n_valid, 0} per block
// pair; chunk index w decodes as kv = w & 1, layer = (w >> 1) % L,
// pair = (w >> 1) / L, so neighbouring CTAs stream K and V of one block.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tkv {

struct HandoffArgs {
    const uint4* work;
    const uint64_t* src_k;  // [n_layers] device addresses, shard-relative
    const uint64_t* src_v;
    const uint64_t* dst_k;
    const uint64_t* dst_v;
    float* dst_k_scales;    // [pool layers][total_blocks][pool heads] or null
    float* dst_v_scales;
    const float* src_k_scales;  // same layout on the source side; set only when a same-dtype
    const float* src_v_scales;  // E4M3 move carries its per-block scales along
    uint32_t* done_counter; // in plan memory on the launching device
    uint32_t* done_flag;    // anywhere reachable (peer ok) or null
    uint64_t src_block_stride;  // bytes
    uint64_t dst_block_stride;
    uint32_t n_pairs;           // block pairs per layer
    uint32_t work_layer_stride; // 0 = one list for all layers
    uint32_t n_layers;
    uint32_t n_heads;
    uint32_t head_dim;
    uint32_t block_size;
    uint32_t src_row_bytes, dst_row_bytes;   // bytes moved per token row
    uint32_t src_row_stride, dst_row_stride; // bytes between token rows
    uint32_t src_head_off, dst_head_off;     // byte offset of the first moved head in a row
    uint32_t dst_total_blocks, dst_pool_heads, dst_head_begin, dst_layer_begin;
    uint32_t src_total_blocks, src_pool_heads, src_head_begin, src_layer_begin;
    uint32_t flag_value;
    uint32_t contiguous;        // rows abut on both sides
    const uint32_t* n_pairs_dev; // set = the work list was built on the device: its length is read here (n_pairs is the capacity)
    uint32_t local_fences;      // 1 = both pools are this GPU's memory: CTAs count themselves with a GPU-scope release, only the last one fences at system scope
};

// Block pairs the launch really has: the host's count, or the device-built list's (never above the capacity).
__device__ __forceinline__ uint32_t live_pairs(const HandoffArgs& a) {
    return a.n_pairs_dev ? min(*reinterpret_cast<const volatile uint32_t*>(a.n_pairs_dev), a.n_pairs) : a.n_pairs;
}

struct Chunk {
    const char* src;
    char* dst;
    uint32_t n_valid, layer, is_v, dst_block, src_block;
};

__device__ __forceinline__ Chunk decode_chunk(const HandoffArgs& a, uint32_t w) {
    Chunk c;
    c.is_v = w & 1u;
    uint32_t q = w >> 1;
    c.layer = q % a.n_layers;
    uint32_t pair = q / a.n_layers;
    uint4 t = __ldg(a.work + (size_t)c.layer * a.work_layer_stride + pair);
    uint64_t sb = c.is_v ? a.src_v[c.layer] : a.src_k[c.layer];
    uint64_t db = c.is_v ? a.dst_v[c.layer] : a.dst_k[c.layer];
    c.src = reinterpret_cast<const char*>(sb + (uint64_t)t.x * a.src_block_stride + a.src_head_off);
    c.dst = reinterpret_cast<char*>(db + (uint64_t)t.y * a.dst_block_stride + a.dst_head_off);
    c.n_valid = t.z;
    c.dst_block = t.y;
    c.src_block = t.x;
    return c;
}

// A short work list carried in the kernel's parameter block: the pairs and the four layer-pointer arrays sit in the
// constant bank the launch fills, so a small handoff starts its first payload load without a dependent fetch of the
// list from device memory (and the host uploads nothing).
constexpr uint32_t INLINE_PAIRS = 256, INLINE_LAYERS = 64;
struct InlineList {
    uint4 pairs[INLINE_PAIRS];
    uint64_t ptr[4][INLINE_LAYERS];   // src K, src V, dst K, dst V
};

__device__ __forceinline__ Chunk decode_chunk_inline(const HandoffArgs& a, const InlineList& il, uint32_t w) {
    Chunk c;
    c.is_v = w & 1u;
    uint32_t q = w >> 1;
    c.layer = q % a.n_layers;
    uint4 t = il.pairs[q / a.n_layers];
    uint64_t sb = il.ptr[c.is_v][c.layer];
    uint64_t db = il.ptr[2u + c.is_v][c.layer];
    c.src = reinterpret_cast<const char*>(sb + (uint64_t)t.x * a.src_block_stride + a.src_head_off);
    c.dst = reinterpret_cast<char*>(db + (uint64_t)t.y * a.dst_block_stride + a.dst_head_off);
    c.n_valid = t.z;
    c.dst_block = t.y;
    c.src_block = t.x;
    return c;
}

// Last CTA to finish publishes the completion flag.  Every CTA fences its
// payload stores to system scope before counting itself, so a reader that
// acquires the flag (host, peer GPU) sees all of them.
__device__ __forceinline__ void signal_done(const HandoffArgs& a) {
    if (a.done_flag == nullptr) return;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t prev;
        if (a.local_fences) {
            // The payload went to this GPU's own memory: a release at GPU scope orders it before the count, the last
            // CTA's acquire of the count and its system-scope release below carry it on to the flag's reader.
            asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(a.done_counter) : "memory");
        } else {
            __threadfence_system();
            prev = atomicAdd(a.done_counter, 1u);
        }
        if (prev == gridDim.x - 1) {
            *a.done_counter = 0;  // ready for the next enqueue (stream order)
            __threadfence_system();
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.done_flag), "r"(a.flag_value) : "memory");
        }
    }
}

// ---- streaming loads / stores of a given width ---------------------------------
template <int BYTES> struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<2> { using type = uint16_t; };
template <> struct VecT<1> { using type = uint8_t; };

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename T> __device__ __forceinline__ T ld_stream(const T* p) { return __ldg(p); }

// ---------------------------------------------------------------------------------
// Same-dtype handoff, register path: 16-byte (or narrower) loads, UNROLL in
// flight per thread, then the stores.  Also the peer-store path: the stores go
// wherever the destination pointers point.
// ---------------------------------------------------------------------------------
template <int VEC, int UNROLL>
__global__ void __launch_bounds__(256) handoff_copy_vec(const HandoffArgs a) {
    using V = typename VecT<VEC>::type;
    const uint32_t total = live_pairs(a) * a.n_layers * 2u;
    const uint32_t vec_per_row = a.src_row_bytes / VEC;
    for (uint32_t w = blockIdx.x; w < total; w += gridDim.x) {
        const Chunk c = decode_chunk(a, w);
        const uint32_t nvec = c.n_valid * vec_per_row;
        if (a.contiguous) {
            const V* s = reinterpret_cast<const V*>(c.src);
            V* d = reinterpret_cast<V*>(c.dst);
            for (uint32_t base = 0; base < nvec; base += 256u * UNROLL) {
                V v[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) v[u] = ld_stream(s + i);
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) d[i] = v[u];
                }
            }
        } else {
            for (uint32_t base = 0; base < nvec; base += 256u * UNROLL) {
                V v[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) {
                        uint32_t r = i / vec_per_row, col = i - r * vec_per_row;
                        v[u] = ld_stream(reinterpret_cast<const V*>(c.src + (size_t)r * a.src_row_stride) + col);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) {
                        uint32_t r = i / vec_per_row, col = i - r * vec_per_row;
                        reinterpret_cast<V*>(c.dst + (size_t)r * a.dst_row_stride)[col] = v[u];
                    }
                }
            }
        }
        if (a.src_k_scales != nullptr) {
            // E4M3 blocks travel with their per-(layer, block, kv-head) scales
            const float* ss = c.is_v ? a.src_v_scales : a.src_k_scales;
            float* ds = c.is_v ? a.dst_v_scales : a.dst_k_scales;
            for (uint32_t h = threadIdx.x; h < a.n_heads; h += 256u)
                ds[((size_t)(a.dst_layer_begin + c.layer) * a.dst_total_blocks + c.dst_block) * a.dst_pool_heads +
                   a.dst_head_begin + h] =
                    ss[((size_t)(a.src_layer_begin + c.layer) * a.src_total_blocks + c.src_block) * a.src_pool_heads +
                       a.src_head_begin + h];
        }
    }
    signal_done(a);
}

// ---------------------------------------------------------------------------------
// Same-dtype handoff, 32 bytes per access (contiguous chunks, everything 32-byte aligned):
// a warp's load or store instruction covers 1 KiB of one chunk, so a store that leaves the
// GPU travels in the widest packets the link takes.  Built for peer destinations; HINT picks
// the store's cache policy (0 default, 1 streaming, 2 no L1 allocation).
// ---------------------------------------------------------------------------------
struct Vec32 {
    uint32_t r[8];
};
__device__ __forceinline__ Vec32 ld_stream32(const void* p) {
    Vec32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]), "=r"(v.r[7])
                 : "l"(p));
    return v;
}
template <int HINT> __device__ __forceinline__ void st32(void* p, const Vec32& v) {
    if (HINT == 1)
        asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]), "r"(v.r[1]), "r"(v.r[2]), "r"(v.r[3]),
                     "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7]) : "memory");
    else if (HINT == 2)
        asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]), "r"(v.r[1]), "r"(v.r[2]),
                     "r"(v.r[3]), "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7]) : "memory");
    else
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]), "r"(v.r[1]), "r"(v.r[2]), "r"(v.r[3]),
                     "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7]) : "memory");
}

template <int UNROLL, int HINT>
__global__ void __launch_bounds__(256) handoff_copy_wide(const HandoffArgs a) {
    const uint32_t total = live_pairs(a) * a.n_layers * 2u;
    const uint32_t vec_per_row = a.src_row_bytes / 32u;
    const uint32_t vpc = a.block_size * vec_per_row;              // 32-byte vectors of a whole chunk
    constexpr uint32_t PER_PASS = 256u * UNROLL;
    // Measured over NVLink (pulled handoff, one CTA per SM): four 32-byte loads in flight per thread -- one 32 KiB chunk per
    // pass -- fetch 786 GB/s; sixteen in flight, spread over four chunks, 763.  So a pass covers 32 KiB whatever the chunk size.
    constexpr int UG = UNROLL < 4 ? UNROLL : 4;
    constexpr uint32_t GROUP_PASS = 256u * UG;
    if (vpc >= GROUP_PASS) {
        for (uint32_t w = blockIdx.x; w < total; w += gridDim.x) {
            const Chunk c = decode_chunk(a, w);
            const uint32_t nvec = c.n_valid * vec_per_row;
            for (uint32_t base = 0; base < nvec; base += PER_PASS) {
                Vec32 v[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    const uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) v[u] = ld_stream32(c.src + (size_t)i * 32u);
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    const uint32_t i = base + u * 256u + threadIdx.x;
                    if (i < nvec) st32<HINT>(c.dst + (size_t)i * 32u, v[u]);
                }
            }
        }
    } else {
        // Chunks shorter than one pass (few kv heads per pool): a pass spans several chunks, so that a thread's loads in flight do
        // not shrink with the chunk.
        const uint32_t group = GROUP_PASS / vpc;                   // whole chunks per pass
        for (uint64_t w0 = (uint64_t)blockIdx.x * group; w0 < total; w0 += (uint64_t)gridDim.x * group) {
            Vec32 v[UG];
#pragma unroll
            for (int u = 0; u < UG; u++) {
                const uint32_t q = u * 256u + threadIdx.x, off = q / vpc, i = q - off * vpc;
                if (off < group && w0 + off < total) {
                    const Chunk c = decode_chunk(a, (uint32_t)(w0 + off));
                    if (i < c.n_valid * vec_per_row) v[u] = ld_stream32(c.src + (size_t)i * 32u);
                }
            }
#pragma unroll
            for (int u = 0; u < UG; u++) {
                const uint32_t q = u * 256u + threadIdx.x, off = q / vpc, i = q - off * vpc;
                if (off < group && w0 + off < total) {
                    const Chunk c = decode_chunk(a, (uint32_t)(w0 + off));   // the list and the layer pointers are cache hits by now
                    if (i < c.n_valid * vec_per_row) st32<HINT>(c.dst + (size_t)i * 32u, v[u]);
                }
            }
        }
    }
    signal_done(a);
}

// ---------------------------------------------------------------------------------
// Same-dtype handoff, bulk-copy path (same device, contiguous chunks): one warp per
// CTA; lane 0 drives a ring of shared-memory stages with the bulk async-copy engine
// (cp.async.bulk global->shared completing on an mbarrier, then shared->global as a
// bulk group).  No thread touches the payload.  All lanes decode work items 32 at a
// time into a small shared table so lane 0 never waits on a dependent global load.
// Every wait is bounded: on a timeout the CTA records an error, drains its copies and
// leaves.
// ---------------------------------------------------------------------------------
struct BulkItem {
    uint64_t src, dst;
    uint32_t bytes, pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
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

#ifndef TKV_KERNELS_TEMPLATES_ONLY
template <bool INLINE>
__device__ __forceinline__ void bulk_copy_body(const HandoffArgs& a, const InlineList* il, uint32_t stage_bytes, uint32_t n_stages,
                                               uint32_t pieces, uint32_t* error_flag) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                    // up to 8 barriers
    BulkItem* items = reinterpret_cast<BulkItem*>(smem + 64);              // 64 decoded items
    unsigned char* data = smem + 64 + 64 * sizeof(BulkItem);               // 1600: 16-byte aligned
    const uint32_t lane = threadIdx.x;
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint64_t total = (uint64_t)chunks * pieces;
    const uint32_t n_mine = blockIdx.x < total ? (uint32_t)((total - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0u;

    if (lane == 0) {
        for (uint32_t s = 0; s < n_stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bars + s)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();

    // decode items [32*b, 32*b + 32) of this CTA into the half of the table that batch b owns
    auto decode_batch = [&](uint32_t b) {
        uint32_t k = b * 32u + lane;
        if (k < n_mine) {
            uint64_t it = (uint64_t)blockIdx.x + (uint64_t)k * gridDim.x;
            uint32_t piece = (uint32_t)(it % pieces);
            Chunk c = INLINE ? decode_chunk_inline(a, *il, (uint32_t)(it / pieces)) : decode_chunk(a, (uint32_t)(it / pieces));
            uint32_t cb = c.n_valid * a.src_row_bytes;                     // valid bytes of this chunk
            uint32_t off = piece * stage_bytes;
            BulkItem bi;
            bi.bytes = off < cb ? min(stage_bytes, cb - off) : 0u;
            bi.src = reinterpret_cast<uint64_t>(c.src) + off;
            bi.dst = reinterpret_cast<uint64_t>(c.dst) + off;
            bi.pad = 0;
            items[(b & 1u) * 32u + lane] = bi;
        }
        __syncwarp();
    };

    auto issue_load = [&](uint32_t k) {                                    // lane 0 only
        const BulkItem bi = items[k & 63u];
        const uint32_t s = k % n_stages;
        const uint32_t bar = smem_u32(bars + s);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bi.bytes) : "memory");
        if (bi.bytes)
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(data + (size_t)s * stage_bytes)), "l"(bi.src), "r"(bi.bytes), "r"(bar) : "memory");
    };

    uint32_t decoded = 0;                                                  // batches decoded so far
    if (n_mine) {
        decode_batch(0);
        decoded = 1;
    }
    const uint32_t pre = min(n_stages, n_mine);
    if (pre > 32u) {                                                        // cannot happen: n_stages <= 8
        decode_batch(1);
        decoded = 2;
    }
    if (lane == 0)
        for (uint32_t k = 0; k < pre; k++) issue_load(k);

    uint32_t failed = 0;
    for (uint32_t k = 0; k < n_mine; k++) {
        const uint32_t refill = k + n_stages - 1u;                         // item that reuses stage (k-1) % S
        if (k >= 1u && refill < n_mine && refill / 32u >= decoded) {
            decode_batch(refill / 32u);
            decoded = refill / 32u + 1u;
        }
        if (lane == 0) {
            const uint32_t s = k % n_stages;
            if (!mbar_wait_bounded(smem_u32(bars + s), (k / n_stages) & 1u)) {
                failed = 1;
            } else {
                const BulkItem bi = items[k & 63u];
                if (bi.bytes)
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 ::"l"(bi.dst), "r"(smem_u32(data + (size_t)s * stage_bytes)), "r"(bi.bytes) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                if (k >= 1u && refill < n_mine) {
                    // the store issued one iteration ago has read its stage: refill it
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    issue_load(refill);
                }
            }
        }
        failed = __shfl_sync(0xFFFFFFFFu, failed, 0);
        if (failed) {
            // give the loads still in flight a bounded chance to land before leaving
            if (lane == 0)
                for (uint32_t j = k + 1u; j < n_mine && j < k + n_stages; j++)
                    mbar_wait_bounded(smem_u32(bars + j % n_stages), (j / n_stages) & 1u);
            break;
        }
    }
    if (lane == 0) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (failed && error_flag) atomicExch(error_flag, 1u);
    }
    __syncwarp();
    signal_done(a);
}

__global__ void __launch_bounds__(32) handoff_copy_bulk(const HandoffArgs a, uint32_t stage_bytes, uint32_t n_stages,
                                                        uint32_t pieces, uint32_t* error_flag) {
    bulk_copy_body<false>(a, nullptr, stage_bytes, n_stages, pieces, error_flag);
}

// The same ring with the work list in the parameter block (at most INLINE_PAIRS pairs and INLINE_LAYERS layers).
__global__ void __launch_bounds__(32) handoff_copy_bulk_inline(const __grid_constant__ HandoffArgs a, const __grid_constant__ InlineList il,
                                                               uint32_t stage_bytes, uint32_t n_stages, uint32_t pieces, uint32_t* error_flag) {
    bulk_copy_body<true>(a, &il, stage_bytes, n_stages, pieces, error_flag);
}
#endif  // TKV_KERNELS_TEMPLATES_ONLY

// ---------------------------------------------------------------------------------
// FP8 E4M3 encoders.
// ---------------------------------------------------------------------------------

// Integer bit-math statement of the element rule: NaN -> 0x7F, clamp to +-448,
// f32 exponent below 121 -> signed zero, round to nearest even on the 20 dropped
// mantissa bits with carry into the exponent.
__device__ __forceinline__ uint32_t e4m3_encode_int(float x) {
    uint32_t bits = __float_as_uint(x);
    uint32_t sign = (bits >> 24) & 0x80u;
    uint32_t abs = bits & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return 0x7Fu;
    abs = min(abs, 0x43E00000u);  // 448.0f; also catches Inf
    uint32_t exp = abs >> 23;
    if (exp < 121u) return sign;
    uint32_t man = abs & 0x7FFFFFu;
    uint32_t mag = ((exp - 120u) << 3) | (man >> 20);  // exponent and kept bits, carry-ready
    uint32_t dropped = man & 0xFFFFFu;
    uint32_t up = (dropped > 0x80000u) || (dropped == 0x80000u && (mag & 1u));
    return sign | (mag + up);
}

// Hardware conversion (round to nearest even, saturate to +-448) with the
// reference's flush applied first: inputs below 2^-6 in magnitude become a
// signed zero instead of an e4m3 subnormal.  NaN of either sign -> 0x7F.
// Returns {byte(hi) << 8 | byte(lo)}.
__device__ __forceinline__ uint32_t e4m3_encode_pair_hw(float lo, float hi) {
    uint32_t bl = __float_as_uint(lo), bh = __float_as_uint(hi);
    if ((bl & 0x7FFFFFFFu) < 0x3C800000u) bl &= 0x80000000u;
    if ((bh & 0x7FFFFFFFu) < 0x3C800000u) bh &= 0x80000000u;
    if ((bl & 0x7FFFFFFFu) > 0x7F800000u) bl = 0x7FC00000u;
    if ((bh & 0x7FFFFFFFu) > 0x7F800000u) bh = 0x7FC00000u;
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(__uint_as_float(bh)), "f"(__uint_as_float(bl)));
    return r;
}

template <bool HW> __device__ __forceinline__ uint32_t e4m3_encode_pair(float lo, float hi) {
    if (HW) return e4m3_encode_pair_hw(lo, hi);
    return e4m3_encode_int(lo) | (e4m3_encode_int(hi) << 8);
}

// Scale rule: amax taken as the integer maximum of (bits & 0x7FFF); a zero or
// non-finite amax leaves the block unscaled; otherwise the stored scale is
// amax / 448 and elements are multiplied by 448 / amax, each one IEEE
// round-to-nearest operation.
__device__ __forceinline__ float block_scale(uint32_t amax_bits, float& inv) {
    if (amax_bits == 0u || amax_bits >= 0x7C00u) {
        inv = 1.0f;
        return 1.0f;
    }
    float amax = __half2float(__ushort_as_half((unsigned short)amax_bits));
    inv = __fdiv_rn(448.0f, amax);
    return __fdiv_rn(amax, 448.0f);
}

// two F16 in a u32 -> two e4m3 bytes in the low 16 bits
template <bool HW> __device__ __forceinline__ uint32_t quant_h2(uint32_t h2, float inv) {
    float lo = __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
    float hi = __half2float(__ushort_as_half((unsigned short)(h2 >> 16)));
    return e4m3_encode_pair<HW>(__fmul_rn(lo, inv), __fmul_rn(hi, inv));
}

// ---- fast path of the scaled encoder ---------------------------------------------
// For a block whose amax is finite and non-zero no element is NaN or Inf, and the
// only place the hardware conversion departs from the element rule is the flush of
// products below 2^-6.  RN(x * inv) is monotone in |x|, so the flush is a single
// threshold on the F16 magnitude: the smallest half h with RN(float(h) * inv) >= 2^-6.
// The guess T / inv is off by far less than the F16 spacing; start one below its
// floor and step up while the exact test fails.
__device__ __forceinline__ uint32_t flush_threshold_bits(float inv) {
    const float T = 0.015625f;
    uint32_t c = (uint32_t)__half_as_ushort(__float2half_rd(__fdiv_rn(T, inv)));
    c = c > 0u ? c - 1u : 0u;
#pragma unroll
    for (int k = 0; k < 3; k++) {
        float y = __fmul_rn(__half2float(__ushort_as_half((unsigned short)c)), inv);
        if (y < T) c++;
    }
    return c;
}

// two F16 in a u32 -> two e4m3 bytes in the low 16 bits; thr2 holds the flush
// threshold in both halves.  Magnitudes below it become signed zeros before widening.
__device__ __forceinline__ uint32_t quant_h2_fast(uint32_t w, float inv, __half2 thr2) {
    __half2 x = *reinterpret_cast<__half2*>(&w);
    uint32_t keep = __hge2_mask(__habs2(x), thr2) | 0x80008000u;
    w &= keep;
    x = *reinterpret_cast<__half2*>(&w);
    float lo = __fmul_rn(__low2float(x), inv), hi = __fmul_rn(__high2float(x), inv);
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// max over |a|, |b| lanes; a NaN lane stays NaN (bits 0x7FFF), so an integer compare
// of the result against 0x7C00 still detects Inf and NaN.
__device__ __forceinline__ uint32_t amax_h2(uint32_t m, uint32_t w) {
    __half2 r = __hmax2_nan(*reinterpret_cast<__half2*>(&m), __habs2(*reinterpret_cast<__half2*>(&w)));
    return *reinterpret_cast<uint32_t*>(&r);
}

// ---------------------------------------------------------------------------------
// F16 -> E4M3 handoff, one warp per (chunk, kv head).  The warp keeps its
// BS x D halves in registers between the absmax pass and the encode pass, so the
// source is read once.  Each lane owns 16 contiguous source bytes of a token row per
// pass, so one load instruction of the warp covers whole, adjacent 32-byte sectors
// (two rows of a 128-wide head); the 8 encoded bytes go out as one 8-byte store.
// ---------------------------------------------------------------------------------
template <int D, int BS, bool HW, bool SCALED>
__global__ void __launch_bounds__(256) handoff_f16_e4m3_warp(const HandoffArgs a) {
    constexpr int LPR = D / 8;         // lanes per token row
    constexpr int RPP = 32 / LPR;      // token rows per pass
    constexpr int NP = (BS + RPP - 1) / RPP;
    static_assert(D % 8 == 0 && LPR >= 1 && LPR <= 32 && (32 % LPR) == 0, "head_dim");
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t r0 = lane / LPR, col = lane % LPR;
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint64_t total = (uint64_t)chunks * a.n_heads;
    for (uint64_t wi = (uint64_t)blockIdx.x * 8u + warp; wi < total; wi += (uint64_t)gridDim.x * 8u) {
        const uint32_t h = (uint32_t)(wi % a.n_heads);
        const Chunk c = decode_chunk(a, (uint32_t)(wi / a.n_heads));
        const char* s = c.src + (size_t)h * D * 2 + col * 16;
        char* d = c.dst + (size_t)h * D + col * 8;
        uint4 v[NP];
        uint32_t m = 0, amax = 0x7C00u;  // amax stays 'non-finite' when no scale pass runs
#pragma unroll
        for (int p = 0; p < NP; p++) {
            uint32_t row = p * RPP + r0;
            if (row < c.n_valid) v[p] = ld_stream(reinterpret_cast<const uint4*>(s + (size_t)row * a.src_row_stride));
            else v[p] = make_uint4(0, 0, 0, 0);
        }
        float inv = 1.0f;
        if (SCALED) {
#pragma unroll
            for (int p = 0; p < NP; p++) {
                m = amax_h2(m, v[p].x);
                m = amax_h2(m, v[p].y);
                m = amax_h2(m, v[p].z);
                m = amax_h2(m, v[p].w);
            }
            amax = max(m & 0xFFFFu, m >> 16);
            amax = __reduce_max_sync(0xFFFFFFFFu, amax);
            float scale = block_scale(amax, inv);
            if (lane == 0) {
                float* sc = c.is_v ? a.dst_v_scales : a.dst_k_scales;
                sc[((size_t)(a.dst_layer_begin + c.layer) * a.dst_total_blocks + c.dst_block) * a.dst_pool_heads +
                   a.dst_head_begin + h] = scale;
            }
        }
        if (SCALED && HW && amax < 0x7C00u) {
            // finite block: threshold flush on the F16 bits, hardware conversion
            const uint32_t t = flush_threshold_bits(inv);
            const uint32_t t2u = t | (t << 16);
            const __half2 thr2 = *reinterpret_cast<const __half2*>(&t2u);
#pragma unroll
            for (int p = 0; p < NP; p++) {
                uint32_t row = p * RPP + r0;
                if (row < c.n_valid) {
                    uint2 o;
                    o.x = __byte_perm(quant_h2_fast(v[p].x, inv, thr2), quant_h2_fast(v[p].y, inv, thr2), 0x5410);
                    o.y = __byte_perm(quant_h2_fast(v[p].z, inv, thr2), quant_h2_fast(v[p].w, inv, thr2), 0x5410);
                    *reinterpret_cast<uint2*>(d + (size_t)row * a.dst_row_stride) = o;
                }
            }
            continue;
        }
        // unscaled destination, integer encoder, or a block holding Inf / NaN
#pragma unroll
        for (int p = 0; p < NP; p++) {
            uint32_t row = p * RPP + r0;
            if (row < c.n_valid) {
                uint2 o;
                o.x = quant_h2<HW>(v[p].x, inv) | (quant_h2<HW>(v[p].y, inv) << 16);
                o.y = quant_h2<HW>(v[p].z, inv) | (quant_h2<HW>(v[p].w, inv) << 16);
                *reinterpret_cast<uint2*>(d + (size_t)row * a.dst_row_stride) = o;
            }
        }
    }
    signal_done(a);
}

// ---------------------------------------------------------------------------------
// F16 -> E4M3 handoff, shared-memory staged (whole rows on the source side, 16 tokens
// per block).  Thread 0 keeps a ring of source chunks in flight with the bulk async-copy
// engine (cp.async.bulk global->shared completing on an mbarrier); the CTA's 8 warps
// encode one kv head each out of shared memory into an output tile; the tile leaves as
// ONE bulk store (destination on this device, whole rows) or as coalesced 16-byte stores
// (peer destination or strided rows).  Memory latency is hidden by the ring, not by
// registers.  Every wait is bounded: on a timeout the CTA records an error, drains its
// copies and leaves.
// ---------------------------------------------------------------------------------
struct StagedItem {
    uint64_t src, dst;
    uint32_t n_valid, layer, is_v, dst_block;
};

template <int D, bool HW, bool SCALED>
__global__ void __launch_bounds__(256) handoff_f16_e4m3_staged(const HandoffArgs a, uint32_t n_stages, uint32_t bulk_store,
                                                               uint32_t* error_flag) {
    constexpr int BS = 16;
    constexpr int LPR = D / 8;         // lanes per token row
    constexpr int RPP = 32 / LPR;      // token rows per pass
    constexpr int NP = BS / RPP;
    static_assert(D % 8 == 0 && LPR >= 2 && LPR <= 32 && (32 % LPR) == 0, "head_dim");
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);                      // up to 8 barriers
    uint32_t* fail_word = reinterpret_cast<uint32_t*>(smem + 64);
    StagedItem* items = reinterpret_cast<StagedItem*>(smem + 128);           // 64 decoded items
    const uint32_t in_bytes = BS * a.src_row_bytes, out_bytes = BS * a.dst_row_bytes;
    unsigned char* in_base = smem + 128 + 64 * sizeof(StagedItem);           // 2176: 128-byte aligned
    unsigned char* out_base = in_base + (size_t)n_stages * in_bytes;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t r0 = lane / LPR, col = lane % LPR;
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint32_t n_mine = blockIdx.x < chunks ? (chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;

    if (tid == 0) {
        for (uint32_t s = 0; s < n_stages; s++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bars + s)));
        *fail_word = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // items [32*b, 32*b + 32) of this CTA, decoded by warp 0 into the half of the table batch b owns
    auto decode_batch = [&](uint32_t b) {
        uint32_t k = b * 32u + lane;
        if (warp == 0 && k < n_mine) {
            Chunk c = decode_chunk(a, blockIdx.x + k * gridDim.x);
            StagedItem it;
            it.src = reinterpret_cast<uint64_t>(c.src);
            it.dst = reinterpret_cast<uint64_t>(c.dst);
            it.n_valid = c.n_valid;
            it.layer = c.layer;
            it.is_v = c.is_v;
            it.dst_block = c.dst_block;
            items[(b & 1u) * 32u + lane] = it;
        }
    };
    auto issue_load = [&](uint32_t k) {                                      // thread 0 only
        const StagedItem it = items[k & 63u];
        const uint32_t s = k % n_stages, bar = smem_u32(bars + s), bytes = it.n_valid * a.src_row_bytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(in_base + (size_t)s * in_bytes)), "l"(it.src), "r"(bytes), "r"(bar) : "memory");
    };

    uint32_t decoded = 0;
    if (n_mine) {
        decode_batch(0);
        decoded = 1;
    }
    __syncthreads();
    if (tid == 0)
        for (uint32_t k = 0; k < min(n_stages, n_mine); k++) issue_load(k);

    uint32_t failed = 0, k_fail = 0;
    for (uint32_t k = 0; k < n_mine; k++) {
        const uint32_t s = k % n_stages, o = k & 1u;
        const uint32_t refill = k + n_stages;
        if (refill < n_mine && refill / 32u >= decoded) {
            decode_batch(refill / 32u);                                      // visible to thread 0 after the barrier below
            decoded = refill / 32u + 1u;
        }
        const StagedItem it = items[k & 63u];
        const bool ok = mbar_wait_bounded(smem_u32(bars + s), (k / n_stages) & 1u);
        if (!ok) *fail_word = 1u;
        const unsigned char* in = in_base + (size_t)s * in_bytes;
        unsigned char* out = out_base + (size_t)o * out_bytes;
        if (ok) {
            for (uint32_t h = warp; h < a.n_heads; h += 8u) {
                const unsigned char* sp = in + (size_t)h * D * 2 + col * 16;
                unsigned char* dp = out + (size_t)h * D + col * 8;
                uint4 v[NP];
                uint32_t m = 0, amax = 0x7C00u;
#pragma unroll
                for (int p = 0; p < NP; p++) {
                    uint32_t row = p * RPP + r0;
                    if (row < it.n_valid) v[p] = *reinterpret_cast<const uint4*>(sp + (size_t)row * a.src_row_bytes);
                    else v[p] = make_uint4(0, 0, 0, 0);
                }
                float inv = 1.0f;
                if (SCALED) {
#pragma unroll
                    for (int p = 0; p < NP; p++) {
                        m = amax_h2(m, v[p].x);
                        m = amax_h2(m, v[p].y);
                        m = amax_h2(m, v[p].z);
                        m = amax_h2(m, v[p].w);
                    }
                    amax = max(m & 0xFFFFu, m >> 16);
                    amax = __reduce_max_sync(0xFFFFFFFFu, amax);
                    float scale = block_scale(amax, inv);
                    if (lane == 0) {
                        float* sc = it.is_v ? a.dst_v_scales : a.dst_k_scales;
                        sc[((size_t)(a.dst_layer_begin + it.layer) * a.dst_total_blocks + it.dst_block) * a.dst_pool_heads +
                           a.dst_head_begin + h] = scale;
                    }
                }
                if (SCALED && HW && amax < 0x7C00u) {
                    const uint32_t t = flush_threshold_bits(inv);
                    const uint32_t t2u = t | (t << 16);
                    const __half2 thr2 = *reinterpret_cast<const __half2*>(&t2u);
#pragma unroll
                    for (int p = 0; p < NP; p++) {
                        uint32_t row = p * RPP + r0;
                        uint2 q;
                        q.x = __byte_perm(quant_h2_fast(v[p].x, inv, thr2), quant_h2_fast(v[p].y, inv, thr2), 0x5410);
                        q.y = __byte_perm(quant_h2_fast(v[p].z, inv, thr2), quant_h2_fast(v[p].w, inv, thr2), 0x5410);
                        if (row < it.n_valid) *reinterpret_cast<uint2*>(dp + (size_t)row * a.dst_row_bytes) = q;
                    }
                } else {
#pragma unroll
                    for (int p = 0; p < NP; p++) {
                        uint32_t row = p * RPP + r0;
                        uint2 q;
                        q.x = quant_h2<HW>(v[p].x, inv) | (quant_h2<HW>(v[p].y, inv) << 16);
                        q.y = quant_h2<HW>(v[p].z, inv) | (quant_h2<HW>(v[p].w, inv) << 16);
                        if (row < it.n_valid) *reinterpret_cast<uint2*>(dp + (size_t)row * a.dst_row_bytes) = q;
                    }
                }
            }
            if (bulk_store) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();   // tile complete, stage s read by every warp
        failed = *fail_word;
        if (failed) {
            k_fail = k;
            break;
        }
        if (bulk_store) {
            if (tid == 0) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(it.dst), "r"(smem_u32(out)), "r"(it.n_valid * a.dst_row_bytes) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                if (refill < n_mine) issue_load(refill);
                // the store issued one iteration ago has read its tile: the next iteration may overwrite it
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            }
        } else {
            if (tid == 0 && refill < n_mine) issue_load(refill);
            const uint32_t vec_per_row = a.dst_row_bytes / 16u, nvec = it.n_valid * vec_per_row;
            for (uint32_t i = tid; i < nvec; i += 256u) {
                uint32_t r = i / vec_per_row, c16 = i - r * vec_per_row;
                uint4 q = *reinterpret_cast<const uint4*>(out + (size_t)i * 16);
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(it.dst) + (size_t)r * a.dst_row_stride + c16 * 16) = q;
            }
        }
        __syncthreads();   // the other tile is free again
    }
    if (tid == 0) {
        if (failed) {
            // give the loads still in flight a bounded chance to land before leaving
            for (uint32_t j = k_fail; j < n_mine && j < k_fail + n_stages; j++)
                mbar_wait_bounded(smem_u32(bars + j % n_stages), (j / n_stages) & 1u);
            if (error_flag) atomicExch(error_flag, 1u);
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    signal_done(a);
}

// Any head_dim / block_size: one warp per (chunk, kv head), two passes over the
// source (the second one hits L2), element-wide accesses.
template <bool HW, bool SCALED>
__global__ void __launch_bounds__(256) handoff_f16_e4m3_generic(const HandoffArgs a) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint64_t total = (uint64_t)chunks * a.n_heads;
    const uint32_t D = a.head_dim;
    for (uint64_t wi = (uint64_t)blockIdx.x * 8u + warp; wi < total; wi += (uint64_t)gridDim.x * 8u) {
        const uint32_t h = (uint32_t)(wi % a.n_heads);
        const Chunk c = decode_chunk(a, (uint32_t)(wi / a.n_heads));
        const uint32_t n = c.n_valid * D;
        float inv = 1.0f;
        if (SCALED) {
            uint32_t amax = 0;
            for (uint32_t i = lane; i < n; i += 32u) {
                uint32_t r = i / D, e = i - r * D;
                uint16_t b = *reinterpret_cast<const uint16_t*>(c.src + (size_t)r * a.src_row_stride + ((size_t)h * D + e) * 2);
                amax = max(amax, (uint32_t)(b & 0x7FFFu));
            }
            amax = __reduce_max_sync(0xFFFFFFFFu, amax);
            float scale = block_scale(amax, inv);
            if (lane == 0) {
                float* sc = c.is_v ? a.dst_v_scales : a.dst_k_scales;
                sc[((size_t)(a.dst_layer_begin + c.layer) * a.dst_total_blocks + c.dst_block) * a.dst_pool_heads +
                   a.dst_head_begin + h] = scale;
            }
        }
        for (uint32_t i = lane; i < n; i += 32u) {
            uint32_t r = i / D, e = i - r * D;
            uint16_t b = *reinterpret_cast<const uint16_t*>(c.src + (size_t)r * a.src_row_stride + ((size_t)h * D + e) * 2);
            float y = __fmul_rn(__half2float(__ushort_as_half(b)), inv);
            uint32_t q = HW ? (e4m3_encode_pair_hw(y, 0.0f) & 0xFFu) : e4m3_encode_int(y);
            *reinterpret_cast<uint8_t*>(c.dst + (size_t)r * a.dst_row_stride + (size_t)h * D + e) = (uint8_t)q;
        }
    }
    signal_done(a);
}

// F32 source with a narrower destination (append_kv's casts): element-wide.
// MODE 0: F32 -> F16 (round to nearest even; NaN -> 0x7FFF as cvt.rn.f16.f32 does)
// MODE 1: F32 -> E4M3, unscaled
template <int MODE>
__global__ void __launch_bounds__(256) handoff_f32_cast_generic(const HandoffArgs a) {
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint32_t row_elems = a.n_heads * a.head_dim;
    for (uint32_t w = blockIdx.x; w < chunks; w += gridDim.x) {
        const Chunk c = decode_chunk(a, w);
        const uint32_t n = c.n_valid * row_elems;
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            uint32_t r = i / row_elems, e = i - r * row_elems;
            float x = *reinterpret_cast<const float*>(c.src + (size_t)r * a.src_row_stride + (size_t)e * 4);
            if (MODE == 0) {
                *reinterpret_cast<__half*>(c.dst + (size_t)r * a.dst_row_stride + (size_t)e * 2) = __float2half_rn(x);
            } else {
                *reinterpret_cast<uint8_t*>(c.dst + (size_t)r * a.dst_row_stride + e) = (uint8_t)e4m3_encode_int(x);
            }
        }
    }
    signal_done(a);
}

__device__ __forceinline__ float e4m3_decode(uint32_t b) {
    uint32_t sign = (b & 0x80u) << 24, exp = (b >> 3) & 0xFu, man = b & 7u;
    return __uint_as_float(exp == 0u ? sign : (sign | ((exp + 120u) << 23) | (man << 20)));
}

// E4M3 source with a wider destination: the reader's side of the FP8 cache
// (Fp8PagedKvCache::k_contiguous widens while it gathers).  Element rule: exact decode
// (subnormal encodings read as signed zero), times the block's scale when the source pool
// carries scales (one round-to-nearest multiply), then round to nearest even for F16.
// One thread per 16 source bytes when everything is 16-byte aligned (VEC16), else per byte.
// DST16: destination is F16 (else F32).
template <bool DST16, bool VEC16>
__global__ void __launch_bounds__(256) handoff_e4m3_dequant(const HandoffArgs a) {
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint32_t D = a.head_dim;
    constexpr uint32_t W = VEC16 ? 16u : 1u;
    const uint32_t per_row = a.src_row_bytes / W;             // work items per token row
    for (uint32_t w = blockIdx.x; w < chunks; w += gridDim.x) {
        const Chunk c = decode_chunk(a, w);
        const float* sc = c.is_v ? a.src_v_scales : a.src_k_scales;
        const float* sc_blk = sc ? sc + ((size_t)(a.src_layer_begin + c.layer) * a.src_total_blocks + c.src_block) * a.src_pool_heads +
                                       a.src_head_begin
                                 : nullptr;
        const uint32_t n = c.n_valid * per_row;
        for (uint32_t i = threadIdx.x; i < n; i += 256u) {
            const uint32_t r = i / per_row, e0 = (i - r * per_row) * W;   // first element of this item within the row
            const float scale = sc_blk ? __ldg(sc_blk + e0 / D) : 1.0f;
            const unsigned char* sp = reinterpret_cast<const unsigned char*>(c.src) + (size_t)r * a.src_row_stride + e0;
            char* dp = c.dst + (size_t)r * a.dst_row_stride + (size_t)e0 * (DST16 ? 2 : 4);
            if (VEC16) {
                const uint4 q = ld_stream(reinterpret_cast<const uint4*>(sp));
                const uint32_t words[4] = {q.x, q.y, q.z, q.w};
                float x[16];
#pragma unroll
                for (int k = 0; k < 16; k++) x[k] = __fmul_rn(e4m3_decode((words[k >> 2] >> ((k & 3) * 8)) & 0xFFu), scale);
                if (DST16) {
                    uint32_t h[8];
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        h[k] = (uint32_t)__half_as_ushort(__float2half_rn(x[2 * k])) |
                               ((uint32_t)__half_as_ushort(__float2half_rn(x[2 * k + 1])) << 16);
                    reinterpret_cast<uint4*>(dp)[0] = make_uint4(h[0], h[1], h[2], h[3]);
                    reinterpret_cast<uint4*>(dp)[1] = make_uint4(h[4], h[5], h[6], h[7]);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        reinterpret_cast<float4*>(dp)[k] = make_float4(x[4 * k], x[4 * k + 1], x[4 * k + 2], x[4 * k + 3]);
                }
            } else {
                const float x = __fmul_rn(e4m3_decode(*sp), scale);
                if (DST16) *reinterpret_cast<__half*>(dp) = __float2half_rn(x);
                else *reinterpret_cast<float*>(dp) = x;
            }
        }
    }
    signal_done(a);
}

// The same casts, 16-byte accesses: a thread converts 8 floats into one 16-byte store of halves (MODE 0) or 16
// floats into 16 e4m3 bytes (MODE 1).  Needs every row offset and stride to keep 16-byte alignment on both sides.
__device__ __forceinline__ float4 ld_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int MODE>
__global__ void __launch_bounds__(256) handoff_f32_cast_vec(const HandoffArgs a) {
    constexpr uint32_t E = MODE == 0 ? 8u : 16u;               // elements per 16-byte store
    const uint32_t chunks = live_pairs(a) * a.n_layers * 2u;
    const uint32_t row_elems = a.n_heads * a.head_dim, per_row = row_elems / E;
    for (uint32_t w = blockIdx.x; w < chunks; w += gridDim.x) {
        const Chunk c = decode_chunk(a, w);
        const uint32_t n = c.n_valid * per_row;
        for (uint32_t i = threadIdx.x; i < n; i += 256u) {
            const uint32_t r = i / per_row, e0 = (i - r * per_row) * E;
            const float4* sp = reinterpret_cast<const float4*>(c.src + (size_t)r * a.src_row_stride + (size_t)e0 * 4);
            uint4 o;
            if (MODE == 0) {
                const float4 x = ld_stream_f4(sp), y = ld_stream_f4(sp + 1);
                o = make_uint4(h2_bits(x.x, x.y), h2_bits(x.z, x.w), h2_bits(y.x, y.y), h2_bits(y.z, y.w));
                *reinterpret_cast<uint4*>(c.dst + (size_t)r * a.dst_row_stride + (size_t)e0 * 2) = o;
            } else {
                float4 x[4];
#pragma unroll
                for (int k = 0; k < 4; k++) x[k] = ld_stream_f4(sp + k);
                uint32_t q[4];
#pragma unroll
                for (int k = 0; k < 4; k++)
                    q[k] = e4m3_encode_int(x[k].x) | (e4m3_encode_int(x[k].y) << 8) | (e4m3_encode_int(x[k].z) << 16) |
                           (e4m3_encode_int(x[k].w) << 24);
                o = make_uint4(q[0], q[1], q[2], q[3]);
                *reinterpret_cast<uint4*>(c.dst + (size_t)r * a.dst_row_stride + e0) = o;
            }
        }
    }
    signal_done(a);
}

// Non-template kernels have one definition per program: a second translation unit that
// only needs the templates above defines TKV_KERNELS_TEMPLATES_ONLY before including.
#ifndef TKV_KERNELS_TEMPLATES_ONLY
// ---------------------------------------------------------------------------------
// small kernels
// ---------------------------------------------------------------------------------
// ---------------------------------------------------------------------------------
// Work list from block tables that live on the device (one CTA): sequence q contributes its blocks
// past the shared prefix, in table order, sequences in index order -- the list the host builder would
// have produced.  Nothing is trusted: a prefix longer than its sequence or not block-aligned, a
// sequence longer than its table row, a block id outside either pool, or more pairs than the plan
// was sized for leave an EMPTY list (nothing moves, no reference count changes) and a status code.
// ---------------------------------------------------------------------------------
struct DeviceTables {
    const uint32_t* seq_lens;
    const uint32_t* prefix_lens;   // tokens, or null
    const uint32_t* prefix_blocks; // blocks, read when prefix_lens is null; or null
    const uint32_t* src_tables;
    const uint32_t* dst_tables;
    uint32_t* offsets;             // [n_seqs] scratch
    uint4* work;
    uint32_t* n_pairs_out;
    uint32_t* status;              // or null
    int32_t* refcounts;            // destination pool's, or null (no reference counting asked for)
    uint32_t n_seqs, table_stride, block_size, capacity, src_total_blocks, dst_total_blocks;
};

__device__ __forceinline__ uint32_t prefix_tokens_of(const DeviceTables& t, uint32_t q) {
    if (t.prefix_lens) return t.prefix_lens[q];
    if (!t.prefix_blocks) return 0u;
    const uint32_t blocks = t.prefix_blocks[q];
    return blocks > 0xFFFFFFFFu / t.block_size ? 0xFFFFFFFFu : blocks * t.block_size;      // an absurd count fails the prefix <= length check
}

__global__ void __launch_bounds__(1024) worklist_from_device_tables(const DeviceTables t) {
    __shared__ uint32_t scan[1024];
    __shared__ uint32_t carry, err;
    const uint32_t tid = threadIdx.x, bs = t.block_size;
    if (tid == 0) carry = err = 0;
    __syncthreads();
    for (uint32_t q0 = 0; q0 < t.n_seqs; q0 += 1024) {
        const uint32_t q = q0 + tid;
        uint32_t cnt = 0;
        if (q < t.n_seqs) {
            const uint32_t len = t.seq_lens[q], pre = prefix_tokens_of(t, q), nb = (len + bs - 1) / bs;
            if (pre > len || pre % bs || nb > t.table_stride) atomicExch(&err, 2u);
            else cnt = nb - pre / bs;
        }
        scan[tid] = cnt;
        __syncthreads();
        for (uint32_t off = 1; off < 1024; off <<= 1) {
            const uint32_t v = tid >= off ? scan[tid - off] : 0u;
            __syncthreads();
            scan[tid] += v;
            __syncthreads();
        }
        if (q < t.n_seqs) t.offsets[q] = carry + scan[tid] - cnt;
        __syncthreads();
        if (tid == 1023) carry = (carry > 0x7FFFFFFFu - scan[1023]) ? 0x7FFFFFFFu : carry + scan[1023];
        __syncthreads();
    }
    const uint32_t total = carry;
    if (tid == 0 && total > t.capacity && !err) err = 1u;          // more pairs than the plan was sized for
    __syncthreads();
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    if (!err) {
        for (uint32_t q = warp; q < t.n_seqs; q += 32) {
            const uint32_t len = t.seq_lens[q], pre_b = (prefix_tokens_of(t, q)) / bs, nb = (len + bs - 1) / bs;
            const uint32_t* srow = t.src_tables + (size_t)q * t.table_stride;
            const uint32_t* drow = t.dst_tables + (size_t)q * t.table_stride;
            for (uint32_t i = lane; i < nb; i += 32) {
                const uint32_t did = drow[i];
                if (did >= t.dst_total_blocks) atomicExch(&err, 2u);
                if (i < pre_b) continue;
                const uint32_t sid = srow[i];
                if (sid >= t.src_total_blocks) atomicExch(&err, 2u);
                t.work[t.offsets[q] + (i - pre_b)] = make_uint4(sid, did, min(bs, len - i * bs), q);
            }
        }
    }
    __syncthreads();
    if (!err && t.refcounts) {                                       // RadixTree::lookup's count, one per sequence and shared block
        for (uint32_t q = warp; q < t.n_seqs; q += 32) {
            const uint32_t pre_b = (prefix_tokens_of(t, q)) / bs;
            for (uint32_t i = lane; i < pre_b; i += 32) atomicAdd(t.refcounts + t.dst_tables[(size_t)q * t.table_stride + i], 1);
        }
    }
    if (tid == 0) {
        *t.n_pairs_out = err ? 0u : total;
        if (t.status) *t.status = err;                              // 0, 1 = dimension mismatch (capacity), 2 = invalid config
    }
}

__global__ void refcount_apply_kernel(uint32_t* refcounts, const uint32_t* ids, uint32_t n, int delta) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t* p = refcounts + ids[i];
        if (delta > 0) {
            atomicAdd(p, 1u);
        } else {
            uint32_t old = *p;
            while (old != 0u) {  // saturating decrement; ends when the CAS lands or the count is 0
                uint32_t seen = atomicCAS(p, old, old - 1u);
                if (seen == old) break;
                old = seen;
            }
        }
    }
}

// The shared-prefix reference counts of a device batch, applied by the pool's own device: one warp per sequence over the
// first prefix_blocks[q] (or prefix_lens[q] / block_size) entries of its destination table row.  Ids outside the pool
// are skipped and reported through `status`.
__global__ void __launch_bounds__(256) refcount_apply_tables_kernel(uint32_t* refcounts, const uint32_t* dst_tables, const uint32_t* prefix_lens,
                                                                    const uint32_t* prefix_blocks, uint32_t n_seqs, uint32_t table_stride,
                                                                    uint32_t block_size, uint32_t total_blocks, int delta, uint32_t* status) {
    const uint32_t warps = (gridDim.x * blockDim.x) >> 5, lane = threadIdx.x & 31u;
    for (uint32_t q = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; q < n_seqs; q += warps) {
        const uint32_t pre = min(prefix_lens ? prefix_lens[q] / block_size : prefix_blocks[q], table_stride);
        for (uint32_t i = lane; i < pre; i += 32) {
            const uint32_t id = dst_tables[(size_t)q * table_stride + i];
            if (id >= total_blocks) {
                if (status) atomicExch(status, 2u);
                continue;
            }
            uint32_t* p = refcounts + id;
            if (delta > 0) {
                atomicAdd(p, 1u);
            } else {
                uint32_t old = *p;
                while (old != 0u) {
                    const uint32_t seen = atomicCAS(p, old, old - 1u);
                    if (seen == old) break;
                    old = seen;
                }
            }
        }
    }
}

// Bounded wait: gives up after max_spins polls and records a status instead of
// spinning forever.
__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t expected, unsigned long long max_spins,
                                 uint32_t* status) {
    uint32_t v = 0;
    for (unsigned long long i = 0; i < max_spins; i++) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t)(v - expected) >= 0) {   // generation reached or already passed
            if (status) *status = 0u;  // TKV_OK
            return;
        }
        __nanosleep(256);
    }
    if (status) *status = 4u;  // TKV_ERR_TIMEOUT
}

// dtype codes: 0 = F32, 1 = F16, 2 = E4M3
template <int SRC, int DST>
__global__ void cast_kernel(const void* __restrict__ src, void* __restrict__ dst, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float x;
        if (SRC == 0) x = reinterpret_cast<const float*>(src)[i];
        else if (SRC == 1) x = __half2float(reinterpret_cast<const __half*>(src)[i]);
        else x = e4m3_decode(reinterpret_cast<const uint8_t*>(src)[i]);
        if (DST == 0) reinterpret_cast<float*>(dst)[i] = x;
        else if (DST == 1) reinterpret_cast<__half*>(dst)[i] = __float2half_rn(x);
        else reinterpret_cast<uint8_t*>(dst)[i] = (uint8_t)e4m3_encode_int(x);
    }
}

__global__ void selfcheck_e4m3_kernel(uint32_t skip_bits, unsigned long long* mismatches) {
    const uint64_t n = 1ull << (32 - skip_bits);
    unsigned long long bad = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float x = __uint_as_float((uint32_t)(i << skip_bits));
        uint32_t want = e4m3_encode_int(x);
        uint32_t p = e4m3_encode_pair_hw(x, -x);
        if ((p & 0xFFu) != want) bad++;
        uint32_t want_neg = e4m3_encode_int(-x);
        if ((p >> 8) != want_neg) bad++;
    }
    if (bad) atomicAdd(mismatches, bad);
}

// Every finite non-zero amax, every |h| <= amax of both signs: the fast scaled path
// (threshold flush + hardware conversion) against the integer encoder applied to the
// same FP32 product.  One CTA per amax value.
__global__ void selfcheck_scaled_quant_kernel(unsigned long long* mismatches) {
    unsigned long long bad = 0;
    for (uint32_t amax = 1u + blockIdx.x; amax < 0x7C00u; amax += gridDim.x) {
        float inv;
        block_scale(amax, inv);
        const uint32_t t = flush_threshold_bits(inv);
        const uint32_t t2u = t | (t << 16);
        const __half2 thr2 = *reinterpret_cast<const __half2*>(&t2u);
        for (uint32_t h = threadIdx.x; h <= amax; h += blockDim.x) {
            uint32_t got = quant_h2_fast(h | ((h | 0x8000u) << 16), inv, thr2);
            float x = __half2float(__ushort_as_half((unsigned short)h));
            uint32_t want = e4m3_encode_int(__fmul_rn(x, inv)) | (e4m3_encode_int(__fmul_rn(-x, inv)) << 8);
            if (got != want) bad++;
        }
    }
    if (bad) atomicAdd(mismatches, bad);
}

template <int DT>
__global__ void bits_checksum_kernel(const void* __restrict__ data, uint64_t n, unsigned long long* out) {
    unsigned long long s = 0;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        float x;
        if (DT == 0) x = reinterpret_cast<const float*>(data)[i];
        else if (DT == 1) x = __half2float(reinterpret_cast<const __half*>(data)[i]);
        else x = e4m3_decode(reinterpret_cast<const uint8_t*>(data)[i]);
        s += __float_as_uint(x);
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_down_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0 && s) atomicAdd(out, s);
}

#endif  // TKV_KERNELS_TEMPLATES_ONLY

}  // namespace tkv
