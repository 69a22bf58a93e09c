// tkv_handoff_noalloc: the same-dtype handoff for callers that must not allocate device
// memory when a handoff happens (pools that already own almost all of HBM, serving loops
// that cannot take the device-wide stall of cudaMalloc/cudaFree, fixed memory budgets).
// The layer pointers and the work list, which a plan keeps in its own device buffer, live
// here in one fixed array that is part of the library image.
#define TKV_KERNELS_TEMPLATES_ONLY
#include "tkv_kernels.cuh"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/tkv.h"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
bool peer_reachable(int from, int to);
bool imported_on(int from, const uint64_t* ptrs, size_t n);
}

namespace {

// Scratch shared by every call on a device.  In host code this name is only a stand-in for
// the symbol: the address a kernel can use comes from cudaGetSymbolAddress (setup() below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[TKV_NOALLOC_SCRATCH_BYTES];

struct PerDevice {
    void* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
std::mutex g_mu;
PerDevice g_per_device[64];

int32_t fail(int32_t code, const char* fmt, unsigned long long a = 0, unsigned long long b = 0, unsigned long long c = 0) {
    char buf[384];
    snprintf(buf, sizeof buf, fmt, a, b, c);
    return tkv_internal::set_error(code, 0, buf);
}
int32_t cuda_fail(cudaError_t e, const char* what) {
    char buf[384];
    snprintf(buf, sizeof buf, "%s: %s (cuda error %d)", what, cudaGetErrorString(e), (int)e);
    return tkv_internal::set_error(TKV_ERR_CUDA, (int32_t)e, buf);
}

// Once per device, with that device current: resolve the scratch symbol to its device address.
int32_t setup(int dev, PerDevice* out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (dev < 0 || dev >= 64) return fail(TKV_ERR_INVALID_CONFIG, "device ordinal %llu out of range", (unsigned long long)dev);
    PerDevice& pd = g_per_device[dev];
    if (!pd.scratch) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(no-alloc scratch)");
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        pd.sm_count = n;
        pd.scratch = p;
    }
    *out = pd;
    return TKV_OK;
}

uint32_t elem_size(int32_t dt) { return dt == TKV_DTYPE_F32 ? 4u : dt == TKV_DTYPE_F16 ? 2u : dt == TKV_DTYPE_E4M3 ? 1u : 0u; }

template <int VEC> int32_t launch(const tkv::HandoffArgs& a, int sm_count, uint64_t chunks, cudaStream_t st) {
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tkv::handoff_copy_vec<VEC, 8>, 256, 0);
    if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
    uint64_t grid = std::min<uint64_t>((uint64_t)sm_count * std::max(per_sm, 1), chunks);
    tkv::handoff_copy_vec<VEC, 8><<<(uint32_t)grid, 256, 0, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "no-alloc handoff launch");
    return TKV_OK;
}

}  // namespace

extern "C" int32_t tkv_handoff_noalloc(const TkvPool* s, const TkvPool* d, const TkvBatch* b, const TkvShard* shard,
                                       void* stream) {
    if (!s || !d || !b) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (!s->k_layer_ptrs || !s->v_layer_ptrs || !d->k_layer_ptrs || !d->v_layer_ptrs)
        return fail(TKV_ERR_INVALID_CONFIG, "pool layer pointer arrays must not be NULL");
    const uint32_t es = elem_size(s->dtype);
    if (es == 0 || s->dtype != d->dtype)
        return fail(TKV_ERR_INVALID_CONFIG, "the no-alloc handoff copies between pools of one dtype (src %llu, dst %llu)",
                    (unsigned long long)s->dtype, (unsigned long long)d->dtype);
    if (s->dtype == TKV_DTYPE_E4M3 && (s->k_scales || d->k_scales))
        return fail(TKV_ERR_INVALID_CONFIG, "E4M3 -> E4M3 with scale arrays is not supported");
    if (s->head_dim != d->head_dim)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (head_dim)", s->head_dim, d->head_dim);
    if (s->block_size != d->block_size)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (block_size)", s->block_size, d->block_size);
    if (!s->head_dim || !s->block_size || !s->n_kv_heads || !d->n_kv_heads || !s->n_layers || !d->n_layers)
        return fail(TKV_ERR_INVALID_CONFIG, "zero-sized pool geometry");
    TkvShard sh;
    if (shard) {
        sh = *shard;
    } else {
        sh = TkvShard{0, 0, std::min(s->n_kv_heads, d->n_kv_heads), 0, 0, std::min(s->n_layers, d->n_layers)};
    }
    if (!sh.n_heads || !sh.n_layers) return fail(TKV_ERR_INVALID_CONFIG, "empty shard");
    if ((uint64_t)sh.src_head_begin + sh.n_heads > s->n_kv_heads || (uint64_t)sh.dst_head_begin + sh.n_heads > d->n_kv_heads)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (shard heads exceed pool heads)",
                    std::min(s->n_kv_heads, d->n_kv_heads), sh.n_heads);
    if ((uint64_t)sh.src_layer_begin + sh.n_layers > s->n_layers || (uint64_t)sh.dst_layer_begin + sh.n_layers > d->n_layers)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (shard layers exceed pool layers)",
                    std::min(s->n_layers, d->n_layers), sh.n_layers);
    if (sh.n_layers > TKV_NOALLOC_MAX_LAYERS)
        return fail(TKV_ERR_INVALID_CONFIG, "no-alloc handoff: %llu layers exceed the fixed scratch (at most %llu per call)", sh.n_layers,
                    TKV_NOALLOC_MAX_LAYERS);
    if (b->n_seqs && (!b->seq_lens || !b->src_tables || !b->dst_tables))
        return fail(TKV_ERR_INVALID_CONFIG, "batch arrays must not be NULL");

    const uint32_t bs = s->block_size;
    const uint32_t n_tab = b->table_layer_stride ? sh.n_layers : 1u;
    uint64_t pairs = 0;
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        const uint32_t len = b->seq_lens[q], pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
        if (pre > len) return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: prefix_len %llu exceeds seq_len %llu", q, pre, len);
        if (pre % bs) return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: prefix_len %llu is not a multiple of block_size %llu", q, pre, bs);
        const uint32_t nb = (len + bs - 1) / bs;
        if (nb > b->table_stride)
            return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (sequence %llu needs more blocks than table_stride)",
                        b->table_stride, nb, q);
        pairs += nb - pre / bs;
    }
    if (pairs * n_tab > TKV_NOALLOC_MAX_BLOCK_PAIRS)
        return fail(TKV_ERR_INVALID_CONFIG, "no-alloc handoff: %llu block pairs exceed the fixed scratch (at most %llu per call); split the batch or use a plan",
                    pairs * n_tab, TKV_NOALLOC_MAX_BLOCK_PAIRS);

    // host image of the scratch: [4*L layer pointers][256 B, zeroed][work list]
    const size_t L = sh.n_layers;
    const size_t off_zero = 4 * L * sizeof(uint64_t);
    const size_t off_work = (off_zero + 256 + 15) & ~(size_t)15;
    const size_t used = off_work + (size_t)pairs * n_tab * sizeof(uint4);
    static thread_local std::vector<unsigned char> image;   // host heap only
    static thread_local std::vector<uint8_t> seen;
    image.assign(used, 0);   // the zeroed gap holds the completion counter the kernel's arguments point at
    uint64_t* ptrs = reinterpret_cast<uint64_t*>(image.data());
    for (size_t l = 0; l < L; l++) {
        ptrs[0 * L + l] = s->k_layer_ptrs[sh.src_layer_begin + l];
        ptrs[1 * L + l] = s->v_layer_ptrs[sh.src_layer_begin + l];
        ptrs[2 * L + l] = d->k_layer_ptrs[sh.dst_layer_begin + l];
        ptrs[3 * L + l] = d->v_layer_ptrs[sh.dst_layer_begin + l];
    }
    seen.assign(d->total_blocks, 0);
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        const uint32_t pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
        for (uint32_t i = 0; i < pre / bs; i++) {
            const uint32_t id = b->dst_tables[(size_t)q * b->table_stride + i];
            if (id >= d->total_blocks)
                return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: prefix block id %llu outside destination pool (%llu blocks)", q, id, d->total_blocks);
            seen[id] = 2;
        }
    }
    uint4* work = reinterpret_cast<uint4*>(image.data() + off_work);
    for (uint32_t t = 0; t < n_tab; t++) {
        const size_t so = (size_t)(sh.src_layer_begin + t) * b->table_layer_stride;
        const size_t dof = (size_t)(sh.dst_layer_begin + t) * b->table_layer_stride;
        if (t > 0)
            for (auto& x : seen) x &= 2;
        size_t k = 0;
        for (uint32_t q = 0; q < b->n_seqs; q++) {
            const uint32_t len = b->seq_lens[q], pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
            const uint32_t nb = (len + bs - 1) / bs;
            for (uint32_t i = pre / bs; i < nb; i++) {
                const uint32_t sid = b->src_tables[so + (size_t)q * b->table_stride + i];
                const uint32_t did = b->dst_tables[dof + (size_t)q * b->table_stride + i];
                if (sid >= s->total_blocks)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: source id %llu outside pool (%llu blocks)", q, sid, s->total_blocks);
                if (did >= d->total_blocks)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: destination id %llu outside pool (%llu blocks)", q, did, d->total_blocks);
                if (seen[did] == 2)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: destination id %llu is a shared prefix block of this batch", q, did);
                if (seen[did])
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %llu: destination id %llu written twice in one batch", q, did);
                seen[did] = 1;
                work[(size_t)t * pairs + k++] = make_uint4(sid, did, std::min(bs, len - i * bs), q);
            }
        }
    }
    // as for a plan: a destination on another device must have been mapped by tkv_init or tkv_ipc_import
    if (!tkv_internal::peer_reachable(s->device, d->device) &&
        !(tkv_internal::imported_on(s->device, d->k_layer_ptrs, d->n_layers) && tkv_internal::imported_on(s->device, d->v_layer_ptrs, d->n_layers)))
        return fail(TKV_ERR_INVALID_CONFIG, "device %llu cannot store into device %llu: no peer mapping (call tkv_init with both devices, or map the pool with tkv_ipc_import)",
                    (unsigned long long)s->device, (unsigned long long)d->device);
    if (pairs == 0) return TKV_OK;

    // ---- CUDA from here on; nothing below allocates ----
    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (prev != s->device && (e = cudaSetDevice(s->device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    PerDevice pd;
    int32_t rc = setup(s->device, &pd);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rc == TKV_OK) {
        // The work list is uploaded from this thread's host image, which the next call rewrites: a stream that
        // is recording a graph would keep a pointer to it, so such a call is refused.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        e = cudaStreamIsCapturing(st, &cap);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaStreamIsCapturing");
        else if (cap != cudaStreamCaptureStatusNone)
            rc = fail(TKV_ERR_INVALID_CONFIG, "no-alloc handoff: the stream is being captured; the call uploads from host memory that the next call rewrites");
    }
    if (rc == TKV_OK) {
        unsigned char* base = static_cast<unsigned char*>(pd.scratch);
        e = cudaMemcpyAsync(base, image.data(), used, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) rc = cuda_fail(e, "work list upload");
        if (rc == TKV_OK) {
            tkv::HandoffArgs a{};
            const uint64_t* dp = reinterpret_cast<const uint64_t*>(base);
            a.work = reinterpret_cast<const uint4*>(base + off_work);
            a.src_k = dp + 0 * L;
            a.src_v = dp + 1 * L;
            a.dst_k = dp + 2 * L;
            a.dst_v = dp + 3 * L;
            a.done_counter = reinterpret_cast<uint32_t*>(base + off_zero);
            a.done_flag = nullptr;
            a.src_block_stride = (uint64_t)bs * s->n_kv_heads * s->head_dim * es;
            a.dst_block_stride = (uint64_t)bs * d->n_kv_heads * d->head_dim * es;
            a.n_pairs = (uint32_t)pairs;
            a.work_layer_stride = b->table_layer_stride ? (uint32_t)pairs : 0u;
            a.n_layers = sh.n_layers;
            a.n_heads = sh.n_heads;
            a.head_dim = s->head_dim;
            a.block_size = bs;
            a.src_row_bytes = a.dst_row_bytes = sh.n_heads * s->head_dim * es;
            a.src_row_stride = s->n_kv_heads * s->head_dim * es;
            a.dst_row_stride = d->n_kv_heads * d->head_dim * es;
            a.src_head_off = sh.src_head_begin * s->head_dim * es;
            a.dst_head_off = sh.dst_head_begin * d->head_dim * es;
            a.contiguous = (a.src_row_bytes == a.src_row_stride && a.dst_row_bytes == a.dst_row_stride) ? 1u : 0u;
            int vec = 16;
            auto fits = [&](int v) {
                if (a.src_row_bytes % v || a.src_row_stride % v || a.dst_row_stride % v || a.src_head_off % v || a.dst_head_off % v) return false;
                if (a.src_block_stride % v || a.dst_block_stride % v) return false;
                for (size_t l = 0; l < 4 * L; l++)
                    if (ptrs[l] % v) return false;
                return true;
            };
            while (vec > 1 && !fits(vec)) vec >>= 1;
            const uint64_t chunks = pairs * L * 2;
            switch (vec) {
                case 16: rc = launch<16>(a, pd.sm_count, chunks, st); break;
                case 8: rc = launch<8>(a, pd.sm_count, chunks, st); break;
                case 4: rc = launch<4>(a, pd.sm_count, chunks, st); break;
                case 2: rc = launch<2>(a, pd.sm_count, chunks, st); break;
                default: rc = launch<1>(a, pd.sm_count, chunks, st); break;
            }
        }
    }
    if (prev != s->device) cudaSetDevice(prev);
    return rc;
}
