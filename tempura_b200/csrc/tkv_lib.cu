// Host side of the C ABI declared in include/tkv.h: argument validation, work-list
// construction, launches.  No CPU fallback exists: every entry point that moves KV
// bytes launches a kernel on the source device or returns an error.
#include "tkv_kernels.cuh"

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tkv.h"

namespace {

thread_local std::string g_err;
thread_local int32_t g_cuda_err = 0;

int32_t fail(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

int32_t cuda_fail(cudaError_t e, const char* what) {
    g_cuda_err = (int32_t)e;
    return fail(TKV_ERR_CUDA, "%s: %s (cuda error %d)", what, cudaGetErrorString(e), (int)e);
}

#define CU(call)                                             \
    do {                                                     \
        cudaError_t e_ = (call);                             \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);  \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool ok = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && (prev == dev || cudaSetDevice(dev) == cudaSuccess)) ok = true;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

uint32_t elem_size(int32_t dt) { return dt == TKV_DTYPE_F32 ? 4u : dt == TKV_DTYPE_F16 ? 2u : dt == TKV_DTYPE_E4M3 ? 1u : 0u; }

enum Mode { MODE_COPY, MODE_F16_E4M3, MODE_F32_F16, MODE_F32_E4M3, MODE_E4M3_F16, MODE_E4M3_F32 };

struct DevInfo {
    int sm_count = 0;
};
std::mutex g_mu;
DevInfo g_dev[64];
cudaStream_t g_copy_stream[64] = {};
// g_peer[a][b]: device a may store into device b's memory because THIS library enabled the mapping
// (tkv_init) or opened it (tkv_ipc_import).  cudaDeviceCanAccessPeer only says the hardware could.
bool g_peer[64][64] = {};
// Allocations of other processes opened by tkv_ipc_import: [base, base + size) as seen from `device`.
struct Imported {
    int device;
    uint64_t base, size;
};
std::vector<Imported> g_imported;

int32_t dev_info(int dev, DevInfo* out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (dev < 0 || dev >= 64) return fail(TKV_ERR_INVALID_CONFIG, "device ordinal %d out of range", dev);
    if (g_dev[dev].sm_count == 0) {
        int n = 0;
        CU(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        g_dev[dev].sm_count = n;
    }
    *out = g_dev[dev];
    return TKV_OK;
}

// a non-blocking stream per device for the library's own small copies
int32_t copy_stream(int dev, cudaStream_t* out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (dev < 0 || dev >= 64) return fail(TKV_ERR_INVALID_CONFIG, "device ordinal %d out of range", dev);
    if (!g_copy_stream[dev]) CU(cudaStreamCreateWithFlags(&g_copy_stream[dev], cudaStreamNonBlocking));
    *out = g_copy_stream[dev];
    return TKV_OK;
}

}  // namespace

// Lets other translation units of this library report through tkv_last_error().
namespace tkv_internal {
bool peer_reachable(int from, int to) {
    if (from == to) return true;
    if (from < 0 || to < 0 || from >= 64 || to >= 64) return false;
    std::lock_guard<std::mutex> lk(g_mu);
    return g_peer[from][to];
}
// Every address lies in an allocation that `from` opened through tkv_ipc_import (the mapping itself is what makes it reachable).
bool imported_on(int from, const uint64_t* ptrs, size_t n) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (size_t i = 0; i < n; i++) {
        bool hit = false;
        for (const Imported& m : g_imported)
            if (m.device == from && ptrs[i] >= m.base && ptrs[i] < m.base + m.size) {
                hit = true;
                break;
            }
        if (!hit) return false;
    }
    return n > 0;
}
void note_import(int device, uint64_t base, uint64_t size) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_imported.push_back(Imported{device, base, size});
}
void forget_import(uint64_t base) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (size_t i = 0; i < g_imported.size(); i++)
        if (g_imported[i].base == base) {
            g_imported.erase(g_imported.begin() + i);
            break;
        }
}
void mark_peer(int from, int to) {
    if (from < 0 || to < 0 || from >= 64 || to >= 64) return;
    std::lock_guard<std::mutex> lk(g_mu);
    g_peer[from][to] = true;
}
int32_t set_error(int32_t code, int32_t cuda_code, const char* text) {
    g_err = text ? text : "";
    if (cuda_code) g_cuda_err = cuda_code;
    return code;
}
}  // namespace tkv_internal

struct tkv_plan {
    TkvPool src{}, dst{};
    std::vector<uint64_t> src_k, src_v, dst_k, dst_v;  // owned copies of the layer pointers
    TkvShard shard{};
    uint32_t flags = 0;
    int launch_dev = 0;   // the device whose kernel moves the bytes: the source pool's, or (TKV_PLAN_PULL) the destination pool's
    Mode mode = MODE_COPY;
    uint32_t variant = 0;
    int vec = 16;
    // device block on src.device: [4*L u64 layer ptrs][u32 done counter .. pad 16][work list][prefix ids]
    char* d_buf = nullptr;
    size_t d_cap = 0;
    char* h_buf = nullptr;  // pinned mirror
    size_t h_cap = 0;
    size_t off_work = 0, off_prefix = 0, used = 0;
    // The pinned mirror goes to the device in stream order, at the head of the next enqueue (or
    // refcount launch): `dirty` = mirror newer than the device copy, `upload_ev` = last upload.
    bool dirty = false, upload_pending = false;
    bool list_clobbered = false;   // a device-built work list sits where the host-built one was uploaded
    cudaEvent_t upload_ev = nullptr;
    uint32_t n_pairs = 0, n_prefix = 0;
    tkv::HandoffArgs args{};
    TkvStats stats{};
    uint32_t grid = 0;
    uint32_t bulk_stages = 3, bulk_ctas_per_sm = 0, bulk_stage_bytes = 0;  // ctas 0 = derive from the stage size; stage 0 = 32 KiB, 8 KiB for few chunks
    uint32_t fp8_stages = 2;         // staged FP8 kernel: ring depth per CTA
    uint32_t vec_bytes = 0, vec_unroll = 8, vec_hint = 0;   // register copy kernel: bytes per access (0 = the library's choice), loads in flight per thread, store cache policy
    // Small handoffs: where the completion flag is written from (0 = the library's choice, 1 = by the kernel's last CTA,
    // 2 = by a stream-ordered 32-bit write behind the kernel) and whether a short work list rides in the kernel's parameter
    // block (0 = the library's choice, 1 = never, 2 = whenever it fits).
    uint32_t flag_mode = 0, inline_mode = 0;
    bool ever_uploaded = false;      // the device block (counter, error word, layer pointers) has been initialised once
    uint64_t flag_checked = 0;       // the last completion-flag address classified, and whether a stream write may target it
    bool flag_stream_ok = false;
    uint32_t grid_ctas_per_sm = 0;   // cap for the register kernels (0 = occupancy limit)   // ring depth and residency of the bulk-copy kernel
    std::vector<uint8_t> seen;  // scratch bitmap over destination blocks
    std::vector<char> image;    // host image of the device block, built before any CUDA call
    // Transfer plans: one side is a contiguous transfer buffer, described as a pool whose
    // block ids are 0, 1, 2, ... in work-list order (virt 1 = source side, 2 = destination).
    int virt = 0;
    TkvTransfer xfer{};
    bool host_side = false;     // the transfer buffer is page-locked host memory (and a kernel touches it directly)
    // TKV_PLAN_STAGE_HOST: a host transfer buffer is brought in by the copy engine, one layer (K plane + V plane) at a time into two
    // device buffers, and the handoff kernel of a layer reads its buffer while the next layer's copy runs
    bool staged = false;
    char* stage = nullptr;
    size_t stage_cap = 0, stage_plane = 0;
    uint32_t stage_group = 1;        // layers per staged copy
    std::vector<uint64_t> stage_host;   // per layer: where its K plane starts in the host buffer
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_copied[2] = {nullptr, nullptr}, ev_read[2] = {nullptr, nullptr};
    // device-built work lists (tkv_handoff_enqueue_device_tables): [u32 live pairs][pad][u32 offsets per sequence]
    uint32_t* dev_scratch = nullptr;
    size_t dev_scratch_seqs = 0;
    bool layer_tables = false;  // the batch carried one table per layer
};

namespace {

int32_t validate_pools(const TkvPool* s, const TkvPool* d, const TkvShard& sh, Mode* mode) {
    if (!s->k_layer_ptrs || !s->v_layer_ptrs || !d->k_layer_ptrs || !d->v_layer_ptrs)
        return fail(TKV_ERR_INVALID_CONFIG, "pool layer pointer arrays must not be NULL");
    if (elem_size(s->dtype) == 0 || elem_size(d->dtype) == 0)
        return fail(TKV_ERR_INVALID_CONFIG, "unknown pool dtype (src %d, dst %d)", s->dtype, d->dtype);
    if (s->head_dim != d->head_dim) {
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (head_dim)", s->head_dim, d->head_dim);
    }
    if (s->block_size != d->block_size)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (block_size)", s->block_size, d->block_size);
    if (s->head_dim == 0 || s->block_size == 0 || s->n_kv_heads == 0 || d->n_kv_heads == 0 || s->n_layers == 0 || d->n_layers == 0)
        return fail(TKV_ERR_INVALID_CONFIG, "zero-sized pool geometry");
    if (sh.n_heads == 0 || sh.n_layers == 0) return fail(TKV_ERR_INVALID_CONFIG, "empty shard");
    if ((uint64_t)sh.src_head_begin + sh.n_heads > s->n_kv_heads || (uint64_t)sh.dst_head_begin + sh.n_heads > d->n_kv_heads)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (shard heads exceed pool heads)",
                    std::min(s->n_kv_heads, d->n_kv_heads), sh.n_heads);
    if ((uint64_t)sh.src_layer_begin + sh.n_layers > s->n_layers || (uint64_t)sh.dst_layer_begin + sh.n_layers > d->n_layers)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (shard layers exceed pool layers)",
                    std::min(s->n_layers, d->n_layers), sh.n_layers);
    if (s->dtype == d->dtype) *mode = MODE_COPY;
    else if (s->dtype == TKV_DTYPE_F16 && d->dtype == TKV_DTYPE_E4M3) *mode = MODE_F16_E4M3;
    else if (s->dtype == TKV_DTYPE_F32 && d->dtype == TKV_DTYPE_F16) *mode = MODE_F32_F16;
    else if (s->dtype == TKV_DTYPE_F32 && d->dtype == TKV_DTYPE_E4M3) *mode = MODE_F32_E4M3;
    else if (s->dtype == TKV_DTYPE_E4M3 && d->dtype == TKV_DTYPE_F16) *mode = MODE_E4M3_F16;
    else if (s->dtype == TKV_DTYPE_E4M3 && d->dtype == TKV_DTYPE_F32) *mode = MODE_E4M3_F32;
    else return fail(TKV_ERR_INVALID_CONFIG, "unsupported dtype pair %d -> %d", s->dtype, d->dtype);
    if ((d->k_scales == 0) != (d->v_scales == 0))
        return fail(TKV_ERR_INVALID_CONFIG, "k_scales and v_scales must both be set or both be 0");
    if ((s->k_scales == 0) != (s->v_scales == 0))
        return fail(TKV_ERR_INVALID_CONFIG, "k_scales and v_scales must both be set or both be 0");
    if (*mode == MODE_COPY && s->dtype == TKV_DTYPE_E4M3 && ((d->k_scales == 0) != (s->k_scales == 0)))
        return fail(TKV_ERR_INVALID_CONFIG, "E4M3 -> E4M3: both pools carry per-block scales or neither does");
    return TKV_OK;
}

// Builds the host image of the plan's device block from a batch.
int32_t build_worklist(tkv_plan* p, const TkvBatch* b) {
    const TkvPool &s = p->src, &d = p->dst;
    const TkvShard& sh = p->shard;
    const uint32_t bs = s.block_size;
    if (b->n_seqs && (!b->seq_lens || (!b->src_tables && p->virt != 1) || (!b->dst_tables && p->virt != 2)))
        return fail(TKV_ERR_INVALID_CONFIG, "batch arrays must not be NULL");
    const uint32_t n_tab = b->table_layer_stride ? sh.n_layers : 1u;

    uint64_t pairs = 0, prefix_refs = 0, tokens = 0;
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        uint32_t len = b->seq_lens[q], pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
        if (pre > len) return fail(TKV_ERR_INVALID_CONFIG, "sequence %u: prefix_len %u exceeds seq_len %u", q, pre, len);
        if (pre % bs) return fail(TKV_ERR_INVALID_CONFIG, "sequence %u: prefix_len %u is not a multiple of block_size %u", q, pre, bs);
        uint32_t nb = (len + bs - 1) / bs;
        if (nb > b->table_stride)
            return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (sequence %u needs more blocks than table_stride)",
                        b->table_stride, nb, q);
        pairs += nb - pre / bs;
        if (p->virt != 2) prefix_refs += pre / bs;   // a transfer buffer holds no shared prefix blocks
        tokens += len - pre;
    }
    if (pairs * n_tab > 0x7FFFFFFFull / (2ull * sh.n_layers))
        return fail(TKV_ERR_INVALID_CONFIG, "batch too large: %llu block pairs", (unsigned long long)pairs);

    const size_t L = sh.n_layers;
    if (p->virt) {
        // the transfer buffer as a pool: `pairs` blocks, layer l's K at 2l, V at 2l + 1
        TkvPool& vp = p->virt == 1 ? p->src : p->dst;
        std::vector<uint64_t>& vk = p->virt == 1 ? p->src_k : p->dst_k;
        std::vector<uint64_t>& vv = p->virt == 1 ? p->src_v : p->dst_v;
        const uint64_t plane = pairs * (uint64_t)bs * vp.n_kv_heads * vp.head_dim * elem_size(vp.dtype);
        if (2 * L * plane > p->xfer.bytes)
            return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (transfer buffer bytes)",
                        (unsigned long long)(2 * L * plane), (unsigned long long)p->xfer.bytes);
        if (pairs > 0xFFFFFFFFull) return fail(TKV_ERR_INVALID_CONFIG, "batch too large");
        vp.total_blocks = (uint32_t)pairs;
        vk.resize(L);
        vv.resize(L);
        if (p->staged) {
            // Layers travel in groups of G (one copy of at least 4 MiB where the layers are small); group g is read from device
            // buffer g % 2; the host address of each group's planes is kept for the copies.
            const size_t G = std::min<size_t>(std::max<size_t>(L, 1), std::max<size_t>(1, ((4u << 20) + 2 * plane - 1) / std::max<size_t>(2 * plane, 1)));
            if (4 * G * plane > p->stage_cap) {
                DeviceGuard g(p->launch_dev);
                if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->launch_dev);
                if (p->stage) {
                    CU(cudaDeviceSynchronize());               // a larger batch than the plan was made for: nothing may still read the old buffers
                    CU(cudaFree(p->stage));
                    p->stage = nullptr;
                    p->stage_cap = 0;
                }
                const size_t cap = std::max<size_t>(4 * G * plane, 256);
                CU(cudaMalloc(&p->stage, cap));
                p->stage_cap = cap;
            }
            p->stage_plane = plane;
            p->stage_group = (uint32_t)G;
            p->stage_host.resize(L);
            for (size_t l = 0; l < L; l++) {
                p->stage_host[l] = p->xfer.data + (2 * l) * plane;
                vk[l] = reinterpret_cast<uint64_t>(p->stage) + (((l / G) & 1) * G + l % G) * 2 * plane;
                vv[l] = vk[l] + plane;
            }
        } else {
            for (size_t l = 0; l < L; l++) {
                vk[l] = p->xfer.data + (2 * l) * plane;
                vv[l] = p->xfer.data + (2 * l + 1) * plane;
            }
        }
        vp.k_layer_ptrs = vk.data();
        vp.v_layer_ptrs = vv.data();
        if (p->xfer.scales) {
            vp.k_scales = p->xfer.scales;
            vp.v_scales = p->xfer.scales + L * pairs * vp.n_kv_heads * sizeof(float);
        }
    }
    const size_t off_counter = 4 * L * sizeof(uint64_t);
    const size_t off_work = (off_counter + 16 + 15) & ~(size_t)15;
    const size_t off_prefix = off_work + (size_t)pairs * n_tab * sizeof(uint4);
    const size_t need = off_prefix + (size_t)prefix_refs * sizeof(uint32_t) + 16;

    p->image.assign(need, 0);
    char* h = p->image.data();
    uint64_t* ptrs = reinterpret_cast<uint64_t*>(h);
    for (size_t l = 0; l < L; l++) {
        ptrs[0 * L + l] = p->src_k[sh.src_layer_begin + l];
        ptrs[1 * L + l] = p->src_v[sh.src_layer_begin + l];
        ptrs[2 * L + l] = p->dst_k[sh.dst_layer_begin + l];
        ptrs[3 * L + l] = p->dst_v[sh.dst_layer_begin + l];
    }
    memset(h + off_counter, 0, off_work - off_counter);

    // destination blocks written by this call must be unique and must not be
    // one of the call's own shared prefix blocks
    const bool check_unique = !(p->flags & TKV_PLAN_ALLOW_SHARED_DST);
    p->seen.assign(d.total_blocks, 0);
    uint32_t* pre_ids = reinterpret_cast<uint32_t*>(h + off_prefix);
    size_t np = 0;
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        uint32_t pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
        for (uint32_t i = 0; i < pre / bs && p->virt != 2; i++) {
            uint32_t id = b->dst_tables[(size_t)q * b->table_stride + i];
            if (id >= d.total_blocks)
                return fail(TKV_ERR_INVALID_CONFIG, "sequence %u: prefix block id %u outside destination pool (%u blocks)", q, id, d.total_blocks);
            p->seen[id] = 2;
            pre_ids[np++] = id;
        }
    }
    uint4* work = reinterpret_cast<uint4*>(h + off_work);
    for (uint32_t t = 0; t < n_tab; t++) {
        const size_t so = (size_t)(sh.src_layer_begin + t) * b->table_layer_stride;
        const size_t dof = (size_t)(sh.dst_layer_begin + t) * b->table_layer_stride;
        if (t > 0 && check_unique)
            for (auto& x : p->seen) x &= 2;
        size_t k = 0;
        for (uint32_t q = 0; q < b->n_seqs; q++) {
            uint32_t len = b->seq_lens[q], pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
            uint32_t nb = (len + bs - 1) / bs;
            for (uint32_t i = pre / bs; i < nb; i++) {
                uint32_t sid = p->virt == 1 ? (uint32_t)k : b->src_tables[so + (size_t)q * b->table_stride + i];
                uint32_t did = p->virt == 2 ? (uint32_t)k : b->dst_tables[dof + (size_t)q * b->table_stride + i];
                if (sid >= s.total_blocks)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %u block %u: source id %u outside pool (%u blocks)", q, i, sid, s.total_blocks);
                if (did >= d.total_blocks)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %u block %u: destination id %u outside pool (%u blocks)", q, i, did, d.total_blocks);
                if (p->seen[did] == 2)
                    return fail(TKV_ERR_INVALID_CONFIG, "sequence %u block %u: destination id %u is a shared prefix block of this batch", q, i, did);
                if (check_unique) {
                    if (p->seen[did])
                        return fail(TKV_ERR_INVALID_CONFIG, "sequence %u block %u: destination id %u written twice in one batch", q, i, did);
                    p->seen[did] = 1;
                }
                uint32_t valid = std::min(bs, len - i * bs);
                work[(size_t)t * pairs + k++] = make_uint4(sid, did, valid, q);
            }
        }
    }

    p->off_work = off_work;
    p->off_prefix = off_prefix;
    p->used = need;
    p->n_pairs = (uint32_t)pairs;
    p->n_prefix = (uint32_t)prefix_refs;

    // A kernel on the source device stores into the destination pool: refuse a pair whose peer mapping this
    // library has not set up, rather than launch stores at addresses the device cannot reach.
    const bool pull = (p->flags & TKV_PLAN_PULL) != 0;
    p->launch_dev = pull ? d.device : s.device;
    const int far_dev = pull ? s.device : d.device;
    const std::vector<uint64_t>&far_k = pull ? p->src_k : p->dst_k, &far_v = pull ? p->src_v : p->dst_v;
    if (!tkv_internal::peer_reachable(p->launch_dev, far_dev) && !(tkv_internal::imported_on(p->launch_dev, far_k.data(), far_k.size()) &&
                                                                  tkv_internal::imported_on(p->launch_dev, far_v.data(), far_v.size())))
        return fail(TKV_ERR_INVALID_CONFIG, "device %d cannot %s device %d: no peer mapping (call tkv_init with both devices, or map the pool with tkv_ipc_import)",
                    p->launch_dev, pull ? "load from" : "store into", far_dev);
    if (pull && (p->mode != MODE_COPY || p->virt || (p->flags & (TKV_PLAN_FORCE_BULK | TKV_PLAN_PEER_BULK_STORES))))
        return fail(TKV_ERR_INVALID_CONFIG, "TKV_PLAN_PULL is for same-dtype pool-to-pool moves with the register kernels (no bulk copy reads a peer's memory)");
    // ---- everything above is pure host logic; CUDA starts here ----
    {
        DeviceGuard g(p->launch_dev);
        if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->launch_dev);
        if (!p->upload_ev) CU(cudaEventCreateWithFlags(&p->upload_ev, cudaEventDisableTiming));
        // the previous upload must have left the pinned mirror before it is rewritten
        if (p->upload_pending) {
            CU(cudaEventSynchronize(p->upload_ev));
            p->upload_pending = false;
        }
        if (need > p->h_cap) {
            size_t cap = std::max(need, p->h_cap * 2);
            if (p->h_buf) cudaFreeHost(p->h_buf);
            if (p->d_buf) cudaFree(p->d_buf);
            p->h_buf = nullptr;
            p->d_buf = nullptr;
            p->h_cap = p->d_cap = 0;
            CU(cudaMallocHost((void**)&p->h_buf, cap));
            CU(cudaMalloc((void**)&p->d_buf, cap));
            CU(cudaMemset(p->d_buf, 0, cap));
            p->h_cap = p->d_cap = cap;
        }
        memcpy(p->h_buf, p->image.data(), need);
        p->dirty = true;
    }

    // kernel arguments
    tkv::HandoffArgs& a = p->args;
    const uint32_t se = elem_size(s.dtype), de = elem_size(d.dtype);
    const uint64_t* dp = reinterpret_cast<const uint64_t*>(p->d_buf);
    a.work = reinterpret_cast<const uint4*>(p->d_buf + off_work);
    a.src_k = dp + 0 * L;
    a.src_v = dp + 1 * L;
    a.dst_k = dp + 2 * L;
    a.dst_v = dp + 3 * L;
    a.dst_k_scales = reinterpret_cast<float*>(d.k_scales);
    a.dst_v_scales = reinterpret_cast<float*>(d.v_scales);
    const bool dequant = p->mode == MODE_E4M3_F16 || p->mode == MODE_E4M3_F32;
    const bool carry_scales = (p->mode == MODE_COPY && s.dtype == TKV_DTYPE_E4M3 && s.k_scales && d.k_scales) || (dequant && s.k_scales);
    a.src_k_scales = carry_scales ? reinterpret_cast<const float*>(s.k_scales) : nullptr;
    a.src_v_scales = carry_scales ? reinterpret_cast<const float*>(s.v_scales) : nullptr;
    a.src_total_blocks = s.total_blocks;
    a.src_pool_heads = s.n_kv_heads;
    a.src_head_begin = sh.src_head_begin;
    a.src_layer_begin = sh.src_layer_begin;
    a.done_counter = reinterpret_cast<uint32_t*>(p->d_buf + off_counter);
    a.done_flag = nullptr;
    a.src_block_stride = (uint64_t)bs * s.n_kv_heads * s.head_dim * se;
    a.dst_block_stride = (uint64_t)bs * d.n_kv_heads * d.head_dim * de;
    a.n_pairs = (uint32_t)pairs;
    a.work_layer_stride = b->table_layer_stride ? (uint32_t)pairs : 0u;
    p->layer_tables = b->table_layer_stride != 0;
    a.n_layers = sh.n_layers;
    a.n_heads = sh.n_heads;
    a.head_dim = s.head_dim;
    a.block_size = bs;
    a.src_row_bytes = sh.n_heads * s.head_dim * se;
    a.dst_row_bytes = sh.n_heads * s.head_dim * de;
    a.src_row_stride = s.n_kv_heads * s.head_dim * se;
    a.dst_row_stride = d.n_kv_heads * d.head_dim * de;
    a.src_head_off = sh.src_head_begin * s.head_dim * se;
    a.dst_head_off = sh.dst_head_begin * d.head_dim * de;
    a.dst_total_blocks = d.total_blocks;
    a.dst_pool_heads = d.n_kv_heads;
    a.dst_head_begin = sh.dst_head_begin;
    a.dst_layer_begin = sh.dst_layer_begin;
    a.flag_value = 0;
    a.contiguous = (a.src_row_bytes == a.src_row_stride && a.dst_row_bytes == a.dst_row_stride) ? 1u : 0u;
    a.local_fences = (s.device == d.device && !p->host_side) ? 1u : 0u;

    // widest vector that divides every offset and address involved
    int vec = 16;
    auto fits = [&](int v) {
        if (a.src_row_bytes % v || a.src_row_stride % v || a.dst_row_stride % v || a.src_head_off % v || a.dst_head_off % v) return false;
        if (a.src_block_stride % v || a.dst_block_stride % v) return false;
        for (size_t l = 0; l < 4 * L; l++)
            if (ptrs[l] % v) return false;
        return true;
    };
    while (vec > 1 && !fits(vec)) vec >>= 1;
    p->vec = vec;

    TkvStats& st = p->stats;
    st = TkvStats{};
    st.n_blocks = pairs;
    st.n_chunks = pairs * L * 2;
    st.n_tokens = tokens;
    st.n_prefix_refs = prefix_refs;
    st.payload_bytes = tokens * L * 2ull * a.src_row_bytes;
    st.bytes_read = st.payload_bytes;
    st.bytes_written = tokens * L * 2ull * a.dst_row_bytes;
    if (p->mode == MODE_F16_E4M3 && d.k_scales) st.bytes_written += pairs * L * 2ull * sh.n_heads * sizeof(float);
    if (carry_scales) {
        st.bytes_read += pairs * L * 2ull * sh.n_heads * sizeof(float);
        if (!dequant) st.bytes_written += pairs * L * 2ull * sh.n_heads * sizeof(float);
    }
    st.worklist_bytes = need;
    st.peer = s.device != d.device;
    return TKV_OK;
}

// Puts the plan's work list on the device in the order of `st`, ahead of whatever is launched
// next on it; a stream that did not carry the upload waits for it.
int32_t ensure_uploaded(tkv_plan* p, cudaStream_t st, bool need_host_list = true) {
    if (p->dirty || (need_host_list && p->list_clobbered)) {
        CU(cudaMemcpyAsync(p->d_buf, p->h_buf, p->used, cudaMemcpyHostToDevice, st));
        CU(cudaEventRecord(p->upload_ev, st));
        p->dirty = false;
        p->list_clobbered = false;
        p->upload_pending = true;
        p->ever_uploaded = true;
    } else if (p->upload_pending) {
        CU(cudaStreamWaitEvent(st, p->upload_ev, 0));
    }
    return TKV_OK;
}

// cudaFuncSetAttribute is a driver call; remember the largest dynamic shared memory size granted
// to each kernel on each device and only raise it.
template <typename K> int32_t grant_smem(K kernel, int dev, size_t smem) {
    static std::mutex mu;
    static std::vector<std::pair<const void*, size_t>> granted[64];
    std::lock_guard<std::mutex> lk(mu);
    const void* key = reinterpret_cast<const void*>(kernel);
    for (auto& g : granted[dev])
        if (g.first == key) {
            if (g.second >= smem) return TKV_OK;
            CU(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            g.second = smem;
            return TKV_OK;
        }
    CU(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    granted[dev].push_back({key, smem});
    return TKV_OK;
}

template <typename K> int32_t occupancy_grid(K kernel, int dev, uint64_t work_ctas, uint32_t* grid) {
    DevInfo di;
    int32_t rc = dev_info(dev, &di);
    if (rc) return rc;
    int per_sm = 0;
    CU(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0));
    if (per_sm < 1) per_sm = 1;
    uint64_t g = (uint64_t)di.sm_count * per_sm;
    *grid = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(g, work_ctas));
    return TKV_OK;
}

template <typename K> int32_t launch(K kernel, tkv_plan* p, uint64_t work_ctas, cudaStream_t st) {
    uint32_t grid = 0;
    int32_t rc = occupancy_grid(kernel, p->launch_dev, work_ctas, &grid);
    if (rc) return rc;
    // Measured on B200 (Llama-3.1-8B shape): the FP8 warp kernel peaks at 3 resident CTAs per
    // SM (90.7 % of the copy peak against 83 % at the occupancy limit of 4).
    // ... and the vectorized F32 cast at 4 (92.8 % against 91.5 % at the occupancy limit of 8).
    uint32_t cap = p->grid_ctas_per_sm ? p->grid_ctas_per_sm
                                       : (p->variant == TKV_VARIANT_FP8_WARP ? 3u : p->variant == TKV_VARIANT_CAST_VEC ? 4u : 0u);
    if (cap) {
        DevInfo di;
        rc = dev_info(p->launch_dev, &di);
        if (rc) return rc;
        grid = std::max(1u, std::min(grid, (uint32_t)di.sm_count * cap));
    }
    p->grid = grid;
    kernel<<<grid, 256, 0, st>>>(p->args);
    CU(cudaGetLastError());
    return TKV_OK;
}

// Bulk-copy variant: only for same-device, contiguous, 16-byte aligned chunks.
bool bulk_eligible(const tkv_plan* p) {
    const bool reach = (p->src.device == p->dst.device || (p->flags & TKV_PLAN_PEER_BULK_STORES)) && !(p->flags & TKV_PLAN_PULL);
    // a host-memory side takes the ring only when asked to (TKV_PLAN_FORCE_BULK)
    const bool host_ok = !p->host_side || (p->flags & TKV_PLAN_FORCE_BULK);
    return p->mode == MODE_COPY && p->args.contiguous && p->vec == 16 && reach && host_ok && p->args.src_k_scales == nullptr;
}

// The work list fits the kernel's parameter block: one list for all layers, built on the host, short enough.
bool inline_eligible(const tkv_plan* p) {
    const tkv::HandoffArgs& a = p->args;
    if (p->inline_mode == 1 || a.n_pairs_dev != nullptr || a.work_layer_stride != 0 || p->staged) return false;
    if (a.n_pairs > tkv::INLINE_PAIRS || a.n_layers > tkv::INLINE_LAYERS) return false;
    if (p->inline_mode == 2) return true;
    // the library's choice: only where the list fetch is a visible share of the launch (few chunks per SM)
    DevInfo di;
    if (dev_info(p->launch_dev, &di)) return false;
    return (uint64_t)a.n_pairs * a.n_layers * 2 <= 16ull * di.sm_count;
}

// A 32-bit write the stream performs behind everything enqueued before it (cuStreamWriteValue32: the driver orders it
// after the preceding kernel's writes at system scope).  Taken from the driver by name; 0 where the driver lacks it.
typedef int (*write_value_fn)(cudaStream_t, unsigned long long, unsigned int, unsigned int);
write_value_fn stream_write_value() {
    static write_value_fn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &f, cudaEnableDefault, &qr) != cudaSuccess) f = nullptr;
        cudaGetLastError();
        return reinterpret_cast<write_value_fn>(f);
    }();
    return fn;
}

// May the completion flag at `flag` be written by a stream operation of the launching device?  Yes for that device's own
// memory and for page-locked host memory whose device address equals its host address; a peer GPU's word stays with the
// kernel's last CTA (whose release store is known to reach it).
bool flag_by_stream(tkv_plan* p, uint64_t flag) {
    if (p->flag_mode == 1 || !flag || !stream_write_value()) return false;
    if (p->flag_checked == flag) return p->flag_stream_ok;
    p->flag_checked = flag;
    p->flag_stream_ok = false;
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, reinterpret_cast<void*>(flag)) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (at.type == cudaMemoryTypeDevice) p->flag_stream_ok = at.device == p->launch_dev;
    else if (at.type == cudaMemoryTypeHost) p->flag_stream_ok = reinterpret_cast<uint64_t>(at.devicePointer) == flag;
    return p->flag_stream_ok;
}

int32_t launch_bulk(tkv_plan* p, cudaStream_t st) {
    const tkv::HandoffArgs& a = p->args;
    DevInfo di;
    int32_t rc = dev_info(p->launch_dev, &di);
    if (rc) return rc;
    const uint32_t chunk = a.block_size * a.src_row_bytes;
    // Few chunks per SM: cut them into 8 KiB pieces so that every SM carries loads from the first cycle and the last
    // piece of the slowest CTA is short.
    const uint64_t n_chunks = (uint64_t)a.n_pairs * a.n_layers * 2;
    const uint32_t stage_cap = p->bulk_stage_bytes ? p->bulk_stage_bytes : (n_chunks < 4ull * di.sm_count ? 8192u : 32768u);
    const uint32_t stage = std::min<uint32_t>(stage_cap, (chunk + 127u) & ~127u);
    const uint32_t pieces = (chunk + stage - 1) / stage;
    const uint32_t stages = std::max(2u, std::min(8u, p->bulk_stages));
    const size_t smem = 64 + 64 * sizeof(tkv::BulkItem) + (size_t)stages * stage;
    if (smem > 227 * 1024) return fail(TKV_ERR_INVALID_CONFIG, "bulk ring of %u x %u bytes exceeds shared memory", stages, stage);
    rc = grant_smem(tkv::handoff_copy_bulk, p->launch_dev, smem);
    if (rc) return rc;
    // Measured on B200: throughput peaks near 96 KiB of ring per SM (3 x 32 KiB, one CTA) and
    // falls off when more is in flight, so smaller stages get proportionally more CTAs.
    uint32_t want = p->bulk_ctas_per_sm ? p->bulk_ctas_per_sm : std::max(1u, 98304u / (stages * stage));
    uint32_t per_sm = std::max<uint32_t>(1u, std::min<uint32_t>(std::min(want, 8u), (uint32_t)((227 * 1024) / (smem + 1024))));
    const uint64_t items = (uint64_t)a.n_pairs * a.n_layers * 2 * pieces;
    p->grid = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)di.sm_count * per_sm, items));
    p->variant = TKV_VARIANT_BULK;
    uint32_t* err = a.done_counter + 1;   // second word of the zeroed slot in the plan's device block
    if (inline_eligible(p)) {
        rc = grant_smem(tkv::handoff_copy_bulk_inline, p->launch_dev, smem);
        if (rc) return rc;
        static thread_local tkv::InlineList il;
        const size_t L = a.n_layers;
        const uint64_t* ptrs = reinterpret_cast<const uint64_t*>(p->h_buf);           // [src K | src V | dst K | dst V][L]
        for (int k = 0; k < 4; k++) memcpy(il.ptr[k], ptrs + k * L, L * sizeof(uint64_t));
        memcpy(il.pairs, p->h_buf + p->off_work, (size_t)a.n_pairs * sizeof(uint4));
        tkv::handoff_copy_bulk_inline<<<p->grid, 32, smem, st>>>(a, il, stage, stages, pieces, err);
    } else {
        tkv::handoff_copy_bulk<<<p->grid, 32, smem, st>>>(a, stage, stages, pieces, err);
    }
    CU(cudaGetLastError());
    return TKV_OK;
}

// Shared-memory staged FP8 variant: whole rows at the source (one contiguous run per chunk),
// 16 tokens per block, device memory on the source side, and a ring that fits shared memory.
bool staged_eligible(const tkv_plan* p, uint32_t* stages_out, size_t* smem_out) {
    const tkv::HandoffArgs& a = p->args;
    if (p->mode != MODE_F16_E4M3 || a.block_size != 16 || p->vec != 16) return false;
    if (a.head_dim != 64 && a.head_dim != 128 && a.head_dim != 256) return false;
    if (a.src_row_bytes != a.src_row_stride || p->host_side) return false;
    const size_t in = 16 * (size_t)a.src_row_bytes, out = 16 * (size_t)a.dst_row_bytes;
    // Measured on B200 (Llama-3.1-8B shape): the encode needs 16 resident warps per SM; two CTAs
    // with a 2-deep ring each reach 1.00 of the copy peak, one CTA with any ring depth 0.76.
    uint32_t stages = std::max(2u, std::min(8u, p->fp8_stages));
    while (stages > 2 && 2176 + stages * in + 2 * out > 200 * 1024) stages--;
    const size_t smem = 2176 + stages * in + 2 * out;
    if (smem > 227 * 1024 || in >= (1u << 20)) return false;
    *stages_out = stages;
    *smem_out = smem;
    return true;
}

template <int D, bool HW, bool SCALED> int32_t launch_fp8_staged(tkv_plan* p, uint32_t stages, size_t smem, cudaStream_t st) {
    const tkv::HandoffArgs& a = p->args;
    DevInfo di;
    int32_t rc = dev_info(p->launch_dev, &di);
    if (rc) return rc;
    auto kernel = tkv::handoff_f16_e4m3_staged<D, HW, SCALED>;
    rc = grant_smem(kernel, p->launch_dev, smem);
    if (rc) return rc;
    uint32_t per_sm = std::max<uint32_t>(1u, (uint32_t)((227 * 1024) / (smem + 1024)));
    if (p->bulk_ctas_per_sm) per_sm = std::min(per_sm, p->bulk_ctas_per_sm);
    per_sm = std::min(per_sm, 8u);
    const uint64_t chunks = (uint64_t)a.n_pairs * a.n_layers * 2;
    p->grid = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)di.sm_count * per_sm, chunks));
    p->variant = TKV_VARIANT_FP8_STAGED;
    // Whole destination rows leave as one bulk store, on this device or on a peer (measured over
    // NVLink on the Llama-3.1-8B shape: 704 GB/s on the wire against 690 GB/s with register stores).
    const uint32_t bulk_store = a.dst_row_bytes == a.dst_row_stride ? 1u : 0u;
    uint32_t* err = a.done_counter + 1;
    kernel<<<p->grid, 256, smem, st>>>(a, stages, bulk_store, err);
    CU(cudaGetLastError());
    return TKV_OK;
}

template <bool HW, bool SCALED> int32_t launch_fp8(tkv_plan* p, cudaStream_t st) {
    const tkv::HandoffArgs& a = p->args;
    const uint64_t warps = (uint64_t)a.n_pairs * a.n_layers * 2 * a.n_heads;
    const uint64_t ctas = (warps + 7) / 8;
    uint32_t stages = 0;
    size_t smem = 0;
    const bool can_stage = staged_eligible(p, &stages, &smem);
    if ((p->flags & TKV_PLAN_FORCE_BULK) && !can_stage)
        return fail(TKV_ERR_INVALID_CONFIG, "the staged FP8 kernel needs whole source rows in device memory, 16-token blocks, head_dim 64/128/256 and 16-byte alignment");
    if (can_stage && !(p->flags & TKV_PLAN_FORCE_VECTOR)) {
        if (a.head_dim == 128) return launch_fp8_staged<128, HW, SCALED>(p, stages, smem, st);
        if (a.head_dim == 64) return launch_fp8_staged<64, HW, SCALED>(p, stages, smem, st);
        return launch_fp8_staged<256, HW, SCALED>(p, stages, smem, st);
    }
    const bool fast = p->vec == 16 && a.block_size == 16;
    if (fast && a.head_dim == 128) {
        p->variant = TKV_VARIANT_FP8_WARP;
        return launch(tkv::handoff_f16_e4m3_warp<128, 16, HW, SCALED>, p, ctas, st);
    }
    if (fast && a.head_dim == 64) {
        p->variant = TKV_VARIANT_FP8_WARP;
        return launch(tkv::handoff_f16_e4m3_warp<64, 16, HW, SCALED>, p, ctas, st);
    }
    if (fast && a.head_dim == 256) {
        p->variant = TKV_VARIANT_FP8_WARP;
        return launch(tkv::handoff_f16_e4m3_warp<256, 16, HW, SCALED>, p, ctas, st);
    }
    p->variant = TKV_VARIANT_FP8_GENERIC;
    return launch(tkv::handoff_f16_e4m3_generic<HW, SCALED>, p, ctas, st);
}

// 32-byte accesses: contiguous chunks whose addresses and strides all keep 32-byte alignment, no scales riding along.
bool wide_eligible(const tkv_plan* p) {
    const tkv::HandoffArgs& a = p->args;
    if (p->vec_bytes != 32 || p->mode != MODE_COPY || !a.contiguous || p->vec != 16 || a.src_k_scales != nullptr) return false;
    if (a.src_row_bytes % 32 || a.src_block_stride % 32 || a.dst_block_stride % 32 || a.src_head_off % 32 || a.dst_head_off % 32) return false;
    const uint64_t* ptrs = reinterpret_cast<const uint64_t*>(p->h_buf);
    for (size_t l = 0; l < 4 * (size_t)a.n_layers; l++)
        if (ptrs[l] % 32) return false;
    return true;
}

int32_t launch_wide(tkv_plan* p, uint64_t chunks, cudaStream_t st) {
    const uint32_t u = p->vec_unroll, h = p->vec_hint;
#define TKV_WIDE(U, H) \
    if (u == U && h == H) return launch(tkv::handoff_copy_wide<U, H>, p, chunks, st);
    TKV_WIDE(4, 0) TKV_WIDE(4, 1) TKV_WIDE(4, 2) TKV_WIDE(8, 0) TKV_WIDE(8, 1) TKV_WIDE(8, 2) TKV_WIDE(16, 0) TKV_WIDE(16, 1) TKV_WIDE(16, 2)
#undef TKV_WIDE
    return fail(TKV_ERR_INVALID_CONFIG, "no 32-byte copy kernel for unroll %u, store hint %u", u, h);
}

}  // namespace

static int32_t dispatch(tkv_plan* p, uint64_t chunks, cudaStream_t st);

extern "C" {

void tkv_last_error(char* buf, size_t len) {
    if (!buf || !len) return;
    snprintf(buf, len, "%s", g_err.c_str());
}
int32_t tkv_last_cuda_error(void) { return g_cuda_err; }
const char* tkv_version(void) { return "tkv 0.1 (sm_100a)"; }

int32_t tkv_init(const int32_t* devices, int32_t n) {
    if (n < 0 || (n > 0 && !devices)) return fail(TKV_ERR_INVALID_CONFIG, "bad device list");
    int count = 0;
    CU(cudaGetDeviceCount(&count));
    for (int i = 0; i < n; i++)
        if (devices[i] < 0 || devices[i] >= count)
            return fail(TKV_ERR_INVALID_CONFIG, "device %d not present (%d devices)", devices[i], count);
    int prev = 0;
    CU(cudaGetDevice(&prev));
    for (int i = 0; i < n; i++) {
        for (int j = 0; j < n; j++) {
            if (i == j || devices[i] == devices[j]) continue;
            int can = 0;
            CU(cudaDeviceCanAccessPeer(&can, devices[i], devices[j]));
            if (!can) {
                cudaSetDevice(prev);
                return fail(TKV_ERR_INVALID_CONFIG, "device %d cannot access device %d as a peer", devices[i], devices[j]);
            }
            CU(cudaSetDevice(devices[i]));
            cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) {
                cudaGetLastError();
            } else if (e != cudaSuccess) {
                cudaSetDevice(prev);
                return cuda_fail(e, "cudaDeviceEnablePeerAccess");
            }
            tkv_internal::mark_peer(devices[i], devices[j]);
        }
    }
    CU(cudaSetDevice(prev));
    return TKV_OK;
}

int32_t tkv_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    int prev = 0;
    cudaGetDevice(&prev);
    for (int d = 0; d < 64; d++)
        if (g_copy_stream[d]) {
            cudaSetDevice(d);
            cudaStreamDestroy(g_copy_stream[d]);
            g_copy_stream[d] = nullptr;
        }
    cudaSetDevice(prev);
    return TKV_OK;
}

static int32_t create_plan(const TkvPool* src, const TkvPool* dst, const TkvBatch* batch, const TkvShard* shard,
                           uint32_t flags, int virt, const TkvTransfer* xfer, tkv_plan** out) {
    *out = nullptr;
    TkvShard sh;
    if (shard) {
        sh = *shard;
    } else {
        sh.src_head_begin = sh.dst_head_begin = 0;
        sh.n_heads = std::min(src->n_kv_heads, dst->n_kv_heads);
        sh.src_layer_begin = sh.dst_layer_begin = 0;
        sh.n_layers = std::min(src->n_layers, dst->n_layers);
    }
    Mode mode;
    int32_t rc = validate_pools(src, dst, sh, &mode);
    if (rc) return rc;
    if ((flags & TKV_PLAN_FORCE_VECTOR) && (flags & TKV_PLAN_FORCE_BULK))
        return fail(TKV_ERR_INVALID_CONFIG, "FORCE_VECTOR and FORCE_BULK are exclusive");
    tkv_plan* p = new tkv_plan();
    p->src = *src;
    p->dst = *dst;
    if (virt != 1) {
        p->src_k.assign(src->k_layer_ptrs, src->k_layer_ptrs + src->n_layers);
        p->src_v.assign(src->v_layer_ptrs, src->v_layer_ptrs + src->n_layers);
    }
    if (virt != 2) {
        p->dst_k.assign(dst->k_layer_ptrs, dst->k_layer_ptrs + dst->n_layers);
        p->dst_v.assign(dst->v_layer_ptrs, dst->v_layer_ptrs + dst->n_layers);
    }
    p->src.k_layer_ptrs = p->src_k.data();
    p->src.v_layer_ptrs = p->src_v.data();
    p->dst.k_layer_ptrs = p->dst_k.data();
    p->dst.v_layer_ptrs = p->dst_v.data();
    p->shard = sh;
    p->flags = flags;
    p->mode = mode;
    p->virt = virt;
    if (flags & TKV_PLAN_PULL) {
        // measured over NVLink (Llama-3.1-70B shape, one pair): 32-byte loads, 16 in flight per thread, one CTA per SM
        // fetch 786 GB/s; 16-byte loads 770; stores pushed the other way stop at 718 whatever their shape
        p->vec_bytes = 32;
        p->vec_unroll = 16;
    }
    if (xfer) {
        p->xfer = *xfer;
        p->host_side = xfer->host_memory != 0;
    }
    if (flags & TKV_PLAN_STAGE_HOST) {
        if (virt != 1 || !p->host_side || src->k_scales) {
            delete p;
            return fail(TKV_ERR_INVALID_CONFIG, "TKV_PLAN_STAGE_HOST is for plans that read a host transfer buffer without scales");
        }
        p->staged = true;
        p->host_side = false;          // the kernels read device memory
        p->launch_dev = src->device;
        DeviceGuard g(p->launch_dev);
        cudaError_t e = g.ok ? cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking) : cudaErrorInvalidDevice;
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_begin, cudaEventDisableTiming);
        for (int i = 0; i < 2 && e == cudaSuccess; i++) {
            e = cudaEventCreateWithFlags(&p->ev_copied[i], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_read[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) {
            tkv_plan_destroy(p);
            return fail(TKV_ERR_CUDA, "staging stream / events: %s", cudaGetErrorString(e));
        }
    }
    rc = build_worklist(p, batch);
    if (rc) {
        tkv_plan_destroy(p);
        return rc;
    }
    *out = p;
    return TKV_OK;
}

int32_t tkv_plan_create(const TkvPool* src, const TkvPool* dst, const TkvBatch* batch, const TkvShard* shard,
                        uint32_t flags, tkv_plan** out) {
    if (!src || !dst || !batch || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    return create_plan(src, dst, batch, shard, flags, 0, nullptr, out);
}

// The transfer buffer described as a pool that holds exactly the shard: same geometry as
// `like`, the shard's heads and layers only, block ids assigned later in work-list order.
static int32_t transfer_as_pool(const TkvTransfer* x, const TkvPool* like, const TkvShard* shard, int side,
                                TkvPool* vp, TkvShard* sh) {
    if (!x->data) return fail(TKV_ERR_INVALID_CONFIG, "transfer buffer address is 0");
    if (x->device < 0) return fail(TKV_ERR_INVALID_CONFIG, "transfer buffer names no device");
    if (side == 2 && x->host_memory && x->device != like->device)
        return fail(TKV_ERR_INVALID_CONFIG, "a host transfer buffer is written by the source pool's device %d, not %d", like->device, x->device);
    if (elem_size(x->dtype) == 0) return fail(TKV_ERR_INVALID_CONFIG, "unknown transfer dtype %d", x->dtype);
    if (x->scales && x->dtype != TKV_DTYPE_E4M3) return fail(TKV_ERR_INVALID_CONFIG, "only an E4M3 transfer buffer carries scales");
    if (shard) {
        *sh = *shard;
    } else {
        *sh = TkvShard{0, 0, like->n_kv_heads, 0, 0, like->n_layers};
    }
    // the buffer's own numbering starts at 0 whatever slice of the pool it holds
    if (side == 1) {
        sh->src_head_begin = 0;
        sh->src_layer_begin = 0;
    } else {
        sh->dst_head_begin = 0;
        sh->dst_layer_begin = 0;
    }
    *vp = TkvPool{};
    vp->device = x->device;
    vp->dtype = x->dtype;
    vp->n_layers = sh->n_layers;
    vp->n_kv_heads = sh->n_heads;
    vp->head_dim = like->head_dim;
    vp->block_size = like->block_size;
    vp->total_blocks = 0;
    static const uint64_t none = 0;
    vp->k_layer_ptrs = &none;   // placeholders; the real addresses depend on the batch
    vp->v_layer_ptrs = &none;
    vp->k_scales = x->scales;   // split into K and V halves once the block count is known
    vp->v_scales = x->scales;
    return TKV_OK;
}

int32_t tkv_plan_create_to_transfer(const TkvPool* src, const TkvTransfer* xfer, const TkvBatch* batch,
                                    const TkvShard* shard, uint32_t flags, tkv_plan** out) {
    if (!src || !xfer || !batch || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    TkvPool vp;
    TkvShard sh;
    int32_t rc = transfer_as_pool(xfer, src, shard, 2, &vp, &sh);
    if (rc) return rc;
    return create_plan(src, &vp, batch, &sh, flags | TKV_PLAN_ALLOW_SHARED_DST, 2, xfer, out);
}

int32_t tkv_plan_create_from_transfer(const TkvTransfer* xfer, const TkvPool* dst, const TkvBatch* batch,
                                      const TkvShard* shard, uint32_t flags, tkv_plan** out) {
    if (!dst || !xfer || !batch || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    TkvPool vp;
    TkvShard sh;
    int32_t rc = transfer_as_pool(xfer, dst, shard, 1, &vp, &sh);
    if (rc) return rc;
    return create_plan(&vp, dst, batch, &sh, flags, 1, xfer, out);
}

uint64_t tkv_transfer_bytes(uint32_t n_layers, uint32_t n_heads, uint32_t head_dim, uint32_t block_size, int32_t dtype,
                            uint64_t n_blocks) {
    return 2ull * n_layers * n_blocks * block_size * n_heads * head_dim * elem_size(dtype);
}

uint64_t tkv_batch_blocks(const TkvBatch* b, uint32_t block_size) {
    if (!b || !block_size || (b->n_seqs && !b->seq_lens)) return 0;
    uint64_t n = 0;
    for (uint32_t q = 0; q < b->n_seqs; q++) {
        const uint32_t len = b->seq_lens[q], pre = b->prefix_lens ? b->prefix_lens[q] : 0u;
        if (pre <= len) n += (len + block_size - 1) / block_size - pre / block_size;
    }
    return n;
}

int32_t tkv_plan_update(tkv_plan* p, const TkvBatch* batch) {
    if (!p || !batch) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    return build_worklist(p, batch);
}

int32_t tkv_plan_destroy(tkv_plan* p) {
    if (!p) return TKV_OK;
    {
        DeviceGuard g(p->launch_dev);
        if (p->upload_ev) {
            if (p->upload_pending) cudaEventSynchronize(p->upload_ev);
            cudaEventDestroy(p->upload_ev);
        }
        if (p->h_buf) cudaFreeHost(p->h_buf);
        if (p->d_buf) cudaFree(p->d_buf);
        if (p->dev_scratch) cudaFree(p->dev_scratch);
        if (p->copy_stream) {
            cudaStreamSynchronize(p->copy_stream);
            cudaStreamDestroy(p->copy_stream);
        }
        if (p->ev_begin) cudaEventDestroy(p->ev_begin);
        for (int i = 0; i < 2; i++) {
            if (p->ev_copied[i]) cudaEventDestroy(p->ev_copied[i]);
            if (p->ev_read[i]) cudaEventDestroy(p->ev_read[i]);
        }
        if (p->stage) cudaFree(p->stage);
    }
    delete p;
    return TKV_OK;
}

int32_t tkv_plan_stats(const tkv_plan* p, TkvStats* out) {
    if (!p || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    *out = p->stats;
    out->grid = p->grid;
    out->block = p->variant == TKV_VARIANT_BULK ? 32u : 256u;
    out->kernel_variant = (p->variant == TKV_VARIANT_VECTOR && wide_eligible(p)) ? (uint32_t)TKV_VARIANT_WIDE : p->variant;
    return TKV_OK;
}

int32_t tkv_handoff_enqueue(tkv_plan* p, void* stream, uint64_t done_flag, uint32_t flag_value) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceGuard g(p->launch_dev);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->launch_dev);
    tkv::HandoffArgs& a = p->args;
    a.done_flag = reinterpret_cast<uint32_t*>(done_flag);
    a.flag_value = flag_value;
    const uint64_t chunks = (uint64_t)a.n_pairs * a.n_layers * 2;
    if (chunks == 0) {
        // nothing moves; still publish the flag, in stream order
        if (done_flag) CU(cudaMemcpyAsync(reinterpret_cast<void*>(done_flag), &a.flag_value, 4, cudaMemcpyDefault, st));
        p->grid = 0;
        return TKV_OK;
    }
    a.n_pairs_dev = nullptr;
    // The flag: by a stream-ordered write behind the kernel where the stream can reach it (no fence, counter and
    // flag store inside the kernel: they cost a small handoff several microseconds), else by the kernel's last CTA.
    bool by_stream = flag_by_stream(p, done_flag);
    if (by_stream) {                       // inside a stream capture the kernel's own store is the form every driver can record
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) by_stream = false;
    }
    if (by_stream) a.done_flag = nullptr;
    // A launch that carries its list in the parameter block reads nothing of the device block once that is initialised.
    const bool needs_block = !(p->ever_uploaded && p->mode == MODE_COPY && !(p->flags & TKV_PLAN_FORCE_VECTOR) && bulk_eligible(p) && inline_eligible(p));
    if (needs_block) {
        int32_t rc = ensure_uploaded(p, st);
        if (rc) return rc;
    }
    int32_t rc = TKV_OK;
    if (p->staged) {
        // One group of layers at a time: the copy engine brings the group's K and V planes into device buffer g % 2 on the plan's own
        // stream, the group's kernel follows on the caller's stream, and a buffer is filled again only after the kernel that read it.
        const uint32_t L = a.n_layers;
        const tkv::HandoffArgs whole = a;
        uint32_t* const flag_ptr = a.done_flag;
        auto layers = [&]() -> int32_t {       // a failed call returns from here; the plan's arguments are put back below either way
            CU(cudaEventRecord(p->ev_begin, st));
            CU(cudaStreamWaitEvent(p->copy_stream, p->ev_begin, 0));
            const uint32_t G = p->stage_group;
            for (uint32_t l = 0, g = 0; l < L; l += G, g++) {
                const int buf = g & 1;
                const uint32_t n = std::min(G, L - l);
                if (g >= 2) CU(cudaStreamWaitEvent(p->copy_stream, p->ev_read[buf], 0));
                CU(cudaMemcpyAsync(p->stage + (size_t)buf * G * 2 * p->stage_plane, reinterpret_cast<const void*>(p->stage_host[l]),
                                   (size_t)n * 2 * p->stage_plane, cudaMemcpyHostToDevice, p->copy_stream));
                CU(cudaEventRecord(p->ev_copied[buf], p->copy_stream));
                CU(cudaStreamWaitEvent(st, p->ev_copied[buf], 0));
                a = whole;
                a.src_k += l;
                a.src_v += l;
                a.dst_k += l;
                a.dst_v += l;
                a.work += (size_t)l * a.work_layer_stride;
                a.n_layers = n;
                a.src_layer_begin += l;
                a.dst_layer_begin += l;
                a.done_flag = l + n == L ? flag_ptr : nullptr;   // the last group's kernel publishes (when the kernel is the one to do it)
                const int32_t r = dispatch(p, (uint64_t)a.n_pairs * 2 * n, st);
                if (r != TKV_OK) return r;
                CU(cudaEventRecord(p->ev_read[buf], st));
            }
            return TKV_OK;
        };
        rc = layers();
        a = whole;
    } else {
        rc = dispatch(p, chunks, st);
    }
    if (rc) return rc;
    if (by_stream) {
        int r = stream_write_value()(st, (unsigned long long)done_flag, flag_value, 0u);
        if (r != 0) {                      // not supported here after all: the kernel publishes from now on, this one by a copy
            p->flag_mode = 1;
            CU(cudaMemcpyAsync(reinterpret_cast<void*>(done_flag), &a.flag_value, 4, cudaMemcpyDefault, st));
        }
    }
    return TKV_OK;
}

}  // extern "C"

// picks and launches the kernel for the plan's mode over `chunks` (block, layer, K|V) units
static int32_t dispatch(tkv_plan* p, uint64_t chunks, cudaStream_t st) {
    tkv::HandoffArgs& a = p->args;
    switch (p->mode) {
        case MODE_COPY:
            if (p->flags & TKV_PLAN_FORCE_BULK) {
                if (!bulk_eligible(p))
                    return fail(TKV_ERR_INVALID_CONFIG, "bulk copies need whole rows, 16-byte alignment and same-device pools (or TKV_PLAN_PEER_BULK_STORES)");
                return launch_bulk(p, st);
            }
            if (!(p->flags & TKV_PLAN_FORCE_VECTOR) && bulk_eligible(p)) return launch_bulk(p, st);
            p->variant = TKV_VARIANT_VECTOR;
            if (wide_eligible(p)) return launch_wide(p, chunks, st);
            switch (p->vec) {
                case 16: return launch(tkv::handoff_copy_vec<16, 8>, p, chunks, st);
                case 8: return launch(tkv::handoff_copy_vec<8, 8>, p, chunks, st);
                case 4: return launch(tkv::handoff_copy_vec<4, 8>, p, chunks, st);
                case 2: return launch(tkv::handoff_copy_vec<2, 8>, p, chunks, st);
                default: return launch(tkv::handoff_copy_vec<1, 8>, p, chunks, st);
            }
        case MODE_F16_E4M3: {
            const bool hw = !(p->flags & TKV_PLAN_INT_QUANTIZER);
            const bool scaled = p->dst.k_scales != 0;
            if (hw) return scaled ? launch_fp8<true, true>(p, st) : launch_fp8<true, false>(p, st);
            return scaled ? launch_fp8<false, true>(p, st) : launch_fp8<false, false>(p, st);
        }
        case MODE_F32_F16:
            if (p->vec == 16 && (a.n_heads * a.head_dim) % 8 == 0 && !(p->flags & TKV_PLAN_FORCE_VECTOR)) {
                p->variant = TKV_VARIANT_CAST_VEC;
                return launch(tkv::handoff_f32_cast_vec<0>, p, chunks, st);
            }
            p->variant = TKV_VARIANT_CAST_GENERIC;
            return launch(tkv::handoff_f32_cast_generic<0>, p, chunks, st);
        case MODE_F32_E4M3:
            if (p->vec == 16 && (a.n_heads * a.head_dim) % 16 == 0 && !(p->flags & TKV_PLAN_FORCE_VECTOR)) {
                p->variant = TKV_VARIANT_CAST_VEC;
                return launch(tkv::handoff_f32_cast_vec<1>, p, chunks, st);
            }
            p->variant = TKV_VARIANT_CAST_GENERIC;
            return launch(tkv::handoff_f32_cast_generic<1>, p, chunks, st);
        case MODE_E4M3_F16:
            p->variant = TKV_VARIANT_DEQUANT;
            if (p->vec == 16 && a.head_dim % 16 == 0) return launch(tkv::handoff_e4m3_dequant<true, true>, p, chunks, st);
            return launch(tkv::handoff_e4m3_dequant<true, false>, p, chunks, st);
        case MODE_E4M3_F32:
            p->variant = TKV_VARIANT_DEQUANT;
            if (p->vec == 16 && a.head_dim % 16 == 0) return launch(tkv::handoff_e4m3_dequant<false, true>, p, chunks, st);
            return launch(tkv::handoff_e4m3_dequant<false, false>, p, chunks, st);
    }
    return fail(TKV_ERR_INVALID_CONFIG, "unreachable mode");
}

extern "C" {

int32_t tkv_handoff_enqueue_device_tables(tkv_plan* p, const TkvDeviceBatch* db, void* stream, uint64_t done_flag, uint32_t flag_value) {
    if (!p || !db) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (p->virt) return fail(TKV_ERR_INVALID_CONFIG, "device tables: not for transfer-buffer plans");
    if (p->layer_tables) return fail(TKV_ERR_INVALID_CONFIG, "device tables: the plan was made with one table per layer");
    tkv::HandoffArgs& a = p->args;
    if (a.n_pairs == 0) return fail(TKV_ERR_INVALID_CONFIG, "device tables: the plan has no capacity (it was made from an empty batch)");
    if (db->n_seqs == 0 || db->table_stride == 0 || !db->seq_lens || !db->src_tables || !db->dst_tables)
        return fail(TKV_ERR_INVALID_CONFIG, "device tables: NULL arrays or empty batch");
    if (db->apply_refcounts && !p->dst.refcounts) return fail(TKV_ERR_INVALID_CONFIG, "device tables: apply_refcounts without a refcount array in the destination pool");
    if (db->apply_refcounts && p->src.device != p->dst.device)
        return fail(TKV_ERR_INVALID_CONFIG, "device tables: reference counts of a peer pool are applied by its own device");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    DeviceGuard g(p->src.device);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->src.device);
    if (db->n_seqs > p->dev_scratch_seqs) {                         // first use, or a wider batch than before
        if (p->dev_scratch) CU(cudaFree(p->dev_scratch));
        p->dev_scratch = nullptr;
        p->dev_scratch_seqs = 0;
        const size_t seqs = std::max<size_t>(db->n_seqs, 256);
        CU(cudaMalloc((void**)&p->dev_scratch, (4 + seqs) * sizeof(uint32_t)));
        p->dev_scratch_seqs = seqs;
    }
    {
        int32_t rc = ensure_uploaded(p, st, false);   // layer pointers and counter; the list is built below
        if (rc) return rc;
    }
    tkv::DeviceTables t{};
    t.seq_lens = reinterpret_cast<const uint32_t*>(db->seq_lens);
    t.prefix_lens = reinterpret_cast<const uint32_t*>(db->prefix_lens);
    t.prefix_blocks = reinterpret_cast<const uint32_t*>(db->prefix_blocks);
    t.src_tables = reinterpret_cast<const uint32_t*>(db->src_tables);
    t.dst_tables = reinterpret_cast<const uint32_t*>(db->dst_tables);
    t.offsets = p->dev_scratch + 4;
    t.work = reinterpret_cast<uint4*>(p->d_buf + p->off_work);
    t.n_pairs_out = p->dev_scratch;
    t.status = reinterpret_cast<uint32_t*>(db->status);
    t.refcounts = db->apply_refcounts ? reinterpret_cast<int32_t*>(p->dst.refcounts) : nullptr;
    t.n_seqs = db->n_seqs;
    t.table_stride = db->table_stride;
    t.block_size = a.block_size;
    t.capacity = a.n_pairs;
    t.src_total_blocks = p->src.total_blocks;
    t.dst_total_blocks = p->dst.total_blocks;
    tkv::worklist_from_device_tables<<<1, 1024, 0, st>>>(t);
    CU(cudaGetLastError());
    a.done_flag = reinterpret_cast<uint32_t*>(done_flag);
    a.flag_value = flag_value;
    a.n_pairs_dev = p->dev_scratch;
    const int32_t rc = dispatch(p, (uint64_t)a.n_pairs * a.n_layers * 2, st);
    a.n_pairs_dev = nullptr;
    // the device builder wrote over the slot that holds the plan's host-built list: the next host-table
    // enqueue uploads the pinned mirror again, in stream order
    p->list_clobbered = true;
    return rc;
}

int32_t tkv_plan_tune_bulk(tkv_plan* p, uint32_t stages, uint32_t ctas_per_sm, uint32_t stage_bytes) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    if (stages < 2 || stages > 8 || ctas_per_sm > 16)
        return fail(TKV_ERR_INVALID_CONFIG, "stages must be in [2, 8] and ctas_per_sm in [0, 16]");
    if (stage_bytes < 1024 || stage_bytes > 98304 || stage_bytes % 128)
        return fail(TKV_ERR_INVALID_CONFIG, "stage_bytes must be a multiple of 128 in [1024, 98304]");
    p->bulk_stages = stages;
    p->fp8_stages = stages;
    p->bulk_ctas_per_sm = ctas_per_sm;
    p->bulk_stage_bytes = stage_bytes;
    return TKV_OK;
}

int32_t tkv_plan_tune_vector(tkv_plan* p, uint32_t bytes_per_access, uint32_t unroll, uint32_t store_hint) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    if ((bytes_per_access != 0 && bytes_per_access != 16 && bytes_per_access != 32) || (unroll != 4 && unroll != 8 && unroll != 16) || store_hint > 2)
        return fail(TKV_ERR_INVALID_CONFIG, "bytes_per_access must be 0, 16 or 32, unroll 4, 8 or 16, store_hint 0, 1 or 2");
    p->vec_bytes = bytes_per_access;
    p->vec_unroll = unroll;
    p->vec_hint = store_hint;
    return TKV_OK;
}

int32_t tkv_plan_tune_small(tkv_plan* p, uint32_t flag_mode, uint32_t inline_list) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    if (flag_mode > 2 || inline_list > 2) return fail(TKV_ERR_INVALID_CONFIG, "flag_mode and inline_list must be 0, 1 or 2");
    p->flag_mode = flag_mode;
    p->inline_mode = inline_list;
    p->flag_checked = 0;
    return TKV_OK;
}

int32_t tkv_plan_tune_grid(tkv_plan* p, uint32_t ctas_per_sm) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    if (ctas_per_sm > 32) return fail(TKV_ERR_INVALID_CONFIG, "ctas_per_sm must be in [0, 32]");
    p->grid_ctas_per_sm = ctas_per_sm;
    return TKV_OK;
}

int32_t tkv_plan_error(const tkv_plan* p, uint32_t* device_error) {
    if (!p || !device_error) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    *device_error = 0;
    if (!p->d_buf) return TKV_OK;
    DeviceGuard g(p->launch_dev);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->launch_dev);
    CU(cudaMemcpy(device_error, p->args.done_counter + 1, 4, cudaMemcpyDeviceToHost));
    return TKV_OK;
}

int32_t tkv_flag_wait_host(int32_t device, uint64_t flag, uint32_t expected, uint64_t timeout_us) {
    if (!flag) return fail(TKV_ERR_INVALID_CONFIG, "NULL flag");
    DeviceGuard g(device);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", device);
    // A flag in page-locked host memory is read in place; one in device memory through small copies.
    cudaPointerAttributes attr{};
    const bool in_host = cudaPointerGetAttributes(&attr, reinterpret_cast<const void*>(flag)) == cudaSuccess &&
                         attr.type == cudaMemoryTypeHost && attr.hostPointer != nullptr;
    if (!in_host) cudaGetLastError();
    cudaStream_t cs = nullptr;
    if (!in_host) {
        int32_t rc = copy_stream(device, &cs);
        if (rc) return rc;
    }
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        uint32_t v = 0;
        if (in_host) {
            v = __atomic_load_n(static_cast<const uint32_t*>(attr.hostPointer), __ATOMIC_ACQUIRE);
        } else {
            CU(cudaMemcpyAsync(&v, reinterpret_cast<const void*>(flag), 4, cudaMemcpyDeviceToHost, cs));
            CU(cudaStreamSynchronize(cs));
        }
        if ((int32_t)(v - expected) >= 0) return TKV_OK;   // generation reached or already passed
        const auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        if ((uint64_t)us >= timeout_us)
            return fail(TKV_ERR_TIMEOUT, "flag still %u after %llu us (waiting for generation %u)", v, (unsigned long long)timeout_us, expected);
        // poll tightly while a handoff of ordinary size could still be finishing, then back off
        if (us > 2000) std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
}

int32_t tkv_flag_wait_enqueue(void* stream, uint64_t flag, uint32_t expected, uint64_t max_spins, uint64_t status) {
    if (!flag) return fail(TKV_ERR_INVALID_CONFIG, "NULL flag");
    if (max_spins == 0 || max_spins > (1ull << 26))
        return fail(TKV_ERR_INVALID_CONFIG, "max_spins must be in [1, 2^26] so the wait stays bounded");
    tkv::flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const uint32_t*>(flag), expected,
                                                                          (unsigned long long)max_spins,
                                                                          reinterpret_cast<uint32_t*>(status));
    CU(cudaGetLastError());
    return TKV_OK;
}

int32_t tkv_refcount_apply(tkv_plan* p, int32_t delta, void* stream) {
    if (!p) return fail(TKV_ERR_INVALID_CONFIG, "NULL plan");
    if (delta == 0 || p->n_prefix == 0) return TKV_OK;
    if (!p->dst.refcounts) return fail(TKV_ERR_INVALID_CONFIG, "destination pool has no refcount array");
    DeviceGuard g(p->src.device);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", p->src.device);
    int32_t rc = ensure_uploaded(p, static_cast<cudaStream_t>(stream), false);   // the prefix ids sit past the work list
    if (rc) return rc;
    uint32_t blocks = std::min<uint32_t>((p->n_prefix + 255) / 256, 1024);
    tkv::refcount_apply_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<uint32_t*>(p->dst.refcounts), reinterpret_cast<const uint32_t*>(p->d_buf + p->off_prefix),
        p->n_prefix, delta);
    CU(cudaGetLastError());
    return TKV_OK;
}

int32_t tkv_refcount_apply_device_tables(const TkvPool* dst, const TkvDeviceBatch* b, int32_t delta, void* stream) {
    if (!dst || !b) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (!dst->refcounts) return fail(TKV_ERR_INVALID_CONFIG, "destination pool has no refcount array");
    if (delta == 0 || b->n_seqs == 0) return TKV_OK;
    if (!b->dst_tables || b->table_stride == 0 || (!b->prefix_lens && !b->prefix_blocks) || dst->block_size == 0)
        return fail(TKV_ERR_INVALID_CONFIG, "device tables: need dst_tables and prefix_lens or prefix_blocks");
    DeviceGuard g(dst->device);
    if (!g.ok) return fail(TKV_ERR_CUDA, "cannot select device %d", dst->device);
    const uint32_t blocks = std::min<uint32_t>((b->n_seqs + 7) / 8, 1024);
    tkv::refcount_apply_tables_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<uint32_t*>(dst->refcounts), reinterpret_cast<const uint32_t*>(b->dst_tables),
        reinterpret_cast<const uint32_t*>(b->prefix_lens), reinterpret_cast<const uint32_t*>(b->prefix_blocks), b->n_seqs, b->table_stride,
        dst->block_size, dst->total_blocks, delta, reinterpret_cast<uint32_t*>(b->status));
    CU(cudaGetLastError());
    return TKV_OK;
}

int32_t tkv_pairing_make(int32_t n_gpus, uint32_t n_layers, uint32_t n_kv_heads, TkvPairing* out, int32_t cap,
                         int32_t* n_pairs) {
    if (!out || !n_pairs) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (n_gpus < 1 || (n_gpus > 1 && (n_gpus & 1))) return fail(TKV_ERR_INVALID_CONFIG, "n_gpus must be 1 or even, got %d", n_gpus);
    if (n_layers == 0 || n_kv_heads == 0) return fail(TKV_ERR_INVALID_CONFIG, "zero-sized model");
    const uint32_t P = n_gpus == 1 ? 1u : (uint32_t)n_gpus / 2u;
    if ((int32_t)P > cap) return fail(TKV_ERR_INVALID_CONFIG, "output holds %d pairings, need %u", cap, P);
    const bool by_head = n_kv_heads >= P;
    if (by_head && n_kv_heads % P) return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %u, got %u (kv heads not divisible by pairs)", P, n_kv_heads);
    if (!by_head && n_layers < P) return fail(TKV_ERR_INVALID_CONFIG, "neither %u heads nor %u layers cover %u pairs", n_kv_heads, n_layers, P);
    for (uint32_t i = 0; i < P; i++) {
        TkvPairing& pr = out[i];
        pr.prefill_device = (int32_t)i;
        pr.decode_device = n_gpus == 1 ? 0 : (int32_t)(i + P);
        if (by_head) {
            uint32_t per = n_kv_heads / P;
            pr.shard = TkvShard{i * per, i * per, per, 0, 0, n_layers};
        } else {
            uint32_t lo = (uint32_t)((uint64_t)n_layers * i / P), hi = (uint32_t)((uint64_t)n_layers * (i + 1) / P);
            pr.shard = TkvShard{0, 0, n_kv_heads, lo, lo, hi - lo};
        }
    }
    *n_pairs = (int32_t)P;
    return TKV_OK;
}

int32_t tkv_cast(uint64_t src, int32_t sdt, uint64_t dst, int32_t ddt, uint64_t n, void* stream) {
    if (n == 0) return TKV_OK;
    if (!src || !dst) return fail(TKV_ERR_INVALID_CONFIG, "NULL buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const void* s = reinterpret_cast<const void*>(src);
    void* d = reinterpret_cast<void*>(dst);
    uint32_t grid = (uint32_t)std::min<uint64_t>((n + 255) / 256, 148ull * 16);
#define TKV_CAST(S, D)                                            \
    if (sdt == S && ddt == D) {                                   \
        tkv::cast_kernel<S, D><<<grid, 256, 0, st>>>(s, d, n);    \
        CU(cudaGetLastError());                                   \
        return TKV_OK;                                            \
    }
    TKV_CAST(0, 1) TKV_CAST(1, 0) TKV_CAST(0, 2) TKV_CAST(2, 0) TKV_CAST(1, 2) TKV_CAST(2, 1)
#undef TKV_CAST
    return fail(TKV_ERR_INVALID_CONFIG, "unsupported cast %d -> %d", sdt, ddt);
}

int32_t tkv_selfcheck_e4m3(uint32_t skip_bits, uint64_t* mismatches) {
    if (!mismatches || skip_bits > 24) return fail(TKV_ERR_INVALID_CONFIG, "bad argument");
    unsigned long long* d = nullptr;
    CU(cudaMalloc((void**)&d, 8));
    CU(cudaMemset(d, 0, 8));
    tkv::selfcheck_e4m3_kernel<<<148 * 8, 256>>>(skip_bits, d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpy(mismatches, d, 8, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return cuda_fail(e, "selfcheck");
    return TKV_OK;
}

int32_t tkv_selfcheck_scaled_quant(uint64_t* mismatches) {
    if (!mismatches) return fail(TKV_ERR_INVALID_CONFIG, "bad argument");
    unsigned long long* d = nullptr;
    CU(cudaMalloc((void**)&d, 8));
    CU(cudaMemset(d, 0, 8));
    tkv::selfcheck_scaled_quant_kernel<<<148 * 8, 256>>>(d);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpy(mismatches, d, 8, cudaMemcpyDeviceToHost);
    cudaFree(d);
    if (e != cudaSuccess) return cuda_fail(e, "selfcheck");
    return TKV_OK;
}

int32_t tkv_memcpy_enqueue(uint64_t dst, uint64_t src, uint64_t bytes, void* stream) {
    if (bytes == 0) return TKV_OK;
    if (!dst || !src) return fail(TKV_ERR_INVALID_CONFIG, "NULL buffer");
    CU(cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes, cudaMemcpyDefault,
                       static_cast<cudaStream_t>(stream)));
    return TKV_OK;
}

int32_t tkv_bits_checksum(uint64_t data, int32_t dtype, uint64_t n, void* stream, uint64_t* out) {
    if (!out || (!data && n)) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned long long* d = nullptr;
    CU(cudaMalloc((void**)&d, 8));
    cudaError_t e = cudaMemsetAsync(d, 0, 8, st);
    if (e == cudaSuccess && n) {
        uint32_t grid = (uint32_t)std::min<uint64_t>((n + 255) / 256, 148ull * 16);
        const void* p = reinterpret_cast<const void*>(data);
        if (dtype == TKV_DTYPE_F32) tkv::bits_checksum_kernel<0><<<grid, 256, 0, st>>>(p, n, d);
        else if (dtype == TKV_DTYPE_F16) tkv::bits_checksum_kernel<1><<<grid, 256, 0, st>>>(p, n, d);
        else if (dtype == TKV_DTYPE_E4M3) tkv::bits_checksum_kernel<2><<<grid, 256, 0, st>>>(p, n, d);
        else {
            cudaFree(d);
            return fail(TKV_ERR_INVALID_CONFIG, "unknown dtype %d", dtype);
        }
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, d, 8, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d);
    if (e != cudaSuccess) return cuda_fail(e, "bits checksum");
    return TKV_OK;
}

int32_t tkv_ipc_export(uint64_t devptr, uint8_t handle[64], uint64_t* offset) {
    if (!devptr || !handle || !offset) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
    cudaIpcMemHandle_t h;
    CU(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(devptr)));
    memcpy(handle, &h, 64);
    // The handle names the whole allocation; report where devptr sits inside it.
    // cuMemGetAddressRange has no runtime-API twin, so fetch it from the driver.
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    CU(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr));
    if (!fn) return fail(TKV_ERR_CUDA, "cuMemGetAddressRange not found");
    unsigned long long base = 0;
    size_t size = 0;
    int r = reinterpret_cast<range_fn>(fn)(&base, &size, (unsigned long long)devptr);
    if (r != 0) return fail(TKV_ERR_CUDA, "cuMemGetAddressRange failed (%d)", r);
    *offset = devptr - (uint64_t)base;
    return TKV_OK;
}

int32_t tkv_ipc_import(const uint8_t handle[64], uint64_t offset, uint64_t* devptr) {
    if (!handle || !devptr) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* base = nullptr;
    CU(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *devptr = reinterpret_cast<uint64_t>(base) + offset;
    // the mapping is usable from the importing (current) device: remember its extent, so that a plan whose destination
    // pointers lie inside it is accepted whatever ordinal the caller gives the owning device
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess) {
        typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        unsigned long long lo = 0;
        size_t size = 0;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr) == cudaSuccess && fn &&
            reinterpret_cast<range_fn>(fn)(&lo, &size, (unsigned long long)reinterpret_cast<uint64_t>(base)) == 0 && size)
            tkv_internal::note_import(cur, (uint64_t)lo, (uint64_t)size);
        else
            tkv_internal::note_import(cur, reinterpret_cast<uint64_t>(base), ~0ull - reinterpret_cast<uint64_t>(base));   // extent unknown: from the base on
    }
    cudaGetLastError();
    return TKV_OK;
}

int32_t tkv_ipc_close(uint64_t devptr, uint64_t offset) {
    if (!devptr) return TKV_OK;
    tkv_internal::forget_import(devptr - offset);
    CU(cudaIpcCloseMemHandle(reinterpret_cast<void*>(devptr - offset)));
    return TKV_OK;
}

}  // extern "C"
