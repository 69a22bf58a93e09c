// C++ host-side mirror of the reference's prefill / decode worker boundary, on top of the C
// ABI in tkv.h.  Header-only; link libtkv.
//
// What it mirrors (paths inside the tempura repository):
//   trait PrefillWorker / DecodeWorker, DisaggregatedPipeline::{new, generate}
//       engine/src/disaggregated.rs:7-19,130-152
//   SessionTransfer {cache, position, seed, last_logits}      engine/src/session.rs:194-200
//   KvCacheTransfer {k_data, v_data, seq_len, ...}            engine/src/kv_cache.rs:514-522
//   KernelError::{DimensionMismatch, InvalidConfig}           kernel-api/src/lib.rs:5-13
// The one deliberate difference: KvCacheTransfer does not hold the K/V vectors.  The K/V stay
// in the prefill GPU's paged pool and the transfer carries the block table that names them;
// the decode side pulls them with one handoff kernel (KvReceiver::adopt below) instead of
// copying Vec<f32> twice.
#ifndef TKV_WORKERS_HPP
#define TKV_WORKERS_HPP

#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "tkv.h"

namespace tkv_host {

// Result<T, KernelError> becomes an exception carrying the C status code.
struct KernelError : std::runtime_error {
    int32_t code;
    KernelError(int32_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};

inline void check(int32_t rc) {
    if (rc == TKV_OK) return;
    char buf[512];
    tkv_last_error(buf, sizeof buf);
    throw KernelError(rc, buf);
}

// kernels/src/sampling.rs SamplingParams: only the fields the pipeline passes through.
struct SamplingParams {
    float temperature = 0.0f;
    uint32_t top_k = 50;
    float top_p = 1.0f;
};

// PageAllocator (engine/src/kv_cache.rs:762-793) over the C handle.
class PageAllocator {
public:
    explicit PageAllocator(size_t total_pages) : h_(tkv_page_allocator_new(total_pages)) {}
    ~PageAllocator() { tkv_page_allocator_delete(h_); }
    PageAllocator(const PageAllocator&) = delete;
    PageAllocator& operator=(const PageAllocator&) = delete;
    // panics in the reference (kv_cache.rs:980); here the recoverable PoolExhausted of
    // engine/src/cutile_kv_cache.rs:27-44
    uint32_t allocate() {
        size_t page = 0;
        check(tkv_page_allocator_allocate(h_, &page));
        return static_cast<uint32_t>(page);
    }
    void free(uint32_t page) { tkv_page_allocator_free(h_, page); }
    size_t available() const { return tkv_page_allocator_available(h_); }
    size_t in_use() const { return tkv_page_allocator_in_use(h_); }

private:
    tkv_page_allocator* h_;
};

// RadixTree (engine/src/prefix_cache.rs:17-149) over the C handle.
class RadixTree {
public:
    RadixTree() : h_(tkv_radix_tree_new()) {}
    ~RadixTree() { tkv_radix_tree_delete(h_); }
    RadixTree(const RadixTree&) = delete;
    RadixTree& operator=(const RadixTree&) = delete;
    void insert(const std::vector<uint32_t>& tokens, const std::vector<size_t>& pages) {
        tkv_radix_tree_insert(h_, tokens.data(), tokens.size(), pages.data(), pages.size());
    }
    // RadixMatch {matched_len, page_ids}; bumps the reference counts of the matched nodes
    std::pair<size_t, std::vector<size_t>> lookup(const std::vector<uint32_t>& tokens) {
        std::vector<size_t> pages(tokens.size() + 1);
        size_t n = 0;
        size_t matched = tkv_radix_tree_lookup(h_, tokens.data(), tokens.size(), pages.data(), pages.size(), &n);
        pages.resize(n);
        return {matched, pages};
    }
    void release(const std::vector<uint32_t>& tokens) { tkv_radix_tree_release(h_, tokens.data(), tokens.size()); }
    uint64_t hit_count() const { return tkv_radix_tree_hit_count(h_); }

private:
    tkv_radix_tree* h_;
};

// A pool description that owns its layer pointer arrays.
struct Pool {
    TkvPool c{};
    std::vector<uint64_t> k_ptrs, v_ptrs;
    const TkvPool* get() {
        c.k_layer_ptrs = k_ptrs.data();
        c.v_layer_ptrs = v_ptrs.data();
        return &c;
    }
};

// engine/src/kv_cache.rs:514-522, as a handle (see the header comment).
struct KvCacheTransfer {
    Pool* pool = nullptr;               // the prefill side's pool
    std::vector<uint32_t> block_table;  // BlockTable::as_slice of the sequence
    size_t seq_len = 0;
    size_t num_layers = 0, num_kv_heads = 0, head_dim = 0;
};

// engine/src/session.rs:194-200
struct SessionTransfer {
    KvCacheTransfer cache;
    size_t position = 0;
    uint64_t seed = 0;
    std::vector<float> last_logits;
};

// The transfer's metadata as one wire message (tkv_session_pack): what a prefill process sends a
// decode process next to the handoff itself.  The K/V bytes are not in it.
inline std::vector<uint8_t> to_wire(const SessionTransfer& t) {
    const TkvPool& p = t.cache.pool->c;
    TkvSessionHeader h{};
    h.position = t.position;
    h.seed = t.seed;
    h.seq_len = static_cast<uint32_t>(t.cache.seq_len);
    h.n_layers = static_cast<uint32_t>(t.cache.num_layers);
    h.n_kv_heads = static_cast<uint32_t>(t.cache.num_kv_heads);
    h.head_dim = static_cast<uint32_t>(t.cache.head_dim);
    h.block_size = p.block_size;
    h.kv_dtype = static_cast<uint32_t>(p.dtype);
    h.n_blocks = (h.seq_len + p.block_size - 1) / p.block_size;
    h.piece_count = 1;
    h.n_logits = static_cast<uint32_t>(t.last_logits.size());
    if (t.cache.block_table.size() < h.n_blocks)
        throw KernelError(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: block table shorter than the sequence");
    std::vector<uint8_t> out(tkv_session_wire_size(&h));
    size_t written = 0;
    check(tkv_session_pack(&h, t.cache.block_table.data(), t.last_logits.data(), out.data(), out.size(), &written));
    return out;
}

// The receiving side names the prefill pool itself (`source_pool`: the peer or IPC mapping it holds).
inline SessionTransfer from_wire(const std::vector<uint8_t>& msg, Pool* source_pool) {
    TkvSessionHeader h{};
    const uint32_t* blocks = nullptr;
    const float* logits = nullptr;
    check(tkv_session_unpack(msg.data(), msg.size(), &h, &blocks, &logits));
    if (h.piece_count != 1) throw KernelError(TKV_ERR_INVALID_CONFIG, "from_wire reads whole-sequence messages; assemble pieces first");
    const TkvPool& p = source_pool->c;
    if (h.n_layers != p.n_layers || h.n_kv_heads != p.n_kv_heads || h.head_dim != p.head_dim || h.block_size != p.block_size ||
        h.kv_dtype != static_cast<uint32_t>(p.dtype))
        throw KernelError(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: message geometry differs from the source pool");
    SessionTransfer t;
    t.cache.pool = source_pool;
    t.cache.block_table.assign(blocks, blocks + h.n_blocks);
    t.cache.seq_len = h.seq_len;
    t.cache.num_layers = h.n_layers;
    t.cache.num_kv_heads = h.n_kv_heads;
    t.cache.head_dim = h.head_dim;
    t.position = static_cast<size_t>(h.position);
    t.seed = h.seed;
    t.last_logits.assign(logits, logits + h.n_logits);
    return t;
}

// engine/src/disaggregated.rs:7-9
struct PrefillWorker {
    virtual ~PrefillWorker() = default;
    virtual SessionTransfer prefill(const std::vector<uint32_t>& token_ids, uint64_t seed) = 0;
};

// engine/src/disaggregated.rs:11-19
struct DecodeWorker {
    virtual ~DecodeWorker() = default;
    virtual std::vector<uint32_t> decode(SessionTransfer transfer, size_t max_new_tokens, const SamplingParams& params,
                                         std::optional<uint32_t> eos_token) = 0;
};

// engine/src/disaggregated.rs:130-152
class DisaggregatedPipeline {
public:
    DisaggregatedPipeline(std::unique_ptr<PrefillWorker> prefill, std::unique_ptr<DecodeWorker> decode)
        : prefill_(std::move(prefill)), decode_(std::move(decode)) {}
    std::vector<uint32_t> generate(const std::vector<uint32_t>& token_ids, size_t max_new_tokens, const SamplingParams& params,
                                   std::optional<uint32_t> eos_token, uint64_t seed) const {
        SessionTransfer transfer = prefill_->prefill(token_ids, seed);
        return decode_->decode(std::move(transfer), max_new_tokens, params, eos_token);
    }

private:
    std::unique_ptr<PrefillWorker> prefill_;
    std::unique_ptr<DecodeWorker> decode_;
};

// What InferenceSession::from_transfer / KvCache::from_transfer (engine/src/session.rs:137-156,
// engine/src/kv_cache.rs:419-431) become on a GPU decode worker: allocate destination pages
// (all of them, or only the suffix when the caller passes shared prefix pages), move the
// blocks with one handoff, count the shared prefix references, wait (bounded) for the
// completion flag.
class KvReceiver {
public:
    // `flag` is a zero-initialised uint32_t in the decode pool's device memory; `stream` belongs to
    // the device of the transfer's (source) pool.
    KvReceiver(Pool* dst, PageAllocator* pages, uint64_t flag, uint64_t wait_us = 10'000'000)
        : dst_(dst), pages_(pages), flag_(flag), wait_us_(wait_us) {}

    // Returns the destination block table.  `shared_prefix_pages` are destination pages that already
    // hold the first shared_prefix_pages.size() blocks (RadixTree::lookup's page_ids, one per block).
    std::vector<uint32_t> adopt(const SessionTransfer& t, void* stream, const std::vector<uint32_t>& shared_prefix_pages = {}) {
        const uint32_t bs = dst_->c.block_size;
        const uint32_t len = static_cast<uint32_t>(t.cache.seq_len);
        const uint32_t nb = (len + bs - 1) / bs;
        if (t.cache.block_table.size() < nb)
            throw KernelError(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: block table shorter than the sequence");
        if (shared_prefix_pages.size() > len / bs)
            throw KernelError(TKV_ERR_INVALID_CONFIG, "more shared prefix pages than whole blocks in the sequence");
        std::vector<uint32_t> table(shared_prefix_pages);
        try {
            while (table.size() < nb) table.push_back(pages_->allocate());
            const uint32_t prefix_len = static_cast<uint32_t>(shared_prefix_pages.size()) * bs;
            TkvBatch b{};
            b.n_seqs = 1;
            b.table_stride = nb ? nb : 1;
            b.seq_lens = &len;
            b.prefix_lens = &prefix_len;
            b.src_tables = t.cache.block_table.data();
            b.dst_tables = table.data();
            tkv_plan* plan = nullptr;
            check(tkv_plan_create(t.cache.pool->get(), dst_->get(), &b, nullptr, TKV_PLAN_DEFAULT, &plan));
            const uint32_t gen = ++generation_;
            int32_t rc = tkv_handoff_enqueue(plan, stream, flag_, gen);
            if (rc == TKV_OK && dst_->c.refcounts && prefix_len) rc = tkv_refcount_apply(plan, +1, stream);
            if (rc == TKV_OK) rc = tkv_flag_wait_host(dst_->c.device, flag_, gen, wait_us_);
            tkv_plan_destroy(plan);
            check(rc);
        } catch (...) {
            for (size_t i = shared_prefix_pages.size(); i < table.size(); i++) pages_->free(table[i]);
            throw;
        }
        return table;
    }

private:
    Pool* dst_;
    PageAllocator* pages_;
    uint64_t flag_;
    uint64_t wait_us_;
    uint32_t generation_ = 0;
};


// ---- the decode side's admission kept on the device -----------------------------------------
// RadixTree (engine/src/prefix_cache.rs:17-149) and PageAllocator (engine/src/kv_cache.rs:762-797)
// with their state in HBM, and a receiver that goes from token ids to a finished handoff on one
// stream: lookup -> allocate -> handoff, no block id or length crossing to the host.
class DevicePrefixIndex {
public:
    DevicePrefixIndex(int device, uint64_t capacity, uint32_t group_tokens) { check(tkv_prefix_index_create(device, capacity, group_tokens, &h_)); }
    ~DevicePrefixIndex() { tkv_prefix_index_destroy(h_); }
    DevicePrefixIndex(const DevicePrefixIndex&) = delete;
    DevicePrefixIndex& operator=(const DevicePrefixIndex&) = delete;
    void insert(const TkvPrefixBatch& b, void* stream) { check(tkv_prefix_index_insert(h_, &b, stream)); }
    void lookup(const TkvPrefixBatch& b, uint64_t out_pages, uint32_t out_stride, uint64_t out_matched, void* stream) {
        check(tkv_prefix_index_lookup(h_, &b, out_pages, out_stride, out_matched, stream));
    }
    void release(const TkvPrefixBatch& b, void* stream) { check(tkv_prefix_index_release(h_, &b, stream)); }
    void evict_lru(uint32_t max_nodes, uint64_t out_pages, uint32_t out_cap, uint64_t out_count, uint64_t out_nodes, void* stream) {
        check(tkv_prefix_index_evict_lru(h_, max_nodes, out_pages, out_cap, out_count, out_nodes, stream));
    }
    TkvPrefixIndexStats stats(void* stream) {
        TkvPrefixIndexStats st{};
        check(tkv_prefix_index_stats(h_, stream, &st));
        return st;
    }
    tkv_prefix_index* get() { return h_; }

private:
    tkv_prefix_index* h_ = nullptr;
};

class DevicePageAllocator {
public:
    DevicePageAllocator(int device, uint32_t total_pages) { check(tkv_device_page_allocator_create(device, total_pages, &h_)); }
    ~DevicePageAllocator() { tkv_device_page_allocator_destroy(h_); }
    DevicePageAllocator(const DevicePageAllocator&) = delete;
    DevicePageAllocator& operator=(const DevicePageAllocator&) = delete;
    void allocate(const TkvPageBatch& b, uint64_t status, void* stream) { check(tkv_device_page_allocator_allocate(h_, &b, status, stream)); }
    void free(const TkvPageBatch& b, uint64_t status, void* stream) { check(tkv_device_page_allocator_free(h_, &b, status, stream)); }
    uint32_t available(void* stream) {
        uint32_t n = 0;
        check(tkv_device_page_allocator_available(h_, stream, &n));
        return n;
    }

private:
    tkv_device_page_allocator* h_ = nullptr;
};

// Device arrays a batch admission works in; the caller owns them (all on the pools' device, u32):
//   tokens [n][token_stride], seq_lens [n], src_tables / dst_tables [n][table_stride], matched [n], status [2]
//   (allocator, work list).
struct DeviceAdmissionBuffers {
    uint64_t tokens = 0, seq_lens = 0, src_tables = 0, dst_tables = 0, matched = 0, status = 0;
    uint32_t n_seqs = 0, token_stride = 0, table_stride = 0;
};

// DecodeWorker::receive_kv for a batch, with prefix resolution and page placement on the device: three calls on one
// stream, nothing copied to the host.  `plan` is a plan over (source pool, destination pool) made from a host batch at
// least as large as any batch admitted here; the index's group_tokens must be the pools' block size.
class DeviceKvReceiver {
public:
    DeviceKvReceiver(tkv_plan* plan, DevicePrefixIndex* index, DevicePageAllocator* pages, uint64_t flag, uint32_t block_size)
        : plan_(plan), index_(index), pages_(pages), flag_(flag), block_size_(block_size) {}

    uint32_t adopt(const DeviceAdmissionBuffers& b, void* stream) {
        TkvPrefixBatch pb{};
        pb.n_seqs = b.n_seqs;
        pb.stride = b.token_stride;
        pb.tokens = b.tokens;
        pb.lens = b.seq_lens;
        index_->lookup(pb, b.dst_tables, b.table_stride, b.matched, stream);      // matched pages at the head of each row
        TkvPageBatch pg{};
        pg.n_seqs = b.n_seqs;
        pg.table_stride = b.table_stride;
        pg.tables = b.dst_tables;
        pg.first = b.matched;
        pg.seq_lens = b.seq_lens;                                                  // the rest of each row
        pg.block_size = block_size_;
        pages_->allocate(pg, b.status, stream);
        TkvDeviceBatch db{};
        db.n_seqs = b.n_seqs;
        db.table_stride = b.table_stride;
        db.apply_refcounts = 1;
        db.seq_lens = b.seq_lens;
        db.prefix_blocks = b.matched;
        db.src_tables = b.src_tables;
        db.dst_tables = b.dst_tables;
        db.status = b.status + 4;
        const uint32_t gen = ++generation_;
        check(tkv_handoff_enqueue_device_tables(plan_, &db, stream, flag_, gen));
        return gen;       // wait for it with tkv_flag_wait_host / tkv_flag_wait_enqueue, then read the two status words
    }

private:
    tkv_plan* plan_;
    DevicePrefixIndex* index_;
    DevicePageAllocator* pages_;
    uint64_t flag_;
    uint32_t block_size_;
    uint32_t generation_ = 0;
};

}  // namespace tkv_host
#endif  // TKV_WORKERS_HPP
