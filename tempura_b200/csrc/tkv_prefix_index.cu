// Device-resident prefix index: RadixTree (engine/src/prefix_cache.rs:17-149) as an open-addressing
// hash table in HBM, walked by one CTA per sequence (one thread per node), so that a batch of prompts
// resolves its cached prefix (length, page ids, reference counts, LRU stamps) in one launch without
// a host round trip.
//
// A node of the reference's tree is one element of a sequence below one parent.  Here an element is
// `group_tokens` consecutive token ids (1 reproduces the reference's per-token nodes, 16 gives one
// node per KV block) and a node is named by a 64-bit key chained from the root:
//     raw_i = raw_{i-1} * C + hash(tokens of element i)  (mod 2^64),   key_i = mix(raw_i),
// linear so that all keys of a sequence come out of one parallel scan.  Equal keys mean equal
// prefixes up to a 64-bit hash collision (two different prefixes collide with probability ~2^-64 per
// pair; the hash is not hardened against chosen tokens).  The index does not store whole prefixes, but
// every node keeps the first and the last token id of its own element: a walk that finds its key on
// a node whose guard differs treats the node as absent (a checked miss, counted) instead of adopting
// another prompt's page.  What still gets through is a collision between prefixes whose colliding
// elements also begin and end with the same token ids.
//
// Batch semantics: one call handles many sequences and is ONE tick of the reference's clock.  Its
// result equals the reference's methods applied to the sequences in index order at that tick:
//   insert   a node new in this call takes the page of the lowest-numbered sequence that walks it;
//   lookup   matched nodes get stamp = tick and one more reference each, per walking sequence;
//   release  references go down by one per walking sequence, never below zero;
//   evict    one unreferenced childless node, oldest stamp first, earliest-created on a tie, is
//            unlinked and its page reported (an unlinked node is never reported twice, unlike
//            prefix_cache.rs:99-125, which leaves it eligible: a page must not be freed twice).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <new>

#include "../../include/tkv.h"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* message);
}

namespace {

constexpr unsigned long long KEY_EMPTY = 0ull, KEY_TOMB = 1ull;     // real keys are >= 2
constexpr unsigned long long ORDER_FRESH = ~0ull;
constexpr uint32_t NO_PAGE = 0xFFFFFFFFu, NO_SLOT = 0xFFFFFFFFu;
// creation order of a node: tick (34 bits) | sequence in the batch (14 bits) | depth (16 bits)
constexpr int ORDER_SEQ_BITS = 14, ORDER_DEPTH_BITS = 16;

struct Meta {                   // 32 bytes per slot
    unsigned long long order;   // creation order; ORDER_FRESH while the slot is free
    unsigned long long stamp;   // tick of the last insert / lookup that walked the node
    uint32_t page;              // NO_PAGE when the node was inserted without one
    int32_t refs;
    uint32_t parent;            // slot of the parent node, NO_SLOT below the root
    uint32_t children;
};

struct Counters {               // device-side statistics and the eviction scratch
    unsigned long long hits, tokens_saved, live, tombstones, collisions;
    uint32_t error;             // 1 = table full during an insert
    uint32_t evict_ctas_done;
};

struct Candidate {
    unsigned long long stamp, order;
    uint32_t slot, valid;
};

struct View {
    unsigned long long* keys;
    Meta* meta;
    Counters* ctr;
    Candidate* cand;            // one per eviction CTA
    uint2* guard;               // per slot: first and last token id of the node's element
    unsigned long long key_mask;   // all ones; fewer bits only to provoke collisions in tests
    uint32_t mask;              // capacity - 1
    uint32_t group;
};

struct Batch {
    const uint32_t* tokens;     // [n_seqs][stride]
    const uint32_t* lens;       // [n_seqs] tokens
    const uint32_t* pages;      // [n_seqs][page_stride] or null
    const uint32_t* page_lens;  // [n_seqs] or null (then `pages` rows are full)
    uint32_t n_seqs, stride, page_stride;
};

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}

// One multiply per token, one full mix at the end: not a cryptographic hash (nothing here defends against chosen tokens).
__device__ __forceinline__ unsigned long long element_hash(const uint32_t* tok, uint32_t group) {
    unsigned long long h = 0x9E3779B97F4A7C15ull;
    for (uint32_t i = 0; i < group; i++) {
        h = (h ^ __ldg(tok + i)) * 0xD6E8FEB86659FD93ull;
        h ^= h >> 32;
    }
    return mix64(h);
}

// The chain from the root is LINEAR in the element hashes, raw_i = raw_{i-1} * CHAIN_MUL + h_i (mod 2^64), so the raw
// values of a whole chunk come out of one parallel scan over affine maps x -> x * a + b; the table key is a full mix
// of the raw value (real keys are >= 2).
constexpr unsigned long long CHAIN_MUL = 0xBF58476D1CE4E5B9ull, ROOT_RAW = 0x243F6A8885A308D3ull;

__device__ __forceinline__ unsigned long long key_of_raw(unsigned long long raw, unsigned long long key_mask) {
    const unsigned long long k = mix64(raw ^ 0x632BE59BD9B4E019ull) & key_mask;
    return k < 2 ? k + 2 : k;
}

struct Affine {
    unsigned long long a, b;
};
// first `p`, then `q`
__device__ __forceinline__ Affine then(const Affine& p, const Affine& q) { return Affine{p.a * q.a, p.b * q.a + q.b}; }

__device__ __forceinline__ uint32_t find_slot(const View& ix, unsigned long long key) {
    uint32_t h = (uint32_t)(key >> 17) & ix.mask;
    for (uint32_t p = 0; p <= ix.mask; p++, h = (h + 1) & ix.mask) {
        const unsigned long long k = ix.keys[h];
        if (k == key) return h;
        if (k == KEY_EMPTY) return NO_SLOT;
    }
    return NO_SLOT;
}

// Finds the node or claims a slot for it (a tombstone on the probe path before the first empty slot is
// reused).  Exactly one thread of the grid gets `created` for a key that was absent.
__device__ __forceinline__ uint32_t find_or_claim(const View& ix, unsigned long long key, bool& created, bool& reused) {
    created = reused = false;
    uint32_t h = (uint32_t)(key >> 17) & ix.mask, first_tomb = NO_SLOT, scanned = 0;
    volatile unsigned long long* keys = ix.keys;
    for (uint32_t p = 0; p <= 4u * ix.mask + 3u; p++) {
        const unsigned long long k = keys[h];
        if (k == key) return h;
        if (k == KEY_TOMB && first_tomb == NO_SLOT) first_tomb = h;
        const bool path_ends = k == KEY_EMPTY || scanned == ix.mask;      // an empty slot, or the whole table seen (no empty slot left)
        if (path_ends) {
            if (k != KEY_EMPTY && first_tomb == NO_SLOT) return NO_SLOT;  // full of live nodes
            const uint32_t target = first_tomb != NO_SLOT ? first_tomb : h;
            const unsigned long long expect = first_tomb != NO_SLOT ? KEY_TOMB : KEY_EMPTY;
            const unsigned long long old = atomicCAS(ix.keys + target, expect, key);
            if (old == expect) {
                created = true;
                reused = first_tomb != NO_SLOT;
                return target;
            }
            if (old == key) return target;
            h = target;                 // somebody else's key went in: look again from there
            first_tomb = NO_SLOT;
            scanned = 0;
            continue;
        }
        h = (h + 1) & ix.mask;
        scanned++;
    }
    return NO_SLOT;
}

enum Op { OP_LOOKUP = 0, OP_INSERT_CLAIM = 1, OP_INSERT_PAGES = 2, OP_RELEASE = 3 };
constexpr int WALK_THREADS = 512;       // nodes one CTA handles per pass (one thread each)

// One CTA per sequence, one thread per node: element hashes, the key chain by a scan, every probe of the pass in
// flight at once, the first miss by a CTA-wide minimum.  A sequence with more nodes than threads takes more passes.
template <int OP>
__global__ void __launch_bounds__(WALK_THREADS) prefix_walk(View ix, Batch b, unsigned long long tick, uint32_t* out_pages,
                                                            uint32_t out_stride, uint32_t* out_matched) {
    __shared__ Affine warp_total[WALK_THREADS / 32];
    __shared__ uint32_t slots[WALK_THREADS];
    __shared__ unsigned long long carry_raw;
    __shared__ uint32_t first_miss, parent_carry;
    const uint32_t seq = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t n_elems = min(b.lens[seq], b.stride) / ix.group;
    const uint32_t* row = b.tokens + (size_t)seq * b.stride;
    if (tid == 0) {
        carry_raw = ROOT_RAW;
        parent_carry = NO_SLOT;
    }
    uint32_t matched = 0;
    for (uint32_t base = 0; base < n_elems; base += WALK_THREADS) {
        const uint32_t i = base + tid;
        const bool active = i < n_elems;
        if (tid == 0) first_miss = WALK_THREADS;
        // ---- keys of this pass ----
        Affine f = active ? Affine{CHAIN_MUL, element_hash(row + (size_t)i * ix.group, ix.group)} : Affine{1ull, 0ull};
#pragma unroll
        for (uint32_t off = 1; off < 32; off <<= 1) {
            Affine prev;
            prev.a = __shfl_up_sync(0xFFFFFFFFu, f.a, off);
            prev.b = __shfl_up_sync(0xFFFFFFFFu, f.b, off);
            if (lane >= off) f = then(prev, f);
        }
        if (lane == 31) warp_total[warp] = f;
        __syncthreads();
        Affine before{1ull, 0ull};
        for (uint32_t wv = 0; wv < warp; wv++) before = then(before, warp_total[wv]);
        f = then(before, f);
        const unsigned long long raw = carry_raw * f.a + f.b;
        const unsigned long long key = key_of_raw(raw, ix.key_mask);
        const uint2 guard = active ? make_uint2(__ldg(row + (size_t)i * ix.group), __ldg(row + (size_t)i * ix.group + ix.group - 1u)) : make_uint2(0u, 0u);
        __syncthreads();                                   // everyone has read carry_raw
        if (tid == WALK_THREADS - 1) carry_raw = raw;
        // ---- the table ----
        if (OP == OP_INSERT_CLAIM) {
            bool created = false, reused = false;
            const uint32_t slot = active ? find_or_claim(ix, key, created, reused) : NO_SLOT;
            if (active && slot == NO_SLOT) atomicExch(&ix.ctr->error, 1u);
            slots[tid] = slot;
            const uint32_t parent_of_first = parent_carry;
            __syncthreads();
            const uint32_t parent = tid ? slots[tid - 1] : parent_of_first;
            if (active && slot != NO_SLOT) {
                const unsigned long long order = (tick << (ORDER_SEQ_BITS + ORDER_DEPTH_BITS)) |
                                                 ((unsigned long long)seq << ORDER_DEPTH_BITS) | min(i, (1u << ORDER_DEPTH_BITS) - 1u);
                atomicMin(&ix.meta[slot].order, order);     // an older node keeps its (smaller) order
                atomicMax(&ix.meta[slot].stamp, tick);
                if (created) {
                    ix.meta[slot].parent = parent;
                    if (parent != NO_SLOT) atomicAdd(&ix.meta[parent].children, 1u);
                    atomicAdd(&ix.ctr->live, 1ull);
                    if (reused) atomicAdd(&ix.ctr->tombstones, ~0ull);
                }
            }
            __syncthreads();
            if (tid == WALK_THREADS - 1) parent_carry = slot;
        } else {
            uint32_t slot = active ? find_slot(ix, key) : NO_SLOT;
            if (OP == OP_INSERT_PAGES) {
                // The node belongs to the sequence whose creation order the claim pass left on it (the lowest-numbered one
                // that walked the key in this call): that one writes the page and the guard.  Nobody reads a guard here,
                // so none is read while it is being written.
                if (slot != NO_SLOT) {
                    Meta& m = ix.meta[slot];
                    const unsigned long long order = (tick << (ORDER_SEQ_BITS + ORDER_DEPTH_BITS)) |
                                                     ((unsigned long long)seq << ORDER_DEPTH_BITS) | min(i, (1u << ORDER_DEPTH_BITS) - 1u);
                    if (m.order == order) {
                        const uint32_t n_pages = b.pages ? (b.page_lens ? min(b.page_lens[seq], b.page_stride) : b.page_stride) : 0u;
                        m.page = i < n_pages ? b.pages[(size_t)seq * b.page_stride + i] : NO_PAGE;
                        ix.guard[slot] = guard;
                    }
                }
                __syncthreads();
                continue;
            }
            if (slot != NO_SLOT) {
                const uint2 g = ix.guard[slot];
                if (g.x != guard.x || g.y != guard.y) {    // the key of another prefix: not this sequence's node
                    slot = NO_SLOT;
                    atomicAdd(&ix.ctr->collisions, 1ull);
                }
            }
            if (slot == NO_SLOT) atomicMin(&first_miss, tid);
            __syncthreads();
            const uint32_t run = first_miss;               // matched nodes of this pass, from its start
            if (tid < run) {
                Meta& m = ix.meta[slot];
                if (OP == OP_LOOKUP) {
                    atomicAdd(&m.refs, 1);
                    atomicMax(&m.stamp, tick);
                    if (out_pages && i < out_stride) out_pages[(size_t)seq * out_stride + i] = m.page;
                } else {                                                           // OP_RELEASE
                    if (atomicAdd(&m.refs, -1) <= 0) atomicAdd(&m.refs, 1);       // never below zero
                }
            }
            matched += run;
            __syncthreads();                               // first_miss is reset at the top of the next pass
            if (run < (uint32_t)WALK_THREADS) break;
        }
        __syncthreads();
    }
    if (OP == OP_LOOKUP && tid == 0) {
        if (out_matched) out_matched[seq] = matched;
        if (matched) {
            atomicAdd(&ix.ctr->hits, 1ull);
            atomicAdd(&ix.ctr->tokens_saved, (unsigned long long)matched * ix.group);
        }
    }
}

__device__ __forceinline__ bool older(const Candidate& a, const Candidate& b) {      // a before b in eviction order
    if (a.valid != b.valid) return a.valid > b.valid;
    if (a.stamp != b.stamp) return a.stamp < b.stamp;
    if (a.order != b.order) return a.order < b.order;
    return a.slot < b.slot;
}

// One victim per launch: every CTA scans a share of the table for its best candidate; the last CTA to
// finish picks the best of those, unlinks it and appends its page to the output.
__global__ void __launch_bounds__(256) prefix_evict_one(View ix, uint32_t* out_pages, uint32_t out_cap, uint32_t* out_count,
                                                        uint32_t* out_nodes) {
    __shared__ Candidate best[256];
    __shared__ uint32_t last;
    Candidate mine{~0ull, ~0ull, NO_SLOT, 0u};
    for (uint32_t s = blockIdx.x * blockDim.x + threadIdx.x; s <= ix.mask; s += gridDim.x * blockDim.x) {
        if (ix.keys[s] < 2) continue;
        const Meta m = ix.meta[s];
        if (m.refs > 0 || m.children != 0) continue;
        const Candidate c{m.stamp, m.order, s, 1u};
        if (older(c, mine)) mine = c;
    }
    best[threadIdx.x] = mine;
    __syncthreads();
    for (uint32_t off = 128; off > 0; off >>= 1) {
        if (threadIdx.x < off && older(best[threadIdx.x + off], best[threadIdx.x])) best[threadIdx.x] = best[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        ix.cand[blockIdx.x] = best[0];
        __threadfence();
        last = atomicAdd(&ix.ctr->evict_ctas_done, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    mine = Candidate{~0ull, ~0ull, NO_SLOT, 0u};
    for (uint32_t c = threadIdx.x; c < gridDim.x; c += blockDim.x) {
        const Candidate x{__ldcg(&ix.cand[c].stamp), __ldcg(&ix.cand[c].order), __ldcg(&ix.cand[c].slot), __ldcg(&ix.cand[c].valid)};
        if (older(x, mine)) mine = x;
    }
    best[threadIdx.x] = mine;
    __syncthreads();
    for (uint32_t off = 128; off > 0; off >>= 1) {
        if (threadIdx.x < off && older(best[threadIdx.x + off], best[threadIdx.x])) best[threadIdx.x] = best[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        ix.ctr->evict_ctas_done = 0;
        const Candidate v = best[0];
        if (v.valid) {
            Meta& m = ix.meta[v.slot];
            if (m.page != NO_PAGE) {
                const uint32_t at = atomicAdd(out_count, 1u);
                if (at < out_cap) out_pages[at] = m.page;
            }
            if (out_nodes) atomicAdd(out_nodes, 1u);
            if (m.parent != NO_SLOT) atomicSub(&ix.meta[m.parent].children, 1u);
            m = Meta{ORDER_FRESH, 0ull, NO_PAGE, 0, NO_SLOT, 0u};
            ix.keys[v.slot] = KEY_TOMB;
            ix.ctr->live -= 1;
            ix.ctr->tombstones += 1;
        }
    }
}

__global__ void prefix_index_clear(View ix) {
    for (size_t s = blockIdx.x * (size_t)blockDim.x + threadIdx.x; s <= ix.mask; s += (size_t)gridDim.x * blockDim.x) {
        ix.keys[s] = KEY_EMPTY;
        ix.meta[s] = Meta{ORDER_FRESH, 0ull, NO_PAGE, 0, NO_SLOT, 0u};
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *ix.ctr = Counters{};
}


// ---------------------------------------------------------------------------------------------
// Device-side page allocator: PageAllocator (engine/src/kv_cache.rs:762-797), a LIFO stack of free
// page ids, kept in HBM.  One launch serves a whole batch: sequence s takes (or returns) counts[s]
// pages into (from) row s of a block table starting at entry first[s], and gets exactly the ids the
// reference's allocate() would pop for the sequences in index order (a fresh stack hands out 0, 1, 2 ...).
// A batch that asks for more than is free gets nothing and the status word says so.
// ---------------------------------------------------------------------------------------------
struct PageStack {
    uint32_t* ids;      // [total]
    uint32_t* top;      // pages on the stack
    uint32_t total;
};

struct PageBatch {
    uint32_t* tables;           // [n_seqs][stride]
    const uint32_t* first;      // [n_seqs] or null (0)
    const uint32_t* counts;     // [n_seqs], or null: ceil(seq_lens / block_size) - first
    const uint32_t* seq_lens;
    uint32_t n_seqs, stride, block_size;
};

__device__ __forceinline__ uint32_t pages_of(const PageBatch& b, uint32_t s) {
    if (b.counts) return b.counts[s];
    const uint32_t nb = (b.seq_lens[s] + b.block_size - 1) / b.block_size, f = b.first ? b.first[s] : 0u;
    return nb > f ? nb - f : 0u;
}

__global__ void page_stack_init(PageStack st) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < st.total; i += gridDim.x * blockDim.x) st.ids[i] = st.total - 1u - i;
    if (blockIdx.x == 0 && threadIdx.x == 0) *st.top = st.total;
}

// offsets[s] = sum of counts before s, through shared memory in chunks of the CTA; returns the batch total
template <bool FREE>
__global__ void __launch_bounds__(1024) page_stack_batch(PageStack st, PageBatch b, uint32_t* status) {
    __shared__ uint32_t scan[1024];
    __shared__ uint32_t carry, bad;
    const uint32_t t = threadIdx.x;
    if (t == 0) carry = bad = 0;
    __syncthreads();
    // pass 1: validate rows and total the request
    for (uint32_t s0 = 0; s0 < b.n_seqs; s0 += 1024) {
        const uint32_t s = s0 + t;
        const uint32_t c = s < b.n_seqs ? pages_of(b, s) : 0u, f = (s < b.n_seqs && b.first) ? b.first[s] : 0u;
        if (c && ((unsigned long long)f + c > b.stride)) atomicExch(&bad, 1u);
        scan[t] = c;
        __syncthreads();
        for (uint32_t off = 512; off > 0; off >>= 1) {
            if (t < off) scan[t] += scan[t + off];
            __syncthreads();
        }
        if (t == 0) carry = (carry > 0xFFFFFFFFu - scan[0]) ? 0xFFFFFFFFu : carry + scan[0];
        __syncthreads();
    }
    const uint32_t total = carry, top = *st.top;
    uint32_t verdict = 0;
    if (bad) verdict = TKV_ERR_INVALID_CONFIG;
    else if (!FREE && total > top) verdict = TKV_ERR_POOL_EXHAUSTED;
    else if (FREE && total > st.total - top) verdict = TKV_ERR_INVALID_CONFIG;       // more pages returned than were ever handed out
    __syncthreads();
    if (verdict) {
        if (t == 0 && status) *status = verdict;
        return;
    }
    // pass 2: running offsets chunk by chunk, each thread then moves its sequence's ids
    if (t == 0) carry = 0;
    __syncthreads();
    for (uint32_t s0 = 0; s0 < b.n_seqs; s0 += 1024) {
        const uint32_t s = s0 + t;
        const uint32_t c = s < b.n_seqs ? pages_of(b, s) : 0u;
        scan[t] = c;
        __syncthreads();
        for (uint32_t off = 1; off < 1024; off <<= 1) {                              // inclusive scan
            const uint32_t v = t >= off ? scan[t - off] : 0u;
            __syncthreads();
            scan[t] += v;
            __syncthreads();
        }
        const uint32_t before = carry + scan[t] - c;
        if (c) {
            uint32_t* row = b.tables + (size_t)s * b.stride + (b.first ? b.first[s] : 0u);
            for (uint32_t i = 0; i < c; i++) {
                if (FREE) st.ids[top + before + i] = row[i];                          // push in table order
                else row[i] = st.ids[top - 1u - before - i];                         // the i-th pop of this sequence
            }
        }
        __syncthreads();
        if (t == 1023) carry += scan[1023];
        __syncthreads();
    }
    if (t == 0) {
        *st.top = FREE ? top + total : top - total;
        if (status) *status = 0;
    }
}

int32_t fail(int32_t code, const char* msg) { return tkv_internal::set_error(code, 0, msg); }
int32_t fail_cuda(cudaError_t e, const char* what) {
    char buf[200];
    snprintf(buf, sizeof buf, "cuda error: %s: %s", what, cudaGetErrorString(e));
    return tkv_internal::set_error(TKV_ERR_CUDA, (int32_t)e, buf);
}

struct DeviceGuard {
    int prev = -1;
    cudaError_t err;
    explicit DeviceGuard(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
        else if (err == cudaSuccess) prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace

struct tkv_prefix_index {
    int device = 0;
    uint64_t capacity = 0;
    uint32_t group = 1;
    unsigned long long tick = 0;
    int evict_ctas = 1;
    View view{};
};

namespace {

int32_t check_batch(const tkv_prefix_index* ix, const TkvPrefixBatch* b, Batch& out) {
    if (!ix || !b) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (b->n_seqs == 0) return TKV_OK;
    if (!b->tokens || !b->lens || b->stride == 0) return fail(TKV_ERR_INVALID_CONFIG, "prefix batch: NULL tokens / lens or zero stride");
    if (b->n_seqs >= (1u << ORDER_SEQ_BITS)) return fail(TKV_ERR_INVALID_CONFIG, "prefix batch: at most 16383 sequences per call");
    if (b->pages && b->page_stride == 0) return fail(TKV_ERR_INVALID_CONFIG, "prefix batch: pages without page_stride");
    out.tokens = reinterpret_cast<const uint32_t*>(b->tokens);
    out.lens = reinterpret_cast<const uint32_t*>(b->lens);
    out.pages = reinterpret_cast<const uint32_t*>(b->pages);
    out.page_lens = reinterpret_cast<const uint32_t*>(b->page_lens);
    out.n_seqs = b->n_seqs;
    out.stride = b->stride;
    out.page_stride = b->page_stride;
    return TKV_OK;
}

}  // namespace

extern "C" {

int32_t tkv_prefix_index_create(int32_t device, uint64_t capacity, uint32_t group_tokens, tkv_prefix_index** out) {
    if (!out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    *out = nullptr;
    if (capacity < 64 || capacity > (1ull << 31) || (capacity & (capacity - 1)))
        return fail(TKV_ERR_INVALID_CONFIG, "prefix index: capacity must be a power of two in [64, 2^31]");
    if (group_tokens == 0 || group_tokens > 4096) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: group_tokens must be in [1, 4096]");
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    auto* ix = new (std::nothrow) tkv_prefix_index();
    if (!ix) return fail(TKV_ERR_POOL_EXHAUSTED, "prefix index: out of host memory");
    ix->device = device;
    ix->capacity = capacity;
    ix->group = group_tokens;
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    ix->evict_ctas = (int)std::min<uint64_t>(std::max(sms, 1) * 4, (capacity + 255) / 256);
    cudaError_t e = cudaMalloc(&ix->view.keys, capacity * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(&ix->view.meta, capacity * sizeof(Meta));
    if (e == cudaSuccess) e = cudaMalloc(&ix->view.ctr, sizeof(Counters));
    if (e == cudaSuccess) e = cudaMalloc(&ix->view.cand, (size_t)ix->evict_ctas * sizeof(Candidate));
    if (e == cudaSuccess) e = cudaMalloc(&ix->view.guard, capacity * sizeof(uint2));
    if (e == cudaSuccess) {
        ix->view.key_mask = ~0ull;
        ix->view.mask = (uint32_t)(capacity - 1);
        ix->view.group = group_tokens;
        prefix_index_clear<<<std::max(sms, 1) * 2, 256>>>(ix->view);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
    }
    if (e != cudaSuccess) {
        tkv_prefix_index_destroy(ix);
        return fail_cuda(e, "prefix index allocation");
    }
    *out = ix;
    return TKV_OK;
}

void tkv_prefix_index_destroy(tkv_prefix_index* ix) {
    if (!ix) return;
    DeviceGuard guard(ix->device);
    cudaFree(ix->view.keys);
    cudaFree(ix->view.meta);
    cudaFree(ix->view.ctr);
    cudaFree(ix->view.cand);
    cudaFree(ix->view.guard);
    delete ix;
}

// Test hook for the collision guard: keys are cut to `bits` bits, so that different prefixes share keys often.  Only on an
// index that holds nothing yet.
int32_t tkv_prefix_index_set_key_bits(tkv_prefix_index* ix, uint32_t bits) {
    if (!ix) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (bits < 4 || bits > 64) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: key bits must be in [4, 64]");
    if (ix->tick) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: key bits can only be set before the first call that walks the index");
    ix->view.key_mask = bits == 64 ? ~0ull : ((1ull << bits) - 1ull);
    return TKV_OK;
}

int32_t tkv_prefix_index_insert(tkv_prefix_index* ix, const TkvPrefixBatch* batch, void* stream) {
    Batch b{};
    if (int32_t rc = check_batch(ix, batch, b)) return rc;
    if (b.n_seqs == 0) return TKV_OK;
    DeviceGuard guard(ix->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const unsigned long long tick = ++ix->tick;
    if (tick >> (64 - ORDER_SEQ_BITS - ORDER_DEPTH_BITS)) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: call counter exhausted");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t ctas = b.n_seqs;
    // two launches: every node is found or claimed first, then the sequence that created a node writes its page
    prefix_walk<OP_INSERT_CLAIM><<<ctas, WALK_THREADS, 0, st>>>(ix->view, b, tick, nullptr, 0, nullptr);
    prefix_walk<OP_INSERT_PAGES><<<ctas, WALK_THREADS, 0, st>>>(ix->view, b, tick, nullptr, 0, nullptr);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "prefix index insert");
}

int32_t tkv_prefix_index_lookup(tkv_prefix_index* ix, const TkvPrefixBatch* batch, uint64_t out_pages, uint32_t out_stride,
                                uint64_t out_matched, void* stream) {
    Batch b{};
    if (int32_t rc = check_batch(ix, batch, b)) return rc;
    if (b.n_seqs == 0) return TKV_OK;
    if (out_pages && out_stride == 0) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: out_pages without out_stride");
    DeviceGuard guard(ix->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const unsigned long long tick = ++ix->tick;
    const uint32_t ctas = b.n_seqs;
    prefix_walk<OP_LOOKUP><<<ctas, WALK_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        ix->view, b, tick, reinterpret_cast<uint32_t*>(out_pages), out_stride, reinterpret_cast<uint32_t*>(out_matched));
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "prefix index lookup");
}

int32_t tkv_prefix_index_release(tkv_prefix_index* ix, const TkvPrefixBatch* batch, void* stream) {
    Batch b{};
    if (int32_t rc = check_batch(ix, batch, b)) return rc;
    if (b.n_seqs == 0) return TKV_OK;
    DeviceGuard guard(ix->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    const uint32_t ctas = b.n_seqs;
    prefix_walk<OP_RELEASE><<<ctas, WALK_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(ix->view, b, ix->tick, nullptr, 0, nullptr);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "prefix index release");
}

int32_t tkv_prefix_index_evict_lru(tkv_prefix_index* ix, uint32_t max_nodes, uint64_t out_pages, uint32_t out_cap, uint64_t out_count,
                                   uint64_t out_nodes, void* stream) {
    if (!ix) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (!out_count || (out_cap && !out_pages)) return fail(TKV_ERR_INVALID_CONFIG, "prefix index: evict needs out_count (and out_pages for out_cap > 0)");
    DeviceGuard guard(ix->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(reinterpret_cast<void*>(out_count), 0, sizeof(uint32_t), st);
    if (e == cudaSuccess && out_nodes) e = cudaMemsetAsync(reinterpret_cast<void*>(out_nodes), 0, sizeof(uint32_t), st);
    max_nodes = (uint32_t)std::min<uint64_t>(max_nodes, ix->capacity);      // one launch per node: never more than the table holds
    for (uint32_t i = 0; i < max_nodes && e == cudaSuccess; i++) {
        prefix_evict_one<<<ix->evict_ctas, 256, 0, st>>>(ix->view, reinterpret_cast<uint32_t*>(out_pages), out_cap,
                                                         reinterpret_cast<uint32_t*>(out_count), reinterpret_cast<uint32_t*>(out_nodes));
        e = cudaGetLastError();
    }
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "prefix index evict");
}

int32_t tkv_prefix_index_stats(tkv_prefix_index* ix, void* stream, TkvPrefixIndexStats* out) {
    if (!ix || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    DeviceGuard guard(ix->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    Counters c{};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&c, ix->view.ctr, sizeof c, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail_cuda(e, "prefix index stats");
    out->hits = c.hits;
    out->tokens_saved = c.tokens_saved;
    out->live_nodes = c.live;
    out->tombstones = c.tombstones;
    out->capacity = ix->capacity;
    out->ticks = ix->tick;
    out->group_tokens = ix->group;
    out->table_full = c.error;
    out->key_collisions = c.collisions;
    return TKV_OK;
}

}  // extern "C"

struct tkv_device_page_allocator {
    int device = 0;
    PageStack st{};
};

namespace {
int32_t page_batch(tkv_device_page_allocator* a, const TkvPageBatch* batch, uint64_t status, void* stream, bool release) {
    if (!a || !batch) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (batch->n_seqs == 0) return TKV_OK;
    if (!batch->tables || batch->table_stride == 0) return fail(TKV_ERR_INVALID_CONFIG, "page batch: NULL tables or zero stride");
    if (!batch->counts && (!batch->seq_lens || batch->block_size == 0))
        return fail(TKV_ERR_INVALID_CONFIG, "page batch: give counts, or seq_lens and block_size to derive them");
    DeviceGuard guard(a->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    PageBatch b{reinterpret_cast<uint32_t*>(batch->tables), reinterpret_cast<const uint32_t*>(batch->first),
                reinterpret_cast<const uint32_t*>(batch->counts), reinterpret_cast<const uint32_t*>(batch->seq_lens),
                batch->n_seqs, batch->table_stride, batch->block_size};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (release) page_stack_batch<true><<<1, 1024, 0, st>>>(a->st, b, reinterpret_cast<uint32_t*>(status));
    else page_stack_batch<false><<<1, 1024, 0, st>>>(a->st, b, reinterpret_cast<uint32_t*>(status));
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "device page allocator");
}
}  // namespace

extern "C" {

int32_t tkv_device_page_allocator_create(int32_t device, uint32_t total_pages, tkv_device_page_allocator** out) {
    if (!out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    *out = nullptr;
    if (total_pages == 0) return fail(TKV_ERR_INVALID_CONFIG, "device page allocator: zero pages");
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    auto* a = new (std::nothrow) tkv_device_page_allocator();
    if (!a) return fail(TKV_ERR_POOL_EXHAUSTED, "device page allocator: out of host memory");
    a->device = device;
    a->st.total = total_pages;
    cudaError_t e = cudaMalloc(&a->st.ids, (size_t)total_pages * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&a->st.top, sizeof(uint32_t));
    if (e == cudaSuccess) {
        page_stack_init<<<64, 256>>>(a->st);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
    }
    if (e != cudaSuccess) {
        tkv_device_page_allocator_destroy(a);
        return fail_cuda(e, "device page allocator allocation");
    }
    *out = a;
    return TKV_OK;
}

void tkv_device_page_allocator_destroy(tkv_device_page_allocator* a) {
    if (!a) return;
    DeviceGuard guard(a->device);
    cudaFree(a->st.ids);
    cudaFree(a->st.top);
    delete a;
}

int32_t tkv_device_page_allocator_allocate(tkv_device_page_allocator* a, const TkvPageBatch* batch, uint64_t status, void* stream) {
    return page_batch(a, batch, status, stream, false);
}

int32_t tkv_device_page_allocator_free(tkv_device_page_allocator* a, const TkvPageBatch* batch, uint64_t status, void* stream) {
    return page_batch(a, batch, status, stream, true);
}

int32_t tkv_device_page_allocator_available(tkv_device_page_allocator* a, void* stream, uint32_t* out) {
    if (!a || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    DeviceGuard guard(a->device);
    if (guard.err != cudaSuccess) return fail_cuda(guard.err, "cudaSetDevice");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(out, a->st.top, sizeof(uint32_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? TKV_OK : fail_cuda(e, "device page allocator available");
}

}  // extern "C"
