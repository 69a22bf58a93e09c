// Host-side block bookkeeping behind the C ABI: the page allocator, block table,
// contiguous-run allocator, token radix tree and prefix table that decide WHICH
// blocks a handoff reads and writes.  Pure integer logic, no CUDA.
// Citations are paths inside the tempura repository.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <limits>
#include <map>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/tkv.h"

// ---- PageAllocator: engine/src/kv_cache.rs:762-793 ---------------------------------
// LIFO free stack seeded so that page 0 is handed out first and a freed page is the
// next one returned.
struct tkv_page_allocator {
    std::vector<size_t> stack;
    size_t total = 0;
};

// ---- BlockTable: engine/src/kv_cache.rs:836-893 ------------------------------------
struct tkv_block_table {
    static constexpr uint32_t kEmpty = std::numeric_limits<uint32_t>::max();
    std::vector<uint32_t> ids;
    size_t live = 0;
};

// ---- PageRunAllocator: engine/src/gpu_page_pool.rs:34-218 --------------------------
// Unsorted free list of at most 128 runs; best-fit allocation (first seen wins a
// tie), freeing merges with every adjacent free run before the run is appended.
struct tkv_run_allocator {
    struct Run {
        size_t start, pages;
    };
    static constexpr size_t kMaxRuns = 128;
    std::vector<Run> runs;
    size_t total = 0, allocated = 0;
};

// ---- RadixTree: engine/src/prefix_cache.rs:17-149 ----------------------------------
struct tkv_radix_tree {
    struct Node {
        std::unordered_map<uint32_t, size_t> next;
        std::vector<size_t> pages;
        size_t refs = 0;
        uint64_t stamp = 0;
        bool unlinked = false;
    };
    std::vector<Node> arena{1};
    uint64_t clock = 0, hits = 0, saved = 0;
};

// ---- PrefixCacheTable: engine/src/kv_cache.rs:581-730 ------------------------------
struct tkv_prefix_table {
    struct Key {
        bool salted;
        std::string salt;
        std::vector<uint32_t> tokens;
        bool operator<(const Key& o) const {
            if (salted != o.salted) return salted < o.salted;
            if (salt != o.salt) return salt < o.salt;
            return tokens < o.tokens;
        }
    };
    struct Entry {
        std::vector<uint32_t> blocks;
        size_t seq_len = 0, refs = 0;
        uint64_t stamp = 0;
    };
    std::map<Key, Entry> entries;
    size_t max_entries = 0;
    uint64_t clock = 0, hits = 0, saved = 0;
    static Key key(const uint32_t* t, size_t n, const char* salt) {
        return Key{salt != nullptr, salt ? std::string(salt) : std::string(), std::vector<uint32_t>(t, t + n)};
    }
};

extern "C" {

// ------------------------------------------------------------------ page allocator
tkv_page_allocator* tkv_page_allocator_new(size_t total) {
    auto* a = new tkv_page_allocator();
    a->total = total;
    a->stack.reserve(total);
    for (size_t i = total; i-- > 0;) a->stack.push_back(i);
    return a;
}
void tkv_page_allocator_delete(tkv_page_allocator* a) { delete a; }
int32_t tkv_page_allocator_allocate(tkv_page_allocator* a, size_t* page) {
    if (a->stack.empty()) return TKV_ERR_POOL_EXHAUSTED;
    *page = a->stack.back();
    a->stack.pop_back();
    return TKV_OK;
}
void tkv_page_allocator_free(tkv_page_allocator* a, size_t page) { a->stack.push_back(page); }
size_t tkv_page_allocator_available(const tkv_page_allocator* a) { return a->stack.size(); }
size_t tkv_page_allocator_in_use(const tkv_page_allocator* a) { return a->total - a->stack.size(); }
size_t tkv_page_allocator_total(const tkv_page_allocator* a) { return a->total; }

// ------------------------------------------------------------------ block table
tkv_block_table* tkv_block_table_new(size_t max_blocks) {
    auto* t = new tkv_block_table();
    t->ids.assign(max_blocks, tkv_block_table::kEmpty);
    return t;
}
void tkv_block_table_delete(tkv_block_table* t) { delete t; }
int32_t tkv_block_table_set_block(tkv_block_table* t, size_t logical, size_t page) {
    if (logical >= t->ids.size()) return TKV_ERR_INVALID_CONFIG;  // the reference panics on the index
    t->ids[logical] = static_cast<uint32_t>(page);
    t->live = std::max(t->live, logical + 1);
    return TKV_OK;
}
int32_t tkv_block_table_get_block(const tkv_block_table* t, size_t logical, size_t* page) {
    if (logical >= t->live || t->ids[logical] == tkv_block_table::kEmpty) return 0;
    *page = t->ids[logical];
    return 1;
}
size_t tkv_block_table_num_blocks(const tkv_block_table* t) { return t->live; }
size_t tkv_block_table_max_blocks(const tkv_block_table* t) { return t->ids.size(); }
const uint32_t* tkv_block_table_as_slice(const tkv_block_table* t) { return t->ids.data(); }
size_t tkv_block_table_clear(tkv_block_table* t, size_t* freed, size_t cap) {
    size_t n = 0;
    for (size_t i = 0; i < t->live; i++) {
        if (t->ids[i] == tkv_block_table::kEmpty) continue;
        if (n < cap && freed) freed[n] = t->ids[i];
        n++;
    }
    std::fill(t->ids.begin(), t->ids.end(), tkv_block_table::kEmpty);
    t->live = 0;
    return n;
}

// ------------------------------------------------------------------ run allocator
tkv_run_allocator* tkv_run_allocator_new(size_t total) {
    auto* a = new tkv_run_allocator();
    a->total = total;
    if (total) a->runs.push_back({0, total});
    return a;
}
void tkv_run_allocator_delete(tkv_run_allocator* a) { delete a; }
static void drop_run(tkv_run_allocator* a, size_t i) {
    a->runs[i] = a->runs.back();  // swap-remove keeps the reference's scan order
    a->runs.pop_back();
}
int32_t tkv_run_allocator_alloc(tkv_run_allocator* a, size_t pages, size_t* start) {
    if (pages == 0) return 0;
    size_t best = SIZE_MAX;
    for (size_t i = 0; i < a->runs.size(); i++)
        if (a->runs[i].pages >= pages && (best == SIZE_MAX || a->runs[i].pages < a->runs[best].pages)) best = i;
    if (best == SIZE_MAX) return 0;
    *start = a->runs[best].start;
    if (a->runs[best].pages == pages) {
        drop_run(a, best);
    } else {
        a->runs[best].start += pages;
        a->runs[best].pages -= pages;
    }
    a->allocated += pages;
    return 1;
}
int32_t tkv_run_allocator_free(tkv_run_allocator* a, size_t start, size_t pages) {
    if (pages == 0 || start + pages > a->total) return TKV_OK;  // ignored, as in the reference
    a->allocated -= pages;
    for (bool merged = true; merged;) {
        merged = false;
        for (size_t i = 0; i < a->runs.size(); i++) {
            const auto r = a->runs[i];
            if (r.start + r.pages == start) {
                start = r.start;
                pages += r.pages;
            } else if (r.start == start + pages) {
                pages += r.pages;
            } else {
                continue;
            }
            drop_run(a, i);
            merged = true;
            break;
        }
    }
    if (a->runs.size() >= tkv_run_allocator::kMaxRuns) return TKV_ERR_POOL_EXHAUSTED;  // the reference panics here
    a->runs.push_back({start, pages});
    return TKV_OK;
}
int32_t tkv_run_allocator_try_extend(tkv_run_allocator* a, size_t start, size_t pages, size_t target) {
    if (target <= pages) return 1;
    const size_t extra = target - pages, end = start + pages;
    for (size_t i = 0; i < a->runs.size(); i++) {
        auto& r = a->runs[i];
        if (r.start != end || r.pages < extra) continue;
        if (r.pages == extra) {
            drop_run(a, i);
        } else {
            r.start = end + extra;
            r.pages -= extra;
        }
        a->allocated += extra;
        return 1;
    }
    return 0;
}
size_t tkv_run_allocator_free_pages(const tkv_run_allocator* a) {
    size_t s = 0;
    for (const auto& r : a->runs) s += r.pages;
    return s;
}
size_t tkv_run_allocator_allocated_pages(const tkv_run_allocator* a) { return a->allocated; }
size_t tkv_run_allocator_free_runs(const tkv_run_allocator* a, size_t* starts, size_t* pages, size_t cap) {
    for (size_t i = 0; i < a->runs.size() && i < cap; i++) {
        starts[i] = a->runs[i].start;
        pages[i] = a->runs[i].pages;
    }
    return a->runs.size();
}

// ------------------------------------------------------------------ radix tree
tkv_radix_tree* tkv_radix_tree_new(void) { return new tkv_radix_tree(); }
void tkv_radix_tree_delete(tkv_radix_tree* t) { delete t; }
void tkv_radix_tree_insert(tkv_radix_tree* t, const uint32_t* tokens, size_t n, const size_t* pages, size_t n_pages) {
    const uint64_t now = ++t->clock;
    size_t at = 0;
    for (size_t i = 0; i < n; i++) {
        auto it = t->arena[at].next.find(tokens[i]);
        if (it != t->arena[at].next.end()) {
            at = it->second;
            t->arena[at].stamp = now;
            continue;
        }
        tkv_radix_tree::Node fresh;
        if (i < n_pages) fresh.pages.push_back(pages[i]);  // a page id only lands on a NEW node
        fresh.stamp = now;
        const size_t id = t->arena.size();
        t->arena.push_back(std::move(fresh));
        t->arena[at].next.emplace(tokens[i], id);
        at = id;
    }
}
size_t tkv_radix_tree_lookup(tkv_radix_tree* t, const uint32_t* tokens, size_t n, size_t* pages_out, size_t cap,
                             size_t* n_pages) {
    const uint64_t now = ++t->clock;
    size_t at = 0, matched = 0, np = 0;
    for (size_t i = 0; i < n; i++) {
        auto it = t->arena[at].next.find(tokens[i]);
        if (it == t->arena[at].next.end()) break;
        at = it->second;
        auto& node = t->arena[at];
        node.stamp = now;
        node.refs++;
        matched++;
        for (size_t pg : node.pages) {
            if (np < cap && pages_out) pages_out[np] = pg;
            np++;
        }
    }
    if (matched) {
        t->hits++;
        t->saved += matched;
    }
    if (n_pages) *n_pages = np;
    return matched;
}
void tkv_radix_tree_release(tkv_radix_tree* t, const uint32_t* tokens, size_t n) {
    size_t at = 0;
    for (size_t i = 0; i < n; i++) {
        auto it = t->arena[at].next.find(tokens[i]);
        if (it == t->arena[at].next.end()) break;
        at = it->second;
        if (t->arena[at].refs) t->arena[at].refs--;
    }
}
// Unlinks the least recently used unreferenced leaf and returns its pages.
// Departure from engine/src/prefix_cache.rs:99-125, on purpose: the reference leaves
// the unlinked node eligible, so a second call reports the same page again; here an
// unlinked node is never reported twice (a page must not be freed twice).
size_t tkv_radix_tree_evict_lru(tkv_radix_tree* t, size_t* freed, size_t cap) {
    size_t victim = 0;
    for (size_t i = 1; i < t->arena.size(); i++) {
        const auto& nd = t->arena[i];
        if (nd.unlinked || nd.refs || !nd.next.empty()) continue;
        if (!victim || nd.stamp < t->arena[victim].stamp) victim = i;
    }
    if (!victim) return 0;
    for (auto& nd : t->arena)
        for (auto it = nd.next.begin(); it != nd.next.end();) it = (it->second == victim) ? nd.next.erase(it) : std::next(it);
    t->arena[victim].unlinked = true;
    size_t n = 0;
    for (size_t pg : t->arena[victim].pages) {
        if (n < cap && freed) freed[n] = pg;
        n++;
    }
    return n;
}
uint64_t tkv_radix_tree_hit_count(const tkv_radix_tree* t) { return t->hits; }
uint64_t tkv_radix_tree_tokens_saved(const tkv_radix_tree* t) { return t->saved; }
size_t tkv_radix_tree_node_count(const tkv_radix_tree* t) { return t->arena.size(); }

// ------------------------------------------------------------------ prefix table
tkv_prefix_table* tkv_prefix_table_new(size_t max_entries) {
    auto* t = new tkv_prefix_table();
    t->max_entries = max_entries;
    return t;
}
void tkv_prefix_table_delete(tkv_prefix_table* t) { delete t; }
void tkv_prefix_table_store(tkv_prefix_table* t, const uint32_t* tokens, size_t n, const char* salt,
                            const uint32_t* blocks, size_t n_blocks, size_t seq_len) {
    if (n == 0 || seq_len == 0) return;
    const uint64_t now = ++t->clock;
    if (t->entries.size() >= t->max_entries) {
        // least recently used entry nobody references; none -> the table grows
        auto victim = t->entries.end();
        for (auto it = t->entries.begin(); it != t->entries.end(); ++it)
            if (it->second.refs == 0 && (victim == t->entries.end() || it->second.stamp < victim->second.stamp)) victim = it;
        if (victim != t->entries.end()) t->entries.erase(victim);
    }
    tkv_prefix_table::Entry e;
    e.blocks.assign(blocks, blocks + n_blocks);
    e.seq_len = seq_len;
    e.stamp = now;
    t->entries[tkv_prefix_table::key(tokens, n, salt)] = std::move(e);
}
size_t tkv_prefix_table_probe(tkv_prefix_table* t, const uint32_t* tokens, size_t n, const char* salt,
                              uint32_t* blocks_out, size_t cap, size_t* n_blocks) {
    const uint64_t now = ++t->clock;
    if (n_blocks) *n_blocks = 0;
    for (size_t len = n; len > 0; len--) {  // longest stored prefix wins
        auto it = t->entries.find(tkv_prefix_table::key(tokens, len, salt));
        if (it == t->entries.end()) continue;
        auto& e = it->second;
        e.stamp = now;
        e.refs++;
        t->hits++;
        t->saved += len;
        if (n_blocks) *n_blocks = e.blocks.size();
        for (size_t i = 0; i < e.blocks.size() && i < cap; i++) blocks_out[i] = e.blocks[i];
        return e.seq_len;
    }
    return 0;
}
void tkv_prefix_table_release(tkv_prefix_table* t, const uint32_t* tokens, size_t n, const char* salt) {
    auto it = t->entries.find(tkv_prefix_table::key(tokens, n, salt));
    if (it != t->entries.end() && it->second.refs) it->second.refs--;
}
size_t tkv_prefix_table_len(const tkv_prefix_table* t) { return t->entries.size(); }
uint64_t tkv_prefix_table_hit_count(const tkv_prefix_table* t) { return t->hits; }
uint64_t tkv_prefix_table_tokens_saved(const tkv_prefix_table* t) { return t->saved; }

}  // extern "C"
