// Handoff coordinator: the host-side bookkeeping a disaggregated server needs around the handoff --
// route a new request to a prefill worker, admit its finished prefill to a decode worker only when
// that worker's pool has the pages (the reference gates admission on pool headroom the same way,
// server/src/engine_task.rs:618-660, and keeps per-request state in BatchScheduler,
// server/src/batch.rs:13-56), follow the transfer, and fall back to prefilling on the decode
// worker itself when a handoff times out or keeps failing.  Pure host logic, no CUDA: the callers
// feed it what the device calls reported (free pages, completion flags, status words).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <new>
#include <unordered_map>
#include <vector>

#include "../../include/tkv.h"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* message);
}

namespace {

int32_t fail(int32_t code, const char* fmt, unsigned long long x = 0, unsigned long long y = 0) {
    char buf[200];
    snprintf(buf, sizeof buf, fmt, x, y);
    return tkv_internal::set_error(code, 0, buf);
}

struct Request {
    uint64_t id = 0;
    uint32_t n_tokens = 0, max_new_tokens = 0, priority = 0;
    uint32_t state = TKV_REQ_QUEUED;
    uint32_t prefill_worker = 0, decode_worker = 0;
    uint32_t prefix_tokens = 0;       // resident on the decode side, reported after prefill
    uint32_t reserved_blocks = 0;     // held against the decode worker's headroom
    uint32_t attempts = 0;            // handoffs started
    uint64_t age = 0;                 // submission order
    uint64_t transfer_started = 0;    // coordinator clock
};

}  // namespace

struct tkv_coordinator {
    TkvCoordinatorConfig cfg{};
    std::unordered_map<uint64_t, Request> reqs;
    std::vector<std::deque<uint64_t>> prefill_queues;     // per prefill worker, submission order
    std::vector<uint64_t> prefill_load;                   // queued + running prompt tokens per prefill worker
    std::deque<uint64_t> waiting;                         // prefill done, not yet admitted to a decode worker
    std::vector<uint64_t> free_blocks, reserved;          // per decode worker: last reported free pages, pages promised
    std::vector<uint32_t> inflight;                       // per decode worker: handoffs admitted and not finished
    uint64_t next_age = 0;
    TkvCoordinatorStats stats{};
};

namespace {

uint32_t blocks_needed(const tkv_coordinator* c, const Request& r) {
    const uint64_t bs = c->cfg.block_size;
    const uint64_t total = ((uint64_t)r.n_tokens + r.max_new_tokens + bs - 1) / bs;
    const uint64_t have = r.prefix_tokens / bs;
    return (uint32_t)(total > have ? total - have : 0);
}

Request* find(tkv_coordinator* c, uint64_t id) {
    auto it = c->reqs.find(id);
    return it == c->reqs.end() ? nullptr : &it->second;
}

void unreserve(tkv_coordinator* c, Request& r) {
    if (r.reserved_blocks) {
        c->reserved[r.decode_worker] -= std::min<uint64_t>(c->reserved[r.decode_worker], r.reserved_blocks);
        r.reserved_blocks = 0;
    }
}

}  // namespace

extern "C" {

tkv_coordinator* tkv_coordinator_new(const TkvCoordinatorConfig* cfg) {
    if (!cfg || cfg->n_prefill == 0 || cfg->n_decode == 0 || cfg->block_size == 0) {
        fail(TKV_ERR_INVALID_CONFIG, "coordinator: needs at least one prefill and one decode worker and a block size");
        return nullptr;
    }
    auto* c = new (std::nothrow) tkv_coordinator();
    if (!c) return nullptr;
    c->cfg = *cfg;
    c->prefill_queues.resize(cfg->n_prefill);
    c->prefill_load.assign(cfg->n_prefill, 0);
    c->free_blocks.assign(cfg->n_decode, 0);
    c->reserved.assign(cfg->n_decode, 0);
    c->inflight.assign(cfg->n_decode, 0);
    return c;
}

void tkv_coordinator_delete(tkv_coordinator* c) { delete c; }

int32_t tkv_coordinator_set_headroom(tkv_coordinator* c, uint32_t decode_worker, uint64_t free_blocks) {
    if (!c || decode_worker >= c->cfg.n_decode) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: no decode worker %llu", decode_worker);
    c->free_blocks[decode_worker] = free_blocks;
    return TKV_OK;
}

// Routes to the prefill worker with the fewest prompt tokens queued or running (lowest index on a tie).
int32_t tkv_coordinator_submit(tkv_coordinator* c, uint64_t request_id, uint32_t n_tokens, uint32_t max_new_tokens, uint32_t priority,
                               uint32_t* prefill_worker) {
    if (!c) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (n_tokens == 0) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu has no tokens", request_id);
    if (c->reqs.count(request_id)) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu is already in the system", request_id);
    uint32_t w = 0;
    for (uint32_t i = 1; i < c->cfg.n_prefill; i++)
        if (c->prefill_load[i] < c->prefill_load[w]) w = i;
    Request r;
    r.id = request_id;
    r.n_tokens = n_tokens;
    r.max_new_tokens = max_new_tokens;
    r.priority = priority;
    r.prefill_worker = w;
    r.age = c->next_age++;
    c->reqs.emplace(request_id, r);
    c->prefill_queues[w].push_back(request_id);
    c->prefill_load[w] += n_tokens;
    c->stats.submitted++;
    if (prefill_worker) *prefill_worker = w;
    return TKV_OK;
}

// The next request a prefill worker should run: highest priority first, oldest within a priority.  1 = one was handed out.
int32_t tkv_coordinator_next_prefill(tkv_coordinator* c, uint32_t prefill_worker, uint64_t* request_id) {
    if (!c || !request_id || prefill_worker >= c->cfg.n_prefill) {
        fail(TKV_ERR_INVALID_CONFIG, "coordinator: no prefill worker %llu", prefill_worker);
        return -1;
    }
    auto& q = c->prefill_queues[prefill_worker];
    if (q.empty()) return 0;
    size_t best = 0;
    for (size_t i = 1; i < q.size(); i++)
        if (c->reqs[q[i]].priority > c->reqs[q[best]].priority) best = i;
    const uint64_t id = q[best];
    q.erase(q.begin() + (std::ptrdiff_t)best);
    c->reqs[id].state = TKV_REQ_PREFILL;
    *request_id = id;
    return 1;
}

int32_t tkv_coordinator_prefill_done(tkv_coordinator* c, uint64_t request_id, uint32_t prefix_tokens_resident) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r || r->state != TKV_REQ_PREFILL) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu is not prefilling", request_id);
    if (prefix_tokens_resident > r->n_tokens || prefix_tokens_resident % c->cfg.block_size)
        return fail(TKV_ERR_INVALID_CONFIG, "coordinator: resident prefix %llu is longer than the prompt or not block-aligned", prefix_tokens_resident);
    r->prefix_tokens = prefix_tokens_resident;
    r->state = TKV_REQ_WAITING;
    c->prefill_load[r->prefill_worker] -= std::min<uint64_t>(c->prefill_load[r->prefill_worker], r->n_tokens);
    c->waiting.push_back(request_id);
    return TKV_OK;
}

// Admits waiting requests, oldest first, each to the decode worker paired with its prefill worker if that one
// has the pages and a free handoff slot, else to the worker with the most unpromised pages.  A request that
// fits nowhere stays waiting and does not block younger, smaller ones.  Returns the number written to `out`.
size_t tkv_coordinator_admit(tkv_coordinator* c, TkvAdmission* out, size_t cap) {
    if (!c || !out) return 0;
    size_t n = 0;
    for (auto it = c->waiting.begin(); it != c->waiting.end() && n < cap;) {
        Request& r = c->reqs[*it];
        const uint32_t need = blocks_needed(c, r);
        auto room = [&](uint32_t d) -> uint64_t {                   // pages neither in use, promised, nor kept back as headroom
            const uint64_t free_now = c->free_blocks[d] > c->reserved[d] ? c->free_blocks[d] - c->reserved[d] : 0;
            return free_now > c->cfg.headroom_blocks ? free_now - c->cfg.headroom_blocks : 0;
        };
        auto fits = [&](uint32_t d) { return (!c->cfg.max_inflight_per_decode || c->inflight[d] < c->cfg.max_inflight_per_decode) && room(d) >= need; };
        uint32_t pick = r.prefill_worker % c->cfg.n_decode;
        if (!fits(pick)) {
            bool found = false;
            for (uint32_t d = 0; d < c->cfg.n_decode; d++)
                if (fits(d) && (!found || room(d) > room(pick))) {
                    pick = d;
                    found = true;
                }
            if (!found) {
                ++it;
                continue;
            }
        }
        r.decode_worker = pick;
        r.reserved_blocks = need;
        r.state = TKV_REQ_ADMITTED;
        c->reserved[pick] += need;
        c->inflight[pick]++;
        out[n++] = TkvAdmission{r.id, r.prefill_worker, pick, need, r.prefix_tokens};
        it = c->waiting.erase(it);
        c->stats.admitted++;
    }
    return n;
}

int32_t tkv_coordinator_handoff_started(tkv_coordinator* c, uint64_t request_id, uint64_t now) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r || r->state != TKV_REQ_ADMITTED) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu is not admitted", request_id);
    r->state = TKV_REQ_TRANSFER;
    r->transfer_started = now;
    r->attempts++;
    unreserve(c, *r);       // the pages are the allocator's business from here on: the next set_headroom already counts them
    return TKV_OK;
}

int32_t tkv_coordinator_handoff_complete(tkv_coordinator* c, uint64_t request_id) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r || r->state != TKV_REQ_TRANSFER) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu has no handoff in flight", request_id);
    r->state = TKV_REQ_DECODE;
    c->inflight[r->decode_worker]--;
    c->stats.handoffs_completed++;
    return TKV_OK;
}

// A handoff that did not complete (flag wait timed out, a status word reported an error): the request keeps its
// decode worker (and whatever pages it was given there) and is either admitted again for another attempt (*action =
// TKV_RETRY_HANDOFF) or, after max_retries attempts, prefilled by the decode worker itself (*action = TKV_REPREFILL).
int32_t tkv_coordinator_handoff_failed(tkv_coordinator* c, uint64_t request_id, uint32_t* action) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r || (r->state != TKV_REQ_TRANSFER && r->state != TKV_REQ_ADMITTED))
        return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu has no handoff to fail", request_id);
    c->stats.handoffs_failed++;
    if (r->attempts <= c->cfg.max_retries) {
        r->state = TKV_REQ_ADMITTED;
        c->stats.retries++;
        if (action) *action = TKV_RETRY_HANDOFF;
    } else {
        r->state = TKV_REQ_REPREFILL;
        c->inflight[r->decode_worker]--;
        c->stats.fallbacks++;
        if (action) *action = TKV_REPREFILL;
    }
    return TKV_OK;
}

// Handoffs in flight for longer than handoff_timeout: their ids, oldest first (the caller then reports each as failed).
size_t tkv_coordinator_timed_out(tkv_coordinator* c, uint64_t now, uint64_t* request_ids, size_t cap) {
    if (!c || !request_ids || !c->cfg.handoff_timeout) return 0;
    std::vector<const Request*> late;
    for (auto& kv : c->reqs)
        if (kv.second.state == TKV_REQ_TRANSFER && now - kv.second.transfer_started > c->cfg.handoff_timeout) late.push_back(&kv.second);
    std::sort(late.begin(), late.end(), [](const Request* a, const Request* b) {
        return a->transfer_started != b->transfer_started ? a->transfer_started < b->transfer_started : a->age < b->age;
    });
    size_t n = 0;
    for (const Request* r : late)
        if (n < cap) request_ids[n++] = r->id;
    return n;
}

int32_t tkv_coordinator_reprefill_done(tkv_coordinator* c, uint64_t request_id) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r || r->state != TKV_REQ_REPREFILL) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu is not re-prefilling", request_id);
    r->state = TKV_REQ_DECODE;
    return TKV_OK;
}

// The request leaves the system from any state (finished, cancelled): reservations and queue entries go with it.
int32_t tkv_coordinator_finish(tkv_coordinator* c, uint64_t request_id) {
    Request* r = c ? find(c, request_id) : nullptr;
    if (!r) return fail(TKV_ERR_INVALID_CONFIG, "coordinator: request %llu is not in the system", request_id);
    if (r->state == TKV_REQ_QUEUED || r->state == TKV_REQ_PREFILL) {
        c->prefill_load[r->prefill_worker] -= std::min<uint64_t>(c->prefill_load[r->prefill_worker], r->n_tokens);
        auto& q = c->prefill_queues[r->prefill_worker];
        q.erase(std::remove(q.begin(), q.end(), request_id), q.end());
    }
    if (r->state == TKV_REQ_WAITING) c->waiting.erase(std::remove(c->waiting.begin(), c->waiting.end(), request_id), c->waiting.end());
    if (r->state == TKV_REQ_ADMITTED || r->state == TKV_REQ_TRANSFER) c->inflight[r->decode_worker]--;
    unreserve(c, *r);
    c->reqs.erase(request_id);
    c->stats.finished++;
    return TKV_OK;
}

int32_t tkv_coordinator_request(const tkv_coordinator* c, uint64_t request_id, TkvRequestInfo* out) {
    if (!c || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    auto it = c->reqs.find(request_id);
    if (it == c->reqs.end()) return 0;
    const Request& r = it->second;
    *out = TkvRequestInfo{r.id, r.state, r.prefill_worker, r.decode_worker, r.reserved_blocks, r.prefix_tokens, r.attempts};
    return 1;
}

int32_t tkv_coordinator_stats(const tkv_coordinator* c, TkvCoordinatorStats* out) {
    if (!c || !out) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    *out = c->stats;
    out->in_system = c->reqs.size();
    out->waiting = c->waiting.size();
    uint64_t res = 0;
    for (uint64_t x : c->reserved) res += x;
    out->reserved_blocks = res;
    return TKV_OK;
}

}  // extern "C"
