// The reference's disaggregated-pipeline tests (engine/src/disaggregated.rs:292-400) restated over
// the C++ worker mirror in include/tkv_workers.hpp, with GPU workers whose KV lives in paged
// pools and moves through the handoff kernels.  The transformer forward is outside this
// library's scope, so a toy model stands in: K/V rows are an integer hash of (token, position,
// layer, head, dim) and the logits are an exact integer reduction over EVERY cached K/V element
// read through the session's block table, so a single wrong byte after a handoff changes the
// generated tokens.  Built and run by tests/test_gpu_workers_cpp.py.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "tkv_workers.hpp"

using namespace tkv_host;

#define CUDA_OK(call)                                                                         \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) {                                                              \
            fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
            exit(2);                                                                          \
        }                                                                                     \
    } while (0)
#define REQUIRE(cond)                                                        \
    do {                                                                     \
        if (!(cond)) {                                                       \
            fprintf(stderr, "%s:%d REQUIRE failed: %s\n", __FILE__, __LINE__, #cond); \
            exit(1);                                                         \
        }                                                                    \
    } while (0)

// ModelConfig::tiny_test-like geometry (engine/src/config.rs:262-301) with the GPU pool's 16-token blocks
struct Config {
    uint32_t num_layers = 2, num_kv_heads = 4, head_dim = 16, vocab_size = 64, block_size = 16, total_pages = 64;
    uint32_t kv_dim() const { return num_kv_heads * head_dim; }
};

__host__ __device__ inline uint64_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// "k_proj / v_proj": one row per new token
__global__ void toy_write_kv(__half* layer_base, const uint32_t* table, const uint32_t* tokens, uint32_t n_new, uint32_t start_pos,
                             uint32_t block_size, uint32_t kv_dim, uint32_t layer, uint32_t is_v, uint64_t weights) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_new * kv_dim) return;
    uint32_t t = i / kv_dim, e = i % kv_dim, pos = start_pos + t;
    uint64_t h = mix(weights ^ mix(((uint64_t)tokens[t] << 32) | pos) ^ mix(((uint64_t)layer << 40) | ((uint64_t)is_v << 32) | e));
    float x = (float)((int)(h % 2048u) - 1024) / 512.0f;
    size_t row = (size_t)table[pos / block_size] * block_size + pos % block_size;
    layer_base[row * kv_dim + e] = __float2half_rn(x);
}

// "attention + lm_head": exact integer reduction over every cached element of one layer tensor
__global__ void toy_logits(const __half* layer_base, const uint32_t* table, uint32_t kv_len, uint32_t block_size, uint32_t kv_dim,
                           uint32_t salt, uint32_t vocab, unsigned long long* acc) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= kv_len * kv_dim) return;
    uint32_t pos = i / kv_dim, e = i % kv_dim;
    size_t row = (size_t)table[pos / block_size] * block_size + pos % block_size;
    unsigned long long bits = __half_as_ushort(layer_base[row * kv_dim + e]);
    for (uint32_t v = 0; v < vocab; v++)
        atomicAdd(acc + v, bits * (unsigned long long)((e * 131u + v * 17u + pos * 7u + salt) % 251u + 1u));
}

struct DevicePool {
    Pool pool;
    std::vector<void*> allocs;
    uint32_t* refcounts = nullptr;
    DevicePool(const Config& c, int device) {
        CUDA_OK(cudaSetDevice(device));
        size_t bytes = (size_t)c.total_pages * c.block_size * c.kv_dim() * sizeof(__half);
        for (uint32_t l = 0; l < 2 * c.num_layers; l++) {
            void* p = nullptr;
            CUDA_OK(cudaMalloc(&p, bytes));
            CUDA_OK(cudaMemset(p, 0xA5, bytes));
            allocs.push_back(p);
            (l % 2 ? pool.v_ptrs : pool.k_ptrs).push_back((uint64_t)p);
        }
        CUDA_OK(cudaMalloc((void**)&refcounts, c.total_pages * 4));
        CUDA_OK(cudaMemset(refcounts, 0, c.total_pages * 4));
        pool.c.device = device;
        pool.c.dtype = TKV_DTYPE_F16;
        pool.c.n_layers = c.num_layers;
        pool.c.n_kv_heads = c.num_kv_heads;
        pool.c.head_dim = c.head_dim;
        pool.c.block_size = c.block_size;
        pool.c.total_blocks = c.total_pages;
        pool.c.refcounts = (uint64_t)refcounts;
    }
    ~DevicePool() {
        cudaSetDevice(pool.c.device);
        for (void* p : allocs) cudaFree(p);
        cudaFree(refcounts);
    }
};

// InferenceSession (engine/src/session.rs): paged cache + position + seed
struct Session {
    DevicePool* pool;
    PageAllocator* pages;
    std::vector<uint32_t> table;
    size_t position = 0;
    uint64_t seed = 0;
};

struct ToyModel {
    Config cfg;
    uint64_t weights;
    // TransformerModel::forward: appends the tokens' K/V, returns the logits of the last position
    std::vector<float> forward(Session& s, const std::vector<uint32_t>& tokens) const {
        CUDA_OK(cudaSetDevice(s.pool->pool.c.device));
        const uint32_t bs = cfg.block_size, n = (uint32_t)tokens.size();
        while (s.table.size() * bs < s.position + n) s.table.push_back(s.pages->allocate());
        uint32_t *d_table = nullptr, *d_tokens = nullptr;
        unsigned long long* d_acc = nullptr;
        CUDA_OK(cudaMalloc((void**)&d_table, s.table.size() * 4));
        CUDA_OK(cudaMalloc((void**)&d_tokens, n * 4));
        CUDA_OK(cudaMalloc((void**)&d_acc, cfg.vocab_size * 8));
        CUDA_OK(cudaMemcpy(d_table, s.table.data(), s.table.size() * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(d_tokens, tokens.data(), n * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemset(d_acc, 0, cfg.vocab_size * 8));
        const uint32_t kv_len = (uint32_t)s.position + n;
        for (uint32_t l = 0; l < cfg.num_layers; l++)
            for (uint32_t is_v = 0; is_v < 2; is_v++) {
                __half* base = (__half*)(is_v ? s.pool->pool.v_ptrs[l] : s.pool->pool.k_ptrs[l]);
                toy_write_kv<<<(n * cfg.kv_dim() + 127) / 128, 128>>>(base, d_table, d_tokens, n, (uint32_t)s.position, bs, cfg.kv_dim(), l,
                                                                      is_v, weights);
                toy_logits<<<(kv_len * cfg.kv_dim() + 127) / 128, 128>>>(base, d_table, kv_len, bs, cfg.kv_dim(), l * 2 + is_v,
                                                                         cfg.vocab_size, d_acc);
            }
        CUDA_OK(cudaGetLastError());
        std::vector<unsigned long long> acc(cfg.vocab_size);
        CUDA_OK(cudaMemcpy(acc.data(), d_acc, cfg.vocab_size * 8, cudaMemcpyDeviceToHost));
        cudaFree(d_table);
        cudaFree(d_tokens);
        cudaFree(d_acc);
        s.position += n;
        std::vector<float> logits(cfg.vocab_size);
        for (uint32_t v = 0; v < cfg.vocab_size; v++) logits[v] = (float)(mix(acc[v]) % 1000003ull);
        return logits;
    }
    static uint32_t argmax(const std::vector<float>& x) {   // temperature 0: CpuSampler's greedy pick
        uint32_t best = 0;
        for (uint32_t i = 1; i < x.size(); i++)
            if (x[i] > x[best]) best = i;
        return best;
    }
    // TransformerModel::generate: the single-worker loop the disaggregated one must match
    std::vector<uint32_t> generate(Session& s, const std::vector<uint32_t>& prompt, size_t max_new, std::optional<uint32_t> eos) const {
        std::vector<float> logits = forward(s, prompt);
        std::vector<uint32_t> out{argmax(logits)};
        while (out.size() < max_new) {
            if (eos && *eos == out.back()) break;
            logits = forward(s, {out.back()});
            out.push_back(argmax(logits));
        }
        return out;
    }
};

// LocalPrefillWorker (engine/src/disaggregated.rs:21-48) on a GPU pool
struct GpuPrefillWorker : PrefillWorker {
    const ToyModel* model;
    DevicePool* pool;
    PageAllocator* pages;
    GpuPrefillWorker(const ToyModel* m, DevicePool* p, PageAllocator* a) : model(m), pool(p), pages(a) {}
    SessionTransfer prefill(const std::vector<uint32_t>& token_ids, uint64_t seed) override {
        Session s{pool, pages, {}, 0, seed};
        std::vector<float> logits = model->forward(s, token_ids);
        SessionTransfer t;                                   // InferenceSession::to_transfer_with_logits
        t.cache.pool = &pool->pool;
        t.cache.block_table = s.table;
        t.cache.seq_len = s.position;
        t.cache.num_layers = model->cfg.num_layers;
        t.cache.num_kv_heads = model->cfg.num_kv_heads;
        t.cache.head_dim = model->cfg.head_dim;
        t.position = s.position;
        t.seed = seed;
        t.last_logits = std::move(logits);
        return t;
    }
};

// LocalDecodeWorker (engine/src/disaggregated.rs:50-128) on a GPU pool
struct GpuDecodeWorker : DecodeWorker {
    const ToyModel* model;
    DevicePool* pool;
    PageAllocator* pages;
    PageAllocator* source_pages;   // the prefill side's allocator: its pages are returned once adopted
    KvReceiver receiver;
    cudaStream_t source_stream;
    GpuDecodeWorker(const ToyModel* m, DevicePool* p, PageAllocator* a, PageAllocator* src_pages, uint64_t flag, cudaStream_t st)
        : model(m), pool(p), pages(a), source_pages(src_pages), receiver(&p->pool, a, flag), source_stream(st) {}
    std::vector<uint32_t> decode(SessionTransfer transfer, size_t max_new_tokens, const SamplingParams& params,
                                 std::optional<uint32_t> eos_token) override {
        REQUIRE(params.temperature == 0.0f);
        std::vector<float> last_logits = transfer.last_logits;
        // InferenceSession::from_transfer: the KV arrives by one handoff
        Session s{pool, pages, receiver.adopt(transfer, source_stream), transfer.position, transfer.seed};
        for (uint32_t page : transfer.cache.block_table) source_pages->free(page);
        std::vector<uint32_t> generated{ToyModel::argmax(last_logits)};
        while (generated.size() < max_new_tokens) {
            if (eos_token && *eos_token == generated.back()) break;
            std::vector<float> step_logits = model->forward(s, {generated.back()});
            generated.push_back(ToyModel::argmax(step_logits));
        }
        for (uint32_t page : s.table) pages->free(page);
        return generated;
    }
};

static std::vector<uint16_t> read_rows(DevicePool& p, const std::vector<uint32_t>& table, size_t seq_len, uint32_t layer, bool is_v,
                                       const Config& c) {
    CUDA_OK(cudaSetDevice(p.pool.c.device));
    std::vector<uint16_t> out(seq_len * c.kv_dim());
    const uint16_t* base = (const uint16_t*)(is_v ? p.pool.v_ptrs[layer] : p.pool.k_ptrs[layer]);
    for (size_t pos = 0; pos < seq_len; pos++) {
        size_t row = (size_t)table[pos / c.block_size] * c.block_size + pos % c.block_size;
        CUDA_OK(cudaMemcpy(out.data() + pos * c.kv_dim(), base + row * c.kv_dim(), c.kv_dim() * 2, cudaMemcpyDeviceToHost));
    }
    return out;
}

struct Rig {
    Config cfg;
    ToyModel model;
    int dev_a, dev_b;
    DevicePool a, b;
    PageAllocator pages_a, pages_b;
    uint32_t* flag = nullptr;
    cudaStream_t stream_a = nullptr;
    Rig(int da, int db) : model{cfg, 42}, dev_a(da), dev_b(db), a(cfg, da), b(cfg, db), pages_a(cfg.total_pages), pages_b(cfg.total_pages) {
        CUDA_OK(cudaSetDevice(db));
        CUDA_OK(cudaMalloc((void**)&flag, 4));
        CUDA_OK(cudaMemset(flag, 0, 4));
        CUDA_OK(cudaSetDevice(da));
        CUDA_OK(cudaStreamCreateWithFlags(&stream_a, cudaStreamNonBlocking));
    }
    ~Rig() {
        cudaSetDevice(dev_a);
        cudaStreamDestroy(stream_a);
        cudaSetDevice(dev_b);
        cudaFree(flag);
    }
    DisaggregatedPipeline pipeline() {
        return DisaggregatedPipeline(std::make_unique<GpuPrefillWorker>(&model, &a, &pages_a),
                                     std::make_unique<GpuDecodeWorker>(&model, &b, &pages_b, &pages_a, (uint64_t)flag, stream_a));
    }
};

static std::vector<uint32_t> prompt_of(size_t n, uint32_t salt) {
    std::vector<uint32_t> p(n);
    for (size_t i = 0; i < n; i++) p[i] = (uint32_t)(mix(salt * 1000003ull + i) % 64);
    return p;
}

// engine/src/disaggregated.rs:292-321
static void test_session_transfer_round_trip(int da, int db) {
    Rig r(da, db);
    for (size_t n : {size_t(3), size_t(16), size_t(45)}) {
        GpuPrefillWorker prefill(&r.model, &r.a, &r.pages_a);
        SessionTransfer transfer = prefill.prefill(prompt_of(n, 1), 42);
        REQUIRE(transfer.position == n && transfer.seed == 42 && transfer.cache.seq_len == n);
        REQUIRE(transfer.last_logits.size() == r.cfg.vocab_size);
        // the metadata crosses as one wire message, as it would between two processes
        SessionTransfer received = from_wire(to_wire(transfer), &r.a.pool);
        REQUIRE(received.position == n && received.seed == 42 && received.cache.seq_len == n);
        REQUIRE(received.last_logits == transfer.last_logits && received.cache.block_table == transfer.cache.block_table);
        KvReceiver receiver(&r.b.pool, &r.pages_b, (uint64_t)r.flag);
        std::vector<uint32_t> restored = receiver.adopt(received, r.stream_a);
        REQUIRE(restored.size() == (n + 15) / 16);
        for (uint32_t layer = 0; layer < r.cfg.num_layers; layer++)
            for (bool is_v : {false, true})
                REQUIRE(read_rows(r.a, transfer.cache.block_table, n, layer, is_v, r.cfg) ==
                        read_rows(r.b, restored, n, layer, is_v, r.cfg));
        for (uint32_t p : transfer.cache.block_table) r.pages_a.free(p);
        for (uint32_t p : restored) r.pages_b.free(p);
    }
    REQUIRE(r.pages_a.in_use() == 0 && r.pages_b.in_use() == 0);
}

// engine/src/disaggregated.rs:323-341
static void test_disaggregated_produces_tokens(int da, int db) {
    Rig r(da, db);
    std::vector<uint32_t> tokens = r.pipeline().generate({1, 2, 3}, 5, SamplingParams{}, std::nullopt, 42);
    REQUIRE(tokens.size() == 5);
    REQUIRE(r.pages_a.in_use() == 0 && r.pages_b.in_use() == 0);
}

// engine/src/disaggregated.rs:343-364
static void test_disaggregated_deterministic(int da, int db) {
    Rig r1(da, db), r2(da, db);
    REQUIRE(r1.pipeline().generate({1, 2, 3}, 5, SamplingParams{}, std::nullopt, 42) ==
            r2.pipeline().generate({1, 2, 3}, 5, SamplingParams{}, std::nullopt, 42));
}

// engine/src/disaggregated.rs:366-400
static void test_disaggregated_matches_single_worker(int da, int db) {
    for (size_t n : {size_t(3), size_t(31), size_t(64), size_t(77)}) {
        Rig r(da, db);
        Session single{&r.a, &r.pages_a, {}, 0, 42};
        std::vector<uint32_t> single_tokens = r.model.generate(single, prompt_of(n, 2), 12, std::nullopt);
        for (uint32_t p : single.table) r.pages_a.free(p);
        std::vector<uint32_t> disagg_tokens = r.pipeline().generate(prompt_of(n, 2), 12, SamplingParams{}, std::nullopt, 42);
        REQUIRE(single_tokens == disagg_tokens);
        // an end-of-sequence token stops both the same way
        std::optional<uint32_t> eos = single_tokens[3];
        Session again{&r.a, &r.pages_a, {}, 0, 42};
        std::vector<uint32_t> stopped = r.model.generate(again, prompt_of(n, 2), 12, eos);
        for (uint32_t p : again.table) r.pages_a.free(p);
        REQUIRE(stopped == r.pipeline().generate(prompt_of(n, 2), 12, SamplingParams{}, eos, 42));
        REQUIRE(stopped.size() <= 12 && stopped.back() == *eos);
    }
}

// Prefix sharing on the decode side (RadixTree::lookup, engine/src/prefix_cache.rs:58-85): the second
// prompt adopts the first one's prefix pages and moves only its suffix.
static void test_shared_prefix_pages_are_adopted_not_moved(int da, int db) {
    Rig r(da, db);
    RadixTree tree;
    std::vector<uint32_t> first = prompt_of(40, 3), second = first;
    for (size_t i = 32; i < second.size(); i++) second[i] = (second[i] + 7) % 64;   // same first 2 blocks
    second.resize(52, 9);
    GpuPrefillWorker prefill(&r.model, &r.a, &r.pages_a);
    KvReceiver receiver(&r.b.pool, &r.pages_b, (uint64_t)r.flag);
    SessionTransfer t1 = prefill.prefill(first, 1);
    std::vector<uint32_t> table1 = receiver.adopt(t1, r.stream_a);
    std::vector<size_t> pages1;                      // page_ids[i] belongs to token i (prefix_cache.rs:41-45)
    for (size_t i = 0; i < 32; i++) pages1.push_back(table1[i / 16]);
    tree.insert(std::vector<uint32_t>(first.begin(), first.begin() + 32), pages1);
    auto [matched, page_ids] = tree.lookup(second);
    REQUIRE(matched == 32 && page_ids.size() == 32);
    std::vector<uint32_t> shared{(uint32_t)page_ids[0], (uint32_t)page_ids[16]};
    REQUIRE(shared[0] == table1[0] && shared[1] == table1[1]);
    size_t in_use_before = r.pages_b.in_use();
    SessionTransfer t2 = prefill.prefill(second, 2);
    std::vector<uint32_t> table2 = receiver.adopt(t2, r.stream_a, shared);
    REQUIRE(table2.size() == 4 && table2[0] == table1[0] && table2[1] == table1[1]);
    REQUIRE(r.pages_b.in_use() == in_use_before + 2);            // only the suffix took pages
    uint32_t rc[64];
    CUDA_OK(cudaSetDevice(db));
    CUDA_OK(cudaMemcpy(rc, r.b.refcounts, sizeof rc, cudaMemcpyDeviceToHost));
    REQUIRE(rc[table1[0]] == 1 && rc[table1[1]] == 1 && rc[table2[2]] == 0);
    // decode continues from the adopted cache exactly as a single worker would from its own
    Session single{&r.a, &r.pages_a, {}, 0, 2};
    std::vector<uint32_t> want = r.model.generate(single, second, 6, std::nullopt);
    Session adopted{&r.b, &r.pages_b, table2, t2.position, 2};
    std::vector<uint32_t> got{ToyModel::argmax(t2.last_logits)};
    while (got.size() < 6) got.push_back(ToyModel::argmax(r.model.forward(adopted, {got.back()})));
    REQUIRE(want == got);
}

// KernelError surfaces as an exception with the C status code; pool exhaustion is recoverable
static void test_errors(int da, int db) {
    Rig r(da, db);
    GpuPrefillWorker prefill(&r.model, &r.a, &r.pages_a);
    SessionTransfer t = prefill.prefill(prompt_of(20, 4), 0);
    KvReceiver receiver(&r.b.pool, &r.pages_b, (uint64_t)r.flag);
    SessionTransfer bad = t;
    bad.cache.block_table.resize(1);
    try {
        receiver.adopt(bad, r.stream_a);
        REQUIRE(!"short block table accepted");
    } catch (const KernelError& e) {
        REQUIRE(e.code == TKV_ERR_DIMENSION_MISMATCH);
    }
    std::vector<uint32_t> hog;
    while (r.pages_b.available() > 1) hog.push_back(r.pages_b.allocate());
    try {
        receiver.adopt(t, r.stream_a);                 // needs 2 pages, 1 left
        REQUIRE(!"exhausted pool accepted");
    } catch (const KernelError& e) {
        REQUIRE(e.code == TKV_ERR_POOL_EXHAUSTED);
    }
    REQUIRE(r.pages_b.available() == 1);               // the page taken before the failure went back
    for (uint32_t p : hog) r.pages_b.free(p);
    REQUIRE(receiver.adopt(t, r.stream_a).size() == 2);
}

// The decode side's admission with the prefix index and the page allocator in device memory: the second prompt
// shares its first two blocks with the first one, so it adopts those pages (reference count 1) and moves the rest.
static void test_device_admission(int da) {
    Rig r(da, da);
    const Config& c = r.cfg;
    const uint32_t bs = c.block_size, stride = 8;
    DevicePrefixIndex index(da, 1024, bs);
    DevicePageAllocator pages(da, c.total_pages);
    // a plan sized for up to `stride` block pairs per admission (only its size matters)
    std::vector<uint32_t> ident(stride);
    for (uint32_t i = 0; i < stride; i++) ident[i] = i;
    uint32_t cap_len = stride * bs;
    TkvBatch cap{};
    cap.n_seqs = 1;
    cap.table_stride = stride;
    cap.seq_lens = &cap_len;
    cap.src_tables = ident.data();
    cap.dst_tables = ident.data();
    tkv_plan* plan = nullptr;
    check(tkv_plan_create(r.a.pool.get(), r.b.pool.get(), &cap, nullptr, TKV_PLAN_DEFAULT, &plan));
    DeviceKvReceiver receiver(plan, &index, &pages, (uint64_t)r.flag, bs);

    std::vector<uint32_t> first = prompt_of(40, 3), second(first.begin(), first.begin() + 32);
    for (uint32_t t : prompt_of(18, 9)) second.push_back(t);
    GpuPrefillWorker prefill(&r.model, &r.a, &r.pages_a);
    uint32_t *d_tokens, *d_len, *d_src, *d_dst, *d_matched, *d_status;
    CUDA_OK(cudaMalloc((void**)&d_tokens, 64 * 4));
    CUDA_OK(cudaMalloc((void**)&d_len, 4));
    CUDA_OK(cudaMalloc((void**)&d_src, stride * 4));
    CUDA_OK(cudaMalloc((void**)&d_dst, stride * 4));
    CUDA_OK(cudaMalloc((void**)&d_matched, 4));
    CUDA_OK(cudaMalloc((void**)&d_status, 8));
    std::vector<uint32_t> first_table;
    for (int round = 0; round < 2; round++) {
        const std::vector<uint32_t>& prompt = round ? second : first;
        SessionTransfer t = prefill.prefill(prompt, 7);
        const uint32_t len = (uint32_t)prompt.size(), nb = (len + bs - 1) / bs;
        std::vector<uint32_t> src(stride, 0);
        for (uint32_t i = 0; i < nb; i++) src[i] = t.cache.block_table[i];
        CUDA_OK(cudaMemcpy(d_tokens, prompt.data(), len * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(d_len, &len, 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(d_src, src.data(), stride * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemset(d_dst, 0xFF, stride * 4));
        CUDA_OK(cudaMemset(d_status, 0xFF, 8));
        DeviceAdmissionBuffers b;
        b.tokens = (uint64_t)d_tokens;
        b.seq_lens = (uint64_t)d_len;
        b.src_tables = (uint64_t)d_src;
        b.dst_tables = (uint64_t)d_dst;
        b.matched = (uint64_t)d_matched;
        b.status = (uint64_t)d_status;
        b.n_seqs = 1;
        b.token_stride = 64;
        b.table_stride = stride;
        const uint32_t gen = receiver.adopt(b, r.stream_a);
        check(tkv_flag_wait_host(da, (uint64_t)r.flag, gen, 10'000'000));
        uint32_t status[2], matched = 99;
        std::vector<uint32_t> table(stride);
        CUDA_OK(cudaMemcpy(status, d_status, 8, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(&matched, d_matched, 4, cudaMemcpyDeviceToHost));
        CUDA_OK(cudaMemcpy(table.data(), d_dst, stride * 4, cudaMemcpyDeviceToHost));
        REQUIRE(status[0] == 0 && status[1] == 0);
        REQUIRE(matched == (round ? 2u : 0u));
        table.resize(nb);
        if (round) {
            REQUIRE(table[0] == first_table[0] && table[1] == first_table[1]);      // adopted, not moved
            REQUIRE(table[2] != first_table[2]);
            uint32_t rc[2];
            CUDA_OK(cudaMemcpy(rc, r.b.refcounts + table[0], 4, cudaMemcpyDeviceToHost));
            CUDA_OK(cudaMemcpy(rc + 1, r.b.refcounts + table[1], 4, cudaMemcpyDeviceToHost));
            REQUIRE(rc[0] == 1 && rc[1] == 1);
        } else {
            first_table = table;
        }
        for (uint32_t l = 0; l < c.num_layers; l++)
            for (bool is_v : {false, true})
                REQUIRE(read_rows(r.a, t.cache.block_table, len, l, is_v, c) == read_rows(r.b, table, len, l, is_v, c));
        // index the whole blocks of this prompt under the pages it now has on the decode side
        TkvPrefixBatch pb{};
        pb.n_seqs = 1;
        pb.stride = 64;
        pb.page_stride = stride;
        pb.tokens = (uint64_t)d_tokens;
        pb.lens = (uint64_t)d_len;
        pb.pages = (uint64_t)d_dst;
        index.insert(pb, r.stream_a);
        index.release(pb, r.stream_a);          // the lookup's references, given back once the prompt is indexed
        for (uint32_t page : t.cache.block_table) r.pages_a.free(page);
    }
    REQUIRE(pages.available(r.stream_a) == c.total_pages - 3 - 2);   // 3 blocks for the first prompt, 2 new ones for the second
    TkvPrefixIndexStats st = index.stats(r.stream_a);
    REQUIRE(st.live_nodes == 2 + 1 && st.hits == 1 && st.tokens_saved == 32);
    tkv_plan_destroy(plan);
    for (void* p : {(void*)d_tokens, (void*)d_len, (void*)d_src, (void*)d_dst, (void*)d_matched, (void*)d_status})
        cudaFree(p);
}

int main() {
    int n_dev = 0;
    CUDA_OK(cudaGetDeviceCount(&n_dev));
    REQUIRE(n_dev >= 1);
    int da = 0, db = n_dev >= 2 ? 1 : 0;
    if (db != da) {
        int32_t devs[2] = {da, db};
        check(tkv_init(devs, 2));
    }
    test_session_transfer_round_trip(da, db);
    test_disaggregated_produces_tokens(da, db);
    test_disaggregated_deterministic(da, db);
    test_disaggregated_matches_single_worker(da, db);
    test_shared_prefix_pages_are_adopted_not_moved(da, db);
    test_errors(da, db);
    test_device_admission(da);
    printf("ALL PASSED (prefill device %d, decode device %d)\n", da, db);
    return 0;
}
