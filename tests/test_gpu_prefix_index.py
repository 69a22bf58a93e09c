"""Device-resident prefix index against the RadixTree oracle: the reference's own test cases replayed on the
GPU, seeded batches with shared prefixes through insert / lookup / release / evict, tombstone reuse, and the
shared-prefix benchmark shape (64 prompts x 8 192 tokens, one node per 16-token block)."""
import numpy as np
import pytest

from oracle.prefix_oracle import RadixOracle
from tempura_b200 import _native as N

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    handoff.init([0])
    return handoff


def dev(seqs, pages=None):
    """Ragged python lists -> padded int32 device tensors (tokens, lens[, pages, page_lens])."""
    import torch
    stride = max(max((len(s) for s in seqs), default=1), 1)
    tok = np.zeros((len(seqs), stride), dtype=np.int32)
    for i, s in enumerate(seqs):
        tok[i, :len(s)] = s
    out = [torch.from_numpy(tok).cuda(), torch.tensor([len(s) for s in seqs], dtype=torch.int32).cuda()]
    if pages is not None:
        pstride = max(max((len(p) for p in pages), default=1), 1)
        pg = np.zeros((len(pages), pstride), dtype=np.int32)
        for i, p in enumerate(pages):
            pg[i, :len(p)] = p
        out += [torch.from_numpy(pg).cuda(), torch.tensor([len(p) for p in pages], dtype=torch.int32).cuda()]
    return out


def lookup(ix, seqs):
    matched, pages = ix.lookup(*dev(seqs))
    matched, pages = matched.cpu().numpy(), pages.cpu().numpy()
    return [(int(matched[i]), [None if p < 0 else int(p) for p in pages[i, :matched[i]]]) for i in range(len(seqs))]


def test_reference_cases_on_the_device(H):
    # prefix_cache.rs:153-241, one sequence per call as the reference makes them
    ix = H.PrefixIndex(0, 1024)
    ix.insert(*dev([[1, 2, 3]], [[10, 20, 30]]))
    assert lookup(ix, [[1, 2, 3]]) == [(3, [10, 20, 30])]
    st = ix.stats()
    assert st.hits == 1 and st.tokens_saved == 3 and st.live_nodes == 3
    ix = H.PrefixIndex(0, 1024)
    ix.insert(*dev([[1, 2, 3, 4]], [[10, 20, 30, 40]]))
    assert lookup(ix, [[1, 2, 5]])[0][0] == 2                      # partial match
    assert lookup(ix, [[5, 6, 7]]) == [(0, [])]                    # no match
    ix = H.PrefixIndex(0, 1024)
    ix.insert(*dev([[1, 2, 3]], [[10, 20, 30]]))
    ix.insert(*dev([[1, 2, 4]], [[10, 20, 40]]))
    assert [m for m, _ in lookup(ix, [[1, 2, 3]]) + lookup(ix, [[1, 2, 4]]) + lookup(ix, [[1, 2]])] == [3, 3, 2]
    ix = H.PrefixIndex(0, 1024)                                    # multi-turn reuse
    system = [100, 101, 102, 103]
    ix.insert(*dev([system], [[0, 1, 2, 3]]))
    turn1 = system + [200, 201]
    assert lookup(ix, [turn1])[0][0] == 4
    ix.insert(*dev([turn1], [[0, 1, 2, 3, 4, 5]]))
    assert lookup(ix, [turn1 + [300]]) == [(6, [0, 1, 2, 3, 4, 5])]
    ix = H.PrefixIndex(0, 1024)                                    # evict_lru: [3, 4] was looked up, so [1, 2]'s leaf is older
    ix.insert(*dev([[1, 2]], [[10, 20]]))
    ix.insert(*dev([[3, 4]], [[30, 40]]))
    lookup(ix, [[3, 4]])
    ix.release(*dev([[3, 4]])[:2])
    assert ix.evict_lru(1) == ([20], 1)
    assert ix.evict_lru(8) == ([10, 40, 30], 3) and ix.evict_lru(1) == ([], 0)
    assert ix.stats().live_nodes == 0 and ix.stats().tombstones == 4


def make_sequences(rng, n, group, stems, vocab=40):
    seqs = []
    for _ in range(n):
        stem = stems[int(rng.integers(len(stems)))]
        keep = int(rng.integers(0, len(stem) + 1))
        tail = rng.integers(0, vocab, size=int(rng.integers(0, 5 * group + 3))).tolist()
        seqs.append(stem[:keep] + tail)
    return seqs


@pytest.mark.parametrize("group", [1, 16])
def test_seeded_batches_match_the_oracle(H, group):
    rng = np.random.default_rng(70 + group)
    stems = [rng.integers(0, 40, size=int(rng.integers(2 * group, 12 * group))).tolist() for _ in range(5)]
    ix, ref = H.PrefixIndex(0, 1 << 14, group), RadixOracle(group)
    next_page = 0
    for rnd in range(12):
        seqs = make_sequences(rng, int(rng.integers(1, 40)), group, stems)
        pages = []
        for s in seqs:                                             # sometimes fewer pages than nodes, as the reference allows
            n_nodes = len(s) // group
            n_pages = n_nodes if rng.random() < 0.7 else int(rng.integers(0, n_nodes + 1))
            pages.append(list(range(next_page, next_page + n_pages)))
            next_page += n_pages
        ix.insert(*dev(seqs, pages))
        ref.batch_insert(seqs, pages)
        probes = make_sequences(rng, int(rng.integers(1, 40)), group, stems)
        got, want = lookup(ix, probes), ref.batch_lookup(probes)
        assert [g[0] for g in got] == [w[0] for w in want], f"round {rnd}: matched lengths"
        assert [g[1] for g in got] == [w[2] for w in want], f"round {rnd}: pages per matched node"
        keep = [p for p in probes if rng.random() < 0.3]           # some lookups stay referenced
        rel = [p for p in probes if p not in keep]
        if rel:
            ix.release(*dev(rel)[:2])
            ref.batch_release(rel)
        k = int(rng.integers(0, 6))
        got_pages, got_nodes = ix.evict_lru(k)
        want_pages, want_nodes = [], 0
        for _ in range(k):
            hit, pg = ref.evict_lru_node()
            want_nodes += int(hit)
            want_pages += pg
        assert (got_pages, got_nodes) == (want_pages, want_nodes), f"round {rnd}: eviction order"
        st = ix.stats()
        assert (st.hits, st.tokens_saved, st.live_nodes) == (ref.hits, ref.tokens_saved, ref.live_nodes()), f"round {rnd}"
        assert st.table_full == 0


def test_tombstones_are_reused(H):
    ix = H.PrefixIndex(0, 256)
    for rnd in range(20):                                          # 20 x 100 nodes through a 256-slot table
        seq = [[1000 * rnd + i for i in range(100)]]
        ix.insert(*dev(seq, [list(range(100))]))
        assert lookup(ix, seq)[0][0] == 100
        ix.release(*dev(seq)[:2])
        pages, nodes = ix.evict_lru(100)
        assert nodes == 100 and pages == list(range(99, -1, -1))   # leaf first, then its parent, ...
    st = ix.stats()
    assert st.live_nodes == 0 and st.table_full == 0 and st.tombstones <= 256


def test_full_table_is_reported_not_overrun(H):
    ix = H.PrefixIndex(0, 64)
    ix.insert(*dev([list(range(200))]))
    st = ix.stats()
    assert st.table_full == 1 and st.live_nodes == 64


def test_shared_prefix_benchmark_shape(H):
    """64 prompts x 8 192 tokens sharing their first 2 048 (the prefix-reuse benchmark configuration), one node
    per 16-token block: the shared nodes keep the first prompt's pages, every prompt matches all of its 512 nodes,
    and a new prompt with the same system prompt matches exactly the shared 128."""
    import torch
    rng = np.random.default_rng(77)
    shared = rng.integers(0, 32000, size=2048)
    tok = np.stack([np.concatenate([shared, rng.integers(0, 32000, size=8192 - 2048)]) for _ in range(64)]).astype(np.int32)
    pages = (np.arange(64 * 512, dtype=np.int32)).reshape(64, 512)
    t, l, p = torch.from_numpy(tok).cuda(), torch.full((64,), 8192, dtype=torch.int32).cuda(), torch.from_numpy(pages).cuda()
    ix = H.PrefixIndex(0, 1 << 17, 16)
    ix.insert(t, l, p)
    matched, got = ix.lookup(t, l)
    assert bool((matched == 512).all())
    want = pages.copy()
    want[:, :128] = pages[0, :128]                                 # the shared nodes were created by prompt 0
    assert np.array_equal(got.cpu().numpy(), want)
    st = ix.stats()
    assert st.live_nodes == 128 + 64 * 384 and st.hits == 64 and st.tokens_saved == 64 * 8192
    fresh = np.concatenate([shared, rng.integers(0, 32000, size=1000)]).astype(np.int32)[None, :]
    m, g = ix.lookup(torch.from_numpy(fresh).cuda(), torch.tensor([fresh.shape[1]], dtype=torch.int32).cuda())
    assert int(m[0]) == 128 and np.array_equal(g.cpu().numpy()[0, :128], pages[0, :128])


def test_lookup_feeds_the_handoff_plan(H):
    """The index's answer is the handoff batch's prefix: matched nodes x 16 = prefix_lens, the pages are the
    destination block ids of the resident prefix.  The plan then moves only the suffixes and raises the
    reference counts of the shared blocks, as with a host-side RadixTree."""
    import torch
    from tempura_b200 import workloads as W
    w = W.llama8b_prefix(pool_blocks=2048, n_seqs=6, prefix=64, lo=20, hi=90, seed=91)
    rng = np.random.default_rng(5)
    system = rng.integers(0, 32000, size=64).tolist()
    prompts = [system + rng.integers(0, 32000, size=int(n) - 64).tolist() for n in w.seq_lens]
    # the decode side already holds the system prompt in w.shared_prefix_blocks (4 blocks) and has indexed it
    ix = H.PrefixIndex(0, 4096, 16)
    ix.insert(*dev([system], [w.shared_prefix_blocks.tolist()]))
    matched, pages = ix.lookup(*dev(prompts))
    matched, pages = matched.cpu().numpy(), pages.cpu().numpy()
    assert matched.tolist() == [4] * 6
    prefix_lens = (matched * 16).astype(np.uint32)
    dst_tables = w.dst_tables.copy()
    for q in range(6):
        dst_tables[q, :matched[q]] = pages[q, :matched[q]]
    assert np.array_equal(dst_tables, w.dst_tables) and np.array_equal(prefix_lens, w.prefix_lens)   # what the host tree would have said
    src = H.Pool.allocate(0, 2, 8, 128, 16, 2048, "f16")
    dst = H.Pool.allocate(0, 2, 8, 128, 16, 2048, "f16", refcounts=True, fill_byte=0x5A)
    src.storage.view(torch.int16).copy_(torch.randint(-3000, 3000, src.storage.view(torch.int16).shape, dtype=torch.int16, device="cuda"))
    plan = H.Plan(src, dst, H.Batch(w.seq_lens, w.src_tables, dst_tables, w.table_stride, prefix_lens))
    plan.enqueue()
    plan.refcount_apply(+1)
    torch.cuda.synchronize()
    st = plan.stats()
    assert st.n_prefix_refs == 6 * 4 and st.n_tokens == int((w.seq_lens - 64).sum())
    shared = torch.from_numpy(w.shared_prefix_blocks.astype(np.int64)).cuda()
    assert bool((dst.refcounts[shared] == 6).all()) and int(dst.refcounts.sum()) == 24
    assert bool((dst.blocks(0).index_select(0, shared).view(torch.uint8) == 0x5A).all())            # nothing moved into the prefix
    for q in range(6):                                                                              # the suffix blocks did move
        nb = (int(w.seq_lens[q]) + 15) // 16
        if nb > 4:
            s_id, d_id = int(w.src_tables[q, 4]), int(dst_tables[q, 4])
            n_valid = min(16, int(w.seq_lens[q]) - 64)
            assert torch.equal(src.blocks(1)[s_id, :n_valid].view(torch.int16), dst.blocks(1)[d_id, :n_valid].view(torch.int16))


def test_device_page_allocator_matches_the_reference_stack(H):
    import torch
    from oracle.prefix_oracle import PageStackOracle
    rng = np.random.default_rng(88)
    total, stride = 5000, 40
    dev_alloc, ref = H.DevicePageAllocator(0, total), PageStackOracle(total)
    held = []                                                      # (rows as lists) still allocated
    for rnd in range(30):
        n = int(rng.integers(1, 2500 if rnd == 7 else 60))         # one batch wider than the CTA (1 024 threads)
        counts = rng.integers(0, 4 if n > 1024 else stride // 2, size=n).astype(np.int32)
        first = rng.integers(0, stride // 2, size=n).astype(np.int32)
        tables = torch.full((n, stride), -1, dtype=torch.int32, device="cuda")
        dev_alloc.allocate(tables, torch.from_numpy(counts).cuda(), torch.from_numpy(first).cuda())
        want = ref.batch_allocate(counts.tolist())
        got = tables.cpu().numpy()
        if want is None:
            assert int(dev_alloc.status.item()) == N.ERR_POOL_EXHAUSTED and bool((got == -1).all())
        else:
            assert int(dev_alloc.status.item()) == 0
            for s in range(n):
                assert got[s, first[s]:first[s] + counts[s]].tolist() == want[s], f"round {rnd} sequence {s}"
                assert bool((np.delete(got[s], np.s_[first[s]:first[s] + counts[s]]) == -1).all())
            held.append((tables, counts, first, want))
        if held and rng.random() < 0.6:                            # give one earlier batch back
            tables, counts, first, rows = held.pop(int(rng.integers(len(held))))
            dev_alloc.free(tables, torch.from_numpy(counts).cuda(), torch.from_numpy(first).cuda())
            ref.batch_free(rows)
            assert int(dev_alloc.status.item()) == 0
        assert dev_alloc.available() == ref.available()
    # a row that would overrun the table, and more pages returned than were handed out: refused, nothing changes
    before = dev_alloc.available()
    t = torch.zeros((1, 8), dtype=torch.int32, device="cuda")
    dev_alloc.allocate(t, torch.tensor([6], dtype=torch.int32).cuda(), torch.tensor([4], dtype=torch.int32).cuda())
    assert int(dev_alloc.status.item()) == N.ERR_INVALID_CONFIG and dev_alloc.available() == before
    big = torch.zeros((1, total + 8), dtype=torch.int32, device="cuda")
    dev_alloc.free(big, torch.tensor([total - before + 1], dtype=torch.int32).cuda())
    assert int(dev_alloc.status.item()) == N.ERR_INVALID_CONFIG and dev_alloc.available() == before


@pytest.mark.parametrize("bits", [64, 9])
def test_a_key_collision_is_a_checked_miss_not_another_prompts_page(H, bits):
    """The index keeps no whole prefixes, only 64-bit keys plus the first and last token id of each node's element.  With the
    keys cut to 9 bits (test hook) different prefixes share keys all the time: a lookup may then match less than the
    reference would, but every page it returns is the page inserted for exactly that prefix."""
    rng = np.random.default_rng(5)
    group = 4
    seqs = [list(map(int, rng.integers(1, 50_000, size=int(rng.integers(2, 12)) * group))) for _ in range(120)]
    for s in range(0, 120, 5):                                     # some share a stem
        seqs[s + 1][: 2 * group] = seqs[s][: 2 * group]
    pages, owner, nxt = [], {}, 0
    for s in seqs:                                                 # the page of a node = what its first inserter brought
        row = []
        for i in range(len(s) // group):
            row.append(nxt)
            owner.setdefault(tuple(s[: (i + 1) * group]), nxt)
            nxt += 1
        pages.append(row)
    ix = H.PrefixIndex(0, 8192, group_tokens=group)
    if bits != 64:
        ix.set_key_bits(bits)
    ix.insert(*dev(seqs, pages))
    got = lookup(ix, seqs)
    short = 0
    for s, (matched, pg) in zip(seqs, got):
        assert matched <= len(s) // group
        short += matched < len(s) // group
        for i in range(matched):
            assert pg[i] == owner[tuple(s[: (i + 1) * group])], (i, pg[i])
    st = ix.stats()
    if bits == 64:
        assert short == 0 and st.key_collisions == 0
    else:
        assert short > 0 and st.key_collisions > 0                 # collisions happened, and each was refused
    with pytest.raises(N.TkvError):
        ix.set_key_bits(32)                                        # not on an index that has been walked
