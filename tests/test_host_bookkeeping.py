"""Host-side block bookkeeping of the C ABI (page allocator, block table, run
allocator, radix tree, prefix table, pairing): the reference's own unit-test
scenarios, and a randomised walk against the CPU oracle.  No GPU needed."""
import ctypes as C

import numpy as np
import pytest

import oracle
from tempura_b200 import _build, _native
from tempura_b200._native import TkvError


@pytest.fixture(scope="module")
def L():
    _build.build()
    return _native.lib()


@pytest.fixture(scope="module")
def O():
    return oracle.lib()


def _u32(xs):
    a = np.asarray(xs, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def _sz(xs):
    a = np.asarray(xs, dtype=np.uint64)
    return a, a.ctypes.data_as(C.POINTER(C.c_size_t))


# engine/src/kv_cache.rs:1946-1962
def test_page_allocator_reference_scenario(L):
    a = L.tkv_page_allocator_new(4)
    assert L.tkv_page_allocator_available(a) == 4 and L.tkv_page_allocator_in_use(a) == 0
    p0, p1 = C.c_size_t(), C.c_size_t()
    assert L.tkv_page_allocator_allocate(a, C.byref(p0)) == 0
    assert L.tkv_page_allocator_allocate(a, C.byref(p1)) == 0
    assert (p0.value, p1.value) == (0, 1)
    assert L.tkv_page_allocator_available(a) == 2 and L.tkv_page_allocator_in_use(a) == 2
    L.tkv_page_allocator_free(a, p0.value)
    assert L.tkv_page_allocator_available(a) == 3
    p2 = C.c_size_t()
    L.tkv_page_allocator_allocate(a, C.byref(p2))
    assert p2.value == p0.value
    L.tkv_page_allocator_allocate(a, C.byref(p2)); L.tkv_page_allocator_allocate(a, C.byref(p2))
    assert L.tkv_page_allocator_allocate(a, C.byref(p2)) == _native.ERR_POOL_EXHAUSTED
    L.tkv_page_allocator_delete(a)


def test_page_allocator_random_walk_vs_oracle(L, O):
    rng = np.random.default_rng(1)
    a, o = L.tkv_page_allocator_new(64), O.orc_pa_new(64)
    held = []
    for _ in range(2000):
        if held and rng.random() < 0.45:
            pg = held.pop(int(rng.integers(len(held))))
            L.tkv_page_allocator_free(a, pg); O.orc_pa_free(o, pg)
        else:
            p = C.c_size_t()
            rc = L.tkv_page_allocator_allocate(a, C.byref(p))
            want = O.orc_pa_allocate(o)
            assert (rc == 0) == (want >= 0)
            if rc == 0:
                assert p.value == want
                held.append(p.value)
        assert L.tkv_page_allocator_available(a) == O.orc_pa_available(o)
    L.tkv_page_allocator_delete(a); O.orc_pa_delete(o)


# engine/src/kv_cache.rs:1965-1981
def test_block_table_reference_scenario(L):
    bt = L.tkv_block_table_new(8)
    assert L.tkv_block_table_num_blocks(bt) == 0 and L.tkv_block_table_max_blocks(bt) == 8
    L.tkv_block_table_set_block(bt, 0, 5)
    L.tkv_block_table_set_block(bt, 1, 3)
    assert L.tkv_block_table_num_blocks(bt) == 2
    pg = C.c_size_t()
    assert L.tkv_block_table_get_block(bt, 0, C.byref(pg)) == 1 and pg.value == 5
    assert L.tkv_block_table_get_block(bt, 1, C.byref(pg)) == 1 and pg.value == 3
    assert L.tkv_block_table_get_block(bt, 2, C.byref(pg)) == 0
    sl = L.tkv_block_table_as_slice(bt)
    assert [sl[0], sl[1]] == [5, 3] and sl[2] == 0xFFFFFFFF
    freed = (C.c_size_t * 8)()
    assert L.tkv_block_table_clear(bt, freed, 8) == 2 and set(freed[:2]) == {5, 3}
    assert L.tkv_block_table_num_blocks(bt) == 0
    assert L.tkv_block_table_set_block(bt, 8, 1) == _native.ERR_INVALID_CONFIG
    L.tkv_block_table_delete(bt)


# engine/src/gpu_page_pool.rs:224-295
def _alloc(L, a, n):
    s = C.c_size_t()
    return s.value if L.tkv_run_allocator_alloc(a, n, C.byref(s)) else None


def _runs(L, a):
    st, pg = (C.c_size_t * 128)(), (C.c_size_t * 128)()
    n = L.tkv_run_allocator_free_runs(a, st, pg, 128)
    return [(st[i], pg[i]) for i in range(n)]


def test_run_allocator_reference_scenarios(L):
    a = L.tkv_run_allocator_new(64)
    r0, r1, r2 = _alloc(L, a, 16), _alloc(L, a, 16), _alloc(L, a, 16)
    assert (r0, r1, r2) == (0, 16, 32) and L.tkv_run_allocator_free_pages(a) == 16
    L.tkv_run_allocator_free(a, r1, 16)
    assert len(_runs(L, a)) == 2
    r3 = _alloc(L, a, 16)
    assert r3 in (16, 48)
    for r in (r0, r2, r3):
        L.tkv_run_allocator_free(a, r, 16)
    assert _runs(L, a) == [(0, 64)] and L.tkv_run_allocator_allocated_pages(a) == 0
    L.tkv_run_allocator_delete(a)
    a = L.tkv_run_allocator_new(10)
    assert _alloc(L, a, 11) is None and L.tkv_run_allocator_free_pages(a) == 10
    assert _alloc(L, a, 0) is None
    L.tkv_run_allocator_delete(a)
    a = L.tkv_run_allocator_new(32)
    r0, r1 = _alloc(L, a, 8), _alloc(L, a, 8)
    assert not L.tkv_run_allocator_try_extend(a, r0, 8, 12)
    L.tkv_run_allocator_free(a, r1, 8)
    assert L.tkv_run_allocator_try_extend(a, r0, 8, 12)
    assert L.tkv_run_allocator_allocated_pages(a) == 12 and L.tkv_run_allocator_free_pages(a) == 20
    assert _alloc(L, a, 16) == 12 and L.tkv_run_allocator_free_pages(a) == 4
    L.tkv_run_allocator_delete(a)


def test_run_allocator_random_walk_vs_oracle(L, O):
    rng = np.random.default_rng(7)
    a, o = L.tkv_run_allocator_new(512), O.orc_ra_new(512)
    live = []
    for _ in range(3000):
        r = rng.random()
        if live and r < 0.4:
            st, pg = live.pop(int(rng.integers(len(live))))
            L.tkv_run_allocator_free(a, st, pg); O.orc_ra_free(o, st, pg)
        elif live and r < 0.5:
            i = int(rng.integers(len(live)))
            st, pg = live[i]
            tgt = pg + int(rng.integers(1, 9))
            got = L.tkv_run_allocator_try_extend(a, st, pg, tgt)
            assert got == O.orc_ra_try_extend(o, st, pg, tgt)
            if got:
                live[i] = (st, tgt)
        else:
            n = int(rng.integers(1, 24))
            got = _alloc(L, a, n)
            s = C.c_size_t()
            want = s.value if O.orc_ra_alloc(o, n, C.byref(s)) else None
            assert got == want
            if got is not None:
                live.append((got, n))
        assert L.tkv_run_allocator_free_pages(a) == O.orc_ra_free_pages(o)
        st, pg = (C.c_size_t * 128)(), (C.c_size_t * 128)()
        n = O.orc_ra_free_runs(o, st, pg, 128)
        assert _runs(L, a) == [(st[i], pg[i]) for i in range(n)]
    L.tkv_run_allocator_delete(a); O.orc_ra_delete(o)


# engine/src/prefix_cache.rs:155-241
def _lookup(L, t, toks):
    a, p = _u32(toks)
    out = (C.c_size_t * 256)()
    n = C.c_size_t(0)
    m = L.tkv_radix_tree_lookup(t, p, len(toks), out, 256, C.byref(n))
    return m, list(out[: n.value])


def _insert(L, t, toks, pages):
    a, p = _u32(toks)
    b, q = _sz(pages)
    L.tkv_radix_tree_insert(t, p, len(toks), q, len(pages))


def test_radix_tree_reference_scenarios(L):
    t = L.tkv_radix_tree_new()
    _insert(L, t, [1, 2, 3], [10, 20, 30])
    assert _lookup(L, t, [1, 2, 3]) == (3, [10, 20, 30])
    assert L.tkv_radix_tree_hit_count(t) == 1 and L.tkv_radix_tree_tokens_saved(t) == 3
    assert _lookup(L, t, [5, 6, 7]) == (0, [])
    L.tkv_radix_tree_delete(t)
    t = L.tkv_radix_tree_new()
    _insert(L, t, [1, 2, 3, 4], [10, 20, 30, 40])
    assert _lookup(L, t, [1, 2, 5])[0] == 2
    L.tkv_radix_tree_delete(t)
    t = L.tkv_radix_tree_new()
    _insert(L, t, [1, 2, 3], [10, 20, 30]); _insert(L, t, [1, 2, 4], [10, 20, 40])
    assert _lookup(L, t, [1, 2, 3])[0] == 3 and _lookup(L, t, [1, 2, 4]) == (3, [10, 20, 40])
    assert _lookup(L, t, [1, 2])[0] == 2
    L.tkv_radix_tree_delete(t)
    t = L.tkv_radix_tree_new()
    _insert(L, t, [100, 101, 102, 103], [0, 1, 2, 3])
    turn1 = [100, 101, 102, 103, 200, 201]
    assert _lookup(L, t, turn1)[0] == 4
    _insert(L, t, turn1, [0, 1, 2, 3, 4, 5])
    assert _lookup(L, t, turn1 + [300])[0] == 6
    L.tkv_radix_tree_delete(t)
    t = L.tkv_radix_tree_new()
    _insert(L, t, [1, 2], [10, 20]); _insert(L, t, [3, 4], [30, 40])
    _lookup(L, t, [3, 4])
    a, p = _u32([3, 4])
    L.tkv_radix_tree_release(t, p, 2)
    freed = (C.c_size_t * 4)()
    assert L.tkv_radix_tree_evict_lru(t, freed, 4) == 1 and freed[0] == 20
    L.tkv_radix_tree_delete(t)


def test_radix_tree_random_walk_vs_oracle_and_no_double_free(L, O):
    rng = np.random.default_rng(3)
    t, o = L.tkv_radix_tree_new(), O.orc_radix_new()
    seqs = []
    next_page = 0
    for _ in range(400):
        r = rng.random()
        if r < 0.4 or not seqs:
            base = list(seqs[int(rng.integers(len(seqs)))][: int(rng.integers(1, 6))]) if seqs and rng.random() < 0.6 else []
            toks = base + [int(x) for x in rng.integers(0, 6, size=int(rng.integers(1, 5)))]
            pages = list(range(next_page, next_page + len(toks)))
            next_page += len(toks)
            _insert(L, t, toks, pages)
            a, p = _u32(toks); b, q = _sz(pages)
            O.orc_radix_insert(o, p, len(toks), q, len(pages))
            seqs.append(toks)
        elif r < 0.8:
            toks = seqs[int(rng.integers(len(seqs)))] + [int(rng.integers(0, 6))]
            a, p = _u32(toks)
            out = (C.c_size_t * 256)(); n = C.c_size_t()
            want_m = O.orc_radix_lookup(o, p, len(toks), out, 256, C.byref(n))
            assert _lookup(L, t, toks) == (want_m, list(out[: n.value]))
        else:
            toks = seqs[int(rng.integers(len(seqs)))]
            a, p = _u32(toks)
            L.tkv_radix_tree_release(t, p, len(toks)); O.orc_radix_release(o, p, len(toks))
        assert L.tkv_radix_tree_node_count(t) == O.orc_radix_node_count(o)
        assert L.tkv_radix_tree_hit_count(t) == O.orc_radix_hit_count(o)
        assert L.tkv_radix_tree_tokens_saved(t) == O.orc_radix_tokens_saved(o)
    # first eviction agrees with the reference's rule ...
    f1, f2 = (C.c_size_t * 4)(), (C.c_size_t * 4)()
    n1, n2 = L.tkv_radix_tree_evict_lru(t, f1, 4), O.orc_radix_evict_lru(o, f2, 4)
    assert (n1, list(f1[:n1])) == (n2, list(f2[:n2]))
    # ... but the library never reports a page twice (the reference would: it leaves
    # the unlinked node eligible, engine/src/prefix_cache.rs:99-125)
    seen = set(f1[:n1])
    for _ in range(2000):
        n = L.tkv_radix_tree_evict_lru(t, f1, 4)
        if n == 0:
            break
        for pg in f1[:n]:
            assert pg not in seen
            seen.add(pg)
    L.tkv_radix_tree_delete(t); O.orc_radix_delete(o)


# engine/src/kv_cache.rs:1686-1787, 2083-2110
def _store(L, t, toks, blocks, seq_len, salt=None):
    a, p = _u32(toks); b, q = _u32(blocks)
    L.tkv_prefix_table_store(t, p, len(toks), salt, q, len(blocks), seq_len)


def _probe(L, t, toks, salt=None):
    a, p = _u32(toks)
    out = (C.c_uint32 * 64)(); n = C.c_size_t()
    m = L.tkv_prefix_table_probe(t, p, len(toks), salt, out, 64, C.byref(n))
    return m, list(out[: n.value])


def test_prefix_table_reference_scenarios(L):
    t = L.tkv_prefix_table_new(10)
    _store(L, t, [1, 2, 3], [7], 3)
    assert L.tkv_prefix_table_len(t) == 1
    assert _probe(L, t, [1, 2, 3]) == (3, [7])
    assert L.tkv_prefix_table_hit_count(t) == 1 and L.tkv_prefix_table_tokens_saved(t) == 3
    assert _probe(L, t, [1, 2, 3]) == (3, [7])
    assert _probe(L, t, [99])[0] == 0
    assert _probe(L, t, [1, 2, 3, 9, 9]) == (3, [7])
    L.tkv_prefix_table_delete(t)
    t = L.tkv_prefix_table_new(2)
    for i in range(3):
        _store(L, t, [i], [i], 1)
    assert L.tkv_prefix_table_len(t) == 2 and _probe(L, t, [0])[0] == 0
    L.tkv_prefix_table_delete(t)
    t = L.tkv_prefix_table_new(10)
    _store(L, t, [1, 2, 3], [1], 1, b"tenant-a"); _store(L, t, [1, 2, 3], [2], 1, b"tenant-b")
    assert L.tkv_prefix_table_len(t) == 2
    assert _probe(L, t, [1, 2, 3], b"tenant-a") == (1, [1]) and _probe(L, t, [1, 2, 3], b"tenant-b") == (1, [2])
    assert _probe(L, t, [1, 2, 3], b"tenant-c")[0] == 0 and _probe(L, t, [1, 2, 3], None)[0] == 0
    L.tkv_prefix_table_delete(t)
    t = L.tkv_prefix_table_new(1)          # a referenced entry is never evicted
    _store(L, t, [1], [1], 1); _probe(L, t, [1]); _store(L, t, [2], [2], 1)
    assert L.tkv_prefix_table_len(t) == 2
    a, p = _u32([1])
    L.tkv_prefix_table_release(t, p, 1, None)
    _store(L, t, [3], [3], 1)              # now [1] (unreferenced, oldest) goes
    assert _probe(L, t, [1])[0] == 0 and _probe(L, t, [2])[0] == 1
    L.tkv_prefix_table_delete(t)


def test_prefix_table_random_walk_vs_oracle(L, O):
    rng = np.random.default_rng(5)
    t, o = L.tkv_prefix_table_new(6), O.orc_pt_new(6)
    keys = []
    for step in range(1500):
        r = rng.random()
        salt = [None, b"a", b"b"][int(rng.integers(3))]
        if r < 0.3 or not keys:
            toks = [int(x) for x in rng.integers(0, 4, size=int(rng.integers(1, 5)))]
            blocks = [int(x) for x in rng.integers(0, 100, size=int(rng.integers(0, 4)))]
            _store(L, t, toks, blocks, len(toks), salt)
            a, p = _u32(toks); b, q = _u32(blocks)
            O.orc_pt_store(o, p, len(toks), salt, q, len(blocks), len(toks))
            keys.append(toks)
        elif r < 0.75:
            toks = keys[int(rng.integers(len(keys)))] + [int(x) for x in rng.integers(0, 4, size=int(rng.integers(0, 3)))]
            a, p = _u32(toks)
            out = (C.c_uint32 * 64)(); n = C.c_size_t()
            want = O.orc_pt_probe(o, p, len(toks), salt, out, 64, C.byref(n))
            assert _probe(L, t, toks, salt) == (want, list(out[: n.value])), step
        else:
            toks = keys[int(rng.integers(len(keys)))]
            a, p = _u32(toks)
            L.tkv_prefix_table_release(t, p, len(toks), salt); O.orc_pt_release(o, p, len(toks), salt)
        assert L.tkv_prefix_table_len(t) == O.orc_pt_len(o)
        assert L.tkv_prefix_table_hit_count(t) == O.orc_pt_hit_count(o)
        assert L.tkv_prefix_table_tokens_saved(t) == O.orc_pt_tokens_saved(o)
    L.tkv_prefix_table_delete(t); O.orc_pt_delete(o)


# ---- pairing ---------------------------------------------------------------------
def _pairs(L, n_gpus, layers, heads):
    out = (_native.TkvPairing * 8)(); n = C.c_int32()
    _native.check(L.tkv_pairing_make(n_gpus, layers, heads, out, 8, C.byref(n)))
    return [(p.prefill_device, p.decode_device, p.shard.src_head_begin, p.shard.n_heads,
             p.shard.src_layer_begin, p.shard.n_layers) for p in out[: n.value]]


def test_pairing_shards_heads_then_layers(L):
    assert _pairs(L, 1, 80, 8) == [(0, 0, 0, 8, 0, 80)]
    assert _pairs(L, 2, 80, 8) == [(0, 1, 0, 8, 0, 80)]
    assert _pairs(L, 4, 80, 8) == [(0, 2, 0, 4, 0, 80), (1, 3, 4, 4, 0, 80)]
    assert _pairs(L, 8, 80, 8) == [(i, i + 4, 2 * i, 2, 0, 80) for i in range(4)]
    # fewer heads than pairs -> layer ranges
    assert _pairs(L, 8, 22, 2) == [(0, 4, 0, 2, 0, 5), (1, 5, 0, 2, 5, 6), (2, 6, 0, 2, 11, 5), (3, 7, 0, 2, 16, 6)]
    with pytest.raises(TkvError) as e:
        _pairs(L, 3, 80, 8)
    assert e.value.code == _native.ERR_INVALID_CONFIG
    with pytest.raises(TkvError) as e:
        _pairs(L, 8, 80, 6)
    assert e.value.code == _native.ERR_DIMENSION_MISMATCH
