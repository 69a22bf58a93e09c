"""Pins the CPU oracle against the reference's own known-answer tests.

Every expected value below is the one asserted in the cited reference test
(paths inside the tempura repository).  The reference is Rust and cannot run in
this image, so its test vectors, restated here, are what anchors the oracle.
"""
import ctypes as C
import math
import struct

import numpy as np
import pytest

import oracle
from oracle import lib


def f32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


def bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


# --- kernels/src/e4m3.rs:100-174 ------------------------------------------------
def test_e4m3_roundtrip_exact_all_normals():
    L = lib()
    for b in range(256):
        exp = (b >> 3) & 0xF
        v = L.orc_e4m3_to_f32(b)
        if exp == 0:
            assert v == 0.0 and math.copysign(1.0, v) == (-1.0 if b & 0x80 else 1.0)
            continue
        if exp == 15 and (b & 7) == 7:
            continue
        assert L.orc_f32_to_e4m3(v) == b, hex(b)


def test_e4m3_known_values():
    L = lib()
    enc, dec = L.orc_f32_to_e4m3, L.orc_e4m3_to_f32
    assert enc(0.0) == 0x00 and enc(-0.0) == 0x80
    assert dec(0x00) == 0.0 and dec(0x38) == 1.0
    assert enc(1.0) == 0x38 and enc(-1.0) == 0xB8
    assert dec(0x7E) == 448.0
    assert enc(448.0) == 0x7E and enc(-448.0) == 0xFE
    assert enc(1e30) == 0x7E
    assert enc(float("inf")) == 0x7E and enc(float("-inf")) == 0xFE
    assert enc(float("nan")) == 0x7F
    assert enc(0.015625) == 0x08 and dec(0x08) == 0.015625
    assert enc(0.01) == 0x00 and enc(0.001) == 0x00 and enc(-0.001) == 0x80
    assert dec(0x01) == 0.0
    d = dec(0x81)
    assert d == 0.0 and math.copysign(1.0, d) == -1.0


def test_e4m3_rne_tie_to_even():
    enc = lib().orc_f32_to_e4m3
    assert enc(1.0) == 0x38
    assert enc(1.0625) == 0x38
    assert enc(1.0626) == 0x39
    assert enc(1.1875) == 0x3A
    assert enc(1.125) == 0x39


def test_e4m3_rne_carry_into_exponent():
    L = lib()
    enc, dec = L.orc_f32_to_e4m3, L.orc_e4m3_to_f32
    assert dec(0x53) == 11.0
    assert enc(15.0) == 0x57
    assert enc(15.4375) == 0x57
    assert enc(15.5) == 0x58
    assert enc(15.9375) == 0x58
    assert enc(16.0) == 0x58
    assert dec(0x58) == 16.0


# --- tools/bench-gpu/src/bench_decode_ops.rs:686-701 (adversarial classes) --------
ADVERSARIAL = [0.0, -0.0, 1.0, -1.0, 1.0625, 1.1875, 15.5, 0.015625, 0.01, 0.001, -0.001,
               448.0, -448.0, 449.0, 1e30, -1e30, float("inf"), float("-inf"), float("nan"),
               65505.0, 65520.0, 6.1035156e-5, 5.96e-8, 2.98e-8, 1e-8, -1e-8, 0.5, 0.49999997]


def test_adversarial_e4m3_bytes():
    want = [0x00, 0x80, 0x38, 0xB8, 0x38, 0x3A, 0x58, 0x08, 0x00, 0x00, 0x80,
            0x7E, 0xFE, 0x7E, 0x7E, 0xFE, 0x7E, 0xFE, 0x7F,
            0x7E, 0x7E, 0x00, 0x00, 0x00, 0x00, 0x80, 0x30, 0x30]
    got = [lib().orc_f32_to_e4m3(v) for v in ADVERSARIAL]
    assert got == want


def test_adversarial_f16_bits_match_numpy_and_f16c():
    L = lib()
    for v in ADVERSARIAL:
        got = L.orc_f32_to_f16(v)
        if math.isnan(v):
            assert got & 0x7C00 == 0x7C00 and got & 0x3FF
            continue
        with np.errstate(over="ignore"):
            want = int(np.array([v], dtype=np.float32).astype(np.float16).view(np.uint16)[0])
        assert got == want, v
        if L.orc_have_f16c():
            assert got == L.orc_hw_f32_to_f16(v)
    # 65505 rounds down to the max normal, 65520 ties up to Inf
    assert L.orc_f32_to_f16(65505.0) == 0x7BFF and L.orc_f32_to_f16(65520.0) == 0x7C00


def test_f32_to_f16_sweep_against_f16c_instruction():
    """engine/src/kv_cache.rs:29-47 calls vcvtps2ph directly; sweep 2^22 inputs
    (every f32 whose low 10 bits are zero) plus random ones against it."""
    L = lib()
    if not L.orc_have_f16c():
        pytest.skip("compiler does not target F16C")
    fn = C.cast(L.orc_f32_to_f16, C.c_void_p)
    assert L.orc_sweep_f32_to_f16(fn, 10) == 0
    rng = np.random.default_rng(0)
    for u in rng.integers(0, 2**32, size=20000, dtype=np.uint64):
        x = struct.unpack("<f", struct.pack("<I", int(u)))[0]
        assert L.orc_f32_to_f16(x) == L.orc_hw_f32_to_f16(x)


def test_f16_to_f32_all_patterns():
    L = lib()
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32).view(np.uint32)
    for i in range(65536):
        got = bits(L.orc_f16_to_f32(i))
        if (i & 0x7C00) == 0x7C00 and (i & 0x3FF):
            assert got & 0x7F800000 == 0x7F800000 and got & 0x7FFFFF
            continue
        assert got == int(want[i]), hex(i)


def test_scalar_fallback_truncates():
    # engine/src/kv_cache.rs:77-89: mantissa truncation, subnormal flush
    L = lib()
    assert L.orc_f32_to_f16_scalar_fallback(1.0) == 0x3C00
    assert L.orc_f32_to_f16_scalar_fallback(f32(1.0 + 2**-11 + 2**-12)) == 0x3C00   # RNE would give 0x3C01
    assert L.orc_f32_to_f16_scalar_fallback(1e-6) == 0x0000
    assert L.orc_f32_to_f16_scalar_fallback(1e6) == 0x7C00


def test_legacy_engine_quantizer_differs_from_oracle_quantizer():
    """engine/src/kv_cache.rs:1078-1123 is NOT the oracle quantizer; this records
    where it departs from kernels/src/e4m3.rs (half-up ties, [256,448) -> 448,
    NaN -> 0x7E)."""
    L = lib()
    assert L.orc_f32_to_e4m3(1.0625) == 0x38 and L.orc_f32_to_e4m3_legacy(1.0625) == 0x39
    assert L.orc_f32_to_e4m3(300.0) == 0x79 and L.orc_f32_to_e4m3_legacy(300.0) == 0x7E
    assert L.orc_f32_to_e4m3(float("nan")) == 0x7F and L.orc_f32_to_e4m3_legacy(float("nan")) == 0x7E
    # ...and agrees where neither rule is exercised
    for v in (0.0, 1.0, -1.0, 0.5, 15.0, 16.0, 0.015625, 192.0):
        assert L.orc_f32_to_e4m3(v) == L.orc_f32_to_e4m3_legacy(v)


# --- engine/src/kv_cache.rs:1946-1981 --------------------------------------------
def test_page_allocator():
    L = lib()
    a = L.orc_pa_new(4)
    assert L.orc_pa_available(a) == 4 and L.orc_pa_in_use(a) == 0
    p0, p1 = L.orc_pa_allocate(a), L.orc_pa_allocate(a)
    assert (p0, p1) == (0, 1)     # first page handed out is 0 (kv_cache.rs:768-770)
    assert L.orc_pa_available(a) == 2 and L.orc_pa_in_use(a) == 2
    L.orc_pa_free(a, p0)
    assert L.orc_pa_available(a) == 3
    assert L.orc_pa_allocate(a) == p0
    L.orc_pa_allocate(a); L.orc_pa_allocate(a)
    assert L.orc_pa_allocate(a) == -1
    L.orc_pa_delete(a)


def test_block_table():
    L = lib()
    bt = L.orc_bt_new(8)
    assert L.orc_bt_num_blocks(bt) == 0
    L.orc_bt_set_block(bt, 0, 5)
    L.orc_bt_set_block(bt, 1, 3)
    assert L.orc_bt_num_blocks(bt) == 2
    assert L.orc_bt_get_block(bt, 0) == 5 and L.orc_bt_get_block(bt, 1) == 3
    assert L.orc_bt_get_block(bt, 2) == -1
    freed = (C.c_size_t * 8)()
    n = L.orc_bt_clear(bt, freed, 8)
    assert n == 2 and set(freed[:2]) == {5, 3}
    assert L.orc_bt_num_blocks(bt) == 0
    L.orc_bt_delete(bt)


# --- engine/src/kv_cache.rs:1914-1943: paged == contiguous -------------------------
def test_paged_matches_contiguous():
    L = lib()
    heads, dim, bs, pages = 4, 16, 4, 32       # ModelConfig::tiny_test kv geometry
    stride = heads * dim
    pool = np.zeros(pages * bs * stride, dtype=np.float32)
    alloc, bt = L.orc_pa_new(pages), L.orc_bt_new(32)
    contiguous = np.zeros((10, stride), dtype=np.float32)
    for t in range(10):
        k = np.array([(t * 100 + i) * 0.1 for i in range(stride)], dtype=np.float32)
        contiguous[t] = k
        while L.orc_bt_num_blocks(bt) < -(-(t + 1) // bs):        # ensure_blocks_for
            L.orc_bt_set_block(bt, L.orc_bt_num_blocks(bt), L.orc_pa_allocate(alloc))
        L.orc_paged_scatter(pool.ctypes.data, L.orc_bt_as_slice(bt), bs, stride, 4, t, 1, k.ctypes.data)
    out = np.zeros((10, stride), dtype=np.float32)
    L.orc_paged_gather(pool.ctypes.data, L.orc_bt_as_slice(bt), bs, stride, 4, 10, out.ctypes.data)
    assert np.array_equal(out.view(np.uint32), contiguous.view(np.uint32))
    assert [L.orc_bt_get_block(bt, i) for i in range(3)] == [0, 1, 2]
    L.orc_pa_delete(alloc); L.orc_bt_delete(bt)


# --- engine/src/disaggregated.rs:292-321: transfer round trip ----------------------
def test_transfer_round_trip_f32_and_f16():
    L = lib()
    rng = np.random.default_rng(42)
    seq, stride = 5, 4 * 16
    src = rng.standard_normal(seq * stride).astype(np.float32)
    dst = np.zeros_like(src)
    L.orc_transfer_layer(src.ctypes.data_as(C.POINTER(C.c_float)), seq, stride, 0, dst.ctypes.data)
    assert np.array_equal(src.view(np.uint32), dst.view(np.uint32))
    dst16 = np.zeros(seq * stride, dtype=np.uint16)
    L.orc_transfer_layer(src.ctypes.data_as(C.POINTER(C.c_float)), seq, stride, 1, dst16.ctypes.data)
    assert np.array_equal(dst16, src.astype(np.float16).view(np.uint16))


# --- kernels/src/attention.rs:472-484 + bench_decode_ops.rs:2965-2980 ---------------
def test_paged_row_offset_matches_probe_loop():
    L = lib()
    d, nkv, bs = 128, 8, 16
    table = oracle.gen_permutation(64, 92)
    tp = table.ctypes.data_as(C.POINTER(C.c_uint32))
    for tok in (0, 1, 15, 16, 17, 999, 1000, 1023):
        for kv_h in (0, 3, 7):
            page = int(table[tok // bs])
            row = (page * bs + tok % bs) * nkv + kv_h
            assert L.orc_paged_row_offset(tp, bs, nkv * d, tok, kv_h, d) == row * d


# --- engine/src/prefix_cache.rs:155-241 --------------------------------------------
def _u32(xs):
    a = np.asarray(xs, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def _sz(xs):
    a = np.asarray(xs, dtype=np.uint64)
    return a, a.ctypes.data_as(C.POINTER(C.c_size_t))


def _lookup(L, t, toks):
    a, p = _u32(toks)
    out = (C.c_size_t * 64)()
    n = C.c_size_t(0)
    m = L.orc_radix_lookup(t, p, len(toks), out, 64, C.byref(n))
    return m, list(out[: n.value])


def _insert(L, t, toks, pages):
    a, p = _u32(toks)
    b, q = _sz(pages)
    L.orc_radix_insert(t, p, len(toks), q, len(pages))


def test_radix_insert_lookup_partial_nomatch():
    L = lib()
    t = L.orc_radix_new()
    _insert(L, t, [1, 2, 3], [10, 20, 30])
    m, pages = _lookup(L, t, [1, 2, 3])
    assert m == 3 and pages == [10, 20, 30]
    assert L.orc_radix_hit_count(t) == 1 and L.orc_radix_tokens_saved(t) == 3
    L.orc_radix_delete(t)
    t = L.orc_radix_new()
    _insert(L, t, [1, 2, 3, 4], [10, 20, 30, 40])
    assert _lookup(L, t, [1, 2, 5])[0] == 2
    m, pages = _lookup(L, t, [5, 6, 7])
    assert m == 0 and pages == []
    L.orc_radix_delete(t)


def test_radix_shared_prefix_and_multi_turn():
    L = lib()
    t = L.orc_radix_new()
    _insert(L, t, [1, 2, 3], [10, 20, 30])
    _insert(L, t, [1, 2, 4], [10, 20, 40])
    assert _lookup(L, t, [1, 2, 3])[0] == 3
    assert _lookup(L, t, [1, 2, 4]) == (3, [10, 20, 40])
    assert _lookup(L, t, [1, 2])[0] == 2
    L.orc_radix_delete(t)
    t = L.orc_radix_new()
    _insert(L, t, [100, 101, 102, 103], [0, 1, 2, 3])
    turn1 = [100, 101, 102, 103, 200, 201]
    assert _lookup(L, t, turn1)[0] == 4
    _insert(L, t, turn1, [0, 1, 2, 3, 4, 5])
    assert _lookup(L, t, turn1 + [300])[0] == 6
    L.orc_radix_delete(t)


def test_radix_refcount_release_evict():
    L = lib()
    t = L.orc_radix_new()
    _insert(L, t, [1, 2, 3], [10, 20, 30])
    _lookup(L, t, [1, 2, 3]); _lookup(L, t, [1, 2, 3])
    a, p = _u32([1, 2, 3])
    L.orc_radix_release(t, p, 3)
    assert L.orc_radix_hit_count(t) == 2
    assert L.orc_radix_ref_count(t, p, 3) == 1
    L.orc_radix_release(t, p, 3); L.orc_radix_release(t, p, 3)    # saturates at 0
    assert L.orc_radix_ref_count(t, p, 3) == 0
    L.orc_radix_delete(t)
    t = L.orc_radix_new()
    _insert(L, t, [1, 2], [10, 20])
    _insert(L, t, [3, 4], [30, 40])
    _lookup(L, t, [3, 4])
    a, p = _u32([3, 4])
    L.orc_radix_release(t, p, 2)
    freed = (C.c_size_t * 4)()
    n = L.orc_radix_evict_lru(t, freed, 4)
    assert n == 1 and freed[0] == 20      # leaf of the least recently used branch
    L.orc_radix_delete(t)


# --- engine/src/kv_cache.rs:1686-1787, 2083-2110 -----------------------------------
def _pt_store(L, t, toks, blocks, seq_len, salt=None):
    a, p = _u32(toks)
    b, q = _u32(blocks)
    L.orc_pt_store(t, p, len(toks), salt, q, len(blocks), seq_len)


def _pt_probe(L, t, toks, salt=None):
    a, p = _u32(toks)
    out = (C.c_uint32 * 64)()
    n = C.c_size_t(0)
    m = L.orc_pt_probe(t, p, len(toks), salt, out, 64, C.byref(n))
    return m, list(out[: n.value])


def test_prefix_table_store_probe_reuse_miss():
    L = lib()
    t = L.orc_pt_new(10)
    _pt_store(L, t, [1, 2, 3], [7], 3)
    assert L.orc_pt_len(t) == 1
    assert _pt_probe(L, t, [1, 2, 3]) == (3, [7])
    assert L.orc_pt_hit_count(t) == 1 and L.orc_pt_tokens_saved(t) == 3
    assert _pt_probe(L, t, [1, 2, 3]) == (3, [7])          # identical reuse
    a, p = _u32([1, 2, 3])
    assert L.orc_pt_ref_count(t, p, 3, None) == 2
    assert _pt_probe(L, t, [99])[0] == 0                    # novel prefix
    assert _pt_probe(L, t, [1, 2, 3, 4, 5]) == (3, [7])     # longest stored prefix wins
    L.orc_pt_release(t, p, 3, None)
    assert L.orc_pt_ref_count(t, p, 3, None) == 2
    for _ in range(5):
        L.orc_pt_release(t, p, 3, None)
    assert L.orc_pt_ref_count(t, p, 3, None) == 0           # saturating
    L.orc_pt_delete(t)


def test_prefix_table_lru_eviction_and_salt():
    L = lib()
    t = L.orc_pt_new(2)
    for i in range(3):
        _pt_store(L, t, [i], [i], 1)
    assert L.orc_pt_len(t) == 2
    assert _pt_probe(L, t, [0])[0] == 0
    L.orc_pt_delete(t)
    t = L.orc_pt_new(10)
    _pt_store(L, t, [1, 2, 3], [1], 1, b"tenant-a")
    _pt_store(L, t, [1, 2, 3], [2], 1, b"tenant-b")
    assert L.orc_pt_len(t) == 2
    assert _pt_probe(L, t, [1, 2, 3], b"tenant-a") == (1, [1])
    assert _pt_probe(L, t, [1, 2, 3], b"tenant-b") == (1, [2])
    assert _pt_probe(L, t, [1, 2, 3], b"tenant-c")[0] == 0
    assert _pt_probe(L, t, [1, 2, 3], None)[0] == 0
    L.orc_pt_delete(t)


def test_prefix_table_referenced_entry_is_not_evicted():
    L = lib()
    t = L.orc_pt_new(1)
    _pt_store(L, t, [1], [1], 1)
    _pt_probe(L, t, [1])                   # ref_count 1
    _pt_store(L, t, [2], [2], 1)           # nothing evictable: table grows past max
    assert L.orc_pt_len(t) == 2
    L.orc_pt_delete(t)


# --- engine/src/gpu_page_pool.rs:224-295 -------------------------------------------
def _ra_alloc(L, a, n):
    s = C.c_size_t(0)
    return s.value if L.orc_ra_alloc(a, n, C.byref(s)) else None


def _ra_runs(L, a):
    st, pg = (C.c_size_t * 128)(), (C.c_size_t * 128)()
    n = L.orc_ra_free_runs(a, st, pg, 128)
    return [(st[i], pg[i]) for i in range(n)]


def test_run_allocator_sequential_free_coalesce():
    L = lib()
    a = L.orc_ra_new(64)
    r0, r1, r2 = _ra_alloc(L, a, 16), _ra_alloc(L, a, 16), _ra_alloc(L, a, 16)
    assert (r0, r1, r2) == (0, 16, 32) and L.orc_ra_free_pages(a) == 16
    L.orc_ra_free(a, r1, 16)
    assert len(_ra_runs(L, a)) == 2
    r3 = _ra_alloc(L, a, 16)
    assert r3 in (16, 48)
    for r in (r0, r2, r3):
        L.orc_ra_free(a, r, 16)
    assert _ra_runs(L, a) == [(0, 64)] and L.orc_ra_allocated_pages(a) == 0
    L.orc_ra_delete(a)


def test_run_allocator_triple_fragmentation_oversize_extend():
    L = lib()
    a = L.orc_ra_new(48)
    r0, r1, r2 = _ra_alloc(L, a, 16), _ra_alloc(L, a, 16), _ra_alloc(L, a, 16)
    L.orc_ra_free(a, r0, 16); L.orc_ra_free(a, r2, 16)
    assert len(_ra_runs(L, a)) == 2
    L.orc_ra_free(a, r1, 16)
    assert _ra_runs(L, a) == [(0, 48)]
    L.orc_ra_delete(a)
    a = L.orc_ra_new(10)
    assert _ra_alloc(L, a, 11) is None and L.orc_ra_free_pages(a) == 10
    L.orc_ra_delete(a)
    a = L.orc_ra_new(32)
    r0, r1 = _ra_alloc(L, a, 8), _ra_alloc(L, a, 8)
    assert not L.orc_ra_try_extend(a, r0, 8, 12)
    L.orc_ra_free(a, r1, 8)
    assert L.orc_ra_try_extend(a, r0, 8, 12)
    assert L.orc_ra_allocated_pages(a) == 12 and L.orc_ra_free_pages(a) == 20
    assert _ra_alloc(L, a, 16) == 12 and L.orc_ra_free_pages(a) == 4
    L.orc_ra_delete(a)


# --- engine/src/cutile_kv_cache.rs:1274-1286 ----------------------------------------
def test_bits_checksum():
    L = lib()
    v = np.array([1.0, -2.0, 0.5, 0.0], dtype=np.float32)
    want = int(v.view(np.uint32).astype(np.uint64).sum())
    assert L.orc_bits_checksum_f32(v.ctypes.data_as(C.POINTER(C.c_float)), 4) == want
    h = v.astype(np.float16).view(np.uint16)
    assert L.orc_bits_checksum_f16_as_f32(h.ctypes.data_as(C.POINTER(C.c_uint16)), 4) == want


# --- frozen scale rule (no reference test pins it) ----------------------------------
def test_block_scale_rule():
    L = lib()
    inv = C.c_float(0)
    assert L.orc_block_scale(0, C.byref(inv)) == 1.0 and inv.value == 1.0          # all-zero block
    assert L.orc_block_scale(0x7C00, C.byref(inv)) == 1.0 and inv.value == 1.0     # Inf in block
    assert L.orc_block_scale(0x7E00, C.byref(inv)) == 1.0 and inv.value == 1.0     # NaN in block
    s = L.orc_block_scale(0x3C00, C.byref(inv))                                    # amax 1.0
    assert s == f32(np.float32(1.0) / np.float32(448.0)) and inv.value == 448.0
    assert L.orc_quantize_scaled(0x3C00, inv.value) == 0x7E                        # amax -> 448
    assert L.orc_quantize_scaled(0xBC00, inv.value) == 0xFE
    s = L.orc_block_scale(0x4900, C.byref(inv))                                    # amax 10.0
    assert s == f32(np.float32(10.0) / np.float32(448.0))
    assert inv.value == f32(np.float32(448.0) / np.float32(10.0))


def test_widening_gather_is_decode_times_scale():
    """The reader's side of the FP8 cache: every byte value decodes as kernels/src/e4m3.rs:27-41
    says (exp 0 -> signed zero, exp 15 through the normal path: 0x7F -> 480.0) and is multiplied
    by the block's scale with one rounding; F16 output rounds that product to nearest even."""
    from tempura_b200 import workloads as W
    w = W.Workload("widen", 1, 2, 128, 16, 4, 4, np.array([16], dtype=np.uint32), src_dtype="e4m3", dst_dtype="f32", seed=1).build_tables()
    src = oracle.HostPool.filled(1, 2, 128, 16, 4, np.uint8, 0, with_scales=True)
    dst32 = oracle.HostPool.filled(1, 2, 128, 16, 4, np.float32, 0x5A)
    dst16 = oracle.HostPool.filled(1, 2, 128, 16, 4, np.uint16, 0x5A)
    sb, db = int(w.src_tables[0][0]), int(w.dst_tables[0][0])
    view = src.block_view(src.k[0])
    view[sb, 0, 0, :] = np.arange(128, dtype=np.uint8)
    view[sb, 0, 1, :] = np.arange(128, 256, dtype=np.uint8)
    src.k_scales[:] = 1.0
    src.v_scales[:] = 1.0
    src.k_scales[0, sb, 0] = np.float32(0.3)
    src.k_scales[0, sb, 1] = np.float32(150.0)
    batch = oracle.make_batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride)
    oracle.handoff(src, dst32, batch, None, "e4m3_f32")
    oracle.handoff(src, dst16, batch, None, "e4m3_f16")
    got32 = dst32.block_view(dst32.k[0])[db, 0]
    got16 = dst16.block_view(dst16.k[0])[db, 0]
    dec = np.array([oracle.e4m3_to_f32(b) for b in range(256)], dtype=np.float32)
    assert dec[0x7F] == 480.0 and dec[0x07] == 0.0 and dec[0x08] == 2.0 ** -6 and dec[0xFE] == -448.0
    want0 = dec[:128] * np.float32(0.3)
    want1 = dec[128:] * np.float32(150.0)
    assert np.array_equal(got32[0].view(np.uint32), want0.view(np.uint32))
    assert np.array_equal(got32[1].view(np.uint32), want1.view(np.uint32))
    with np.errstate(over="ignore"):
        assert np.array_equal(got16[0], want0.astype(np.float16).view(np.uint16))
        assert np.array_equal(got16[1], want1.astype(np.float16).view(np.uint16))     # 480 * 150 overflows to -Inf / Inf
    assert got16[1][0x7E] == 0xFC00                      # -448 * 150 -> -Inf in F16


def test_paged_attention_oracle_against_plain_softmax_and_table_invariance():
    """The oracle's paged decode attention equals a plain numpy softmax attention over the widened
    rows, and does not depend on where the blocks sit (the reference's own property,
    kernels/src/attention.rs test_paged_attention_identity_and_shuffled_match_flash)."""
    rng = np.random.default_rng(5)
    H_, D, bs, nb = 2, 128, 16, 8
    lens = np.array([37, 100], dtype=np.uint32)

    def make(table):
        pool = oracle.HostPool.filled(1, H_, D, bs, 32, np.uint16, 0xA5)
        return pool

    rows = [rng.standard_normal((int(n), 2, H_, D)).astype(np.float16) for n in lens]      # [token][K|V][head][dim]
    outs = []
    for tables in (np.array([[0, 1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12, 13]], dtype=np.uint32),
                   np.array([[30, 2, 17, 9, 4, 25, 11], [1, 29, 3, 14, 8, 20, 6]], dtype=np.uint32)):
        pool = make(tables)
        for s, n in enumerate(lens):
            for t in range(int(n)):
                blk, off = tables[s, t // bs], t % bs
                pool.block_view(pool.k[0])[blk, off] = rows[s][t, 0].view(np.uint16)
                pool.block_view(pool.v[0])[blk, off] = rows[s][t, 1].view(np.uint16)
        q = np.random.default_rng(6).standard_normal((2, 4, D)).astype(np.float32)         # 2 query heads per kv head
        outs.append(oracle.paged_decode_attention(pool, 0, q, tables, lens, 0.125))
    assert np.array_equal(outs[0], outs[1])
    for s, n in enumerate(lens):
        for h in range(4):
            k = rows[s][:, 0, h // 2].astype(np.float64)
            v = rows[s][:, 1, h // 2].astype(np.float64)
            sc = k @ q[s, h].astype(np.float64) * 0.125
            p = np.exp(sc - sc.max())
            want = (p / p.sum()) @ v
            assert np.allclose(outs[0][s, h], want, rtol=1e-4, atol=1e-5)
