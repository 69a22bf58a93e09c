"""The reference's own device-side KV movement (engine/src/cutile_kv_cache.rs): a sequence whose run of pages must grow is
moved to a larger run INSIDE the same pool (try_ensure_capacity, :402-482: copy the live prefix, free the old run), and a
preempted sequence is swapped out to page-locked host memory and later swapped in to a different run, verified
bit-for-bit by a wrapping sum of the values' f32 bit patterns taken before and after (:1256-1268).  Here both go through
the handoff plans; the oracle replays the relocation on the host, the checksum is tkv_bits_checksum (pinned to the
oracle's by test_gpu_handoff.py)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, to_device_pool
from tempura_b200 import _native as N

pytestmark = pytest.mark.gpu

LAYERS, HEADS, DIM, BS, BLOCKS = 3, 8, 128, 16, 64
LIVE = 150                       # live tokens: 9 full pages + 6 rows of the tenth
OLD_BASE, OLD_PAGES = 5, 10
NEW_BASE, NEW_PAGES = 32, 20     # "2x the current run" (:414-417)
ROW = HEADS * DIM


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    return handoff


def seeded_pool(dtype: str, seed: int) -> oracle.HostPool:
    """Every page holds seeded values (the pool is shared: other sequences live around the runs)."""
    np_dt = np.uint16 if dtype == "f16" else np.uint8
    hp = oracle.HostPool.filled(LAYERS, HEADS, DIM, BS, BLOCKS, np_dt, 0, with_scales=dtype == "e4m3")
    n = BLOCKS * BS * ROW
    for l in range(LAYERS):
        for kv, arrs in enumerate((hp.k, hp.v)):
            vals = oracle.gen_normal_f16(n, seed, 2 * l + kv, 1.0)
            if dtype == "f16":
                arrs[l][:] = vals
            else:
                b = (vals >> 7).astype(np.uint8)                         # sign + mixed exponent/mantissa bits
                b[(b & 0x7F) == 0x7F] = 0x7E                             # no NaN codes: their f32 bit pattern is a convention, not data
                arrs[l][:] = b
    if hp.k_scales is not None:
        rng = np.random.default_rng(seed)
        hp.k_scales[:] = rng.uniform(0.01, 3.0, hp.k_scales.shape).astype(np.float32)
        hp.v_scales[:] = rng.uniform(0.01, 3.0, hp.v_scales.shape).astype(np.float32)
    return hp


def run_table(base: int, pages: int) -> np.ndarray:
    return np.arange(base, base + pages, dtype=np.uint32)


def prefix_checksum(H, pool, base: int, dtype: str) -> int:
    """device_prefix_bits_checksum: the live prefix of a run is contiguous in every layer tensor."""
    total = 0
    for l in range(LAYERS):
        for t in (pool.k[l], pool.v[l]):
            total = (total + H.bits_checksum(t.reshape(-1)[base * BS * ROW: base * BS * ROW + LIVE * ROW], dtype)) & (2 ** 64 - 1)
    return total


def live_scales(pool, base: int):
    n = (LIVE + BS - 1) // BS
    return pool.k_scales[:, base:base + n].clone(), pool.v_scales[:, base:base + n].clone()


@pytest.mark.parametrize("dtype", ["f16", "e4m3"])
def test_a_growing_run_is_relocated_inside_its_pool(H, dtype):
    import torch
    hp = seeded_pool(dtype, 41)
    pool = to_device_pool(hp, dtype)
    before = prefix_checksum(H, pool, OLD_BASE, dtype)
    lens = np.array([LIVE], dtype=np.uint32)
    old, new = run_table(OLD_BASE, OLD_PAGES), run_table(NEW_BASE, NEW_PAGES)
    n_live = (LIVE + BS - 1) // BS
    plan = H.Plan(pool, pool, H.Batch(lens, old[:n_live], new[:n_live], n_live), None, N.PLAN_ALLOW_SHARED_DST)
    plan.enqueue()
    torch.cuda.synchronize()
    assert plan.device_error() == 0
    assert prefix_checksum(H, pool, NEW_BASE, dtype) == before            # the live prefix arrived bit for bit
    assert prefix_checksum(H, pool, OLD_BASE, dtype) == before            # ... and the freed run was only read
    if dtype == "e4m3":                                                   # a page's scales move with the page
        ok, ov = live_scales(pool, OLD_BASE)
        nk, nv = live_scales(pool, NEW_BASE)
        assert torch.equal(ok.view(torch.int32), nk.view(torch.int32)) and torch.equal(ov.view(torch.int32), nv.view(torch.int32))
        for s in (hp.k_scales, hp.v_scales):
            s[:, NEW_BASE:NEW_BASE + n_live] = s[:, OLD_BASE:OLD_BASE + n_live]
    # the whole pool against the oracle's replay: the rows past the live prefix in the new run's last page, the rest of the
    # new run and every other sequence's pages are untouched
    oracle.handoff(hp, hp, oracle.make_batch(lens, old[:n_live], new[:n_live], n_live), None, "copy")
    assert_pool_equals_host(pool, hp, "relocated run")
    # a relocation whose runs overlap is refused unless the caller says the destination may be shared -- and the flag does
    # not excuse a sequence longer than its table
    with pytest.raises(N.TkvError):
        H.Plan(pool, pool, H.Batch(np.array([LIVE + 200], dtype=np.uint32), old[:n_live], new[:n_live], n_live), None, N.PLAN_ALLOW_SHARED_DST)


@pytest.mark.parametrize("dtype", ["f16", "e4m3"])
def test_swap_out_then_swap_in_elsewhere_keeps_the_bits_checksum(H, dtype):
    import torch
    hp = seeded_pool(dtype, 43)
    pool = to_device_pool(hp, dtype)
    lens = np.array([LIVE], dtype=np.uint32)
    n_live = (LIVE + BS - 1) // BS
    old, new = run_table(OLD_BASE, OLD_PAGES)[:n_live], run_table(NEW_BASE, NEW_PAGES)[:n_live]
    cs_out = prefix_checksum(H, pool, OLD_BASE, dtype)
    if dtype == "e4m3":
        sk, sv = live_scales(pool, OLD_BASE)
    # swap_out: the live prefix into the page-locked host mirror
    mirror = H.Transfer.allocate(LAYERS, HEADS, DIM, BS, n_live, dtype, host=True, scales=dtype == "e4m3", fill_byte=0xEE)
    out = H.Plan.to_transfer(pool, mirror, H.Batch(lens, old, old, n_live))
    out.enqueue()
    torch.cuda.synchronize()
    assert out.device_error() == 0
    # the mirror's own checksum, taken on the host by the oracle (mirror_bits_checksum)
    L = oracle.lib()
    es = 2 if dtype == "f16" else 1
    planes = mirror.planes(LAYERS, n_live).numpy().reshape(LAYERS, 2, -1)
    fn, ct = (L.orc_bits_checksum_f16_as_f32, C.c_uint16) if dtype == "f16" else (L.orc_bits_checksum_e4m3_as_f32, C.c_uint8)
    cs_mirror = 0
    for l in range(LAYERS):
        for kv in range(2):
            live = np.ascontiguousarray(planes[l, kv, : LIVE * ROW * es]).view(np.uint16 if dtype == "f16" else np.uint8)
            cs_mirror = (cs_mirror + fn(live.ctypes.data_as(C.POINTER(ct)), live.size)) & (2 ** 64 - 1)
    assert cs_mirror == cs_out
    # the pages go to someone else while the sequence is out
    pool.storage.fill_(0x5A)
    if dtype == "e4m3":
        pool.k_scales.fill_(-7.0)
        pool.v_scales.fill_(-7.0)
    assert prefix_checksum(H, pool, OLD_BASE, dtype) != cs_out
    # swap_in: a fresh run elsewhere in the pool
    back = H.Plan.from_transfer(mirror, pool, H.Batch(lens, new, new, n_live))
    back.enqueue()
    torch.cuda.synchronize()
    assert back.device_error() == 0
    assert prefix_checksum(H, pool, NEW_BASE, dtype) == cs_out            # "EXACT"
    if dtype == "e4m3":
        nk, nv = live_scales(pool, NEW_BASE)
        assert torch.equal(sk.view(torch.int32), nk.view(torch.int32)) and torch.equal(sv.view(torch.int32), nv.view(torch.int32))
    # and only the live rows of the new run were written: the oracle's replay onto a wiped pool
    np_dt = np.uint16 if dtype == "f16" else np.uint8
    wiped = oracle.HostPool.filled(LAYERS, HEADS, DIM, BS, BLOCKS, np_dt, 0x5A, with_scales=dtype == "e4m3", scale_fill=-7.0)
    oracle.handoff(hp, wiped, oracle.make_batch(lens, old, new, n_live), None, "copy")
    if dtype == "e4m3":
        for s, d in ((hp.k_scales, wiped.k_scales), (hp.v_scales, wiped.v_scales)):
            d[:, NEW_BASE:NEW_BASE + n_live] = s[:, OLD_BASE:OLD_BASE + n_live]
    assert_pool_equals_host(pool, wiped, "swapped-in run")
