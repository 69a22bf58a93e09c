"""The allocation-free handoff entry point (tkv_handoff_noalloc), called through the C ABI.

Some callers cannot allocate device memory when a handoff happens: the KV pools of a
serving engine already own nearly all of HBM, and a cudaMalloc in the steady-state loop
stalls every stream of the device.  For them the work list lives in a fixed array inside
the library.  This file checks that entry point against the planned handoff
(tkv_plan_create + tkv_handoff_enqueue) and against the CPU oracle on the same inputs,
byte for byte, on two calls in a row, and that oversized batches are refused.  It is
named to be collected last.
"""
import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, device_batch, host_pools, oracle_batch, to_device_pool
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _pool_bytes(p):
    import torch
    torch.cuda.synchronize()
    return [t.view(torch.uint8).cpu().numpy().copy() for t in list(p.k) + list(p.v)]


def _workload(seed, n_seqs, lo, hi):
    return W.Workload("noalloc", 3, 8, 128, 16, 256, 256, W.lengths(n_seqs, lo, hi, seed, 7), seed=seed).build_tables()


def test_noalloc_matches_planned_handoff_twice_in_a_row():
    import torch
    from tempura_b200 import handoff as H

    # first call: a larger batch; second call: a smaller, different one, so anything the
    # first call left in the shared array would show up as wrong or extra blocks
    for call, (seed, n_seqs, lo, hi) in enumerate([(31, 7, 40, 300), (32, 3, 5, 90)]):
        w = _workload(seed, n_seqs, lo, hi)
        hs, hd = host_pools(w)
        src = to_device_pool(hs, "f16")
        dst_plan = to_device_pool(hd, "f16")
        dst_noalloc = to_device_pool(hd, "f16")
        batch = device_batch(w)

        H.Plan(src, dst_plan, batch).enqueue()
        if call == 1:
            free_before, _ = torch.cuda.mem_get_info()
        H.handoff_noalloc(src, dst_noalloc, batch)
        torch.cuda.synchronize()
        if call == 1:                       # set-up happened on the first call; this one allocates nothing
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before
        want, got = _pool_bytes(dst_plan), _pool_bytes(dst_noalloc)
        for i, (a, b) in enumerate(zip(want, got)):
            assert np.array_equal(a, b), f"call {call}: tensor {i} differs from the planned handoff"
        oracle.handoff(hs, hd, oracle_batch(w), None, "copy")           # and directly against the checker
        assert_pool_equals_host(dst_noalloc, hd, f"no-alloc call {call}")
        assert any((a != 0x5A).any() for a in got)          # something was actually moved


def test_noalloc_head_shard_matches_planned_handoff():
    import torch
    from tempura_b200 import handoff as H

    w = W.Workload("noalloc-shard", 2, 8, 128, 16, 64, 64, np.array([70, 33], dtype=np.uint32), seed=33).build_tables()
    hs, hd = host_pools(w, dst_heads=2)
    src = to_device_pool(hs, "f16")
    a, b = to_device_pool(hd, "f16"), to_device_pool(hd, "f16")
    shard = H.Shard(4, 0, 2, 0, 0, 2)
    H.Plan(src, a, device_batch(w), shard).enqueue()
    H.handoff_noalloc(src, b, device_batch(w), shard)
    torch.cuda.synchronize()
    for x, y in zip(_pool_bytes(a), _pool_bytes(b)):
        assert np.array_equal(x, y)


def test_noalloc_refuses_what_does_not_fit_or_is_invalid():
    from tempura_b200 import handoff as H

    # 1 layer keeps the pools small; 16385 block pairs is one more than the array holds
    n_blocks = 16385
    pool = H.Pool.allocate(0, 1, 1, 16, 16, n_blocks, "f16", fill_byte=None)
    dst = H.Pool.allocate(0, 1, 1, 16, 16, n_blocks, "f16", fill_byte=None)
    ids = np.arange(n_blocks, dtype=np.uint32)[None, :]
    big = H.Batch(np.array([n_blocks * 16]), ids, ids, n_blocks)
    with pytest.raises(N.TkvError) as e:
        H.handoff_noalloc(pool, dst, big)
    assert e.value.code == N.ERR_INVALID_CONFIG and "16384" in e.value.message
    fits = H.Batch(np.array([16384 * 16]), ids[:, :16384], ids[:, :16384], 16384)
    H.handoff_noalloc(pool, dst, fits)                       # exactly the maximum is accepted
    # dtype pairs that need a cast go through a plan, not through this entry point
    e4 = H.Pool.allocate(0, 1, 1, 16, 16, 8, "e4m3", fill_byte=None)
    small = H.Batch(np.array([16]), np.array([[0]]), np.array([[0]]), 1)
    with pytest.raises(N.TkvError) as e:
        H.handoff_noalloc(pool, e4, small)
    assert e.value.code == N.ERR_INVALID_CONFIG
    dup = H.Batch(np.array([16, 16]), np.array([[0], [1]]), np.array([[3], [3]]), 1)
    with pytest.raises(N.TkvError) as e:
        H.handoff_noalloc(pool, dst, dup)
    assert "written twice" in e.value.message
