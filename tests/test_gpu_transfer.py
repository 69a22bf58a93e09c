"""GPU parity tests of the two halves of the handoff against a contiguous transfer buffer:
to_transfer (KvCache::to_transfer / PagedKvCache::k_contiguous, engine/src/kv_cache.rs:
402-417,1032-1060) and from_transfer (KvCache::from_transfer / append_kv, :419-431,986-1004),
called through the C ABI and compared with the oracle's gather and scatter loops byte for
byte.  The buffer lives in device memory or in pinned host memory (the swap tier)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, device_batch, host_pools, oracle_batch, to_device_pool
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu
FILL = 0xEE


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    return handoff


def workload(n_layers=3, n_seqs=5, lo=1, hi=200, pool=128, seed=3, heads=8, dim=128, **kw):
    return W.Workload("xfer", n_layers, heads, dim, 16, pool, pool, W.lengths(n_seqs, lo, hi, seed, 7), seed=seed,
                      **kw).build_tables()


def moved_blocks(w):
    bs = w.block_size
    pre = w.prefix_lens if w.prefix_lens is not None else np.zeros(len(w.seq_lens), dtype=np.uint32)
    return [(int(l) + bs - 1) // bs - int(p) // bs for l, p in zip(w.seq_lens, pre)]


def expected_buffer(w, hs, head_begin=0, n_heads=None, layer_begin=0, n_layers=None):
    """The oracle's per-sequence contiguous gather, laid into the buffer's planes; bytes the
    gather does not produce (rows past a sequence's end in its last block) keep FILL."""
    n_heads = n_heads or hs.n_kv_heads
    n_layers = n_layers or hs.n_layers
    L = oracle.lib()
    bs, D = w.block_size, w.head_dim
    es = hs.dtype.itemsize
    nb = moved_blocks(w)
    total = sum(nb)
    row = n_heads * D * es
    buf = np.full((n_layers, 2, total * bs * row), FILL, dtype=np.uint8)
    stride = hs.n_kv_heads * D
    for l in range(n_layers):
        for kv, arrs in enumerate((hs.k, hs.v)):
            at = 0
            for q, length in enumerate(w.seq_lens):
                length = int(length)
                pre = int(w.prefix_lens[q]) if w.prefix_lens is not None else 0
                out = np.empty(length * stride, dtype=hs.dtype)
                tab = np.ascontiguousarray(w.src_tables[q])
                L.orc_paged_gather(arrs[layer_begin + l].ctypes.data, tab.ctypes.data_as(C.POINTER(C.c_uint32)), bs, stride, es,
                                   length, out.ctypes.data)
                rows = out.reshape(length, hs.n_kv_heads, D)[pre:, head_begin:head_begin + n_heads, :]
                rows = np.ascontiguousarray(rows).view(np.uint8).reshape(-1)
                buf[l, kv, at * bs * row: at * bs * row + rows.size] = rows
                at += nb[q]
    return buf, total


@pytest.mark.parametrize("where", ["device", "host"])
def test_to_transfer_matches_oracle_gather(H, where):
    import torch
    w = workload()
    hs, _ = host_pools(w)
    ds = to_device_pool(hs, "f16")
    want, total = expected_buffer(w, hs)
    x = H.Transfer.allocate(w.n_layers, 8, 128, 16, total, "f16", host=(where == "host"), fill_byte=FILL)
    batch = device_batch(w)
    assert H.batch_blocks(batch, 16) == total
    plan = H.Plan.to_transfer(ds, x, batch)
    plan.enqueue()
    torch.cuda.synchronize()
    got = x.data.cpu().numpy()[: want.size].reshape(want.shape)
    assert np.array_equal(got, want)
    assert plan.stats().kernel_variant == (N.VARIANT_BULK if where == "device" else N.VARIANT_VECTOR)
    assert_pool_equals_host(ds, hs, "source untouched")


@pytest.mark.parametrize("where", ["device", "host", "host-bulk", "host-staged"])
def test_from_transfer_matches_oracle_scatter(H, where):
    import torch
    w = workload(seed=4)
    _, hd = host_pools(w)
    L = oracle.lib()
    bs, D, stride = 16, 128, 8 * 128
    nb = moved_blocks(w)
    total = sum(nb)
    x = H.Transfer.allocate(w.n_layers, 8, 128, 16, total, "f16", host=where.startswith("host"), fill_byte=FILL)
    planes = np.full((w.n_layers, 2, total * bs * stride), 0, dtype=np.uint16)
    for l in range(w.n_layers):
        for kv, arrs in enumerate((hd.k, hd.v)):
            at = 0
            for q, length in enumerate(w.seq_lens):
                length = int(length)
                rows = oracle.gen_normal_f16(length * stride, 9, 100 * l + 10 * kv + q)
                planes[l, kv, at * bs * stride: at * bs * stride + rows.size] = rows
                tab = np.ascontiguousarray(w.dst_tables[q])
                L.orc_paged_scatter(arrs[l].ctypes.data, tab.ctypes.data_as(C.POINTER(C.c_uint32)), bs, stride, 2, 0, length,
                                    rows.ctypes.data)
                at += nb[q]
    x.data[: planes.nbytes].copy_(torch.from_numpy(planes.view(np.uint8).reshape(-1)))
    dd = to_device_pool(host_pools(w)[1], "f16")
    # "host-bulk": the bulk-copy ring reading the pinned buffer (measured equal to the register kernel over PCIe)
    # "host-staged": the copy engine brings one layer at a time into two device buffers of the plan, the kernels read those
    flags = {"host-bulk": N.PLAN_FORCE_BULK, "host-staged": N.PLAN_STAGE_HOST}.get(where, 0)
    plan = H.Plan.from_transfer(x, dd, device_batch(w), None, flags)
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    for gen in (1, 2):                                    # twice: the staging buffers and their events are reused
        plan.enqueue(done_flag=flag.data_ptr(), flag_value=gen)
        H.flag_wait_host(0, flag.data_ptr(), gen, 10_000_000)
    torch.cuda.synchronize()
    assert plan.stats().kernel_variant == (N.VARIANT_VECTOR if where == "host" else N.VARIANT_BULK) and plan.device_error() == 0
    assert_pool_equals_host(dd, hd, "from_transfer")


def test_round_trip_equals_direct_handoff_with_prefix_and_shard(H):
    """to_transfer then from_transfer of a head + layer shard of a prefix batch lands exactly
    what the one-kernel handoff (and the oracle) lands."""
    import torch
    suf = W.lengths(6, 5, 90, 2, 11)
    w = W.Workload("xfer-prefix", 4, 8, 128, 16, 256, 256, (suf + np.uint32(64)).astype(np.uint32),
                   prefix_lens=np.full(6, 64, dtype=np.uint32), seed=2).build_tables()
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    osh = oracle.OrcShard(2, 2, 4, 1, 1, 3)
    oracle.handoff(hs, hd, oracle_batch(w), osh, "copy")
    total = sum(moved_blocks(w))
    x = H.Transfer.allocate(3, 4, 128, 16, total, "f16", fill_byte=FILL)
    sh = H.Shard(2, 2, 4, 1, 1, 3)
    batch = device_batch(w)
    H.Plan.to_transfer(ds, x, batch, sh).enqueue()
    H.Plan.from_transfer(x, dd, batch, sh).enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "round trip")
    want, _ = expected_buffer(w, hs, head_begin=2, n_heads=4, layer_begin=1, n_layers=3)
    got = x.data.cpu().numpy()[: want.size].reshape(want.shape)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("where", ["device", "host"])
def test_fp8_cast_before_the_wire_then_scatter_equals_direct_fp8_handoff(H, where):
    """F16 pool -> E4M3 buffer with scales -> E4M3 pool with scales: bytes and scales equal
    the oracle's direct F16 -> E4M3 handoff."""
    import torch
    w = workload(n_layers=2, seed=6, dst_dtype="e4m3", outlier_channels=(5,), outlier_gain=20.0)
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "e4m3")
    oracle.handoff(hs, hd, oracle_batch(w), None, "f16_e4m3")
    total = sum(moved_blocks(w))
    x = H.Transfer.allocate(2, 8, 128, 16, total, "e4m3", host=(where == "host"), scales=True, fill_byte=FILL)
    batch = device_batch(w)
    H.Plan.to_transfer(ds, x, batch).enqueue()
    p2 = H.Plan.from_transfer(x, dd, batch)
    p2.enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "fp8 via transfer buffer")
    assert p2.stats().kernel_variant == N.VARIANT_VECTOR
    sc = x.scales.cpu().numpy()
    assert np.all(sc[:, :, :total, :] > 0)


def test_f32_transfer_into_f16_pool(H):
    """The reference's own transfer is F32 and its destination may be F16
    (engine/src/kv_cache.rs:209-221): F32 buffer -> F16 pool with round to nearest even."""
    import torch
    w = workload(n_layers=2, n_seqs=3, hi=70, seed=8, heads=2, dim=64, src_dtype="f32", dst_dtype="f16")
    hs, hd = host_pools(w)
    oracle.handoff(hs, hd, oracle_batch(w), None, "f32_f16")
    # build the F32 buffer from the source pool with the GPU gather, then scatter with the cast
    ds = to_device_pool(hs, "f32")
    dd = to_device_pool(host_pools(w)[1], "f16")
    total = sum(moved_blocks(w))
    x = H.Transfer.allocate(2, 2, 64, 16, total, "f32", fill_byte=0)
    batch = device_batch(w)
    H.Plan.to_transfer(ds, x, batch).enqueue()
    H.Plan.from_transfer(x, dd, batch).enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "f32 transfer -> f16 pool")


def test_transfer_plan_validation(H):
    w = workload(n_layers=2, n_seqs=2, hi=40)
    hs, _ = host_pools(w)
    ds = to_device_pool(hs, "f16")
    total = sum(moved_blocks(w))
    small = H.Transfer.allocate(2, 8, 128, 16, max(total - 1, 0), "f16")
    with pytest.raises(N.TkvError) as e:
        H.Plan.to_transfer(ds, small, device_batch(w))
    assert e.value.code == N.ERR_DIMENSION_MISMATCH
    bad = H.Transfer.allocate(2, 8, 128, 16, total, "f32")
    with pytest.raises(N.TkvError) as e:
        H.Plan.to_transfer(ds, bad, device_batch(w))     # F16 pool -> F32 buffer is not a supported pair
    assert e.value.code == N.ERR_INVALID_CONFIG
    # an update with a batch that outgrows the buffer is refused and the plan stays usable
    ok = H.Transfer.allocate(2, 8, 128, 16, total, "f16")
    plan = H.Plan.to_transfer(ds, ok, device_batch(w))
    w2 = workload(n_layers=2, n_seqs=4, lo=100, hi=200, seed=5)
    with pytest.raises(N.TkvError):
        plan.update(device_batch(w2))
    plan.update(device_batch(w))
    plan.enqueue()
    import torch
    torch.cuda.synchronize()


@pytest.mark.parametrize("dst_dtype", ["f16", "e4m3"])
def test_staged_host_buffer_follows_plan_updates_and_casts(H, dst_dtype):
    """TKV_PLAN_STAGE_HOST over several layers (both device buffers are reused), an F16 host buffer into an F16 pool and into
    an E4M3 + scales pool, then a plan update to a larger batch (the staging buffers grow): every byte and scale equal to
    the oracle's handoff from a pool that holds the same rows."""
    import torch
    for seed, n_seqs in ((11, 3), (12, 7)):               # the second batch is larger than the one the plan was made for
        w = workload(n_layers=5, n_seqs=n_seqs, seed=seed, dst_dtype=dst_dtype, outlier_channels=(5,), outlier_gain=20.0)
        hs, hd = host_pools(w)
        ds = to_device_pool(hs, "f16")
        total = sum(moved_blocks(w))
        x = H.Transfer.allocate(5, 8, 128, 16, total, "f16", host=True, fill_byte=FILL)
        H.Plan.to_transfer(ds, x, device_batch(w)).enqueue()           # the host buffer: this batch's rows in transfer layout
        torch.cuda.synchronize()
        dd = to_device_pool(hd, dst_dtype)
        oracle.handoff(hs, hd, oracle_batch(w), None, "copy" if dst_dtype == "f16" else "f16_e4m3")
        if seed == 11:
            plan = H.Plan.from_transfer(x, dd, device_batch(w), None, N.PLAN_STAGE_HOST)
            first = (x, dd)
        else:
            # same plan object cannot change its pools: make a plan for the small batch over these pools, then update it
            small = workload(n_layers=5, n_seqs=3, seed=11, dst_dtype=dst_dtype, outlier_channels=(5,), outlier_gain=20.0)
            plan = H.Plan.from_transfer(x, dd, device_batch(small), None, N.PLAN_STAGE_HOST)
            plan.update(device_batch(w))
        plan.enqueue()
        torch.cuda.synchronize()
        assert plan.device_error() == 0
        assert_pool_equals_host(dd, hd, f"staged host buffer -> {dst_dtype} pool, {n_seqs} sequences")
    with pytest.raises(N.TkvError):                       # only for host buffers that a from_transfer plan reads
        H.Plan(ds, dd, device_batch(w), None, N.PLAN_STAGE_HOST)
