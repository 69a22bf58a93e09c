"""Two-GPU parity: the prefill GPU's kernel stores straight into the decode GPU's pool
over NVLink (one process, peer access).  Skipped on a single-GPU box."""
import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, device_batch, host_pools, oracle_batch, to_device_pool
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tempura_b200 import handoff
    handoff.init([0, 1])
    return handoff


def _run(H, w, mode, shard=None, oshard=None, dst_heads=None, flags=0):
    import torch
    hs, hd = host_pools(w, dst_heads=dst_heads)
    src = to_device_pool(hs, w.src_dtype, device=0)
    dst = to_device_pool(hd, w.dst_dtype, device=1)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:1")
    oracle.handoff(hs, hd, oracle_batch(w), oshard, mode)
    plan = H.Plan(src, dst, device_batch(w), shard, flags)
    with torch.cuda.device(0):
        plan.enqueue(torch.cuda.current_stream(0), done_flag=flag.data_ptr(), flag_value=9)
    H.flag_wait_host(1, flag.data_ptr(), 9, 10_000_000)      # decode side sees the flag ...
    with torch.cuda.device(1):
        assert_pool_equals_host(dst, hd, f"peer {w.name}")    # ... and every byte behind it
    st = plan.stats()
    assert st.peer == 1
    return plan


def test_peer_f16_copy_uses_register_stores(H):
    w = W.Workload("peer-f16", 3, 8, 128, 16, 256, 256, W.lengths(6, 40, 300, 50, 7), seed=50).build_tables()
    plan = _run(H, w, "copy")
    assert plan.stats().kernel_variant == 1          # peer destinations never take the bulk-copy path


def test_peer_f16_copy_32_byte_stores(H):
    import torch
    w = W.Workload("peer-f16-wide", 3, 8, 128, 16, 256, 256, W.lengths(6, 40, 300, 52, 7), seed=52).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16", device=0), to_device_pool(hd, "f16", device=1)
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    plan = H.Plan(src, dst, device_batch(w))
    plan.tune_vector(32, 8, 0)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:1")
    with torch.cuda.device(0):
        plan.enqueue(torch.cuda.current_stream(0), done_flag=flag.data_ptr(), flag_value=3)
    H.flag_wait_host(1, flag.data_ptr(), 3, 10_000_000)
    with torch.cuda.device(1):
        assert_pool_equals_host(dst, hd, "peer 32-byte stores")


@pytest.mark.parametrize("tune", [None, (16, 8, 0), (32, 4, 0)])
def test_peer_pull_kernel_on_the_decode_gpu_loads_over_nvlink(H, tune):
    """TKV_PLAN_PULL: the kernel runs on the destination pool's GPU, fetches the source blocks with ordinary loads over
    the peer mapping and stores locally; the flag it publishes is local to the receiver.  Same bytes as the oracle,
    ragged tails and untouched fill included; the source pool is not written."""
    import torch
    w = W.Workload("peer-pull", 3, 8, 128, 16, 256, 256, W.lengths(6, 40, 300, 53, 7), seed=53).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16", device=0), to_device_pool(hd, "f16", device=1)
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    plan = H.Plan(src, dst, device_batch(w), None, N.PLAN_PULL)
    if tune:
        plan.tune_vector(*tune)
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    with torch.cuda.device(1):
        plan.enqueue(torch.cuda.current_stream(1), done_flag=flag.data_ptr(), flag_value=4)
    H.flag_wait_host(1, flag.data_ptr(), 4, 10_000_000)
    with torch.cuda.device(1):
        assert_pool_equals_host(dst, hd, "peer pull")
    with torch.cuda.device(0):
        assert_pool_equals_host(src, hs, "peer pull (source untouched)")
    assert plan.stats().peer == 1 and plan.stats().kernel_variant == (N.VARIANT_VECTOR if tune and tune[0] == 16 else N.VARIANT_WIDE)
    # a pull cannot use the bulk-copy pipelines (they would load a peer's memory with the bulk engine) nor cast
    with pytest.raises(N.TkvError):
        H.Plan(src, dst, device_batch(w), None, N.PLAN_PULL | N.PLAN_FORCE_BULK)


def test_peer_bulk_refused(H):
    import torch
    w = W.Workload("peer-bulk", 1, 8, 128, 16, 32, 32, np.array([20], dtype=np.uint32), seed=51).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16", device=0), to_device_pool(hd, "f16", device=1)
    plan = H.Plan(src, dst, device_batch(w), None, N.PLAN_FORCE_BULK)
    with pytest.raises(N.TkvError):
        plan.enqueue(torch.cuda.current_stream(0))


def test_peer_bulk_stores_opt_in(H):
    """With TKV_PLAN_PEER_BULK_STORES the shared-memory pipelines store into the peer pool
    with bulk copies; same bytes as the register path."""
    w = W.Workload("peer-bulk-f16", 3, 8, 128, 16, 256, 256, W.lengths(6, 40, 300, 54, 7), seed=54).build_tables()
    plan = _run(H, w, "copy", flags=N.PLAN_PEER_BULK_STORES)
    assert plan.stats().kernel_variant == 2 and plan.device_error() == 0
    w = W.Workload("peer-bulk-fp8", 2, 8, 128, 16, 256, 256, W.lengths(5, 30, 200, 55, 7), dst_dtype="e4m3",
                   outlier_channels=(9,), outlier_gain=20.0, seed=55).build_tables()
    plan = _run(H, w, "f16_e4m3", flags=N.PLAN_PEER_BULK_STORES)
    assert plan.stats().kernel_variant == 6 and plan.device_error() == 0


def test_peer_fp8_scaled_cast_before_the_wire(H):
    w = W.Workload("peer-fp8", 2, 8, 128, 16, 256, 256, W.lengths(5, 30, 200, 52, 7), dst_dtype="e4m3",
                   outlier_channels=(9,), outlier_gain=20.0, seed=52).build_tables()
    plan = _run(H, w, "f16_e4m3")
    st = plan.stats()
    assert st.bytes_written < st.bytes_read          # half the payload (+ scales) crosses NVLink


def test_peer_head_shard_pair(H):
    """One pair of the 4 -> 4 layout: source holds 8 heads, this pair's decode pool its 2."""
    w = W.Workload("peer-shard", 4, 8, 128, 16, 128, 128, np.full(5, 70, dtype=np.uint32), seed=53).build_tables()
    _run(H, w, "copy", shard=H.Shard(2, 0, 2, 0, 0, 4), oshard=oracle.OrcShard(2, 0, 2, 0, 0, 4), dst_heads=2)


def test_peer_handoff_from_device_tables(H):
    """The work list built on the prefill GPU from tables in its memory, the stores going to the decode GPU."""
    import torch
    w = W.Workload("peer-dt", 2, 8, 128, 16, 256, 256, W.lengths(6, 20, 280, 56, 7), seed=56).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16", device=0), to_device_pool(hd, "f16", device=1)
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    n = len(w.seq_lens)
    to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).to("cuda:0")
    plan = H.Plan.with_capacity(src, dst, 200)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda:0")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:1")
    with torch.cuda.device(0):
        plan.enqueue_device_tables(to_dev(w.seq_lens), to_dev(w.src_tables.reshape(n, -1)), to_dev(w.dst_tables.reshape(n, -1)),
                                   status=status, done_flag=flag.data_ptr(), flag_value=3)
    H.flag_wait_host(1, flag.data_ptr(), 3, 10_000_000)
    assert int(status.item()) == 0 and plan.stats().peer == 1
    with torch.cuda.device(1):
        assert_pool_equals_host(dst, hd, "peer device tables")


def test_peer_admission_on_the_decode_gpu_handoff_from_the_prefill_gpu(H):
    """Two GPUs: the decode GPU resolves the prefix, places the pages and counts the references in its own memory;
    the prefill GPU's handoff builds its work list from those tables over NVLink and stores into the decode pool."""
    import torch
    from oracle.prefix_oracle import PageStackOracle
    rng = np.random.default_rng(57)
    bs, n, total = 16, 5, 256
    system = rng.integers(0, 32000, size=48).tolist()                # 3 blocks resident on the decode side
    lens = rng.integers(60, 150, size=n)
    prompts = [system + rng.integers(0, 32000, size=int(m) - 48).tolist() for m in lens]
    w = W.Workload("peer-admit", 2, 8, 128, 16, total, total, lens.astype(np.uint32), seed=57).build_tables()
    stride = w.table_stride
    hs, hd = host_pools(w)
    src = to_device_pool(hs, "f16", device=0)
    dst = to_device_pool(hd, "f16", device=1, refcounts=np.zeros(total, dtype=np.int32))
    d1 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).to("cuda:1")
    d0 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).to("cuda:0")
    tok = np.zeros((n, int(lens.max())), dtype=np.int32)
    for q, p in enumerate(prompts):
        tok[q, :len(p)] = p
    with torch.cuda.device(1):
        alloc, ix = H.DevicePageAllocator(1, total), H.PrefixIndex(1, 2048, bs)
        pre_tab = torch.full((1, 3), -1, dtype=torch.int32, device="cuda:1")
        alloc.allocate(pre_tab, d1([3]))
        ix.insert(d1([system]), d1([48]), pre_tab)
        lens1 = d1(lens)
        dst_tables = torch.full((n, stride), -1, dtype=torch.int32, device="cuda:1")
        matched, _ = ix.lookup(d1(tok), lens1, out_pages=dst_tables)
        alloc.allocate(dst_tables, first=matched, seq_lens=lens1, block_size=bs)
        H.refcount_apply_device_tables(dst, dst_tables, matched, +1)
        ready = torch.cuda.Event()
        ready.record()
    plan = H.Plan.with_capacity(src, dst, n * stride)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda:0")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:1")
    with torch.cuda.device(0):
        s0 = torch.cuda.current_stream(0)
        s0.wait_event(ready)                                          # the tables are complete before the prefill GPU reads them
        plan.enqueue_device_tables(d0(lens), d0(w.src_tables.reshape(n, -1)), dst_tables, prefix_blocks=matched, status=status,
                                   done_flag=flag.data_ptr(), flag_value=11)
    H.flag_wait_host(1, flag.data_ptr(), 11, 10_000_000)
    assert int(status.item()) == 0 and int(alloc.status.item()) == 0 and matched.tolist() == [3] * n
    ref = PageStackOracle(total)
    resident = ref.batch_allocate([3])[0]
    fresh = ref.batch_allocate([(int(m) + bs - 1) // bs - 3 for m in lens])
    want = np.zeros((n, stride), dtype=np.uint32)
    for q in range(n):
        want[q, :3] = resident
        want[q, 3:3 + len(fresh[q])] = fresh[q]
    got = dst_tables.cpu().numpy()
    for q in range(n):
        nb = (int(lens[q]) + bs - 1) // bs
        assert got[q, :nb].tolist() == want[q, :nb].tolist()
    w.dst_tables, w.prefix_lens = want, np.full(n, 48, dtype=np.uint32)
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    with torch.cuda.device(1):
        assert_pool_equals_host(dst, hd, "peer admission")
        rc = np.zeros(total, dtype=np.int32)
        rc[resident] = n
        assert np.array_equal(dst.refcounts.cpu().numpy(), rc)
