"""The handoff with its work list built on the device: same bytes as the host-built plan on seeded batches (copy,
FP8 cast, prefix + reference counts), the refusals, and the whole decode-side admission without a host round trip:
prefix index lookup -> page allocator -> device tables -> handoff."""
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
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    handoff.init([0])
    return handoff


def dev_i32(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).cuda()


def run_device_tables(H, w, mode, flags=0, refcounts=False):
    import torch
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, w.src_dtype), to_device_pool(hd, w.dst_dtype)
    oracle.handoff(hs, hd, oracle_batch(w), None, mode)
    pairs = int(((w.seq_lens.astype(np.int64) + 15) // 16).sum())
    plan = H.Plan.with_capacity(src, dst, pairs + 7, flags=flags)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    n = len(w.seq_lens)
    plan.enqueue_device_tables(dev_i32(w.seq_lens), dev_i32(w.src_tables.reshape(n, -1)), dev_i32(w.dst_tables.reshape(n, -1)),
                               dev_i32(w.prefix_lens) if w.prefix_lens is not None else None, apply_refcounts=refcounts, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and plan.device_error() == 0
    assert_pool_equals_host(dst, hd, f"device tables {w.name}")
    return plan, dst


@pytest.mark.parametrize("flags", [0, N.PLAN_FORCE_VECTOR])
def test_copy_matches_oracle(H, flags):
    w = W.Workload("dt-f16", 3, 8, 128, 16, 256, 256, W.lengths(9, 1, 300, 31, 7), seed=31).build_tables()
    plan, _ = run_device_tables(H, w, "copy", flags)
    assert plan.stats().kernel_variant == (N.VARIANT_VECTOR if flags else N.VARIANT_BULK)


@pytest.mark.parametrize("flags", [0, N.PLAN_FORCE_VECTOR])
def test_fp8_scaled_cast_matches_oracle(H, flags):
    w = W.Workload("dt-fp8", 2, 8, 128, 16, 256, 256, W.lengths(7, 5, 260, 32, 7), dst_dtype="e4m3",
                   outlier_channels=(3,), outlier_gain=20.0, seed=32).build_tables()
    run_device_tables(H, w, "f16_e4m3", flags)


def test_prefix_blocks_stay_and_are_counted(H):
    import torch
    suffix = W.lengths(9, 3, 120, 33, 11)
    w = W.Workload("dt-prefix", 2, 8, 128, 16, 1024, 1024, (suffix + np.uint32(48)).astype(np.uint32),
                   prefix_lens=np.full(9, 48, dtype=np.uint32), seed=33).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16"), to_device_pool(hd, "f16", refcounts=np.zeros(1024, dtype=np.int32))
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    plan = H.Plan.with_capacity(src, dst, 200)
    n = len(w.seq_lens)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    plan.enqueue_device_tables(dev_i32(w.seq_lens), dev_i32(w.src_tables.reshape(n, -1)), dev_i32(w.dst_tables.reshape(n, -1)),
                               dev_i32(w.prefix_lens), apply_refcounts=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_pool_equals_host(dst, hd, "device tables prefix")
    want = np.zeros(1024, dtype=np.int32)
    want[w.shared_prefix_blocks] = n
    assert np.array_equal(dst.refcounts.cpu().numpy(), want)


def test_refusals_move_nothing(H):
    import torch
    w = W.Workload("dt-bad", 1, 8, 128, 16, 64, 64, np.array([40, 70], dtype=np.uint32), seed=34).build_tables()
    hs, hd = host_pools(w)
    src, dst = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    before = dst.storage.clone()
    lens, st, dt = dev_i32(w.seq_lens), dev_i32(w.src_tables.reshape(2, -1)), dev_i32(w.dst_tables.reshape(2, -1))
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def expect(code, plan, *args, **kw):
        status.fill_(-1)
        flag.zero_()
        plan.enqueue_device_tables(*args, status=status, done_flag=flag.data_ptr(), flag_value=5, **kw)
        torch.cuda.synchronize()
        assert int(status.item()) == code and torch.equal(dst.storage, before) and int(flag.item()) == 5   # still published

    plan = H.Plan.with_capacity(src, dst, 8)
    small = H.Plan.with_capacity(src, dst, 7)                        # the batch has 3 + 5 = 8 pairs
    expect(N.ERR_DIMENSION_MISMATCH, small, lens, st, dt)
    bad = dt.clone()
    bad[1, 2] = 64                                                   # one id past the pool
    expect(N.ERR_INVALID_CONFIG, plan, lens, st, bad)
    expect(N.ERR_INVALID_CONFIG, plan, lens, st, dt, prefix_lens=dev_i32([8, 0]))     # not a multiple of the block size
    expect(N.ERR_INVALID_CONFIG, plan, lens, st, dt, prefix_lens=dev_i32([48, 0]))    # longer than the sequence
    expect(N.ERR_INVALID_CONFIG, plan, dev_i32([40, 16 * st.shape[1] + 1]), st, dt)   # longer than a table row
    with pytest.raises(N.TkvError):
        plan.enqueue_device_tables(lens, st, dt, apply_refcounts=True)                # the pool has no refcount array
    plan.enqueue_device_tables(lens, st, dt, status=status)          # and the good batch still goes through afterwards
    torch.cuda.synchronize()
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    assert int(status.item()) == 0
    assert_pool_equals_host(dst, hd, "device tables after refusals")


def test_admission_without_a_host_round_trip(H):
    """Decode side, all on the stream: look the prompts up in the device prefix index, take pages for the blocks
    that are not resident from the device allocator, and hand off through the tables they filled.  Checked against
    the host-side answer (RadixTree oracle, page stack oracle, host-built plan through the handoff oracle)."""
    import torch
    from oracle.prefix_oracle import PageStackOracle, RadixOracle
    rng = np.random.default_rng(35)
    bs, n, total = 16, 7, 512
    system = rng.integers(0, 32000, size=64).tolist()                # 4 blocks, already resident on the decode side
    lens = rng.integers(70, 180, size=n)
    prompts = [system + rng.integers(0, 32000, size=int(m) - 64).tolist() for m in lens]
    w = W.Workload("admit", 2, 8, 128, 16, total, total, lens.astype(np.uint32), seed=35).build_tables()
    stride = w.table_stride
    hs, hd = host_pools(w)
    # decode-side state: allocator with the first 4 pages given to the resident prefix, index holding it
    alloc, ref_alloc = H.DevicePageAllocator(0, total), PageStackOracle(total)
    ix, ref_ix = H.PrefixIndex(0, 4096, bs), RadixOracle(bs)
    pre_tab = torch.full((1, stride), -1, dtype=torch.int32, device="cuda")
    alloc.allocate(pre_tab, dev_i32([4]))
    resident = ref_alloc.batch_allocate([4])[0]
    ix.insert(dev_i32([system]), dev_i32([64]), pre_tab[:, :4].contiguous())
    ref_ix.batch_insert([system], [resident])
    # ---- the admission, device only ----
    tok = np.zeros((n, int(lens.max())), dtype=np.int32)
    for q, p in enumerate(prompts):
        tok[q, :len(p)] = p
    lens_t = dev_i32(lens)
    dst_tables = torch.full((n, stride), -1, dtype=torch.int32, device="cuda")
    matched, _ = ix.lookup(dev_i32(tok), lens_t, out_pages=dst_tables)     # matched nodes' pages at the head of each row
    alloc.allocate(dst_tables, first=matched, seq_lens=lens_t, block_size=bs)   # the rest of each row
    hs2, hd2 = host_pools(w)
    src, dst = to_device_pool(hs2, "f16"), to_device_pool(hd2, "f16", refcounts=np.zeros(total, dtype=np.int32))
    plan = H.Plan.with_capacity(src, dst, n * stride)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    plan.enqueue_device_tables(lens_t, dev_i32(w.src_tables.reshape(n, -1)[:, :stride]), dst_tables, prefix_blocks=matched,
                               apply_refcounts=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(alloc.status.item()) == 0
    # ---- the same on the host ----
    want_tables = np.full((n, stride), -1, dtype=np.int64)
    got = ref_ix.batch_lookup(prompts)
    fresh = ref_alloc.batch_allocate([(int(m) + bs - 1) // bs - g[0] for m, g in zip(lens, got)])
    for q in range(n):
        m = got[q][0]
        assert m == 4
        want_tables[q, :m] = got[q][2]
        want_tables[q, m:m + len(fresh[q])] = fresh[q]
    got_tables = dst_tables.cpu().numpy()
    for q in range(n):
        nb = (int(lens[q]) + bs - 1) // bs
        assert got_tables[q, :nb].tolist() == want_tables[q, :nb].tolist()
    w.dst_tables = np.where(want_tables < 0, 0, want_tables).astype(np.uint32)
    w.src_tables = w.src_tables.reshape(n, -1)[:, :stride].copy()
    w.table_stride = stride
    w.prefix_lens = np.full(n, 64, dtype=np.uint32)
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    assert_pool_equals_host(dst, hd, "admission")
    rc = np.zeros(total, dtype=np.int32)
    rc[resident] = n
    assert np.array_equal(dst.refcounts.cpu().numpy(), rc)


def test_more_sequences_than_the_builder_has_threads(H):
    """1 500 short prompts (the builder's scan runs in chunks of 1 024 sequences), some of them empty."""
    rng = np.random.default_rng(36)
    lens = rng.integers(0, 40, size=1500).astype(np.uint32)
    lens[[0, 1023, 1024, 1499]] = [0, 17, 0, 33]
    w = W.Workload("dt-wide", 1, 4, 64, 16, 4096, 4096, lens, seed=36).build_tables()
    run_device_tables(H, w, "copy")


def test_index_and_allocator_edge_cases(H):
    import torch
    ix = H.PrefixIndex(0, 64, 16)
    empty_tok = torch.zeros((3, 20), dtype=torch.int32, device="cuda")
    lens = torch.tensor([0, 15, 16], dtype=torch.int32, device="cuda")          # no whole group, no whole group, exactly one
    ix.insert(empty_tok, lens)
    matched, pages = ix.lookup(empty_tok, lens)
    assert matched.tolist() == [0, 0, 1] and int(pages[2, 0]) == -1               # inserted without a page
    st = ix.stats()
    assert st.live_nodes == 1 and st.hits == 1 and st.tokens_saved == 16
    assert ix.evict_lru(4) == ([], 0)                                             # still referenced by the lookup
    ix.release(empty_tok, lens)
    ix.release(empty_tok, lens)                                                   # a second release does not go below zero
    assert ix.evict_lru(4) == ([], 1)                                             # unlinked; it had no page to report
    with pytest.raises(N.TkvError):
        H.PrefixIndex(0, 100)                                                     # capacity must be a power of two
    alloc = H.DevicePageAllocator(0, 8)
    t = torch.full((2, 4), -1, dtype=torch.int32, device="cuda")
    alloc.allocate(t, torch.tensor([0, 0], dtype=torch.int32, device="cuda"))     # nothing asked for
    assert int(alloc.status.item()) == 0 and alloc.available() == 8 and bool((t == -1).all())
    alloc.allocate(t, torch.tensor([4, 4], dtype=torch.int32, device="cuda"))     # exactly everything
    assert int(alloc.status.item()) == 0 and alloc.available() == 0 and sorted(t.flatten().tolist()) == list(range(8))
    alloc.allocate(t, torch.tensor([1, 0], dtype=torch.int32, device="cuda"))
    assert int(alloc.status.item()) == N.ERR_POOL_EXHAUSTED


def test_refcounts_from_device_tables_up_and_down(H):
    import torch
    dst = H.Pool.allocate(0, 1, 4, 64, 16, 64, "f16", refcounts=True)
    dst.refcounts.zero_()
    tables = dev_i32([[3, 4, 5, 9], [3, 4, 7, 8], [60, 61, 62, 63]])
    pre = dev_i32([2, 3, 0])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    H.refcount_apply_device_tables(dst, tables, pre, +1, status)
    want = np.zeros(64, dtype=np.int32)
    want[[3, 4]] = 2
    want[7] = 1
    assert np.array_equal(dst.refcounts.cpu().numpy(), want) and int(status.item()) == 0
    H.refcount_apply_device_tables(dst, tables, pre, -1)
    H.refcount_apply_device_tables(dst, tables, pre, -1)             # never below zero
    assert int(dst.refcounts.abs().sum()) == 0
    H.refcount_apply_device_tables(dst, dev_i32([[64, 1]]), dev_i32([2]), +1, status)     # id 64 is outside the pool
    assert int(status.item()) == N.ERR_INVALID_CONFIG and int(dst.refcounts[1]) == 1


def test_host_tables_and_device_tables_alternate_on_one_plan(H):
    """The device builder writes its list where the plan's host-built list was uploaded.  A host-table enqueue
    that follows must move the plan's own batch again (the list is uploaded anew, in stream order), and a
    device-table enqueue after that its device batch: both against the oracle, twice round."""
    import torch
    w_host = W.Workload("alt-host", 2, 8, 128, 16, 256, 256, W.lengths(6, 20, 200, 41, 7), seed=41).build_tables()
    w_dev = W.Workload("alt-dev", 2, 8, 128, 16, 256, 256, W.lengths(4, 5, 90, 42, 7), seed=42).build_tables()
    hs, hd0 = host_pools(w_host)
    src = to_device_pool(hs, "f16")
    # the device batch reads the same source pool through its own tables (seeded blocks or the 0xA5 filler alike)
    dst = to_device_pool(hd0, "f16")
    fresh = dst.storage.clone()
    plan = H.Plan(src, dst, device_batch(w_host))
    n = len(w_dev.seq_lens)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    for rnd in range(2):
        for which in ("host", "device"):
            _, hd = host_pools(w_host)                               # the oracle's fresh 0x5A destination
            oracle.handoff(hs, hd, oracle_batch(w_host if which == "host" else w_dev), None, "copy")
            dst.storage.copy_(fresh)
            if which == "host":
                plan.enqueue()
            else:
                plan.enqueue_device_tables(dev_i32(w_dev.seq_lens), dev_i32(w_dev.src_tables.reshape(n, -1)),
                                           dev_i32(w_dev.dst_tables.reshape(n, -1)), status=status)
            torch.cuda.synchronize()
            if which == "device":
                assert int(status.item()) == 0
            assert_pool_equals_host(dst, hd, f"round {rnd} {which} tables")
