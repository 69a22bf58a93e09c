"""GPU parity tests: the CUDA handoff, called through the C ABI, against the CPU oracle
on the same seeded inputs.  Bit-exact everywhere (byte, index and FP8 work; the FP8
scale is compared as FP32 bit patterns)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from helpers import (assert_pool_equals_host, device_batch, host_pools, mode_of, oracle_batch, to_device_pool)
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    return handoff


def run_case(H, w, shard=None, oshard=None, flags=0, src_heads=None, dst_heads=None, src_layers=None,
             dst_layers=None, table_layer_stride=0, scales=None, refcounts=None):
    import torch
    hs, hd = host_pools(w, src_heads, dst_heads, src_layers, dst_layers, scales)
    ds = to_device_pool(hs, w.src_dtype)
    dd = to_device_pool(hd, w.dst_dtype, refcounts=refcounts)
    oracle.handoff(hs, hd, oracle_batch(w, table_layer_stride), oshard, mode_of(w))
    plan = H.Plan(ds, dd, device_batch(w, table_layer_stride), shard, flags)
    plan.enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, w.name)
    assert_pool_equals_host(ds, hs, w.name + " (source untouched)")
    return plan, ds, dd, hs, hd


def small(w_fn, **kw):
    """A workload with the full shape but fewer layers/blocks so the oracle finishes fast."""
    w = w_fn(**kw)
    return w


def reduced_8b(n_layers=3, n_seqs=6, lo=40, hi=300, pool=256, seed=0, **kw):
    w = W.Workload("8b-reduced", n_layers, 8, 128, 16, pool, pool, W.lengths(n_seqs, lo, hi, seed, 7), seed=seed, **kw)
    return w.build_tables()


# ---- config 1: TinyLlama shape, full size -------------------------------------------
def test_config1_tinyllama_full_size(H):
    w = W.tinyllama_cpu()
    plan, *_ = run_case(H, w)
    st = plan.stats()
    assert st.payload_bytes == 11_534_336 and st.n_blocks == 32 and st.n_chunks == 32 * 22 * 2
    assert st.bytes_read + st.bytes_written == 23_068_672


# ---- config 2 shape: F16 -> F16, ragged lengths ---------------------------------------
@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("flags,variant", [(0, 2), (N.PLAN_FORCE_VECTOR, 1)])
def test_config2_shape_f16_copy(H, seed, flags, variant):
    plan, *_ = run_case(H, reduced_8b(seed=seed), flags=flags)
    assert plan.stats().kernel_variant == variant     # 2 = bulk-copy ring, 1 = register copy


@pytest.mark.parametrize("unroll,hint", [(4, 0), (8, 1), (16, 2)])
def test_config2_shape_f16_copy_32_byte_accesses(H, unroll, hint):
    """The 32-byte register kernel (the peer path's store shape), here on one GPU: same bytes, ragged tails included."""
    import torch
    w = reduced_8b(seed=2)
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    plan = H.Plan(ds, dd, device_batch(w), None, N.PLAN_FORCE_VECTOR)
    plan.tune_vector(32, unroll, hint)
    plan.enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, f"32-byte copy unroll {unroll} hint {hint}")
    assert plan.stats().kernel_variant == N.VARIANT_WIDE
    # two kv heads per pool (one pair's share of a batch split over four pairs): 8 KiB chunks, several per pass
    w = W.Workload("two-heads", 3, 2, 128, 16, 256, 256, W.lengths(7, 1, 300, 5, 3), seed=6).build_tables()
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    oracle.handoff(hs, hd, oracle_batch(w), None, "copy")
    plan = H.Plan(ds, dd, device_batch(w), None, N.PLAN_FORCE_VECTOR)
    plan.tune_vector(32, unroll, hint)
    plan.enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, f"32-byte copy of 8 KiB chunks, unroll {unroll}")
    assert plan.stats().kernel_variant == N.VARIANT_WIDE


def test_config2_lengths_exact_multiple_and_single_token(H):
    w = W.Workload("edge-lens", 2, 8, 128, 16, 64, 64, np.array([16, 1, 17, 32, 15], dtype=np.uint32), seed=3).build_tables()
    run_case(H, w)


# ---- config 3 shape: F16 -> E4M3 + scales ----------------------------------------------
@pytest.mark.parametrize("flags,variant", [(0, 6), (N.PLAN_INT_QUANTIZER, 6), (N.PLAN_FORCE_VECTOR, 3),
                                           (N.PLAN_FORCE_VECTOR | N.PLAN_INT_QUANTIZER, 3), (N.PLAN_FORCE_BULK, 6)])
def test_config3_shape_fp8_scaled(H, flags, variant):
    w = reduced_8b(dst_dtype="e4m3", outlier_channels=(5, 77), outlier_gain=20.0, seed=2)
    plan, *_ = run_case(H, w, flags=flags)
    # 6: shared-memory staged kernel (default for whole rows); 3: warp-per-(block, head) register kernel
    assert plan.stats().kernel_variant == variant and plan.device_error() == 0


@pytest.mark.parametrize("tune", [(2, 0), (2, 1), (4, 1), (8, 1)])
def test_fp8_staged_ring_depths_and_completion_flag(H, tune):
    import torch
    w = reduced_8b(n_layers=2, n_seqs=9, lo=1, hi=200, dst_dtype="e4m3", outlier_channels=(9,), outlier_gain=20.0, seed=21)
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "e4m3")
    oracle.handoff(hs, hd, oracle_batch(w), None, "f16_e4m3")
    plan = H.Plan(ds, dd, device_batch(w), None, N.PLAN_FORCE_BULK)
    plan.tune_bulk(tune[0], tune[1], 32768)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    for gen in (1, 2):                                   # twice: the completion counter re-arms itself
        plan.enqueue(done_flag=flag.data_ptr(), flag_value=gen)
        H.flag_wait_host(0, flag.data_ptr(), gen, 5_000_000)
    assert plan.stats().kernel_variant == 6 and plan.device_error() == 0
    assert_pool_equals_host(dd, hd, f"staged fp8 {tune}")


def test_fp8_staged_into_strided_destination_rows(H):
    """Whole source rows, destination pool with more heads than the source: the staged
    kernel leaves through plain stores instead of one bulk store."""
    w = W.Workload("fp8-staged-strided", 2, 4, 128, 16, 64, 64, np.array([40, 33, 7], dtype=np.uint32), dst_dtype="e4m3", seed=22).build_tables()
    sh, osh = H.Shard(0, 2, 4, 0, 0, 2), oracle.OrcShard(0, 2, 4, 0, 0, 2)
    p, *_ = run_case(H, w, shard=sh, oshard=osh, dst_heads=8)
    assert p.stats().kernel_variant == 6


def test_config3_fp8_special_blocks(H):
    """All-zero block, Inf and NaN blocks (unscaled fallback), tiny subnormal-only block,
    exact ties: the classes the reference's GPU probe lists
    (tools/bench-gpu/src/bench_decode_ops.rs:686-701), pushed through the scaled path."""
    import torch
    w = W.Workload("fp8-special", 1, 8, 128, 16, 16, 16, np.array([16 * 6 + 5], dtype=np.uint32), dst_dtype="e4m3", seed=4).build_tables()
    hs, hd = host_pools(w)
    blk = hs.block_view(hs.k[0])
    t = w.src_tables[0]
    blk[t[0]] = 0                                            # all zero -> scale 1
    blk[t[1], 3, 2, 7] = 0x7C00                              # +Inf in head 2
    blk[t[1], 4, 3, 9] = 0xFC00                              # -Inf in head 3
    blk[t[2], 0, 0, 0] = 0x7E00                              # NaN in head 0
    blk[t[2], 1, 1, 1] = 0xFFFF                              # negative NaN in head 1
    blk[t[3]] = 0x0001                                       # smallest subnormal everywhere
    blk[t[3], 0, 0, 0] = 0x8003
    adv = np.array([0.0, -0.0, 1.0, -1.0, 1.0625, 1.1875, 15.5, 0.015625, 0.01, 0.001, -0.001, 448.0, -448.0, 449.0,
                    65504.0, -65504.0, 6.1035156e-5, 5.96e-8, 0.5, 0.49999997], dtype=np.float32).astype(np.float16)
    blk[t[4], 0, 4, : len(adv)] = adv.view(np.uint16)
    hv = hs.block_view(hs.v[0])
    hv[t[5], :, 5, :] = np.float16(448.0).view(np.uint16)    # amax exactly 448 -> inv exactly 1
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "e4m3")
    oracle.handoff(hs, hd, oracle_batch(w), None, "f16_e4m3")
    for flags in (0, N.PLAN_INT_QUANTIZER, N.PLAN_FORCE_VECTOR, N.PLAN_FORCE_VECTOR | N.PLAN_INT_QUANTIZER):
        dd.k[0].fill_(0x5A)                                  # every variant starts from an unwritten pool
        dd.v[0].fill_(0x5A)
        dd.k_scales.fill_(-123.0)
        dd.v_scales.fill_(-123.0)
        plan = H.Plan(ds, dd, device_batch(w), None, flags)
        plan.enqueue()
        torch.cuda.synchronize()
        assert_pool_equals_host(dd, hd, f"special flags={flags}")
    d = w.dst_tables[0]
    assert hd.k_scales[0, d[0], 0] == 1.0 and hd.k_scales[0, d[1], 2] == 1.0 and hd.k_scales[0, d[2], 1] == 1.0


def test_fp8_unscaled_destination(H):
    """An E4M3 pool without scale arrays takes raw e4m3 bytes, as the reference's pools do
    (engine/src/cutile_kv_cache.rs:1593-1595)."""
    w = reduced_8b(n_layers=2, dst_dtype="e4m3", seed=5)
    run_case(H, w, scales=False)


# ---- config 4 shape: shared resident prefix, suffix-only move, refcounts -----------------
def test_config4_shape_prefix_suffix_and_refcounts(H):
    import torch
    n = 12
    suf = W.lengths(n, 20, 90, 0, 11)
    w = W.Workload("prefix-reduced", 2, 8, 128, 16, 512, 512, (suf + np.uint32(128)).astype(np.uint32),
                   prefix_lens=np.full(n, 128, dtype=np.uint32), seed=6).build_tables()
    r0 = (W.mix64(9, 9, np.arange(512, dtype=np.uint64)) % np.uint64(5)).astype(np.uint32)
    plan, ds, dd, hs, hd = run_case(H, w, refcounts=r0)
    st = plan.stats()
    assert st.n_prefix_refs == n * 8 and st.n_tokens == int(suf.sum())
    want = r0.copy()
    oracle.refcount_apply(want, oracle_batch(w), 16, +1)
    plan.refcount_apply(+1)
    torch.cuda.synchronize()
    got = dd.refcounts.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, want)
    assert all(got[b] == r0[b] + n for b in w.shared_prefix_blocks)
    # release: saturating decrement, driven past zero on purpose
    for _ in range(n + 6):
        oracle.refcount_apply(want, oracle_batch(w), 16, -1)
        plan.refcount_apply(-1)
    torch.cuda.synchronize()
    got = dd.refcounts.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, want) and got[w.shared_prefix_blocks].max() == 0
    assert_pool_equals_host(dd, hd, "prefix blocks unchanged after refcounting")


# ---- config 5 shape: head / layer shards -------------------------------------------------
def test_config5_shape_head_shard_into_local_pool(H):
    """Prefill pool holds all 8 heads; the decode pool of this pair holds its 2 local heads."""
    w = W.Workload("70b-reduced", 4, 8, 128, 16, 128, 128, np.full(5, 70, dtype=np.uint32), seed=7).build_tables()
    sh = H.Shard(4, 0, 2, 0, 0, 4)
    osh = oracle.OrcShard(4, 0, 2, 0, 0, 4)
    run_case(H, w, shard=sh, oshard=osh, dst_heads=2)


def test_config5_shape_local_to_local_and_layer_shard(H):
    w = W.Workload("70b-local", 6, 2, 128, 16, 128, 128, np.full(4, 64, dtype=np.uint32), seed=8).build_tables()
    run_case(H, w)                                           # both pools hold the pair's 2 heads
    sh, osh = H.Shard(0, 0, 2, 2, 1, 3), oracle.OrcShard(0, 0, 2, 2, 1, 3)
    run_case(H, w, shard=sh, oshard=osh, dst_layers=5)       # layers [2,5) -> [1,4)
    sh, osh = H.Shard(1, 0, 1, 0, 0, 6), oracle.OrcShard(1, 0, 1, 0, 0, 6)
    run_case(H, w, shard=sh, oshard=osh)                     # strided rows on both sides


def test_fp8_with_head_shard(H):
    w = W.Workload("fp8-shard", 2, 8, 128, 16, 64, 64, np.array([40, 33], dtype=np.uint32), dst_dtype="e4m3", seed=9).build_tables()
    sh, osh = H.Shard(2, 1, 4, 0, 0, 2), oracle.OrcShard(2, 1, 4, 0, 0, 2)
    run_case(H, w, shard=sh, oshard=osh, dst_heads=6)


# ---- other shapes the reference's CPU types use --------------------------------------------
def test_tiny_test_shape_f32_and_casts(H):
    """ModelConfig::tiny_test geometry (4 kv heads, head_dim 16; engine/src/config.rs:262-301)
    with the CPU cache's block size 4 (engine/src/kv_cache.rs:1918)."""
    base = dict(n_layers=2, n_kv_heads=4, head_dim=16, block_size=4, src_blocks=32, dst_blocks=32)
    lens = np.array([10, 3, 4], dtype=np.uint32)
    run_case(H, W.Workload("tiny-f32", seq_lens=lens, src_dtype="f32", dst_dtype="f32", seed=10, **base).build_tables())
    run_case(H, W.Workload("tiny-f32-f16", seq_lens=lens, src_dtype="f32", dst_dtype="f16", seed=11, **base).build_tables())
    p, *_ = run_case(H, W.Workload("tiny-f16-e4m3", seq_lens=lens, src_dtype="f16", dst_dtype="e4m3", seed=12, **base).build_tables())
    assert p.stats().kernel_variant == 4                     # generic FP8 kernel


def test_head_dim_64_and_256_fp8(H):
    for d, seed in ((64, 13), (256, 14)):
        w = W.Workload(f"d{d}", 2, 4, d, 16, 64, 64, np.array([37, 16, 5], dtype=np.uint32), dst_dtype="e4m3", seed=seed).build_tables()
        p, *_ = run_case(H, w)
        assert p.stats().kernel_variant == 6
        p, *_ = run_case(H, w, flags=N.PLAN_FORCE_VECTOR)
        assert p.stats().kernel_variant == 3


def test_per_layer_block_tables(H):
    """PagedKvCache keeps one table per layer drawing from one allocator
    (engine/src/kv_cache.rs:925-936,975-984)."""
    L, n, stride = 3, 2, 4
    lens = np.array([50, 20], dtype=np.uint32)
    w = W.Workload("per-layer", L, 8, 128, 16, 64, 64, lens, seed=15).build_tables()
    src_free, dst_free = W.permutation(64, 1, 1), W.permutation(64, 2, 2)
    src = np.zeros((L, n, stride), dtype=np.uint32)
    dst = np.zeros((L, n, stride), dtype=np.uint32)
    k = 0
    for l in range(L):
        for q in range(n):
            nb = (int(lens[q]) + 15) // 16
            src[l, q, :nb] = src_free[k:k + nb]
            dst[l, q, :nb] = dst_free[k:k + nb]
            k += nb
    w.src_tables, w.dst_tables, w.table_stride = src.reshape(L * n, stride), dst.reshape(L * n, stride), stride
    # host_pools seeds the blocks named by the first n rows only; seed all of them
    w2 = W.Workload("per-layer-all", L, 8, 128, 16, 64, 64, np.tile(lens, L), seed=15)
    w2.src_tables, w2.dst_tables, w2.table_stride = w.src_tables, w.dst_tables, stride
    import torch
    hs, hd = host_pools(w2)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    oracle.handoff(hs, hd, oracle.make_batch(lens, w.src_tables, w.dst_tables, stride, None, n * stride))
    H.Plan(ds, dd, H.Batch(lens, w.src_tables, w.dst_tables, stride, None, n * stride)).enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "per-layer tables")


def test_empty_batch_and_zero_suffix(H):
    import torch
    w = reduced_8b(n_layers=1, n_seqs=2)
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    empty = H.Batch(np.zeros(0, np.uint32), np.zeros((0, 1), np.uint32), np.zeros((0, 1), np.uint32), 1)
    p = H.Plan(ds, dd, empty)
    p.enqueue(done_flag=flag.data_ptr(), flag_value=7)
    torch.cuda.synchronize()
    assert int(flag.item()) == 7 and p.stats().n_chunks == 0
    # every token already resident: nothing moves
    b = H.Batch(np.array([32]), np.array([[1, 2]]), np.array([[3, 4]]), 2, np.array([32]))
    p = H.Plan(ds, dd, b)
    p.enqueue()
    torch.cuda.synchronize()
    assert p.stats().n_chunks == 0 and p.stats().n_prefix_refs == 2
    assert_pool_equals_host(dd, hd, "nothing written")


def test_plan_update_reuses_plan(H):
    import torch
    w1, w2 = reduced_8b(n_layers=2, seed=20), reduced_8b(n_layers=2, seed=21, n_seqs=9)
    hs, hd = host_pools(w1)
    hs2, _ = host_pools(w2)
    for l in range(2):                                       # both batches' source blocks in one pool
        m = hs2.k[l] != np.uint16(0xA5A5)
        hs.k[l][m] = hs2.k[l][m]
        m = hs2.v[l] != np.uint16(0xA5A5)
        hs.v[l][m] = hs2.v[l][m]
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    plan = H.Plan(ds, dd, device_batch(w1))
    plan.enqueue()
    oracle.handoff(hs, hd, oracle_batch(w1))
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "first batch")
    plan.update(device_batch(w2))
    plan.enqueue()
    oracle.handoff(hs, hd, oracle_batch(w2))
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, hd, "second batch through the same plan")


# ---- bulk-copy variant of the same-dtype handoff ---------------------------------------------
@pytest.mark.parametrize("tune", [(3, 2, 32768), (2, 1, 32768), (8, 1, 8192), (4, 4, 4096)])
def test_bulk_variant_parity(H, tune):
    import torch
    cases = [W.tinyllama_cpu(),                                              # 8 KiB chunks
             reduced_8b(seed=40),                                            # 32 KiB chunks, ragged tails
             W.Workload("bs32", 2, 8, 128, 32, 64, 64, np.array([100, 31, 64], dtype=np.uint32), seed=41).build_tables()]  # 64 KiB chunks
    for w in cases:
        hs, hd = host_pools(w)
        ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
        oracle.handoff(hs, hd, oracle_batch(w))
        plan = H.Plan(ds, dd, device_batch(w), None, N.PLAN_FORCE_BULK)
        plan.tune_bulk(*tune)
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        plan.enqueue(done_flag=flag.data_ptr(), flag_value=5)
        H.flag_wait_host(0, flag.data_ptr(), 5, 5_000_000)
        assert plan.stats().kernel_variant == 2 and plan.device_error() == 0
        assert_pool_equals_host(dd, hd, f"bulk {w.name} {tune}")


@pytest.mark.parametrize("flag_mode", [0, 1, 2])
@pytest.mark.parametrize("inline_list", [0, 1, 2])
@pytest.mark.parametrize("where", ["device", "host"])
def test_small_handoff_choices_change_no_byte(H, flag_mode, inline_list, where):
    """Who publishes the flag (the kernel's last CTA or a stream-ordered write behind the kernel) and where the work list
    sits (device memory or the kernel's parameter block) are latency choices: same bytes, same flag, plan updates included."""
    import torch
    flag = torch.zeros(1, dtype=torch.int32, device="cuda") if where == "device" else torch.zeros(1, dtype=torch.int32).pin_memory()
    w = W.tinyllama_cpu()
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    oracle.handoff(hs, hd, oracle_batch(w))
    plan = H.Plan(ds, dd, device_batch(w))
    plan.tune_small(flag_mode, inline_list)
    for gen in (1, 2, 3):
        plan.enqueue(done_flag=flag.data_ptr(), flag_value=gen)
        H.flag_wait_host(0, flag.data_ptr(), gen, 5_000_000)
        if gen == 1:
            assert_pool_equals_host(dd, hd, f"small flag {flag_mode} inline {inline_list}")
    assert plan.device_error() == 0
    # a new batch through the same plan: the parameter-block list must follow the update, not the first batch
    w2 = W.Workload("small-update", w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.src_blocks, w.dst_blocks,
                    np.array([33, 7], dtype=np.uint32), seed=78).build_tables()
    hs2, hd2 = host_pools(w2)
    ds2, dd2 = to_device_pool(hs2, "f16"), to_device_pool(hd2, "f16")
    oracle.handoff(hs2, hd2, oracle_batch(w2))
    plan2 = H.Plan(ds2, dd2, device_batch(w))             # created for the first batch ...
    plan2.tune_small(flag_mode, inline_list)
    plan2.enqueue(done_flag=flag.data_ptr(), flag_value=4)
    H.flag_wait_host(0, flag.data_ptr(), 4, 5_000_000)
    for arrs in (dd2.k, dd2.v):                           # ... whose rows are wiped again before the update
        for l in range(w2.n_layers):
            arrs[l].view(torch.uint8).fill_(0x5A)
    plan2.update(device_batch(w2))
    plan2.enqueue(done_flag=flag.data_ptr(), flag_value=5)
    H.flag_wait_host(0, flag.data_ptr(), 5, 5_000_000)
    assert_pool_equals_host(dd2, hd2, "after update")
    with pytest.raises(N.TkvError):
        plan.tune_small(3, 0)


def test_bulk_variant_refuses_strided_rows(H):
    w = W.Workload("bulk-shard", 2, 8, 128, 16, 64, 64, np.array([40], dtype=np.uint32), seed=42).build_tables()
    hs, hd = host_pools(w, dst_heads=2)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    plan = H.Plan(ds, dd, device_batch(w), H.Shard(4, 0, 2, 0, 0, 2), N.PLAN_FORCE_BULK)
    with pytest.raises(N.TkvError) as e:
        plan.enqueue()
    assert e.value.code == N.ERR_INVALID_CONFIG


# ---- completion flag and bounded waits ------------------------------------------------------
def test_done_flag_and_bounded_waits(H):
    import torch
    w = reduced_8b(n_layers=2)
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    flag = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.full((1,), 99, dtype=torch.int32, device="cuda")
    plan = H.Plan(ds, dd, device_batch(w))
    side = torch.cuda.Stream()
    for gen in (1, 2, 3):                                     # the counter re-arms itself
        plan.enqueue(done_flag=flag.data_ptr(), flag_value=gen)
        H.flag_wait_host(0, flag.data_ptr(), gen, 5_000_000)
        H.flag_wait_enqueue(side, flag.data_ptr(), gen, 1 << 20, status.data_ptr())
        side.synchronize()
        assert int(status.item()) == 0
    oracle.handoff(hs, hd, oracle_batch(w))
    assert_pool_equals_host(dd, hd, "after flagged handoffs")
    # a waiter that polls late: the flag (3) has passed the generation it waits for (1, 2)
    for late in (1, 2):
        H.flag_wait_host(0, flag.data_ptr(), late, 20_000)
        H.flag_wait_enqueue(side, flag.data_ptr(), late, 2000, status.data_ptr())
        side.synchronize()
        assert int(status.item()) == 0
    # a flag in page-locked host memory: the kernel's release store lands there, the host reads it in place
    hflag = torch.zeros(1, dtype=torch.int32).pin_memory()
    plan.enqueue(done_flag=hflag.data_ptr(), flag_value=11)
    H.flag_wait_host(0, hflag.data_ptr(), 11, 5_000_000)
    assert int(hflag[0]) == 11
    with pytest.raises(N.TkvError) as e:
        H.flag_wait_host(0, hflag.data_ptr(), 12, 20_000)
    assert e.value.code == N.ERR_TIMEOUT
    # a flag nothing sets: both waits give up and say so; the context stays usable
    with pytest.raises(N.TkvError) as e:
        H.flag_wait_host(0, flag[1:].data_ptr(), 5, 20_000)
    assert e.value.code == N.ERR_TIMEOUT
    H.flag_wait_enqueue(side, flag[1:].data_ptr(), 5, 2000, status.data_ptr())
    side.synchronize()
    assert int(status.item()) == N.ERR_TIMEOUT
    assert int((flag[0] + 1).item()) == 4                     # device still answers


# ---- element casts and checksum -----------------------------------------------------------------
def test_fast_fp8_encoder_equals_integer_port_on_every_f32(H):
    assert H.selfcheck_e4m3(0) == 0


def test_scaled_fast_path_equals_integer_port_for_every_amax_and_value(H):
    assert H.selfcheck_scaled_quant() == 0


def test_cast_kernels_against_oracle(H):
    import torch
    L = oracle.lib()
    rng = np.random.default_rng(0)
    adv = np.array([0.0, -0.0, 1.0, -1.0, 1.0625, 1.1875, 15.5, 0.015625, 0.01, 0.001, -0.001, 448.0, -448.0, 449.0,
                    1e30, -1e30, np.inf, -np.inf, np.nan, 65505.0, 65520.0, 6.1035156e-5, 5.96e-8, 2.98e-8, 1e-8, -1e-8,
                    0.5, 0.49999997], dtype=np.float32)
    x = np.concatenate([adv, rng.standard_normal(4000).astype(np.float32) * 30,
                        rng.integers(0, 2**32, 4000, dtype=np.uint64).astype(np.uint32).view(np.float32)])
    xd = torch.from_numpy(x).cuda()
    out8 = torch.zeros(len(x), dtype=torch.uint8, device="cuda")
    H.cast(xd, out8, "f32", "e4m3")
    want8 = np.array([L.orc_f32_to_e4m3(C.c_float(v)) for v in x], dtype=np.uint8)
    assert np.array_equal(out8.cpu().numpy(), want8)
    out16 = torch.zeros(len(x), dtype=torch.float16, device="cuda")
    H.cast(xd, out16, "f32", "f16")
    want16 = np.array([L.orc_f32_to_f16(C.c_float(v)) for v in x], dtype=np.uint16)
    got16 = out16.view(torch.int16).cpu().numpy().view(np.uint16)
    nan = np.isnan(x)
    assert np.array_equal(got16[~nan], want16[~nan])
    assert np.all(got16[nan] == 0x7FFF)      # GPU NaN convention (bench_decode_ops.rs:711-726)
    # decode direction: every byte
    b = torch.arange(256, dtype=torch.uint8, device="cuda")
    f = torch.zeros(256, dtype=torch.float32, device="cuda")
    H.cast(b, f, "e4m3", "f32")
    want = np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    assert np.array_equal(f.cpu().numpy().view(np.uint32), want.view(np.uint32))
    h = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.float16)
    f = torch.zeros(65536, dtype=torch.float32, device="cuda")
    H.cast(h, f, "f16", "f32")
    wantf = np.array([L.orc_f16_to_f32(i) for i in range(65536)], dtype=np.float32)
    keep = ~np.isnan(wantf)
    assert np.array_equal(f.cpu().numpy().view(np.uint32)[keep], wantf.view(np.uint32)[keep])


def test_bits_checksum_matches_oracle(H):
    import torch
    L = oracle.lib()
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100_003) * 3).astype(np.float32)
    assert H.bits_checksum(torch.from_numpy(x).cuda(), "f32") == L.orc_bits_checksum_f32(x.ctypes.data_as(C.POINTER(C.c_float)), len(x))
    h = x.astype(np.float16).view(np.uint16)
    hd = torch.from_numpy(h.view(np.int16)).cuda().view(torch.float16)
    assert H.bits_checksum(hd, "f16") == L.orc_bits_checksum_f16_as_f32(h.ctypes.data_as(C.POINTER(C.c_uint16)), len(h))
    b = rng.integers(0, 256, 50_001, dtype=np.uint8)
    assert H.bits_checksum(torch.from_numpy(b).cuda(), "e4m3") == L.orc_bits_checksum_e4m3_as_f32(b.ctypes.data_as(C.POINTER(C.c_uint8)), len(b))


# ---- the reader's side of the FP8 cache: gather + widen ----------------------------------------
@pytest.mark.parametrize("dst_dtype", ["f16", "f32"])
@pytest.mark.parametrize("scaled", [True, False])
def test_e4m3_pool_widens_into_f16_and_f32(H, dst_dtype, scaled):
    """Every E4M3 byte value (NaN encodings and subnormal encodings included) under seeded
    per-block scales, against the oracle's decode * scale (kernels/src/e4m3.rs:27-41)."""
    import torch
    w = W.Workload("dequant", 2, 8, 128, 16, 64, 64, np.array([70, 16, 33, 1], dtype=np.uint32), src_dtype="e4m3",
                   dst_dtype=dst_dtype, seed=31).build_tables()
    hs, hd = host_pools(w, scales=False)
    if scaled:
        rng = np.random.default_rng(7)
        hs.k_scales = (rng.random((2, 64, 8), dtype=np.float32) * 4 + 1e-3).astype(np.float32)
        hs.v_scales = (rng.random((2, 64, 8), dtype=np.float32) * 200 + 1e-3).astype(np.float32)   # some products overflow F16
    hs.block_view(hs.k[0])[w.src_tables[0][0], 0, 0, :] = np.arange(128, dtype=np.uint8)           # all byte values
    hs.block_view(hs.k[0])[w.src_tables[0][0], 1, 0, :] = np.arange(128, 256, dtype=np.uint8)
    ds, dd = to_device_pool(hs, "e4m3"), to_device_pool(hd, dst_dtype)
    oracle.handoff(hs, hd, oracle_batch(w), None, mode_of(w))
    plan = H.Plan(ds, dd, device_batch(w))
    plan.enqueue()
    torch.cuda.synchronize()
    assert plan.stats().kernel_variant == N.VARIANT_DEQUANT
    assert_pool_equals_host(dd, hd, f"dequant {dst_dtype} scaled={scaled}")


def test_e4m3_widen_head_shard_and_odd_geometry(H):
    w = W.Workload("dequant-shard", 2, 8, 128, 16, 64, 64, np.array([40, 33], dtype=np.uint32), src_dtype="e4m3", dst_dtype="f16",
                   seed=32).build_tables()
    hs, hd = host_pools(w, dst_heads=4, scales=False)
    hs.k_scales = np.full((2, 64, 8), 0.5, dtype=np.float32)
    hs.v_scales = np.linspace(0.1, 3.0, 2 * 64 * 8, dtype=np.float32).reshape(2, 64, 8)
    ds, dd = to_device_pool(hs, "e4m3"), to_device_pool(hd, "f16")
    osh, sh = oracle.OrcShard(3, 1, 3, 0, 0, 2), H.Shard(3, 1, 3, 0, 0, 2)
    oracle.handoff(hs, hd, oracle_batch(w), osh, "e4m3_f16")
    H.Plan(ds, dd, device_batch(w), sh).enqueue()
    assert_pool_equals_host(dd, hd, "dequant shard")
    # head_dim 24, block 4: the byte-wide form
    w = W.Workload("dequant-odd", 1, 3, 24, 4, 16, 16, np.array([9, 4], dtype=np.uint32), src_dtype="e4m3", dst_dtype="f32", seed=33).build_tables()
    hs, hd = host_pools(w, scales=False)
    hs.k_scales = np.full((1, 16, 3), 2.0, dtype=np.float32)
    hs.v_scales = np.full((1, 16, 3), 0.25, dtype=np.float32)
    ds, dd = to_device_pool(hs, "e4m3"), to_device_pool(hd, "f32")
    oracle.handoff(hs, hd, oracle_batch(w), None, "e4m3_f32")
    H.Plan(ds, dd, device_batch(w)).enqueue()
    assert_pool_equals_host(dd, hd, "dequant odd")


def test_quantize_then_widen_stays_within_one_e4m3_step(H):
    """Property at the full config-3 shape of one layer: F16 -> scaled E4M3 -> F16 comes back within
    2^-4 relative error of the block's absmax-scaled value (3 mantissa bits), exactly where the scale is 1."""
    import torch
    w = reduced_8b(n_layers=1, n_seqs=4, lo=100, hi=400, pool=256, dst_dtype="e4m3", outlier_channels=(3,), outlier_gain=20.0, seed=34)
    hs, hq = host_pools(w)
    ds, dq = to_device_pool(hs, "f16"), to_device_pool(hq, "e4m3")
    back = H.Pool.allocate(0, 1, 8, 128, 16, 256, "f16", fill_byte=0)
    batch = device_batch(w)
    H.Plan(ds, dq, batch).enqueue()
    own = H.Batch(w.seq_lens, w.dst_tables, w.dst_tables, w.table_stride)
    H.Plan(dq, back, own, None, N.PLAN_ALLOW_SHARED_DST).enqueue()
    torch.cuda.synchronize()
    for q in range(len(w.seq_lens)):
        nfull = int(w.seq_lens[q]) // 16
        s = torch.from_numpy(w.src_tables[q, :nfull].astype(np.int64)).cuda()
        d = torch.from_numpy(w.dst_tables[q, :nfull].astype(np.int64)).cuda()
        x = ds.blocks(0).index_select(0, s).float()
        y = back.blocks(0).index_select(0, d).float()
        amax = x.abs().amax(dim=(1, 3), keepdim=True)
        # an e4m3 step is 2^-3 of the value's binade; after scaling the largest binade is [256, 448]
        assert bool(((x - y).abs() <= amax / 448 * 16 + amax * 2 ** -10 + 1e-6).all())   # half an E4M3 step + F16 rounding of the result
        big = x.abs() >= amax / 448 * 2 ** -6 * 1.01            # not flushed
        rel = ((x - y).abs() / x.abs().clamp_min(1e-9))[big]
        assert float(rel.max()) <= 2 ** -4 + 1e-3


# ---- the reference's own transfer dtype: F32 rows into an F16 (or unscaled E4M3) cache ----------
@pytest.mark.parametrize("dst_dtype", ["f16", "e4m3"])
@pytest.mark.parametrize("flags,variant", [(0, N.VARIANT_CAST_VEC), (N.PLAN_FORCE_VECTOR, N.VARIANT_CAST_GENERIC)])
def test_f32_source_casts_at_the_8b_shape(H, dst_dtype, flags, variant):
    """KvCacheTransfer is F32 (engine/src/kv_cache.rs:514-522) and the cache it lands in may be F16
    (append_kv's cast, :209-221) or the GPU pool's unscaled E4M3 (kernels/src/kv_scatter_write.rs:172-273)."""
    w = reduced_8b(n_layers=2, n_seqs=5, lo=1, hi=150, src_dtype="f32", dst_dtype=dst_dtype, outlier_channels=(11,), outlier_gain=2000.0, seed=71)
    plan, *_ = run_case(H, w, flags=flags, scales=False)     # x2000: values past 448 and past 65504 saturate / overflow as the rules say
    assert plan.stats().kernel_variant == variant


def test_f32_cast_head_shard(H):
    w = W.Workload("f32-shard", 2, 8, 128, 16, 64, 64, np.array([40, 33], dtype=np.uint32), src_dtype="f32", dst_dtype="f16", seed=72).build_tables()
    sh, osh = H.Shard(2, 1, 4, 0, 0, 2), oracle.OrcShard(2, 1, 4, 0, 0, 2)
    p, *_ = run_case(H, w, shard=sh, oshard=osh, dst_heads=6)
    assert p.stats().kernel_variant == N.VARIANT_CAST_VEC
