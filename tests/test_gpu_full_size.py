"""Benchmark configurations 2-5 at their FULL batch sizes on the GPU.  Two layers of every configuration
(the first and the last, with the full batch and the full tables) are compared with the CPU oracle byte
for byte, scales and untouched fill included; all layers are checked through properties that do not need
the oracle to walk gigabytes: every moved block compared with its source block by an independent torch
gather (bit-exact), untouched memory still holding its fill pattern, prefix blocks unchanged with their
refcounts raised, the two FP8 encoders agreeing byte for byte and the quantize -> widen round trip staying
inside one E4M3 step.  Pools hold the blocks the batch needs (not the benchmark's 65 536-block free list)
so two of them fit beside each other; tables stay shuffled."""
import os

import numpy as np
import pytest

import oracle
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    if torch.cuda.get_device_properties(0).total_memory < 120 * 2 ** 30:
        pytest.skip("full-size cases need a 180 GB device")
    from tempura_b200 import handoff
    return handoff


def fill_source(pool, w, seed):
    import torch
    g = torch.Generator(device=f"cuda:{pool.device}")
    g.manual_seed(seed)
    bs = w.block_size
    used = np.unique(np.concatenate([w.src_tables[q, : (int(w.seq_lens[q]) + bs - 1) // bs] for q in range(len(w.seq_lens))]))
    idx = torch.from_numpy(used.astype(np.int64)).to(f"cuda:{pool.device}")
    for l in range(pool.n_layers):
        for is_v in (False, True):
            vals = torch.randn((len(used), bs, pool.n_kv_heads, pool.head_dim), generator=g, device=idx.device) * w.sigma
            for c in w.outlier_channels:
                vals[..., c] *= w.outlier_gain
            pool.blocks(l, is_v).index_copy_(0, idx, vals.to(torch.float16))


_NP = {N.DTYPE_F32: np.float32, N.DTYPE_F16: np.uint16, N.DTYPE_E4M3: np.uint8}


def snapshot_layers(pool, layers):
    """The named layers of a device pool as a host pool of len(layers) layers (what the oracle reads and writes)."""
    import torch
    torch.cuda.synchronize()
    dt = _NP[pool.dtype]
    grab = lambda t: t.view(torch.uint8).cpu().numpy().view(dt).copy()
    hp = oracle.HostPool(len(layers), pool.n_kv_heads, pool.head_dim, pool.block_size, pool.total_blocks, np.dtype(dt),
                         [grab(pool.k[l]) for l in layers], [grab(pool.v[l]) for l in layers])
    if pool.k_scales is not None:
        hp.k_scales = np.stack([pool.k_scales[l].cpu().numpy() for l in layers])
        hp.v_scales = np.stack([pool.v_scales[l].cpu().numpy() for l in layers])
    return hp


def assert_layers_equal_oracle(pool, hp, layers, what):
    """Every byte of the named device layers (moved rows, ragged tails, untouched fill) and every scale bit pattern."""
    import torch
    torch.cuda.synchronize()
    for i, l in enumerate(layers):
        for name, dev, host in (("K", pool.k[l], hp.k[i]), ("V", pool.v[l], hp.v[i])):
            got = dev.view(torch.uint8).cpu().numpy()
            want = host.view(np.uint8)
            if not np.array_equal(got, want):
                bad = np.flatnonzero(got != want)
                raise AssertionError(f"{what} layer {l} {name}: {bad.size} bytes differ from the oracle, first at {bad[0]}")
        if hp.k_scales is not None:
            for name, dev, host in (("k_scales", pool.k_scales[l], hp.k_scales[i]), ("v_scales", pool.v_scales[l], hp.v_scales[i])):
                assert np.array_equal(dev.cpu().numpy().view(np.uint32), host.view(np.uint32)), f"{what} layer {l} {name} differ from the oracle"


def oracle_on_layers(src, dst_before, w, layers, mode):
    """The oracle's handoff of the FULL batch over the snapshot of the named layers; returns the host destination."""
    hs = snapshot_layers(src, layers)
    oracle.handoff(hs, dst_before, oracle.make_batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens), None, mode,
                   n_threads=os.cpu_count() or 1)
    return dst_before


def moved(w):
    """(src ids, dst ids, valid tokens) of every moved block, in table order."""
    bs = w.block_size
    s, d, v = [], [], []
    for q, length in enumerate(w.seq_lens):
        length = int(length)
        pre = int(w.prefix_lens[q]) // bs if w.prefix_lens is not None else 0
        nb = (length + bs - 1) // bs
        s.append(w.src_tables[q, pre:nb])
        d.append(w.dst_tables[q, pre:nb])
        valid = np.full(nb - pre, bs)
        if nb > pre and length % bs:
            valid[-1] = length % bs
        v.append(valid)
    return np.concatenate(s).astype(np.int64), np.concatenate(d).astype(np.int64), np.concatenate(v).astype(np.int64)


def assert_moved_blocks_equal(src, dst, w, fill_byte):
    import torch
    s, d, valid = moved(w)
    dev = f"cuda:{src.device}"
    s_t, d_t = torch.from_numpy(s).to(dev), torch.from_numpy(d).to(dev)
    mask = (torch.arange(w.block_size, device=dev)[None, :] < torch.from_numpy(valid).to(dev)[:, None])[:, :, None, None]
    fill = int(np.array([fill_byte | (fill_byte << 8)], dtype=np.uint16).view(np.int16)[0])
    for l in range(src.n_layers):
        for is_v in (False, True):
            a = src.blocks(l, is_v).view(torch.int16).index_select(0, s_t)
            b = dst.blocks(l, is_v).view(torch.int16).index_select(0, d_t)
            assert bool(((a == b) | ~mask).all()), f"layer {l} {'V' if is_v else 'K'}: a moved row differs"
            assert bool(((b == fill) | mask).all()), f"layer {l}: rows past a sequence's end were written"


def untouched_blocks_keep_fill(dst, w, fill_byte, extra_used=()):
    import torch
    _, d, _ = moved(w)
    keep = np.ones(dst.total_blocks, dtype=bool)
    keep[d] = False
    keep[list(extra_used)] = False
    idx = torch.from_numpy(np.flatnonzero(keep)).to(f"cuda:{dst.device}")
    if idx.numel() == 0:
        return
    for l in (0, dst.n_layers - 1):
        blk = dst.blocks(l).view(torch.uint8).index_select(0, idx[:64])
        assert bool((blk == fill_byte).all()), "a block outside the batch was written"


def test_config2_full_batch_bit_exact(H):
    import torch
    w = W.llama8b_f16(pool_blocks=4096)
    assert w.tokens_moved == 36748 and w.payload_bytes == 4_816_633_856
    src = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "f16")
    dst = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "f16", fill_byte=0x5A)
    fill_source(src, w, 1)
    want = oracle_on_layers(src, snapshot_layers(dst, (0, 31)), w, (0, 31), "copy")
    for flags, variant in ((0, N.VARIANT_BULK), (N.PLAN_FORCE_VECTOR, N.VARIANT_VECTOR)):
        dst.storage.fill_(0x5A)
        plan = H.Plan(src, dst, H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride), None, flags)
        plan.enqueue()
        torch.cuda.synchronize()
        st = plan.stats()
        assert st.kernel_variant == variant and st.payload_bytes == w.payload_bytes and plan.device_error() == 0
        assert_layers_equal_oracle(dst, want, (0, 31), "config 2")
        assert_moved_blocks_equal(src, dst, w, 0x5A)
        untouched_blocks_keep_fill(dst, w, 0x5A)


def test_config3_full_batch_two_encoders_agree_and_round_trip(H):
    import torch
    w = W.llama8b_fp8(pool_blocks=4096)
    src = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "f16")
    fill_source(src, w, 2)
    batch = H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride)
    pools = []
    for flags, variant in ((0, N.VARIANT_FP8_STAGED), (N.PLAN_FORCE_VECTOR | N.PLAN_INT_QUANTIZER, N.VARIANT_FP8_WARP)):
        dst = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "e4m3", scales=True, fill_byte=0x5A)
        plan = H.Plan(src, dst, batch, None, flags)
        plan.enqueue()
        torch.cuda.synchronize()
        assert plan.stats().kernel_variant == variant and plan.device_error() == 0
        pools.append(dst)
    a, b = pools
    # the oracle's own bytes and scales for the first and the last layer of the full batch
    fresh = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "e4m3", scales=True, fill_byte=0x5A)
    want = oracle_on_layers(src, snapshot_layers(fresh, (0, 31)), w, (0, 31), "f16_e4m3")
    del fresh
    assert_layers_equal_oracle(a, want, (0, 31), "config 3")
    # staged kernel + hardware conversion == register kernel + integer bit-math encoder, every byte and scale
    assert torch.equal(a.storage, b.storage)
    assert torch.equal(a.k_scales.view(torch.int32), b.k_scales.view(torch.int32))
    assert torch.equal(a.v_scales.view(torch.int32), b.v_scales.view(torch.int32))
    # widen back and compare with the source: inside one E4M3 step of the block-scaled value
    back = H.Pool.allocate(0, 32, 8, 128, 16, 4096, "f16", fill_byte=0)
    own = H.Batch(w.seq_lens, w.dst_tables, w.dst_tables, w.table_stride)
    H.Plan(a, back, own, None, N.PLAN_ALLOW_SHARED_DST).enqueue()
    torch.cuda.synchronize()
    s, d, valid = moved(w)
    full = valid == 16
    s_t, d_t = torch.from_numpy(s[full]).cuda(), torch.from_numpy(d[full]).cuda()
    for l in (0, 13, 31):
        x = src.blocks(l).index_select(0, s_t).float()
        y = back.blocks(l).index_select(0, d_t).float()
        amax = x.abs().amax(dim=(1, 3), keepdim=True)
        sc = a.k_scales[l].index_select(0, d_t)                          # [block, head]
        am = amax[:, 0, :, 0]
        # scale = amax / 448 as ONE FP32 division (a tensor divisor: torch turns a scalar one into a reciprocal multiply)
        assert torch.equal(sc, am / torch.full_like(am, 448.0))
        assert bool(((x - y).abs() <= amax / 448 * 16 + amax * 2 ** -10 + 1e-6).all())   # half an E4M3 step + F16 rounding of the result


def test_config4_full_batch_prefix_untouched_and_refcounted(H):
    import torch
    w = W.llama8b_prefix(pool_blocks=16384)              # the prefill side holds every prompt's own prefix blocks
    assert len(w.seq_lens) == 64 and w.shared_prefix_blocks.size == 128
    src = H.Pool.allocate(0, 32, 8, 128, 16, 16384, "f16")
    dst = H.Pool.allocate(0, 32, 8, 128, 16, 16384, "f16", refcounts=True, fill_byte=0x5A)
    fill_source(src, w, 3)
    shared = torch.from_numpy(w.shared_prefix_blocks.astype(np.int64)).cuda()
    g = torch.Generator(device="cuda")
    g.manual_seed(9)
    for l in range(32):                                   # the resident prefix, already on the decode side
        for is_v in (False, True):
            dst.blocks(l, is_v).index_copy_(0, shared, torch.randn((128, 16, 8, 128), generator=g, device="cuda").to(torch.float16))
    r0 = torch.randint(0, 5, (16384,), generator=g, device="cuda", dtype=torch.int32)
    dst.refcounts.copy_(r0)
    before = [dst.blocks(l).index_select(0, shared).clone() for l in (0, 31)]
    want = oracle_on_layers(src, snapshot_layers(dst, (0, 31)), w, (0, 31), "copy")
    plan = H.Plan(src, dst, H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens))
    plan.enqueue()
    plan.refcount_apply(+1)
    torch.cuda.synchronize()
    assert_layers_equal_oracle(dst, want, (0, 31), "config 4")
    st = plan.stats()
    assert st.n_prefix_refs == 64 * 128 and st.n_tokens == w.tokens_moved
    assert_moved_blocks_equal(src, dst, w, 0x5A)
    for l, want in zip((0, 31), before):
        assert torch.equal(dst.blocks(l).index_select(0, shared), want)   # 0 bytes moved into the prefix
    want_rc = r0.clone()
    want_rc[shared] += 64
    assert torch.equal(dst.refcounts, want_rc)
    plan.refcount_apply(-1)
    torch.cuda.synchronize()
    assert torch.equal(dst.refcounts, r0)
    untouched_blocks_keep_fill(dst, w, 0x5A, extra_used=w.shared_prefix_blocks.tolist())


def test_config5_full_batch_and_its_head_shards(H):
    """The whole 42.9 GB batch on one device, then the same batch as the 4 -> 4 layout's shares
    (2 of 8 heads each) into one destination: both land the same bytes."""
    import torch
    w = W.llama70b_f16()
    assert w.payload_bytes == 42_949_672_960
    src = H.Pool.allocate(0, 80, 8, 128, 16, 8192, "f16")
    dst = H.Pool.allocate(0, 80, 8, 128, 16, 8192, "f16", fill_byte=0x5A)
    fill_source(src, w, 4)
    batch = H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride)
    want = oracle_on_layers(src, snapshot_layers(dst, (0, 79)), w, (0, 79), "copy")
    plan = H.Plan(src, dst, batch)
    plan.enqueue()
    torch.cuda.synchronize()
    assert plan.stats().n_chunks == 8192 * 80 * 2 and plan.device_error() == 0
    assert_layers_equal_oracle(dst, want, (0, 79), "config 5")
    assert_moved_blocks_equal(src, dst, w, 0x5A)
    whole = [dst.blocks(l).clone() for l in (0, 79)]
    dst.storage.fill_(0x5A)
    for pr in H.pairing_make(8, 80, 8):
        sh = pr.shard
        H.Plan(src, dst, batch, H.Shard(sh.src_head_begin, sh.dst_head_begin, sh.n_heads, 0, 0, 80)).enqueue()
    torch.cuda.synchronize()
    for l, want in zip((0, 79), whole):
        assert torch.equal(dst.blocks(l), want)


def test_config4_full_batch_from_device_tables(H):
    """The prefix-reuse batch at full size with the work list built on the device: the prefix comes from the device
    index, the suffix pages from the device allocator, and the same properties hold as for the host-built plan."""
    import torch
    w = W.llama8b_prefix(pool_blocks=16384)
    n, bs, pre = len(w.seq_lens), 16, 2048
    src = H.Pool.allocate(0, 32, 8, 128, 16, 16384, "f16")
    dst = H.Pool.allocate(0, 32, 8, 128, 16, 16384, "f16", refcounts=True, fill_byte=0x5A)
    fill_source(src, w, 5)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).cuda()
    rng = np.random.default_rng(6)
    system = rng.integers(0, 32000, size=pre)
    tok = np.zeros((n, int(w.seq_lens.max())), dtype=np.int32)
    for q, m in enumerate(w.seq_lens):
        tok[q, :pre] = system
        tok[q, pre:int(m)] = rng.integers(0, 32000, size=int(m) - pre)
    index, alloc = H.PrefixIndex(0, 1 << 16, bs), H.DevicePageAllocator(0, 16384)
    pre_tab = torch.zeros((1, pre // bs), dtype=torch.int32, device="cuda")
    alloc.allocate(pre_tab, i32([pre // bs]))                      # pages 0..127 hold the resident prefix
    index.insert(i32(system[None, :]), i32([pre]), pre_tab)
    lens, src_tables = i32(w.seq_lens), i32(w.src_tables.reshape(n, -1))
    matched, pages = index.lookup(i32(tok), lens)
    dst_tables = torch.zeros_like(src_tables)
    k = min(pages.shape[1], dst_tables.shape[1])
    dst_tables[:, :k] = pages[:, :k]
    need = ((lens + (bs - 1)) // bs - matched).to(torch.int32)
    alloc.allocate(dst_tables, need, matched)
    plan = H.Plan.with_capacity(src, dst, int(need.sum().item()) + 64)
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    plan.enqueue_device_tables(lens, src_tables, dst_tables, (matched * bs).to(torch.int32), apply_refcounts=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(alloc.status.item()) == 0 and matched.tolist() == [128] * n
    w.dst_tables = dst_tables.cpu().numpy().astype(np.uint32)      # what the device chose, for the property checks
    assert_moved_blocks_equal(src, dst, w, 0x5A)
    shared = torch.arange(128, device="cuda")
    assert bool((dst.refcounts[shared] == n).all()) and int(dst.refcounts.sum()) == 128 * n
    assert bool((dst.blocks(0).index_select(0, shared).view(torch.uint8) == 0x5A).all())      # nothing moved into the prefix
    used = np.unique(w.dst_tables[np.arange(w.dst_tables.shape[1])[None, :] < ((w.seq_lens[:, None] + 15) // 16)])
    assert used.size == 128 + int(need.sum().item())               # every suffix block got its own page
    assert alloc.available() == 16384 - used.size
