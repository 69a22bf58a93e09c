"""Decode attention over the paged pool (the consumer of the FP8 cache) against the oracle's
restatement of paged_flash_attention (kernels/src/attention.rs:486-590).  Floating point:
the kernel feeds FP16 operands (q, probabilities; K/V are exact in FP16) to FP32-accumulating
tensor-core MMAs, the oracle computes in FP32, so the comparison is by tolerance:
|got - want| <= 4e-3 * max|V[:, d]| + 2e-3 * |want| per output dim d (2^-11 relative on q and on
each probability: about 3e-3 on a score in the worst case, hence on the weights of V)."""
import numpy as np
import pytest

import oracle
from helpers import device_batch, host_pools, oracle_batch, to_device_pool
from tempura_b200 import _native as N
from tempura_b200 import workloads as W

pytestmark = pytest.mark.gpu
ATOL_REL_V, RTOL = 4e-3, 2e-3


@pytest.fixture(scope="module")
def H():
    import torch
    assert torch.cuda.is_available()
    from tempura_b200 import handoff
    return handoff


def close(got, want, vmax):
    err = np.abs(got - want)
    bound = ATOL_REL_V * vmax + RTOL * np.abs(want)
    assert np.isfinite(got).all()
    assert (err <= bound).all(), f"max err {err.max():.3e} at bound {bound.flat[err.argmax()]:.3e}"


def run(H, pool_host, pool_dev, w, n_q_heads, seed, layers=None, flags=0):
    import torch
    rng = np.random.default_rng(seed)
    n = len(w.seq_lens)
    tables = torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda()
    lens = torch.from_numpy(w.seq_lens.astype(np.int64)).to(torch.int32).cuda()
    for layer in (layers if layers is not None else range(pool_host.n_layers)):
        q = rng.standard_normal((n, n_q_heads, 128)).astype(np.float32)
        got = H.decode_attention(pool_dev, layer, torch.from_numpy(q).cuda(), tables, lens, flags=flags).cpu().numpy()
        want = oracle.paged_decode_attention(pool_host, layer, q, w.dst_tables, w.seq_lens, 1.0 / np.sqrt(128.0))
        yield got, want


def v_max_per_dim(hs, layer=0):
    """max |V| per head_dim channel over the whole F16 source pool's seeded blocks (0xA5 filler excluded by magnitude cap)."""
    v = hs.block_view(hs.v[layer]).view(np.float16).astype(np.float32)
    v = np.where(np.isfinite(v) & (np.abs(v) < 1e3), v, 0.0)
    return np.maximum(np.abs(v).max(axis=(0, 1, 2)), 1e-3)


def quantized_pool(H, w):
    """F16 source -> the handoff's own E4M3 + scales destination, on host (oracle) and device (CUDA)."""
    import torch
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "e4m3")
    oracle.handoff(hs, hd, oracle_batch(w), None, "f16_e4m3")
    H.Plan(ds, dd, device_batch(w)).enqueue()
    torch.cuda.synchronize()
    return hs, hd, dd


def test_tensor_core_operand_plumbing_is_exact(H):
    """The tcgen05 path's tensor-map copy, swizzle, descriptors and tensor-memory reads on operands whose products and
    sums are exact in FP32: E4M3 K-major, E4M3 x E5M2 MN-major, F16 K-major, F16 MN-major."""
    assert H.selfcheck_tensor_cores() == [0, 0, 0, 0]


@pytest.mark.parametrize("flags", [0, N.ATTN_MMA_SYNC, N.ATTN_PER_HEAD_CTAS])
def test_fp8_scaled_pool_matches_oracle_attention(H, flags):
    # ragged lengths around the block (16), tile (32) and split (512) boundaries; 32 query heads on 8 kv heads
    lens = np.array([1, 15, 16, 17, 33, 511, 512, 513, 1300], dtype=np.uint32)
    w = W.Workload("attn-fp8", 2, 8, 128, 16, 512, 512, lens, dst_dtype="e4m3", outlier_channels=(7,), outlier_gain=20.0, seed=61).build_tables()
    hs, hd, dd = quantized_pool(H, w)
    for layer, (got, want) in enumerate(run(H, hd, dd, w, 32, seed=1, flags=flags)):
        close(got, want, v_max_per_dim(hs, layer))          # the x20 outlier channel gets its own bound
    # the split size only changes how partial softmaxes are merged
    import torch
    q = torch.randn((len(lens), 32, 128), generator=torch.Generator().manual_seed(9)).cuda()
    tables = torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda()
    lens_t = torch.from_numpy(lens.astype(np.int64)).to(torch.int32).cuda()
    want = oracle.paged_decode_attention(hd, 1, q.cpu().numpy(), w.dst_tables, lens, 1.0 / np.sqrt(128.0))
    for split in (64, 256, 512, 4096):
        got = H.decode_attention(dd, 1, q, tables, lens_t, split_tokens=split, flags=flags).cpu().numpy()
        close(got, want, v_max_per_dim(hs, 1))
    with pytest.raises(N.TkvError):
        H.decode_attention(dd, 1, q, tables, lens_t, split_tokens=100)


@pytest.mark.parametrize("flags", [0, N.ATTN_PER_HEAD_CTAS])
def test_fp8_unscaled_pool_and_f16_pool(H, flags):
    import torch
    lens = np.array([40, 700, 5], dtype=np.uint32)
    w = W.Workload("attn-raw", 1, 8, 128, 16, 128, 128, lens, dst_dtype="e4m3", seed=62).build_tables()
    hs, hd = host_pools(w, scales=False)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "e4m3")
    oracle.handoff(hs, hd, oracle_batch(w), None, "f16_e4m3")
    H.Plan(ds, dd, device_batch(w)).enqueue()
    torch.cuda.synchronize()
    for got, want in run(H, hd, dd, w, 8, seed=2, flags=flags):          # one query head per kv head
        close(got, want, v_max_per_dim(hs))
    # the F16 pool the E4M3 one was made from, read in place (source tables)
    w2 = W.Workload("attn-f16", 1, 8, 128, 16, 128, 128, lens, seed=62).build_tables()
    w2.dst_tables = w.src_tables
    for got, want in run(H, hs, ds, w2, 64, seed=3, flags=flags):        # 8 query heads per kv head
        close(got, want, v_max_per_dim(hs))


def test_four_kv_heads_and_more_than_eight(H):
    """4 kv heads ride the whole-block form with idle consumer warps; 16 kv heads take the per-head form."""
    import torch
    for heads, n_q in ((4, 16), (16, 32)):
        w = W.Workload(f"attn-h{heads}", 1, heads, 128, 16, 64, 64, np.array([90, 300], dtype=np.uint32), dst_dtype="e4m3", seed=64).build_tables()
        hs, hd, dd = quantized_pool(H, w)
        for got, want in run(H, hd, dd, w, n_q, seed=5):
            close(got, want, v_max_per_dim(hs))


def test_shuffled_tables_equal_identity_tables(H):
    """The reference's own property (test_paged_attention_identity_and_shuffled_match_flash): where the
    blocks sit does not change the result, bit for bit."""
    import torch
    lens = np.array([200, 77], dtype=np.uint32)
    w = W.Workload("attn-perm", 1, 8, 128, 16, 64, 64, lens, dst_dtype="e4m3", seed=63).build_tables()
    hs, hd, dd = quantized_pool(H, w)
    q = torch.randn((2, 32, 128), generator=torch.Generator().manual_seed(4)).cuda()
    lens_t = torch.from_numpy(lens.astype(np.int64)).to(torch.int32).cuda()
    shuffled = H.decode_attention(dd, 0, q, torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda(), lens_t)
    # lay the same blocks out in order in a second pool
    ident = H.Pool.allocate(0, 1, 8, 128, 16, 64, "e4m3", scales=True)
    order = np.full_like(w.dst_tables, 0)
    nxt = 0
    for qi in range(2):
        nb = (int(lens[qi]) + 15) // 16
        for i in range(nb):
            src_id = int(w.dst_tables[qi, i])
            for is_v in (False, True):
                ident.blocks(0, is_v)[nxt].copy_(dd.blocks(0, is_v)[src_id])
            ident.k_scales[0, nxt].copy_(dd.k_scales[0, src_id])
            ident.v_scales[0, nxt].copy_(dd.v_scales[0, src_id])
            order[qi, i] = nxt
            nxt += 1
    same = H.decode_attention(ident, 0, q, torch.from_numpy(order.astype(np.int64)).to(torch.int32).cuda(), lens_t)
    assert torch.equal(shuffled, same)


def test_back_to_back_calls_share_one_scratch(H):
    """Eighteen calls back to back in one stream, all merging through ONE scratch buffer: each call's partials are
    written only after the call before it has merged its own.  Bit-equal to calls run one at a time."""
    import torch
    lens = np.array([900, 33, 1500, 260], dtype=np.uint32)
    w = W.Workload("attn-chain", 2, 8, 128, 16, 512, 512, lens, dst_dtype="e4m3", seed=66).build_tables()
    hs, hd, dd = quantized_pool(H, w)
    tables = torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda()
    lens_t = torch.from_numpy(lens.astype(np.int64)).to(torch.int32).cuda()
    g = torch.Generator().manual_seed(12)
    qs = [torch.randn((len(lens), 32, 128), generator=g).cuda() for _ in range(6)]
    plain = [H.decode_attention(dd, i % 2, q, tables, lens_t, split_tokens=128).clone() for i, q in enumerate(qs)]
    chain = [H.DecodeAttention(dd, q, tables, lens_t, 1500, split_tokens=128) for q in qs]
    for c in chain[1:]:
        c.scratch = chain[0].scratch
    torch.cuda.synchronize()
    for rep in range(3):
        for i, c in enumerate(chain):
            c.enqueue(i % 2)
    torch.cuda.synchronize()
    for c, want in zip(chain, plain):
        assert int(c.status.item()) == 0
        assert torch.equal(c.out, want)
    want0 = oracle.paged_decode_attention(hd, 0, qs[0].cpu().numpy(), w.dst_tables, lens, 1.0 / np.sqrt(128.0))
    close(chain[0].out.cpu().numpy(), want0, v_max_per_dim(hs, 0))


def test_attention_argument_errors(H):
    import torch
    pool = H.Pool.allocate(0, 1, 8, 64, 16, 8, "f16")
    q = torch.zeros((1, 8, 64), device="cuda")
    t = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    n = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(N.TkvError) as e:
        H.decode_attention(pool, 0, q, t, n)
    assert e.value.code == N.ERR_DIMENSION_MISMATCH          # head_dim 64
    pool = H.Pool.allocate(0, 1, 8, 128, 16, 8, "f16")
    with pytest.raises(N.TkvError) as e:
        H.decode_attention(pool, 0, torch.zeros((1, 12, 128), device="cuda"), t, n)
    assert e.value.code == N.ERR_DIMENSION_MISMATCH          # 12 query heads on 8 kv heads
    with pytest.raises(N.TkvError) as e:
        H.decode_attention(pool, 3, torch.zeros((1, 8, 128), device="cuda"), t, n)
    assert e.value.code == N.ERR_INVALID_CONFIG               # layer outside the pool
    with pytest.raises(N.TkvError) as e:
        H.decode_attention(pool, 0, torch.zeros((1, 8, 128), device="cuda"), t, n, max_kv_len=40)
    assert e.value.code == N.ERR_DIMENSION_MISMATCH          # table too short for max_kv_len


def test_causal_chunk_of_new_tokens_matches_oracle(H):
    """A few new tokens of one sequence at once (speculative verification, a short prefill chunk): token t sees
    positions 0 .. start + t.  Checked against the oracle run once per query token with that length."""
    import torch
    lens = np.array([300], dtype=np.uint32)
    w = W.Workload("attn-chunk", 1, 8, 128, 16, 64, 64, lens, dst_dtype="e4m3", outlier_channels=(5,), outlier_gain=20.0, seed=67).build_tables()
    hs, hd, dd = quantized_pool(H, w)
    start, t = 300 - 7, 7
    q = torch.randn((t, 32, 128), generator=torch.Generator().manual_seed(13)).cuda()
    row = torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda()[0]
    got = H.causal_chunk_attention(dd, 0, q, row, start).cpu().numpy()
    tables = np.repeat(w.dst_tables.reshape(1, -1), t, axis=0)
    kv = np.arange(start + 1, start + t + 1, dtype=np.uint32)
    want = oracle.paged_decode_attention(hd, 0, q.cpu().numpy(), tables, kv, 1.0 / np.sqrt(128.0))
    close(got, want, v_max_per_dim(hs, 0))
    # the last row is plain decode attention over the whole sequence
    one = H.decode_attention(dd, 0, q[-1:].contiguous(), row.reshape(1, -1), torch.tensor([300], dtype=torch.int32).cuda())
    assert torch.equal(one.cpu(), torch.from_numpy(got[-1:]))


@pytest.mark.parametrize("flags", [0, N.ATTN_MMA_SYNC, N.ATTN_PER_HEAD_CTAS])
def test_length_above_the_host_bound_and_foreign_block_id_report_instead_of_faulting(H, flags):
    """kv_lens is device memory read when the kernel runs: a value above max_kv_len (which sized the grid, the
    table rows and the scratch) is clamped, and a table entry outside the pool is never turned into an
    address.  Both launches finish, report TKV_ERR_INVALID_CONFIG, and leave the context usable."""
    import torch
    lens = np.array([40, 200], dtype=np.uint32)
    w = W.Workload("attn-guard", 1, 8, 128, 16, 64, 64, lens, seed=5).build_tables()
    hs, _ = host_pools(w)
    ds = to_device_pool(hs, "f16")
    q = torch.randn((2, 32, 128), generator=torch.Generator().manual_seed(3)).cuda()
    tables = torch.from_numpy(w.src_tables.astype(np.int64)).to(torch.int32).cuda()
    good = torch.from_numpy(lens.astype(np.int64)).to(torch.int32).cuda()
    want = H.decode_attention(ds, 0, q, tables, good, max_kv_len=200, flags=flags).cpu().numpy()

    # a device length far above the bound: attended up to the bound, reported
    long = torch.tensor([40, 100000], dtype=torch.int32).cuda()
    attn = H.DecodeAttention(ds, q, tables, long, 200, flags=flags)
    got = attn.enqueue(0).cpu().numpy()
    assert int(attn.status.item()) == N.ERR_INVALID_CONFIG
    np.testing.assert_array_equal(got, want)           # the clamp makes it the max_kv_len answer

    # one table entry outside the pool
    bad = tables.clone()
    bad[1, 3] = 1 << 20
    attn = H.DecodeAttention(ds, q, bad, good, 200, flags=flags)
    attn.enqueue(0)
    torch.cuda.synchronize()
    assert int(attn.status.item()) == N.ERR_INVALID_CONFIG
    # the context still works
    again = H.decode_attention(ds, 0, q, tables, good, max_kv_len=200, flags=flags).cpu().numpy()
    np.testing.assert_array_equal(again, want)


# both forms of both pools are forced: chunks this short take one query tile per CTA by default
@pytest.mark.parametrize("dtype,flags", [("e4m3", N.PREFILL_TWO_TILES), ("e4m3", N.PREFILL_SINGLE_TILE), ("f16", 0), ("f16", N.PREFILL_TWO_TILES)])
@pytest.mark.parametrize("start,t", [(0, 40), (45, 70), (250, 33), (0, 300), (100, 64), (3, 129)])
def test_prefill_attention_on_tensor_cores_matches_oracle(H, dtype, flags, start, t):
    """The prefill-side twin: T new tokens of one sequence, token t attends to positions 0 .. start + t.  Ragged against
    every boundary (start not on a block, T not a multiple of the 32 tokens a CTA takes, the last tile of 128 cached tokens
    partly filled, rows of one CTA ending in different tiles).  Checked against the oracle run once per query token."""
    import torch
    total = start + t
    lens = np.array([total], dtype=np.uint32)
    kw = dict(dst_dtype="e4m3", outlier_channels=(5,), outlier_gain=20.0) if dtype == "e4m3" else {}
    w = W.Workload("prefill-chunk", 1, 8, 128, 16, 64, 64, lens, seed=71, **kw).build_tables()
    if dtype == "e4m3":
        hs, hd, dd = quantized_pool(H, w)
    else:
        hs, _ = host_pools(w)
        hd, dd = hs, to_device_pool(hs, "f16")
        w.dst_tables = w.src_tables
    q = torch.randn((t, 32, 128), generator=torch.Generator().manual_seed(17)).cuda()
    row = torch.from_numpy(w.dst_tables.astype(np.int64)).to(torch.int32).cuda()[0]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = H.prefill_attention(dd, 0, q, row, start, status=status, flags=flags).cpu().numpy()
    assert int(status.item()) == 0
    tables = np.repeat(w.dst_tables.reshape(1, -1), t, axis=0)
    kv = np.arange(start + 1, start + t + 1, dtype=np.uint32)
    want = oracle.paged_decode_attention(hd, 0, q.cpu().numpy(), tables, kv, 1.0 / np.sqrt(128.0))
    close(got, want, v_max_per_dim(hs, 0))


def test_prefill_attention_f16_long_prompt_takes_the_two_tile_form(H):
    """A long prompt over an F16 pool: two query tiles per CTA with two K tiles and one V tile in flight, the K ring a tile ahead
    of V; sampled query tokens of a 6 400-token prompt against the oracle."""
    import torch
    t = 6400
    w = W.Workload("prefill-long", 1, 8, 128, 16, 512, 512, np.array([t], dtype=np.uint32), seed=73).build_tables()
    hs, _ = host_pools(w)
    dd = to_device_pool(hs, "f16")
    q = torch.randn((t, 32, 128), generator=torch.Generator().manual_seed(19)).cuda()
    row = torch.from_numpy(w.src_tables.astype(np.int64)).to(torch.int32).cuda()[0]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = H.prefill_attention(dd, 0, q, row, 0, status=status)
    assert int(status.item()) == 0
    pick = [0, 31, 32, 63, 64, 2047, 4100, 6143, 6399]
    tables = np.repeat(w.src_tables.reshape(1, -1), len(pick), axis=0)
    kv = np.array([p + 1 for p in pick], dtype=np.uint32)
    want = oracle.paged_decode_attention(hs, 0, q[pick].cpu().numpy(), tables, kv, 1.0 / np.sqrt(128.0))
    close(got[pick].cpu().numpy(), want, v_max_per_dim(hs, 0))


def test_prefill_attention_refuses_other_geometries_and_foreign_blocks(H):
    import torch
    w = W.Workload("prefill-guard", 1, 8, 128, 16, 64, 64, np.array([100], dtype=np.uint32), seed=3).build_tables()
    hs, _ = host_pools(w)
    ds = to_device_pool(hs, "f16")
    q = torch.randn((20, 32, 128), generator=torch.Generator().manual_seed(3)).cuda()
    row = torch.from_numpy(w.src_tables.astype(np.int64)).to(torch.int32).cuda()[0]
    with pytest.raises(N.TkvError) as e:                              # 16 query heads: not the geometry the kernel is built for
        H.prefill_attention(ds, 0, q[:, :16].contiguous(), row, 80)
    assert e.value.code == N.ERR_DIMENSION_MISMATCH
    with pytest.raises(N.TkvError) as e:                              # the table does not reach start + T
        H.prefill_attention(ds, 0, q, row[:5], 80)
    assert e.value.code == N.ERR_DIMENSION_MISMATCH
    bad = row.clone()
    bad[2] = 1 << 20                                                  # a block id outside the pool is reported, never read
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    H.prefill_attention(ds, 0, q, bad, 80, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == N.ERR_INVALID_CONFIG
    good = H.prefill_attention(ds, 0, q, row, 80, status=None)       # the context is still usable
    assert bool(torch.isfinite(good).all())
