"""Argument validation of tkv_plan_create runs before any CUDA call, so it is
checked here without a GPU.  Error classes follow the reference's KernelError
(kernel-api/src/lib.rs:5-13)."""
import ctypes as C

import numpy as np
import pytest

from tempura_b200 import _build, _native as N
from tempura_b200 import handoff as H


@pytest.fixture(scope="module", autouse=True)
def _built():
    _build.build()


def fake_pool(layers=2, heads=4, dim=16, bs=4, blocks=32, dtype="f16", scales=False):
    # addresses are never dereferenced: validation fails first
    base = 0x10000000
    k = [base + 0x100000 * (2 * l) for l in range(layers)]
    v = [base + 0x100000 * (2 * l + 1) for l in range(layers)]
    return H.Pool.from_pointers(0, dtype, heads, dim, bs, blocks, k, v,
                                k_scales_ptr=0x7000000 if scales else 0, v_scales_ptr=0x7100000 if scales else 0)


def batch(seq_lens, src, dst, stride, prefix=None):
    return H.Batch(np.array(seq_lens), np.array(src), np.array(dst), stride, None if prefix is None else np.array(prefix))


def expect(code, fn):
    with pytest.raises(N.TkvError) as e:
        fn()
    assert e.value.code == code, e.value
    return e.value.message


def test_dimension_mismatch_head_dim_and_block_size():
    b = batch([4], [[0]], [[0]], 1)
    msg = expect(N.ERR_DIMENSION_MISMATCH, lambda: H.Plan(fake_pool(dim=16), fake_pool(dim=32), b))
    assert "expected 16, got 32" in msg
    expect(N.ERR_DIMENSION_MISMATCH, lambda: H.Plan(fake_pool(bs=4), fake_pool(bs=8), b))


def test_unsupported_dtype_pair_and_half_set_scales():
    b = batch([4], [[0]], [[0]], 1)
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(dtype="f16"), fake_pool(dtype="f32"), b))
    half = fake_pool(dtype="e4m3", scales=True)
    half.k_scales_ptr = 0                                  # a source with only one of its two scale arrays
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(half, fake_pool(dtype="f16"), b))
    # E4M3 -> E4M3 moves scales along: both sides carry them or neither does
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(dtype="e4m3", scales=True), fake_pool(dtype="e4m3"), b))
    p = fake_pool(dtype="e4m3", scales=True)
    p.v_scales_ptr = 0
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), p, b))


def test_shard_out_of_range():
    b = batch([4], [[0]], [[0]], 1)
    expect(N.ERR_DIMENSION_MISMATCH, lambda: H.Plan(fake_pool(), fake_pool(), b, H.Shard(2, 0, 3, 0, 0, 2)))
    expect(N.ERR_DIMENSION_MISMATCH, lambda: H.Plan(fake_pool(), fake_pool(), b, H.Shard(0, 0, 4, 1, 0, 2)))
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), b, H.Shard(0, 0, 0, 0, 0, 2)))


def test_table_too_short_and_ids_out_of_pool():
    expect(N.ERR_DIMENSION_MISMATCH, lambda: H.Plan(fake_pool(), fake_pool(), batch([9], [[0, 1]], [[0, 1]], 2)))
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), batch([8], [[0, 32]], [[0, 1]], 2)))
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), batch([8], [[0, 1]], [[0, 0xFFFFFFFF]], 2)))


def test_prefix_rules():
    # prefix longer than the sequence, and not block-aligned
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), batch([4], [[0, 1]], [[0, 1]], 2, [8])))
    expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), batch([8], [[0, 1]], [[0, 1]], 2, [3])))
    # a moved block may not land on one of the batch's shared prefix blocks
    msg = expect(N.ERR_INVALID_CONFIG,
                 lambda: H.Plan(fake_pool(), fake_pool(), batch([8, 8], [[0, 1], [2, 3]], [[5, 6], [5, 5]], 2, [4, 4])))
    assert "shared prefix block" in msg


def test_duplicate_destination_rejected_unless_allowed():
    b = batch([4, 4], [[0], [1]], [[7], [7]], 1)
    msg = expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), b))
    assert "written twice" in msg
    # with the flag the duplicate passes validation; the next failure is CUDA (no device here)
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if not has_gpu:
        expect(N.ERR_CUDA, lambda: H.Plan(fake_pool(), fake_pool(), b, flags=N.PLAN_ALLOW_SHARED_DST))


def test_null_arguments():
    L = N.lib()
    out = C.c_void_p()
    assert L.tkv_plan_create(None, None, None, None, 0, C.byref(out)) == N.ERR_INVALID_CONFIG
    assert L.tkv_plan_destroy(None) == 0
    assert L.tkv_handoff_enqueue(None, None, 0, 0) == N.ERR_INVALID_CONFIG
    assert L.tkv_flag_wait_enqueue(None, 0, 0, 10, 0) == N.ERR_INVALID_CONFIG
    assert L.tkv_flag_wait_enqueue(None, 0x1000, 0, 0, 0) == N.ERR_INVALID_CONFIG   # unbounded wait refused


def test_batch_beyond_the_chunk_index_range_is_refused():
    """Chunk indices are 32-bit: a batch with more than 2^31 / (2 * layers) block pairs is refused by
    arithmetic on the lengths alone, before any table entry is read."""
    n_blocks = 600_000_000                                    # x 2 layers x 2 > 2^31
    b = H.Batch(np.array([n_blocks * 4], dtype=np.uint32), np.zeros(1, np.uint32), np.zeros(1, np.uint32), n_blocks)
    msg = expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), b))
    assert "too large" in msg


def test_transfer_buffer_plans_validate_without_a_gpu():
    small = N.TkvTransfer(0, N.DTYPE_F16, 0, 0, 0x20000000, 64, 0)          # 64 bytes for a batch that needs far more
    pool, b = fake_pool(), batch([9], [[0, 1, 2]], [[3, 4, 5]], 3)
    for make in (lambda: N.lib().tkv_plan_create_to_transfer(C.byref(pool.c_struct()), C.byref(small), C.byref(b.c_struct()), None, 0,
                                                             C.byref(C.c_void_p())),
                 lambda: N.lib().tkv_plan_create_from_transfer(C.byref(small), C.byref(pool.c_struct()), C.byref(b.c_struct()), None, 0,
                                                               C.byref(C.c_void_p()))):
        assert make() == N.ERR_DIMENSION_MISMATCH
    null = N.TkvTransfer(0, N.DTYPE_F16, 0, 0, 0, 1 << 20, 0)
    assert N.lib().tkv_plan_create_to_transfer(C.byref(pool.c_struct()), C.byref(null), C.byref(b.c_struct()), None, 0,
                                               C.byref(C.c_void_p())) == N.ERR_INVALID_CONFIG
    scaled_f16 = N.TkvTransfer(0, N.DTYPE_F16, 0, 0, 0x20000000, 1 << 20, 0x30000000)
    assert N.lib().tkv_plan_create_to_transfer(C.byref(pool.c_struct()), C.byref(scaled_f16), C.byref(b.c_struct()), None, 0,
                                               C.byref(C.c_void_p())) == N.ERR_INVALID_CONFIG
    assert N.lib().tkv_batch_blocks(C.byref(b.c_struct()), 4) == 3
    assert N.lib().tkv_transfer_bytes(2, 4, 16, 4, N.DTYPE_F16, 3) == 2 * 2 * 3 * 4 * 4 * 16 * 2


def test_copy_engine_staging_is_only_for_host_buffers_read_into_a_pool():
    """TKV_PLAN_STAGE_HOST names the one case it serves (a page-locked host transfer buffer, without scales, scattered
    into a pool); a pool-to-pool plan, a device buffer and a buffer written by the plan are refused before any CUDA call."""
    pool, b = fake_pool(), batch([8], [[0, 1]], [[2, 3]], 2)
    msg = expect(N.ERR_INVALID_CONFIG, lambda: H.Plan(fake_pool(), fake_pool(), b, flags=N.PLAN_STAGE_HOST))
    assert "TKV_PLAN_STAGE_HOST" in msg
    on_device = N.TkvTransfer(0, N.DTYPE_F16, 0, 0, 0x20000000, 1 << 20, 0)
    assert N.lib().tkv_plan_create_from_transfer(C.byref(on_device), C.byref(pool.c_struct()), C.byref(b.c_struct()), None,
                                                 N.PLAN_STAGE_HOST, C.byref(C.c_void_p())) == N.ERR_INVALID_CONFIG
    on_host = N.TkvTransfer(0, N.DTYPE_F16, 1, 0, 0x20000000, 1 << 20, 0)
    assert N.lib().tkv_plan_create_to_transfer(C.byref(pool.c_struct()), C.byref(on_host), C.byref(b.c_struct()), None,
                                               N.PLAN_STAGE_HOST, C.byref(C.c_void_p())) == N.ERR_INVALID_CONFIG


def test_decode_attention_arguments_validate_without_a_gpu():
    pool = fake_pool(layers=1, heads=8, dim=128, bs=16)
    args = N.TkvDecodeAttn(1, 12, 1, 0, 16, 0.1, 0, 0, 0x100, 0x200, 0x300, 0x400, 0x500, 1 << 20, 0, 0)
    assert N.lib().tkv_decode_attn_enqueue(C.byref(pool.c_struct()), C.byref(args), None) == N.ERR_DIMENSION_MISMATCH   # 12 heads on 8
    args = N.TkvDecodeAttn(1, 8, 1, 5, 16, 0.1, 0, 0, 0x100, 0x200, 0x300, 0x400, 0x500, 1 << 20, 0, 0)
    assert N.lib().tkv_decode_attn_enqueue(C.byref(pool.c_struct()), C.byref(args), None) == N.ERR_INVALID_CONFIG       # layer 5 of 1
    f32 = fake_pool(layers=1, heads=8, dim=128, bs=16, dtype="f32")
    assert N.lib().tkv_decode_attn_enqueue(C.byref(f32.c_struct()), C.byref(args), None) == N.ERR_INVALID_CONFIG
    assert N.lib().tkv_decode_attn_scratch_bytes(16, 32, 128, 4096, 1024) == 2 * 16 * 32 * 4 * 130 * 4    # one partial result per token range and softmax group


def test_unmapped_peer_destination_is_refused_on_the_host():
    """A kernel on the source device stores into the destination pool.  Two ordinals the library never
    paired (no tkv_init, no tkv_ipc_import) are refused before any CUDA call, by the planned handoff and
    by the allocation-free one alike: nothing is launched at addresses the source device cannot reach."""
    b = batch([8], [[0, 1]], [[2, 3]], 2)
    src, dst = fake_pool(), fake_pool()
    dst.device = 5
    for call in (lambda: H.Plan(src, dst, b), lambda: H.handoff_noalloc(src, dst, b, stream=_NoStream())):
        msg = expect(N.ERR_INVALID_CONFIG, call)
        assert "device 0 cannot store into device 5" in msg and "tkv_init" in msg
    # the transfer-buffer forms go through the same gate (buffer on one device, pool on another)
    x = H.Transfer(_FakeTensor(0x20000000, 1 << 20), N.DTYPE_F16, 3)
    msg = expect(N.ERR_INVALID_CONFIG, lambda: H.Plan.from_transfer(x, dst, b))
    assert "device 3 cannot store into device 5" in msg


class _NoStream:
    cuda_stream = 0


class _FakeTensor:
    """Address and size of a buffer that is never dereferenced (validation fails first)."""
    def __init__(self, ptr, n):
        self._p, self._n = ptr, n

    def data_ptr(self):
        return self._p

    def numel(self):
        return self._n
