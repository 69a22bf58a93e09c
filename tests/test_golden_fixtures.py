"""Committed golden vectors (tests/golden/handoff_small.npz, made by make_golden.py): the
oracle must still produce them (CPU), and so must the CUDA path (GPU)."""
import os

import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, device_batch, oracle_batch, to_device_pool
from tempura_b200 import workloads as W

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "handoff_small.npz"))


def _case(dst_dtype):
    w = W.Workload("golden", 1, 2, 64, 16, 8, 8, G["seq_lens"], dst_dtype=dst_dtype, seed=123)
    w.src_tables, w.dst_tables, w.table_stride = G["src_tables"], G["dst_tables"], G["src_tables"].shape[1]
    src = oracle.HostPool.filled(1, 2, 64, 16, 8, np.uint16, 0xA5)
    src.k[0][:], src.v[0][:] = G["src_k"], G["src_v"]
    dst = oracle.HostPool.filled(1, 2, 64, 16, 8, np.uint16 if dst_dtype == "f16" else np.uint8, 0x5A,
                                 with_scales=dst_dtype == "e4m3")
    return w, src, dst


def _expected(dst_dtype, dst):
    mode = "copy" if dst_dtype == "f16" else "f16_e4m3"
    dst.k[0][:], dst.v[0][:] = G[f"{mode}_dst_k"], G[f"{mode}_dst_v"]
    if dst_dtype == "e4m3":
        dst.k_scales[:], dst.v_scales[:] = G["k_scales"], G["v_scales"]
    return dst


@pytest.mark.parametrize("dst_dtype", ["f16", "e4m3"])
def test_oracle_reproduces_golden(dst_dtype):
    w, src, dst = _case(dst_dtype)
    oracle.handoff(src, dst, oracle_batch(w), None, "copy" if dst_dtype == "f16" else "f16_e4m3")
    want = _expected(dst_dtype, _case(dst_dtype)[2])
    assert np.array_equal(dst.k[0], want.k[0]) and np.array_equal(dst.v[0], want.v[0])
    if dst_dtype == "e4m3":
        assert np.array_equal(dst.k_scales.view(np.uint32), want.k_scales.view(np.uint32))
        assert np.array_equal(dst.v_scales.view(np.uint32), want.v_scales.view(np.uint32))
        # the frozen rule, spelled out on the fixture: zero block and Inf/NaN blocks carry scale 1
        t = G["dst_tables"]
        assert want.k_scales[0, t[0, 0], 0] == 1.0 and want.k_scales[0, t[0, 1], 1] == 1.0 and want.k_scales[0, t[1, 0], 0] == 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("dst_dtype", ["f16", "e4m3"])
def test_cuda_reproduces_golden(dst_dtype):
    import torch
    from tempura_b200 import handoff as H
    w, src, dst = _case(dst_dtype)
    ds, dd = to_device_pool(src, "f16"), to_device_pool(dst, dst_dtype)
    H.Plan(ds, dd, device_batch(w)).enqueue()
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, _expected(dst_dtype, _case(dst_dtype)[2]), f"golden {dst_dtype}")


# ---- the reader's rule: the golden E4M3 pool widened back to F16 (tests/golden/widen_small.npz) ----
GW = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "widen_small.npz"))


def _widen_case():
    w, _, _ = _case("e4m3")
    src = _expected("e4m3", _case("e4m3")[2])                      # the golden E4M3 bytes and scales
    w.src_tables = w.dst_tables                                    # read where the handoff wrote
    w.src_dtype, w.dst_dtype = "e4m3", "f16"
    dst = oracle.HostPool.filled(1, 2, 64, 16, 8, np.uint16, 0x5A)
    want = oracle.HostPool.filled(1, 2, 64, 16, 8, np.uint16, 0x5A)
    want.k[0][:], want.v[0][:] = GW["widen_dst_k"], GW["widen_dst_v"]
    return w, src, dst, want


def test_oracle_reproduces_golden_widen():
    w, src, dst, want = _widen_case()
    oracle.handoff(src, dst, oracle_batch(w), None, "e4m3_f16")
    assert np.array_equal(dst.k[0], want.k[0]) and np.array_equal(dst.v[0], want.v[0])
    # spot values: the golden source held 1.0 in a block whose scale is amax / 448; it must come back as 1.0 exactly
    # only where the scale is a power of two; in general within one E4M3 step, so pin a decoded byte instead
    assert oracle.e4m3_to_f32(0x38) == 1.0 and oracle.e4m3_to_f32(0x7E) == 448.0


@pytest.mark.gpu
def test_cuda_reproduces_golden_widen():
    import torch
    from tempura_b200 import handoff as H
    w, src, dst, want = _widen_case()
    ds, dd = to_device_pool(src, "e4m3"), to_device_pool(dst, "f16")
    H.Plan(ds, dd, device_batch(w), None, 1).enqueue()            # 1: the ids repeat the source's, fine for a fresh pool
    torch.cuda.synchronize()
    assert_pool_equals_host(dd, want, "golden widen")
