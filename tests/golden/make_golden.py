"""Regenerates the committed golden fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust) cannot run in this image, so the fixtures freeze what the oracle, pinned
to the reference's known-answer tests, produces for one small seeded handoff per dtype pair,
special values included.  The FP8 scale rule is the one part no reference test pins; the
fixture is what keeps it from drifting.  Files: handoff_small.npz, and widen_small.npz (the
E4M3 destination of the former widened back to F16 through its scales: the reader's rule).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from helpers import host_pools, oracle_batch  # noqa: E402
from tempura_b200 import workloads as W  # noqa: E402


def workload(dst_dtype):
    w = W.Workload("golden", 1, 2, 64, 16, 8, 8, np.array([37, 16, 5], dtype=np.uint32), dst_dtype=dst_dtype,
                   outlier_channels=(3,), outlier_gain=20.0, seed=123)
    return w.build_tables()


def special_values(hs, w):
    k = hs.block_view(hs.k[0])
    t = w.src_tables
    k[t[0, 0], :, 0, :] = 0                                   # all-zero (block, head)
    k[t[0, 1], 2, 1, 5] = 0x7C00                              # +Inf -> unscaled fallback
    k[t[1, 0], 0, 0, 0] = 0x7E00                              # NaN  -> unscaled fallback
    adv = np.array([0.0, -0.0, 1.0, -1.0, 1.0625, 1.1875, 15.5, 0.015625, 0.01, 0.001, -0.001, 448.0, -448.0, 449.0,
                    65504.0, 6.1035156e-5, 5.96e-8, 0.5, 0.49999997], dtype=np.float32).astype(np.float16)
    hs.block_view(hs.v[0])[t[0, 2], 1, 1, : len(adv)] = adv.view(np.uint16)


def main():
    out = {}
    for dst_dtype, mode in (("f16", "copy"), ("e4m3", "f16_e4m3")):
        w = workload(dst_dtype)
        hs, hd = host_pools(w)
        special_values(hs, w)
        if mode == "copy":
            out.update(src_k=hs.k[0].copy(), src_v=hs.v[0].copy(), seq_lens=w.seq_lens, src_tables=w.src_tables,
                       dst_tables=w.dst_tables)
        oracle.handoff(hs, hd, oracle_batch(w), None, mode)
        out[f"{mode}_dst_k"], out[f"{mode}_dst_v"] = hd.k[0].copy(), hd.v[0].copy()
        if hd.k_scales is not None:
            out["k_scales"], out["v_scales"] = hd.k_scales.copy(), hd.v_scales.copy()
    np.savez_compressed(os.path.join(HERE, "handoff_small.npz"), **out)
    print({k: (v.shape, str(v.dtype)) for k, v in out.items()})
    # widen the E4M3 pool just produced (hd) back into an F16 pool at the same block ids
    back = oracle.HostPool.filled(1, 2, 64, 16, 8, np.uint16, 0x5A)
    own = oracle.make_batch(w.seq_lens, w.dst_tables, w.dst_tables, w.table_stride)
    oracle.handoff(hd, back, own, None, "e4m3_f16")
    np.savez_compressed(os.path.join(HERE, "widen_small.npz"), widen_dst_k=back.k[0].copy(), widen_dst_v=back.v[0].copy())


if __name__ == "__main__":
    main()
