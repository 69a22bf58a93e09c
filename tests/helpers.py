"""Shared test plumbing: seeded host pools for a workload, the oracle run, and the
device mirror used by the GPU parity tests."""
from __future__ import annotations

import numpy as np

import oracle
from tempura_b200 import workloads as W

NP_DT = {"f32": np.float32, "f16": np.uint16, "e4m3": np.uint8}


def host_pools(w: W.Workload, src_heads=None, dst_heads=None, src_layers=None, dst_layers=None, scales=None):
    """Source pool: 0xA5 pattern everywhere, seeded N(0, sigma) F16 values in every block
    a table names (prefix blocks included).  Destination pool: 0x5A pattern; for a
    prefix workload the shared prefix blocks hold seeded values too, so a stray write
    into them is visible."""
    sh = src_heads or w.n_kv_heads
    dh = dst_heads or w.n_kv_heads
    sl = src_layers or w.n_layers
    dl = dst_layers or w.n_layers
    if scales is None:
        scales = w.dst_dtype == "e4m3" and w.src_dtype == "f16"
    src = oracle.HostPool.filled(sl, sh, w.head_dim, w.block_size, w.src_blocks, NP_DT[w.src_dtype], 0xA5)
    dst = oracle.HostPool.filled(dl, dh, w.head_dim, w.block_size, w.dst_blocks, NP_DT[w.dst_dtype], 0x5A,
                                 with_scales=scales)
    bs = w.block_size
    used = sorted({int(b) for q in range(len(w.seq_lens))
                   for b in w.src_tables[q, : (int(w.seq_lens[q]) + bs - 1) // bs]})
    per_block = bs * sh * w.head_dim
    for l in range(sl):
        for kv, arrs in enumerate((src.k, src.v)):
            view = arrs[l].reshape(w.src_blocks, per_block)
            for b in used:
                vals = oracle.gen_normal_f16(per_block, w.seed, 1000 + 2 * l + kv, w.sigma, w.head_dim,
                                             w.outlier_channels, w.outlier_gain, first_index=b * per_block)
                if w.src_dtype == "f16":
                    view[b] = vals
                elif w.src_dtype == "f32":
                    # full-width mantissas, so a narrowing cast really has to round
                    with np.errstate(over="ignore", invalid="ignore"):
                        view[b] = vals.view(np.float16).astype(np.float32) * np.float32(1.0001234)
                else:
                    view[b] = (vals & 0xFF).astype(np.uint8)
    if w.shared_prefix_blocks is not None:
        per_block_d = bs * dh * w.head_dim
        for l in range(dl):
            for kv, arrs in enumerate((dst.k, dst.v)):
                view = arrs[l].reshape(w.dst_blocks, per_block_d)
                for b in w.shared_prefix_blocks:
                    vals = oracle.gen_normal_f16(per_block_d, w.seed + 77, 2 * l + kv, w.sigma, first_index=int(b) * per_block_d)
                    view[int(b)] = vals if w.dst_dtype == "f16" else (vals & 0xFF).astype(np.uint8)
    return src, dst


def oracle_batch(w: W.Workload, table_layer_stride=0):
    return oracle.make_batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens, table_layer_stride)


def mode_of(w: W.Workload) -> str:
    if w.src_dtype == w.dst_dtype:
        return "copy"
    return {("f16", "e4m3"): "f16_e4m3", ("f32", "f16"): "f32_f16", ("e4m3", "f16"): "e4m3_f16",
            ("e4m3", "f32"): "e4m3_f32", ("f32", "e4m3"): "f32_e4m3"}[(w.src_dtype, w.dst_dtype)]


# ---- device side ------------------------------------------------------------------
def to_device_pool(hp: oracle.HostPool, dtype: str, device: int = 0, refcounts=None):
    import torch
    from tempura_b200 import handoff as H
    p = H.Pool.allocate(device, hp.n_layers, hp.n_kv_heads, hp.head_dim, hp.block_size, hp.total_blocks, dtype,
                        scales=hp.k_scales is not None, refcounts=refcounts is not None, fill_byte=None)
    for l in range(hp.n_layers):
        p.k[l].view(torch.uint8).copy_(torch.from_numpy(hp.k[l].view(np.uint8)))
        p.v[l].view(torch.uint8).copy_(torch.from_numpy(hp.v[l].view(np.uint8)))
    torch.cuda.synchronize(device)
    if hp.k_scales is not None:
        p.k_scales.copy_(torch.from_numpy(hp.k_scales))
        p.v_scales.copy_(torch.from_numpy(hp.v_scales))
    if refcounts is not None:
        p.refcounts.copy_(torch.from_numpy(refcounts.view(np.int32)))
    return p


def assert_pool_equals_host(p, hp: oracle.HostPool, what=""):
    import torch
    torch.cuda.synchronize()
    for l in range(hp.n_layers):
        for name, dev, host in (("K", p.k[l], hp.k[l]), ("V", p.v[l], hp.v[l])):
            got = dev.view(torch.uint8).cpu().numpy()
            want = host.view(np.uint8)
            if not np.array_equal(got, want):
                bad = np.flatnonzero(got != want)
                raise AssertionError(f"{what} layer {l} {name}: {bad.size} bytes differ, first at {bad[0]} "
                                     f"(got {got[bad[0]]:#x}, want {want[bad[0]]:#x})")
    if hp.k_scales is not None:
        for name, dev, host in (("k_scales", p.k_scales, hp.k_scales), ("v_scales", p.v_scales, hp.v_scales)):
            got = dev.cpu().numpy().view(np.uint32)
            want = host.view(np.uint32)
            if not np.array_equal(got, want):
                bad = np.argwhere(got != want)
                raise AssertionError(f"{what} {name}: {len(bad)} scales differ, first at {bad[0]}")


def device_batch(w: W.Workload, table_layer_stride=0):
    from tempura_b200 import handoff as H
    return H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens, table_layer_stride)
