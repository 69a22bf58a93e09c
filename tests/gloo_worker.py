"""One rank of the CPU multi-rank test (launched by test_multirank_gloo.py through
torch.distributed.run, backend gloo).

Every rank derives its role from the C ABI's pairing, prefill ranks gather their share of
the seeded batch into a transfer buffer laid out as the C ABI sizes it and send it to their
partner, decode ranks scatter it into their share of the destination pool, and rank 0
checks the union of the decode pools against one unsharded oracle handoff.  The data
movement here is the oracle's loops (this is a test of the host-side partitioning, run
without a GPU); the GPU tests cover the kernels.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import oracle  # noqa: E402
from helpers import host_pools, oracle_batch  # noqa: E402
from tempura_b200 import _native as N  # noqa: E402
from tempura_b200 import disagg, handoff as H  # noqa: E402
from tempura_b200 import workloads as W  # noqa: E402


def share_of(pool: oracle.HostPool, role: disagg.Role) -> oracle.HostPool:
    """The slice of a full pool that one pair's GPU would hold."""
    def cut(arr):
        v = pool.block_view(arr)[:, :, role.head_begin:role.head_begin + role.n_heads, :]
        return np.ascontiguousarray(v).reshape(-1)
    layers = range(role.layer_begin, role.layer_begin + role.n_layers)
    return oracle.HostPool(role.n_layers, role.n_heads, pool.head_dim, pool.block_size, pool.total_blocks, pool.dtype,
                           [cut(pool.k[l]) for l in layers], [cut(pool.v[l]) for l in layers])


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    case = os.environ.get("GLOO_CASE", "heads")
    heads = 1 if case == "layers" else 8
    lens = W.lengths(5, 1, 150, 11, 7)
    pre = None
    if case == "prefix":
        pre = np.full(5, 32, dtype=np.uint32)
        lens = (lens + np.uint32(32)).astype(np.uint32)
    w = W.Workload("gloo-" + case, 4, heads, 64, 16, 96, 96, lens, prefix_lens=pre, seed=5).build_tables()
    role = disagg.role_of(rank, world, w.n_layers, w.n_kv_heads)
    assert role.partner == (rank + world // 2 if role.is_prefill else rank - world // 2)
    hs_full, hd_full = host_pools(w)                      # identical on every rank (seeded)
    L = oracle.lib()
    bs, es = w.block_size, 2
    stride = role.n_heads * w.head_dim                    # elements per token row of this pair's share
    batch = H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens)
    n_blocks = H.batch_blocks(batch, bs)
    nbytes = int(N.lib().tkv_transfer_bytes(role.n_layers, role.n_heads, w.head_dim, bs, N.DTYPE_F16, n_blocks))
    plane = n_blocks * bs * stride * es
    assert nbytes == 2 * role.n_layers * plane
    buf = np.zeros(max(nbytes, 1), dtype=np.uint8)
    u32p = C.POINTER(C.c_uint32)
    mine = None
    if role.is_prefill:
        src = share_of(hs_full, role)
        for l in range(role.n_layers):
            for kv, arrs in enumerate((src.k, src.v)):
                at = (2 * l + kv) * plane
                for q, length in enumerate(w.seq_lens):
                    length = int(length)
                    p0 = int(pre[q]) if pre is not None else 0
                    out = np.empty(length * stride, dtype=np.uint16)
                    tab = np.ascontiguousarray(w.src_tables[q])
                    L.orc_paged_gather(arrs[l].ctypes.data, tab.ctypes.data_as(u32p), bs, stride, es, length, out.ctypes.data)
                    rows = out[p0 * stride:].view(np.uint8)
                    buf[at:at + rows.size] = rows
                    at += ((length + bs - 1) // bs - p0 // bs) * bs * stride * es
        dist.send(torch.from_numpy(buf), role.partner)
    else:
        dst = share_of(hd_full, role)
        dist.recv(torch.from_numpy(buf), role.partner)
        for l in range(role.n_layers):
            for kv, arrs in enumerate((dst.k, dst.v)):
                at = (2 * l + kv) * plane
                for q, length in enumerate(w.seq_lens):
                    length = int(length)
                    p0 = int(pre[q]) if pre is not None else 0
                    tab = np.ascontiguousarray(w.dst_tables[q])
                    rows = np.ascontiguousarray(buf[at:at + (length - p0) * stride * es])
                    L.orc_paged_scatter(arrs[l].ctypes.data, tab.ctypes.data_as(u32p), bs, stride, es, p0, length - p0,
                                        rows.ctypes.data)
                    at += ((length + bs - 1) // bs - p0 // bs) * bs * stride * es
        mine = (role.head_begin, role.n_heads, role.layer_begin, role.n_layers, dst.k, dst.v)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        oracle.handoff(hs_full, hd_full, oracle_batch(w), None, "copy")
        covered = np.zeros((w.n_layers, w.n_kv_heads), dtype=np.int32)
        for g in gathered:
            if g is None:
                continue
            hb, nh, lb, nl, ks, vs = g
            for i in range(nl):
                for got, want in ((ks[i], hd_full.k[lb + i]), (vs[i], hd_full.v[lb + i])):
                    ref = hd_full.block_view(want)[:, :, hb:hb + nh, :].reshape(-1)
                    assert np.array_equal(got, ref), f"pair share heads {hb}+{nh} layer {lb + i} differs"
                covered[lb + i, hb:hb + nh] += 1
        assert (covered == 1).all(), "shares do not tile the (layer, head) grid exactly once"
        with open(os.environ["GLOO_RESULT"], "w") as f:
            f.write(f"OK {world} {case} pairs={world // 2}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
