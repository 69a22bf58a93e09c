"""One rank of the two-process wire test (launched by test_session_gloo.py through torch.distributed.run, gloo).

Rank 0 is the prefill side: it holds a sequence in a shuffled paged pool and announces it as page-granular
tkv_session_pack messages, delivered OUT OF ORDER and in TWO batches, each followed by the rows of the pages it
names.  Rank 1 is the decode side: for every message that arrives intact it allocates destination pages (the
reference's LIFO PageAllocator through the C ABI), records them in a BlockTable, and moves the named pages'
rows in -- after the first batch the table is partially filled and exactly the announced pages hold data; a
damaged message is refused by its checksum and asked for again.  At the end the decode pool equals one oracle
handoff of the whole sequence.  The row movement here is the oracle's loops (host-side test, no GPU)."""
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
from helpers import host_pools  # noqa: E402
from tempura_b200 import _native as N  # noqa: E402
from tempura_b200 import session as S  # noqa: E402
from tempura_b200 import workloads as W  # noqa: E402

BS, LAYERS, HEADS, DIM = 16, 2, 4, 32


def send_bytes(b: bytes, dst: int):
    dist.send(torch.tensor([len(b)], dtype=torch.int64), dst)
    if b:
        dist.send(torch.frombuffer(bytearray(b), dtype=torch.uint8), dst)


def recv_bytes(src: int) -> bytes:
    n = torch.zeros(1, dtype=torch.int64)
    dist.recv(n, src)
    buf = torch.zeros(int(n.item()), dtype=torch.uint8)
    if int(n.item()):
        dist.recv(buf, src)
    return buf.numpy().tobytes()


def rows_of(pool: oracle.HostPool, blocks) -> bytes:
    """[layer][K|V][block] rows of the named pages, the data that follows a piece on the wire."""
    out = []
    for l in range(pool.n_layers):
        for arrs in (pool.k, pool.v):
            out.append(pool.block_view(arrs[l])[np.asarray(blocks, dtype=np.int64)].tobytes())
    return b"".join(out)


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    w = W.Workload("wire", LAYERS, HEADS, DIM, BS, 64, 64, np.array([150], dtype=np.uint32), seed=17).build_tables()
    hs, hd = host_pools(w)                                    # seeded: identical on both ranks
    n_blocks = (150 + BS - 1) // BS                           # 10 pages
    pieces = [(0, 3), (3, 3), (6, 2), (8, 2)]                 # (first logical block, count)
    lib = N.lib()
    if rank == 0:
        msgs = []
        for i, (b0, n) in enumerate(pieces):
            h = S.header(150, 99, 150, LAYERS, HEADS, DIM, BS, N.DTYPE_F16, b0, n, i, len(pieces), 7 if i == len(pieces) - 1 else 0)
            msgs.append(S.pack(h, w.src_tables[0, b0:b0 + n], np.arange(7, dtype=np.float32) if i == len(pieces) - 1 else ()))
        damaged = bytearray(msgs[2])
        damaged[70] ^= 0x40                                   # one bit inside the message: the checksum must catch it
        # batch 1: pieces 3 and 1 (out of order); batch 2: a damaged piece 2, then pieces 0 and 2
        for batch in ([(3, msgs[3]), (1, msgs[1])], [(2, bytes(damaged)), (0, msgs[0]), (2, msgs[2])]):
            send_bytes(S.frame([m for _, m in batch]), 1)
            for i, _ in batch:
                b0, n = pieces[i]
                send_bytes(rows_of(hs, w.src_tables[0, b0:b0 + n]), 1)
            ack = recv_bytes(1)                               # which pieces the receiver still lacks
            assert ack in (b"need 0 2", b"need "), ack
        dist.barrier()
    else:
        alloc = lib.tkv_page_allocator_new(64)
        table = lib.tkv_block_table_new(n_blocks)
        have, refused, logits, position = set(), 0, None, None
        row_bytes = BS * HEADS * DIM * 2
        for batch_no in range(2):
            for msg in S.unframe(recv_bytes(0)):
                rows = recv_bytes(0)
                try:
                    h, blocks, lg = S.unpack(msg)
                except N.TkvError as e:
                    assert e.code == N.ERR_INVALID_CONFIG and "corrupt" in e.message
                    refused += 1
                    continue
                assert (h.seq_len, h.seed, h.piece_count, h.n_layers, h.n_kv_heads, h.head_dim) == (150, 99, len(pieces), LAYERS, HEADS, DIM)
                position = h.position
                if h.n_logits:
                    logits = lg
                assert len(rows) == 2 * LAYERS * h.n_blocks * row_bytes
                at = 0
                dst_ids = []
                for i in range(h.n_blocks):                   # PageAllocator::allocate + BlockTable::set_block per page
                    page = C.c_size_t()
                    N.check(lib.tkv_page_allocator_allocate(alloc, C.byref(page)))
                    N.check(lib.tkv_block_table_set_block(table, h.block_begin + i, page.value))
                    dst_ids.append(page.value)
                for l in range(LAYERS):                       # the pages' rows land where the table now says
                    for arrs in (hd.k, hd.v):
                        chunk = np.frombuffer(rows[at:at + h.n_blocks * row_bytes], dtype=np.uint16).reshape(h.n_blocks, -1)
                        hd.block_view(arrs[l]).reshape(hd.total_blocks, -1)[np.asarray(dst_ids)] = chunk
                        at += h.n_blocks * row_bytes
                have.add(h.piece_index)
            # a partial transfer is visible as a partially filled block table
            filled = [lib.tkv_block_table_get_block(table, b, C.byref(C.c_size_t())) == 1 for b in range(n_blocks)]
            want = [any(p in have and pieces[p][0] <= b < pieces[p][0] + pieces[p][1] for p in range(len(pieces))) for b in range(n_blocks)]
            assert filled == want, (batch_no, filled)
            if batch_no == 0:
                assert have == {1, 3} and sum(filled) == 5 and lib.tkv_page_allocator_in_use(alloc) == 5
            missing = sorted(set(range(len(pieces))) - have)
            send_bytes(("need " + " ".join(map(str, missing))).encode(), 0)
        assert have == {0, 1, 2, 3} and refused == 1 and position == 150 and np.array_equal(logits, np.arange(7, dtype=np.float32))
        # the decode pool now equals one oracle handoff through the table the pieces built
        dst_table = np.array([[int(lib.tkv_block_table_as_slice(table)[b]) for b in range(n_blocks)]], dtype=np.uint32)
        _, want_pool = host_pools(w)
        oracle.handoff(hs, want_pool, oracle.make_batch(w.seq_lens, w.src_tables, dst_table, n_blocks), None, "copy")
        tail = 150 % BS                                       # the oracle leaves the last page's unused rows at the fill pattern
        for l in range(LAYERS):
            for got, ref in ((hd.k[l], want_pool.k[l]), (hd.v[l], want_pool.v[l])):
                g, r = hd.block_view(got).copy(), want_pool.block_view(ref)
                last = int(dst_table[0, n_blocks - 1])
                g[last, tail:] = r[last, tail:]               # whole pages travelled; only the valid rows are compared there
                assert np.array_equal(g, r)
        with open(os.environ["GLOO_RESULT"], "w") as f:
            f.write("OK wire pieces out of order, one refused and resent")
        lib.tkv_block_table_delete(table)
        lib.tkv_page_allocator_delete(alloc)
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
