"""The handoff coordinator driving real device handoffs: requests are routed, prefilled (their K/V already sit in
the prefill pool), admitted against the decode pool's free pages, moved by the CUDA path and confirmed through the
completion flag; one request's completion never arrives (nothing sets its flag -- the failure is made on the host, the
device is not disturbed), so its wait runs out, the coordinator retries once, then falls back to re-prefill and its
pages go back to the allocator.  The decode pool must equal the oracle's handoff of exactly the completed requests."""
import ctypes as C
import time

import numpy as np
import pytest

import oracle
from helpers import assert_pool_equals_host, host_pools, to_device_pool
from tempura_b200 import _native as N
from tempura_b200 import workloads as W
from tempura_b200.coordinator import Coordinator

pytestmark = pytest.mark.gpu

BS = 16


def now_us() -> int:
    return time.monotonic_ns() // 1000


def test_coordinator_admits_moves_confirms_and_falls_back_on_a_lost_completion():
    import torch
    from tempura_b200 import handoff as H
    lens = np.array([40, 150, 300, 77], dtype=np.uint32)
    max_new = 20
    w = W.Workload("coordinated", 2, 8, 128, BS, 96, 40, lens, seed=5).build_tables()
    hs, hd = host_pools(w)
    ds, dd = to_device_pool(hs, "f16"), to_device_pool(hd, "f16")
    lib = N.lib()
    pages = lib.tkv_page_allocator_new(w.dst_blocks)              # 40 pages: the four requests (42 with their decode room) do not all fit
    coord = Coordinator(n_prefill=1, n_decode=1, block_size=BS, max_inflight_per_decode=2, max_retries=1, handoff_timeout=30_000)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")      # slot q: request q's completion flag
    lost = 2                                                       # this request's completion is never signalled
    for q, n in enumerate(lens):
        assert coord.submit(q, int(n), max_new_tokens=max_new) == 0
    while (rid := coord.next_prefill(0)) is not None:
        coord.prefill_done(rid)                                    # its K/V are in the prefill pool
    owned, dst_rows, done, gen = {}, {}, [], 0
    for _round in range(12):
        coord.set_headroom(0, lib.tkv_page_allocator_available(pages))
        for a in coord.admit():
            q = int(a.request_id)
            assert a.blocks == (int(lens[q]) + max_new + BS - 1) // BS and a.decode_worker == 0
            owned[q] = []
            for _i in range(a.blocks):                             # the allocator refuses when the pool is exhausted: admission must prevent that
                page = C.c_size_t()
                N.check(lib.tkv_page_allocator_allocate(pages, C.byref(page)))
                owned[q].append(page.value)
            dst_rows[q] = np.array(owned[q][: (int(lens[q]) + BS - 1) // BS], dtype=np.uint32)
        for q in sorted(owned):
            if coord.request(q).state != N.REQ_ADMITTED:
                continue
            coord.handoff_started(q, now=now_us())
            gen += 1
            if q != lost:
                nb = len(dst_rows[q])
                plan = H.Plan(ds, dd, H.Batch(lens[q:q + 1], w.src_tables[q, :nb], dst_rows[q], nb))
                plan.enqueue(done_flag=flags[q:].data_ptr(), flag_value=gen)
                H.flag_wait_host(0, flags[q:].data_ptr(), gen, 5_000_000)
                coord.handoff_complete(q)
                assert coord.request(q).state == N.REQ_DECODE
                done.append(q)
                plan.destroy()
                continue
            with pytest.raises(N.TkvError) as e:                   # the wait is bounded: it reports, nothing hangs
                H.flag_wait_host(0, flags[q:].data_ptr(), gen, 40_000)
            assert e.value.code == N.ERR_TIMEOUT
            assert coord.timed_out(now=now_us()) == [q]
            first_attempt = coord.request(q).attempts == 1
            action = coord.handoff_failed(q)
            if first_attempt:
                assert action == N.RETRY_HANDOFF and coord.request(q).state == N.REQ_ADMITTED
            else:                                                  # it keeps its decode worker and pages and is prefilled there
                assert action == N.REPREFILL and coord.request(q).state == N.REQ_REPREFILL
                coord.reprefill_done(q)
        for q in list(done):                                       # a finished request gives its pages back, which lets the waiting one in
            if q in owned and len(done) >= 2 and q == done[0]:
                coord.finish(q)
                for page in owned.pop(q):
                    lib.tkv_page_allocator_free(pages, page)
        if len(done) == 3 and coord.request(lost).state == N.REQ_DECODE:
            break
    st = coord.stats()
    assert sorted(done) == [0, 1, 3] and st.waiting == 0
    assert (st.handoffs_completed, st.handoffs_failed, st.retries, st.fallbacks) == (3, 2, 1, 1)
    assert coord.request(lost).state == N.REQ_DECODE and coord.request(lost).attempts == 2
    # the decode pool: exactly the completed requests' rows, through the pages the allocator handed out
    for q in done:                                                 # one oracle handoff per request, in the order the device ran them
        nb = len(dst_rows[q])                                      # (a finished request's pages may since have gone to a later one)
        oracle.handoff(hs, hd, oracle.make_batch(lens[q:q + 1], w.src_tables[q, :nb], dst_rows[q], nb), None, "copy")
    assert_pool_equals_host(dd, hd, "coordinated handoffs")
    assert_pool_equals_host(ds, hs, "prefill pool untouched")
    assert lib.tkv_page_allocator_in_use(pages) == sum(len(v) for v in owned.values())
    for q in list(owned):
        coord.finish(q)
        for page in owned.pop(q):
            lib.tkv_page_allocator_free(pages, page)
    assert coord.stats().in_system == 0 and lib.tkv_page_allocator_in_use(pages) == 0
    lib.tkv_page_allocator_delete(pages)
