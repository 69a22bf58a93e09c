"""The handoff coordinator's state machine on the host: routing, admission against decode-pool headroom, retries,
timeouts and the fallback to re-prefill, and a seeded run whose books must balance at every step."""
import numpy as np
import pytest

from tempura_b200 import _native as N
from tempura_b200.coordinator import Coordinator


def test_routing_goes_to_the_least_loaded_prefill_worker_and_priority_orders_its_queue():
    c = Coordinator(n_prefill=2, n_decode=2)
    assert [c.submit(1, 1000), c.submit(2, 100), c.submit(3, 100), c.submit(4, 100, priority=9)] == [0, 1, 1, 1]
    assert c.next_prefill(1) == 4 and c.next_prefill(1) == 2 and c.next_prefill(1) == 3 and c.next_prefill(1) is None
    assert c.next_prefill(0) == 1
    c.prefill_done(1)                                    # worker 0 is free again: the next prompt goes there
    assert c.submit(5, 50) == 0
    with pytest.raises(N.TkvError):
        c.submit(5, 50)                                  # already in the system
    with pytest.raises(N.TkvError):
        c.prefill_done(5)                                # still queued


def test_admission_waits_for_pages_and_prefers_the_paired_decode_worker():
    c = Coordinator(n_prefill=2, n_decode=2, block_size=16, headroom_blocks=4)
    for rid, n in ((1, 160), (2, 320), (3, 16)):
        c.submit(rid, n, max_new_tokens=16)
    for w in (0, 1):
        while (rid := c.next_prefill(w)) is not None:
            c.prefill_done(rid)
    assert c.admit() == []                               # no pool has reported free pages yet
    c.set_headroom(0, 14)                                # 10 usable after the headroom: fits only request 3 (2 blocks)
    c.set_headroom(1, 19)                                # 15 usable: request 1 (11 blocks); request 2 needs 21
    got = {a.request_id: (a.decode_worker, a.blocks) for a in c.admit()}
    assert got == {1: (1, 11), 3: (0, 2)}                # request 1's own partner (0) was too small; 3 went to its partner
    assert c.stats().reserved_blocks == 13 and c.stats().waiting == 1
    assert c.admit() == []                               # promised pages are not promised twice
    c.set_headroom(1, 40)
    a = c.admit()
    assert [(x.request_id, x.decode_worker, x.blocks) for x in a] == [(2, 1, 21)]
    for rid in (1, 2, 3):
        c.handoff_started(rid, now=0)
    assert c.stats().reserved_blocks == 0                # taken from the allocator now; the pools report the rest
    for rid in (1, 2, 3):
        c.handoff_complete(rid)
        assert c.request(rid).state == N.REQ_DECODE
        c.finish(rid)
    assert c.stats().in_system == 0 and c.stats().handoffs_completed == 3


def test_resident_prefix_shrinks_the_reservation():
    c = Coordinator(1, 1, block_size=16)
    c.submit(7, 2048 + 300, max_new_tokens=100)
    c.next_prefill(0)
    with pytest.raises(N.TkvError):
        c.prefill_done(7, prefix_tokens_resident=2050)   # not block-aligned
    c.prefill_done(7, prefix_tokens_resident=2048)
    c.set_headroom(0, 1000)
    (a,) = c.admit()
    assert a.blocks == (2048 + 300 + 100 + 15) // 16 - 128 and a.prefix_tokens == 2048


def test_inflight_limit_timeouts_retries_and_fallback():
    c = Coordinator(1, 1, block_size=16, max_inflight_per_decode=1, max_retries=1, handoff_timeout=100)
    c.set_headroom(0, 1000)
    for rid in (1, 2):
        c.submit(rid, 64)
        c.next_prefill(0)
        c.prefill_done(rid)
    assert [a.request_id for a in c.admit()] == [1]      # one handoff at a time into this worker
    c.handoff_started(1, now=1000)
    assert c.timed_out(now=1100) == [] and c.timed_out(now=1101) == [1]
    assert c.handoff_failed(1) == N.RETRY_HANDOFF and c.request(1).state == N.REQ_ADMITTED
    assert c.admit() == []                               # request 1 still holds the slot
    c.handoff_started(1, now=2000)
    assert c.handoff_failed(1) == N.REPREFILL and c.request(1).state == N.REQ_REPREFILL
    assert [a.request_id for a in c.admit()] == [2]      # the slot is free again
    with pytest.raises(N.TkvError):
        c.handoff_complete(1)
    c.reprefill_done(1)
    assert c.request(1).state == N.REQ_DECODE
    st = c.stats()
    assert (st.handoffs_failed, st.retries, st.fallbacks) == (2, 1, 1)
    c.finish(2)                                          # cancelled while admitted: slot and reservation go with it
    assert c.stats().reserved_blocks == 0 and c.request(2) is None


def test_seeded_run_keeps_the_books_balanced():
    rng = np.random.default_rng(3)
    c = Coordinator(n_prefill=3, n_decode=2, block_size=16, max_inflight_per_decode=4, max_retries=1, headroom_blocks=8, handoff_timeout=50)
    pool = [600, 400]                                     # free pages of the two decode pools, as their allocators would report
    held = {}                                             # request -> (decode worker, pages taken)
    now, next_id, done = 0, 0, 0
    for step in range(400):
        now += 1
        for _ in range(int(rng.integers(0, 3))):
            c.submit(next_id, int(rng.integers(1, 900)), int(rng.integers(0, 200)), int(rng.integers(0, 10)))
            next_id += 1
        for w in range(3):
            if rng.random() < 0.5 and (rid := c.next_prefill(w)) is not None:
                c.prefill_done(rid, 0)
        for d in range(2):
            c.set_headroom(d, pool[d])
        for a in c.admit():
            assert a.blocks + 8 <= pool[a.decode_worker]          # never promises pages the pool does not have
            pool[a.decode_worker] -= a.blocks
            held[a.request_id] = (a.decode_worker, a.blocks)
            c.set_headroom(a.decode_worker, pool[a.decode_worker])
            c.handoff_started(a.request_id, now)
        for rid in list(held):
            info = c.request(rid)
            if info.state == N.REQ_TRANSFER and rng.random() < 0.3:
                if rng.random() < 0.85:
                    c.handoff_complete(rid)
                elif c.handoff_failed(rid) == N.RETRY_HANDOFF:
                    c.handoff_started(rid, now)
                else:
                    c.reprefill_done(rid)
            elif info.state == N.REQ_DECODE and rng.random() < 0.2:
                d, blocks = held.pop(rid)
                pool[d] += blocks
                c.finish(rid)
                done += 1
        for rid in c.timed_out(now):
            if c.handoff_failed(rid) == N.RETRY_HANDOFF:
                c.handoff_started(rid, now)
            else:
                c.reprefill_done(rid)
        st = c.stats()
        assert st.reserved_blocks == 0 and st.in_system == next_id - done
        assert pool[0] + sum(b for d, b in held.values() if d == 0) == 600 and pool[1] + sum(b for d, b in held.values() if d == 1) == 400
    assert done > 50 and c.stats().fallbacks > 0 and c.stats().retries > 0
