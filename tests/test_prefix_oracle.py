"""The RadixTree oracle against the reference's own tests (engine/src/prefix_cache.rs:153-241, replayed
here with the same inputs and expectations), plus the two behaviours the device index is checked against."""
from oracle.prefix_oracle import RadixOracle


def test_insert_and_lookup():
    t = RadixOracle()
    t.insert([1, 2, 3], [10, 20, 30])
    n, pages, _ = t.lookup([1, 2, 3])
    assert n == 3 and len(pages) == 3 and t.hits == 1 and t.tokens_saved == 3


def test_partial_match():
    t = RadixOracle()
    t.insert([1, 2, 3, 4], [10, 20, 30, 40])
    assert t.lookup([1, 2, 5])[0] == 2


def test_no_match():
    t = RadixOracle()
    t.insert([1, 2, 3], [10, 20, 30])
    n, pages, _ = t.lookup([5, 6, 7])
    assert n == 0 and pages == []


def test_shared_prefix():
    t = RadixOracle()
    t.insert([1, 2, 3], [10, 20, 30])
    t.insert([1, 2, 4], [10, 20, 40])
    assert t.lookup([1, 2, 3])[0] == 3
    assert t.lookup([1, 2, 4])[0] == 3
    assert t.lookup([1, 2])[0] == 2


def test_multi_turn_reuse():
    t = RadixOracle()
    system = [100, 101, 102, 103]
    t.insert(system, [0, 1, 2, 3])
    turn1 = system + [200, 201]
    assert t.lookup(turn1)[0] == 4
    t.insert(turn1, [0, 1, 2, 3, 4, 5])
    assert t.lookup(turn1 + [300])[0] == 6


def test_ref_count_and_release():
    t = RadixOracle()
    t.insert([1, 2, 3], [10, 20, 30])
    t.lookup([1, 2, 3])
    t.lookup([1, 2, 3])
    t.release([1, 2, 3])
    assert t.hits == 2


def test_evict_lru():
    t = RadixOracle()
    t.insert([1, 2], [10, 20])
    t.insert([3, 4], [30, 40])
    t.lookup([3, 4])
    t.release([3, 4])
    assert t.evict_lru() != []


def test_reference_reports_an_unlinked_node_again_and_report_once_does_not():
    t = RadixOracle()
    t.insert([1, 2], [10, 20])
    assert t.evict_lru() == [20] and t.evict_lru() == [10] and t.evict_lru() == [10]   # prefix_cache.rs:99-125 as written: unlinked nodes stay eligible
    t = RadixOracle()
    t.insert([1, 2], [10, 20])
    assert t.evict_lru(report_once=True) == [20] and t.evict_lru(report_once=True) == [10] and t.evict_lru(report_once=True) == []


def test_groups_and_batches():
    t = RadixOracle(group=2)
    t.batch_insert([[1, 2, 3, 4, 5], [1, 2, 9, 9]], [[7, 8], [70, 80]])
    (n0, p0, _), (n1, p1, _) = t.batch_lookup([[1, 2, 3, 4], [1, 2, 9, 9, 5, 5]])
    assert (n0, p0) == (2, [7, 8]) and (n1, p1) == (2, [7, 80])      # the shared node keeps the first sequence's page
    assert t.tokens_saved == 8 and t.live_nodes() == 3


def test_page_stack_oracle_follows_the_reference_allocator():
    # kv_cache.rs:762-797: pops hand out 0, 1, 2 ...; a freed page is the next one handed out
    from oracle.prefix_oracle import PageStackOracle
    a = PageStackOracle(4)
    assert [a.allocate() for _ in range(3)] == [0, 1, 2] and a.available() == 1
    a.free(1)
    assert a.allocate() == 1 and a.allocate() == 3 and a.allocate() is None
    assert a.batch_allocate([1]) is None
    a.batch_free([[2, 0], [3]])
    assert a.batch_allocate([2, 1]) == [[3, 0], [2]]
