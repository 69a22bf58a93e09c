"""CPU restatement of the reference's RadixTree (engine/src/prefix_cache.rs:17-149) — TEST
INFRASTRUCTURE ONLY: the checker for the device-resident prefix index; nothing in the product
imports it.  Pinned against the reference's own seven tests (prefix_cache.rs:153-241), which
tests/test_prefix_oracle.py replays.

``group`` > 1 treats every ``group`` consecutive tokens as one element (a node per KV block);
``batch_*`` methods apply one tick to several sequences, which is what one call of the device
index means.  ``evict_lru(report_once=True)`` is the stated departure the product makes: the
reference leaves an unlinked node eligible, so a second call reports its page again
(prefix_cache.rs:99-125); with ``report_once`` an unlinked node is never reported twice."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


class _Node:
    __slots__ = ("children", "page_ids", "ref_count", "last_used", "unlinked")

    def __init__(self, page_ids, last_used):
        self.children = {}
        self.page_ids = page_ids
        self.ref_count = 0
        self.last_used = last_used
        self.unlinked = False


class RadixOracle:
    def __init__(self, group: int = 1):
        self.group = group
        self.nodes: List[_Node] = [_Node([], 0)]          # prefix_cache.rs:18-30
        self.tick = 0
        self.hits = 0
        self.tokens_saved = 0

    def _elements(self, token_ids: Sequence[int]):
        g = self.group
        if g == 1:
            return list(token_ids)
        return [tuple(token_ids[i * g:(i + 1) * g]) for i in range(len(token_ids) // g)]

    # prefix_cache.rs:32-58
    def insert(self, token_ids, page_ids=(), tick: Optional[int] = None):
        self.tick = self.tick + 1 if tick is None else tick
        idx = 0
        for i, el in enumerate(self._elements(token_ids)):
            child = self.nodes[idx].children.get(el)
            if child is not None:
                idx = child
                self.nodes[idx].last_used = self.tick
            else:
                new = len(self.nodes)
                self.nodes.append(_Node([page_ids[i]] if i < len(page_ids) else [], self.tick))
                self.nodes[idx].children[el] = new
                idx = new

    # prefix_cache.rs:60-86; also returns one page slot per matched node (None when it has no page)
    def lookup(self, token_ids, tick: Optional[int] = None) -> Tuple[int, List[int], List[Optional[int]]]:
        self.tick = self.tick + 1 if tick is None else tick
        idx, matched, pages, per_node = 0, 0, [], []
        for el in self._elements(token_ids):
            child = self.nodes[idx].children.get(el)
            if child is None:
                break
            idx = child
            n = self.nodes[idx]
            n.last_used = self.tick
            n.ref_count += 1
            matched += 1
            pages.extend(n.page_ids)
            per_node.append(n.page_ids[0] if n.page_ids else None)
        if matched > 0:
            self.hits += 1
            self.tokens_saved += matched * self.group
        return matched, pages, per_node

    # prefix_cache.rs:88-97
    def release(self, token_ids):
        idx = 0
        for el in self._elements(token_ids):
            child = self.nodes[idx].children.get(el)
            if child is None:
                break
            idx = child
            self.nodes[idx].ref_count = max(self.nodes[idx].ref_count - 1, 0)

    # prefix_cache.rs:99-125
    def evict_lru(self, report_once: bool = False) -> List[int]:
        cand = [i for i, n in enumerate(self.nodes)
                if i != 0 and n.ref_count == 0 and not n.children and not (report_once and n.unlinked)]
        if not cand:
            return []
        oldest = min(cand, key=lambda i: self.nodes[i].last_used)      # first minimum = lowest index, as min_by_key
        for n in self.nodes:
            for k in [k for k, c in n.children.items() if c == oldest]:
                del n.children[k]
        self.nodes[oldest].unlinked = True
        return list(self.nodes[oldest].page_ids)

    def evict_lru_node(self) -> Tuple[bool, List[int]]:
        """``evict_lru(report_once=True)`` that also says whether a node was unlinked at all."""
        before = sum(n.unlinked for n in self.nodes)
        pages = self.evict_lru(report_once=True)
        return sum(n.unlinked for n in self.nodes) > before, pages

    def node_count(self) -> int:
        return len(self.nodes)

    def live_nodes(self) -> int:
        return sum(1 for n in self.nodes[1:] if not n.unlinked)

    # one tick for a whole batch, sequences in index order: the meaning of one device call
    def batch_insert(self, seqs, pages):
        self.tick += 1
        for s, p in zip(seqs, pages):
            self.insert(s, p, tick=self.tick)

    def batch_lookup(self, seqs):
        self.tick += 1
        return [self.lookup(s, tick=self.tick) for s in seqs]

    def batch_release(self, seqs):
        for s in seqs:
            self.release(s)


class PageStackOracle:
    """PageAllocator (engine/src/kv_cache.rs:762-797): a LIFO stack of free page ids, 0 on top at the start."""

    def __init__(self, total_pages: int):
        self.free_pages = list(range(total_pages))[::-1]      # (0..total).rev().collect()
        self.total = total_pages

    def allocate(self) -> Optional[int]:
        return self.free_pages.pop() if self.free_pages else None

    def free(self, page_id: int) -> None:
        self.free_pages.append(page_id)

    def available(self) -> int:
        return len(self.free_pages)

    # the device allocator's batch calls: sequences in index order, all or nothing
    def batch_allocate(self, counts: Sequence[int]) -> Optional[List[List[int]]]:
        if sum(counts) > len(self.free_pages):
            return None
        return [[self.allocate() for _ in range(c)] for c in counts]

    def batch_free(self, rows: Sequence[Sequence[int]]) -> None:
        for row in rows:
            for p in row:
                self.free(p)
