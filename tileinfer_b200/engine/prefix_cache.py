"""Prefix cache: a trie over full KV blocks, plus which nodes own a DeltaNet state snapshot.

Keeps the reference's keying (one trie level per block of 16 token ids, so a node identifies the
whole prefix and RoPE positions stay valid; engine/prefix_cache.py:1-8, 51-100).  Differences:

* The cache holds its own reference on every cached block, so a block outlives the sequence that
  produced it and is released only by LRU eviction (`evict`).
* Only blocks that have actually been prefilled are inserted.
* A prefix is reusable only up to the deepest node that also has a recurrent-state snapshot; the
  hybrid model cannot resume from KV blocks alone.
"""
from __future__ import annotations

from itertools import count


class PrefixNode:
    __slots__ = ("node_id", "parent", "key", "block_id", "children", "last_used", "has_state", "depth")
    _ids = count(1)

    def __init__(self, parent, key, block_id, depth):
        self.node_id = next(PrefixNode._ids)
        self.parent, self.key, self.block_id, self.depth = parent, key, block_id, depth
        self.children = {}
        self.last_used = 0
        self.has_state = False


class PrefixCache:
    def __init__(self, block_size: int, block_manager=None):
        self.block_size = block_size
        self.bm = block_manager
        self.root = PrefixNode(None, None, -1, 0)
        self.nodes = {}                 # node_id -> node
        self._clock = 0
        self.on_node_evicted = None     # callable(node_id)
        self.hits = 0
        self.hit_tokens = 0
        self.queries = 0

    def __len__(self):
        return len(self.nodes)

    def _tick(self):
        self._clock += 1
        return self._clock

    def match(self, token_ids: list, max_tokens: int) -> list:
        """Longest chain of cached nodes covering at most `max_tokens` tokens."""
        bs = self.block_size
        node, chain = self.root, []
        for i in range(min(max_tokens, len(token_ids)) // bs):
            child = node.children.get(tuple(token_ids[i * bs:(i + 1) * bs]))
            if child is None:
                break
            chain.append(child)
            node = child
        return chain

    def find_longest_prefix(self, token_ids: list, max_tokens: int | None = None):
        """(nodes, num_tokens) of the longest reusable prefix: KV blocks AND a state snapshot."""
        self.queries += 1
        if max_tokens is None:
            max_tokens = len(token_ids) - 1
        chain = self.match(token_ids, max_tokens)
        while chain and not chain[-1].has_state:
            chain.pop()
        if not chain:
            return [], 0
        t = self._tick()
        for n in chain:
            n.last_used = t
        self.hits += 1
        self.hit_tokens += len(chain) * self.block_size
        return chain, len(chain) * self.block_size

    def insert(self, token_ids: list, block_table: list, num_full_blocks: int) -> list:
        """Register the first `num_full_blocks` prefilled blocks.  Returns the node chain."""
        bs = self.block_size
        node, chain, t = self.root, [], self._tick()
        for i in range(min(num_full_blocks, len(block_table))):
            key = tuple(token_ids[i * bs:(i + 1) * bs])
            if len(key) < bs:
                break
            child = node.children.get(key)
            if child is None:
                child = PrefixNode(node, key, block_table[i], i + 1)
                node.children[key] = child
                self.nodes[child.node_id] = child
                if self.bm is not None:
                    self.bm.incref(child.block_id)
            child.last_used = t
            chain.append(child)
            node = child
        return chain

    def mark_state(self, node_id: int, has_state: bool = True):
        n = self.nodes.get(node_id)
        if n is not None:
            n.has_state = has_state

    # ---- eviction -----------------------------------------------------------
    def _evictable_leaves(self):
        return [n for n in self.nodes.values()
                if not n.children and (self.bm is None or self.bm.ref_count[n.block_id] == 1)]

    def num_evictable(self) -> int:
        """Blocks that eviction could free now or after their descendants go (cache-only references)."""
        if self.bm is None:
            return len(self.nodes)
        # a node is releasable when it and its whole subtree are referenced by the cache alone
        memo = {}

        def ok(n):
            r = memo.get(n.node_id)
            if r is None:
                r = self.bm.ref_count[n.block_id] == 1 and all(ok(c) for c in n.children.values())
                memo[n.node_id] = r
            return r
        return sum(1 for n in self.nodes.values() if ok(n))

    def evict(self, num_blocks: int) -> int:
        freed = 0
        while freed < num_blocks:
            leaves = self._evictable_leaves()
            if not leaves:
                break
            leaves.sort(key=lambda n: n.last_used)
            for n in leaves:
                self._drop(n)
                freed += 1
                if freed >= num_blocks:
                    break
        return freed

    def _drop(self, n: PrefixNode):
        del n.parent.children[n.key]
        del self.nodes[n.node_id]
        if self.on_node_evicted is not None:
            self.on_node_evicted(n.node_id)
        if self.bm is not None:
            self.bm.decref(n.block_id)

    def clear(self):
        while self.nodes:
            if not self.evict(len(self.nodes)):
                break
