"""Prefix (radix) cache over the paged KV blocks: requests whose prompts start with the same tokens share the KV of the
common part instead of recomputing it.

The serving engine the reference drives keeps a radix tree over token sequences and reuses KV across requests — across
the samples of a prompt, and across the turns of a multi-turn rollout where every new prompt extends the previous
conversation (N5 in the component inventory; the reference only turns it off for bit-exact on-policy runs,
`--sglang-disable-radix-cache`).  Here the tree is BLOCK-granular: an edge is one block of `block_size` token ids, a node
owns the KV block that holds exactly those tokens after exactly that prefix.  Only full blocks are cached; the last,
partial block of a prompt is always computed by its request.

Ownership.  The tree holds one allocator reference per node, so a cached block survives the request that computed it.
A request that matches a prefix takes its own reference on every matched block (they appear in its block table) and pins
the nodes (`users`) until it finishes; eviction removes least-recently-used LEAVES nobody pins and gives their blocks back
to the allocator.  `reset()` drops everything — required whenever the weights change, since cached KV belongs to the old
weights.
"""
from __future__ import annotations

import itertools


class _Node:
    __slots__ = ("block", "children", "parent", "key", "users", "last_used")

    def __init__(self, block, parent, key):
        self.block, self.parent, self.key = block, parent, key
        self.children: dict[tuple, _Node] = {}
        self.users = 0
        self.last_used = 0


class PrefixCache:
    def __init__(self, allocator, block_size: int):
        self.allocator, self.bs = allocator, block_size
        self.root = _Node(None, None, None)
        self.clock = itertools.count(1)
        self.num_nodes = 0
        self.num_unpinned = 0                 # nodes nobody uses; kept incrementally: the scheduler asks every step
        self.stats = {"hit_tokens": 0, "lookup_tokens": 0, "inserted_blocks": 0, "evicted_blocks": 0}

    # ---- lookup ------------------------------------------------------------------------------------------------
    def match(self, tokens: list[int], max_blocks: int | None = None) -> list[_Node]:
        """Nodes of the longest cached chain of full blocks at the start of `tokens` (at most `max_blocks`)."""
        bs, node, out = self.bs, self.root, []
        limit = len(tokens) // bs if max_blocks is None else min(max_blocks, len(tokens) // bs)
        for i in range(limit):
            child = node.children.get(tuple(tokens[i * bs:(i + 1) * bs]))
            if child is None:
                break
            out.append(child)
            node = child
        return out

    def acquire(self, tokens: list[int], max_blocks: int | None = None) -> list[_Node]:
        """`match` + pin: the caller's request now uses these blocks (one allocator reference each is taken for it)."""
        nodes = self.match(tokens, max_blocks)
        t = next(self.clock)
        for n in nodes:
            self._pin(n)
            n.last_used = t
        if nodes:
            self.allocator.share([n.block for n in nodes])
        self.stats["hit_tokens"] += len(nodes) * self.bs
        self.stats["lookup_tokens"] += len(tokens)
        return nodes

    def unpin(self, nodes: list[_Node]) -> None:
        """The request is done with the matched nodes (its allocator references are released by the caller as usual)."""
        for n in nodes:
            n.users -= 1
            if n.users == 0 and n.parent is not None:       # nodes dropped by `reset` are no longer counted
                self.num_unpinned += 1

    def _pin(self, n: _Node) -> None:
        if n.users == 0 and n.parent is not None:
            self.num_unpinned -= 1
        n.users += 1

    # ---- insertion -----------------------------------------------------------------------------------------------
    def insert(self, tokens: list[int], blocks: list[int]) -> list[_Node]:
        """Register the full blocks of a sequence whose KV sits in `blocks` (block i holds tokens [i·bs, (i+1)·bs)).
        Chains that exist are kept (first writer wins: the KV is identical by construction).  Returns the WHOLE chain of
        nodes for this sequence; a live request pins all of them — also those that own another request's block for the
        same content — so that pinned nodes always form a prefix of the tree and "unpinned" means "evictable"."""
        bs, node, chain = self.bs, self.root, []
        t = next(self.clock)
        for i in range(min(len(tokens) // bs, len(blocks))):
            key = tuple(tokens[i * bs:(i + 1) * bs])
            child = node.children.get(key)
            if child is None:
                child = _Node(blocks[i], node, key)
                node.children[key] = child
                self.allocator.share([blocks[i]])
                self.num_nodes += 1
                self.num_unpinned += 1
                self.stats["inserted_blocks"] += 1
            chain.append(child)
            child.last_used = t
            node = child
        return chain

    def pin(self, nodes: list[_Node]) -> None:
        for n in nodes:
            self._pin(n)

    # ---- eviction -------------------------------------------------------------------------------------------------
    def evictable(self) -> int:
        """Blocks that could be freed now.  Requests pin prefixes of the tree, so a node nobody pins has no pinned node below
        it: every unpinned node can go (leaves first)."""
        return self.num_unpinned

    def evict(self, num_blocks: int) -> int:
        """Free up to `num_blocks` blocks, least recently used leaves first.  Returns how many were freed."""
        freed = 0
        while freed < num_blocks:
            leaves = [n for n in self._leaves() if n.users == 0]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.last_used)
            for n in leaves:
                if freed >= num_blocks:
                    break
                del n.parent.children[n.key]
                self.allocator.release([n.block])
                self.num_nodes -= 1
                self.num_unpinned -= 1
                freed += 1
        self.stats["evicted_blocks"] += freed
        return freed

    def _leaves(self):
        stack, out = [self.root], []
        while stack:
            n = stack.pop()
            if not n.children and n is not self.root:
                out.append(n)
            stack.extend(n.children.values())
        return out

    def reset(self) -> int:
        """Drop every cached block (weights changed, cache flushed).  Pinned nodes lose their place in the tree; the requests
        that use them keep their own references and finish normally."""
        n = 0
        stack = list(self.root.children.values())
        while stack:
            node = stack.pop()
            stack.extend(node.children.values())
            self.allocator.release([node.block])
            node.parent = None
            n += 1
        self.root = _Node(None, None, None)
        self.num_nodes = 0
        self.num_unpinned = 0
        return n
