"""Page and slot bookkeeping on the host: a free list of page ids
(ullm/core/kv_cache.py:118-134 keeps the same kind of LIFO list over token
slots) and a prefix tree over full pages (ullm/core/kv_cache.py:137-323 keeps a
radix tree over single tokens).

Nothing here touches the device.
"""

from __future__ import annotations

import heapq
import itertools


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    """LIFO free list of page ids with ownership checks: a page is either free
    or held; freeing a free page or an unknown page is an error."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(reversed(range(num_pages)))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list[int] | None:
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} freed twice")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, p: int) -> bool:
        return self._held[p]


class SlotAllocator:
    """Request slots 0..n-1: rows of every fixed-size per-request array
    (ullm/core/req_state.py:14-16 keeps `free_indices` for the same purpose)."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(reversed(range(n)))
        self._held = [False] * n

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int | None:
        if not self._free:
            return None
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, s: int) -> None:
        if not self._held[s]:
            raise ValueError(f"slot {s} released twice")
        self._held[s] = False
        self._free.append(s)


class _Node:
    __slots__ = ("key", "page", "parent", "children", "ref", "stamp", "uid")

    def __init__(self, key, page, parent, uid):
        self.key = key
        self.page = page
        self.parent = parent
        self.children: dict[tuple, "_Node"] = {}
        self.ref = 0
        self.stamp = 0
        self.uid = uid


class PrefixTree:
    """Full pages of finished (or preempted) requests, findable by content.

    One node per page; a node's key is the tuple of the page's token ids and
    its path from the root is the token prefix it completes.  A node with
    ref > 0 is in use by a live request; nodes with ref == 0 and no children
    are evictable, least recently used first.  The tree owns the pages of its
    nodes: they are neither free nor private."""

    def __init__(self, page_size: int):
        self.page_size = page_size
        self.root = _Node((), -1, None, 0)
        self._uid = itertools.count(1)
        self._clock = itertools.count(1)
        self._heap: list[tuple[int, int, _Node]] = []
        self.num_pages = 0
        self._num_unreferenced = 0  # nodes with ref == 0, kept as references come and go

    def _touch(self, node: _Node) -> None:
        node.stamp = next(self._clock)
        if node.ref == 0 and not node.children:
            heapq.heappush(self._heap, (node.stamp, node.uid, node))
            # Entries are only taken out by evictions; a server with room to spare never evicts, and every
            # release adds one.  When stale entries outnumber the tree's pages several times over, the heap is
            # rebuilt from the unreferenced leaves that exist now.
            if len(self._heap) > 4 * self.num_pages + 1024:
                self._rebuild_heap()

    def _rebuild_heap(self) -> None:
        live, stack = [], [self.root]
        while stack:
            n = stack.pop()
            for c in n.children.values():
                if c.ref == 0 and not c.children:
                    live.append((c.stamp, c.uid, c))
                stack.append(c)
        heapq.heapify(live)
        self._heap = live

    def match(self, tokens, max_pages: int) -> list[_Node]:
        """Nodes of the longest chain of full pages that prefixes `tokens`,
        at most `max_pages` of them.  Takes no references."""
        ps = self.page_size
        node, out = self.root, []
        for i in range(min(max_pages, len(tokens) // ps)):
            child = node.children.get(tuple(tokens[i * ps:(i + 1) * ps]))
            if child is None:
                break
            out.append(child)
            node = child
        return out

    def acquire(self, nodes: list[_Node]) -> None:
        for n in nodes:
            if n.ref == 0:
                self._num_unreferenced -= 1
            n.ref += 1
            n.stamp = next(self._clock)

    def release(self, nodes: list[_Node]) -> None:
        for n in reversed(nodes):
            if n.ref <= 0:
                raise ValueError("prefix node released more often than acquired")
            n.ref -= 1
            if n.ref == 0:
                self._num_unreferenced += 1
            self._touch(n)

    def insert(self, tokens, pages: list[int], have: list[_Node]) -> list[int]:
        """Adds the full pages `pages` (page i holds tokens [i*ps, (i+1)*ps))
        below the chain `have` (nodes the caller already holds for pages
        0..len(have)-1).  Returns the pages that were NOT adopted because the
        tree already holds that content: the caller frees them."""
        ps = self.page_size
        node = have[-1] if have else self.root
        dup: list[int] = []
        for i in range(len(have), len(pages)):
            key = tuple(tokens[i * ps:(i + 1) * ps])
            child = node.children.get(key)
            if child is None:
                child = _Node(key, pages[i], node, next(self._uid))
                node.children[key] = child
                self.num_pages += 1
                self._num_unreferenced += 1
            else:
                dup.append(pages[i])
            self._touch(child)
            node = child
        return dup

    def adopt(self, parent: "_Node | None", key: tuple, page: int) -> "_Node | None":
        """Adds one page below `parent` (None: the root) on behalf of a live
        request, which holds it from the start (ref 1).  Returns None when that
        content is already in the tree (the caller keeps its page private)."""
        node = parent if parent is not None else self.root
        if key in node.children:
            return None
        child = _Node(key, page, node, next(self._uid))
        child.ref = 1
        child.stamp = next(self._clock)
        node.children[key] = child
        self.num_pages += 1
        return child

    def evict(self, n: int) -> list[int]:
        """Removes up to n unreferenced leaves, least recently used first, and
        returns their pages."""
        out: list[int] = []
        while len(out) < n and self._heap:
            stamp, _, node = heapq.heappop(self._heap)
            if node.stamp != stamp or node.ref != 0 or node.children or node.parent is None:
                continue  # stale entry
            if node.parent.children.get(node.key) is not node:
                continue
            del node.parent.children[node.key]
            parent = node.parent
            node.parent = None
            self.num_pages -= 1
            self._num_unreferenced -= 1
            out.append(node.page)
            if parent is not self.root and parent.ref == 0 and not parent.children:
                heapq.heappush(self._heap, (parent.stamp, parent.uid, parent))
        return out

    def num_evictable(self) -> int:
        """Pages that eviction could return now: the nodes of unreferenced subtrees.  A request holds the whole
        chain from the root to its last node, so a node that nobody holds has no held descendant either, and the
        count is simply the number of unreferenced nodes, which is kept as references come and go (this is asked
        for every running request in every step)."""
        return self._num_unreferenced

    def count_evictable_by_walk(self) -> int:
        """The same number from a walk over the whole tree (tests compare the two)."""

        def walk(node) -> tuple[int, bool]:
            total, all_free = 0, True
            for c in node.children.values():
                t, f = walk(c)
                total += t
                all_free = all_free and f
            if node is self.root:
                return total, False
            if all_free and node.ref == 0:
                return total + 1, True
            return total, False

        return walk(self.root)[0]

    def pages(self) -> list[int]:
        out, stack = [], [self.root]
        while stack:
            n = stack.pop()
            for c in n.children.values():
                out.append(c.page)
                stack.append(c)
        return out
