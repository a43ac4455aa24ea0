"""The cache manager: keys and values in pages with a block table per request,
one pool per group of layers with the same needs, and rows of fixed-size state
per request.

What it owns
  * the device pools: per group K and V pages, [executions, pages, page_size,
    kv_heads, head_dim] in the engine's dtype (the reference keeps two tensors
    [layers, slots, kv_heads, head_dim], ullm/core/kv_cache.py:79-89, with a
    "page" of one token);
  * per group a page allocator, and for a model whose only group keeps every
    token, a prefix tree over full pages (ullm/core/kv_cache.py:326-398 is the
    reference's manager: match at admission, insert at finish, evict on demand);
  * per request: a slot (row of every per-request array), per group the list
    of its pages, the count of tokens written;
  * device block tables [slots, pages per request] per group, kept up to date
    by small copies of the rows that changed;
  * the fixed-size state rows that mixers asked for, zeroed when a slot is
    handed out.

Groups: executions (schedule entries) with equal CacheNeed share a group; an
execution that reads another's cache has none of its own.  A group with a
window gives pages back as soon as every position in them is out of reach of
any later token; a finished request gives back everything (full pages of a
prefix-cached group go to the tree instead and stay findable until evicted).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed
from .pages import OutOfPages, PageAllocator, PrefixTree, SlotAllocator


logger = logging.getLogger("ullm_b200")


@dataclass
class GroupInfo:
    need: CacheNeed
    executions: list[int]  # schedule entries whose caches live in this group


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: str
    slot: int
    num_tokens: int = 0  # tokens whose keys/values are written (or reserved by the running step)
    pages: list[list[int]] = field(default_factory=list)  # per group; -1 where a window gave the page back
    first_live_page: list[int] = field(default_factory=list)  # per group
    prefix_nodes: list = field(default_factory=list)  # tree nodes this request holds (group 0 only)
    num_cached_tokens: int = 0  # tokens found in the prefix tree at admission


@dataclass
class LayerCache:
    """Handed to a mixer for one execution in one step."""

    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    group: "object | None"  # engine.batch.GroupStep of this execution's group
    writes: bool
    state: torch.Tensor | None  # [slots, *shape] or None


def plan_groups(needs) -> tuple[list[GroupInfo], list[tuple[int, int] | None]]:
    """needs: per schedule entry (CacheNeed | None, StateNeed | None, cache_of).
    Returns the groups and, per entry, (group, index inside the group) of the
    cache it uses (its own or the one it reads), or None."""
    groups: list[GroupInfo] = []
    where: list[tuple[int, int] | None] = []
    for i, (need, _state, cache_of) in enumerate(needs):
        if need is None:
            where.append(None)
            continue
        if cache_of is not None:
            src_need = needs[cache_of][0]
            if src_need is None or (src_need.num_kv_heads, src_need.head_dim) != (need.num_kv_heads, need.head_dim):
                raise ValueError(f"schedule entry {i} cannot read the cache of entry {cache_of}: different geometry")
            where.append(where[cache_of])
            continue
        for g, info in enumerate(groups):
            if info.need == need:
                info.executions.append(i)
                where.append((g, len(info.executions) - 1))
                break
        else:
            groups.append(GroupInfo(need, [i]))
            where.append((len(groups) - 1, 0))
    return groups, where


class CacheManager:
    def __init__(
        self,
        needs,
        page_size: int,
        num_pages: int,
        max_requests: int,
        max_pages_per_request: int,
        device=None,
        dtype: torch.dtype = torch.bfloat16,
        enable_prefix_cache: bool = True,
        poison: bool = False,
    ):
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_pages_per_request = max_pages_per_request
        self.device = torch.device(device) if device is not None else None
        self.dtype = dtype
        self.needs = list(needs)
        self.groups, self.where = plan_groups(self.needs)
        self.allocators = [PageAllocator(num_pages) for _ in self.groups]
        self.slots = SlotAllocator(max_requests)
        has_state = any(s is not None for _, s, _ in self.needs)
        only_full = len(self.groups) == 1 and self.groups[0].need.window is None
        self.tree = PrefixTree(page_size) if (enable_prefix_cache and only_full and not has_state) else None
        if enable_prefix_cache and self.tree is None:
            why = ("a mixer keeps per-request state" if has_state else
                   "a layer keeps only a window of its keys" if len(self.groups) == 1 else
                   f"the layers form {len(self.groups)} cache groups with different needs")
            logger.warning("prefix reuse is off for this model: %s (shared pages would have to hold what every "
                           "layer needs of a prefix)", why)
        self.requests: dict[str, RequestCache] = {}
        # device side
        self.k_pools: list[torch.Tensor] = []
        self.v_pools: list[torch.Tensor] = []
        self.block_tables: list[torch.Tensor] = []
        self.block_tables_host: list[torch.Tensor] = []
        self.states: dict[int, torch.Tensor] = {}
        self._dirty: list[list[tuple[int, int, int]]] = [[] for _ in self.groups]
        # pinned snapshots that the copies to the device read from, taken in turn (see flush_block_tables)
        self._flush_ring: list[torch.Tensor] = []
        self._flush_events: list = []
        self._flush_next = 0
        if self.device is not None:
            pin = self.device.type == "cuda"
            for g in self.groups:
                shape = (len(g.executions), num_pages, page_size, g.need.num_kv_heads, g.need.head_dim)
                k = torch.empty(shape, dtype=dtype, device=self.device)
                v = torch.empty(shape, dtype=dtype, device=self.device)
                if poison:
                    k.fill_(float("nan"))
                    v.fill_(float("nan"))
                else:
                    k.zero_()
                    v.zero_()
                self.k_pools.append(k)
                self.v_pools.append(v)
                self.block_tables.append(
                    torch.full((max_requests, max_pages_per_request), -1, dtype=torch.int32, device=self.device))
                self.block_tables_host.append(
                    torch.full((max_requests, max_pages_per_request), -1, dtype=torch.int32))
            n = max(1, len(self.groups)) * max_requests * max_pages_per_request
            self._flush_ring = [torch.empty(n, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
            self._flush_events = [torch.cuda.Event() if pin else None for _ in range(4)]
            for i, (_need, state, _c) in enumerate(self.needs):
                if state is not None:
                    self.states[i] = torch.zeros((max_requests, *state.shape), dtype=state.dtype, device=self.device)

    # -- sizes --------------------------------------------------------------
    @staticmethod
    def bytes_per_page(needs, page_size: int, itemsize: int) -> int:
        groups, _ = plan_groups(list(needs))
        return sum(2 * len(g.executions) * page_size * g.need.num_kv_heads * g.need.head_dim * itemsize
                   for g in groups)

    def num_free_pages(self, group: int = 0) -> int:
        return self.allocators[group].num_free

    def num_available_pages(self, group: int = 0) -> int:
        """Free pages plus what eviction of the prefix tree could return."""
        n = self.allocators[group].num_free
        if self.tree is not None and group == 0:
            n += self.tree.num_evictable()
        return n

    # -- a request's life -----------------------------------------------------
    def admit(self, request_id: str, tokens=None) -> RequestCache | None:
        """Gives the request a slot; None when every slot is taken.  With
        `tokens` and a prefix tree, full pages already holding a prefix of
        tokens[:-1] are taken over (at least one token is left to run)."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.slots.alloc()
        if slot is None:
            return None
        rc = RequestCache(request_id, slot, 0, [[] for _ in self.groups], [0 for _ in self.groups])
        if self.tree is not None and tokens is not None and len(tokens) > 1:
            nodes = self.tree.match(tokens, (len(tokens) - 1) // self.page_size)
            nodes = nodes[: self.max_pages_per_request]
            if nodes:
                self.tree.acquire(nodes)
                rc.prefix_nodes = nodes
                rc.pages[0] = [n.page for n in nodes]
                rc.num_tokens = rc.num_cached_tokens = len(nodes) * self.page_size
                self._mark(0, slot, 0, len(nodes), rc.pages[0])
        for st in self.states.values():
            st[slot].zero_()
        self.requests[request_id] = rc
        return rc

    def pages_needed(self, rc: RequestCache, n_new: int) -> list[int]:
        """Pages each group must add so that n_new more tokens have a place."""
        total = rc.num_tokens + n_new
        want = -(-total // self.page_size)
        return [max(0, want - len(p)) for p in rc.pages]

    def _fits_held_pages(self, rc: RequestCache, n_new: int) -> bool:
        """The common case of a decode step: the next tokens still fit the pages the request holds."""
        room = rc.num_tokens + n_new
        ps = self.page_size
        for p in rc.pages:
            if room > len(p) * ps:
                return False
        return True

    def can_reserve(self, rc: RequestCache, n_new: int) -> bool:
        if self._fits_held_pages(rc, n_new):
            return True
        if -(-(rc.num_tokens + n_new) // self.page_size) > self.max_pages_per_request:
            return False
        return all(n <= self.num_available_pages(g) for g, n in enumerate(self.pages_needed(rc, n_new)))

    def reserve(self, rc: RequestCache, n_new: int) -> None:
        """Makes room for tokens [num_tokens, num_tokens + n_new); evicts
        unreferenced prefix pages if the free list is short.  All or nothing."""
        if self._fits_held_pages(rc, n_new):
            return
        need = self.pages_needed(rc, n_new)
        if -(-(rc.num_tokens + n_new) // self.page_size) > self.max_pages_per_request:
            raise OutOfPages(f"request {rc.request_id!r} would exceed {self.max_pages_per_request} pages")
        for g, n in enumerate(need):
            short = n - self.allocators[g].num_free
            if short > 0 and self.tree is not None and g == 0:
                self.allocators[g].free(self.tree.evict(short))
            if n > self.allocators[g].num_free:
                raise OutOfPages(f"group {g}: {n} pages needed, {self.allocators[g].num_free} free")
        for g, n in enumerate(need):
            if n:
                new = self.allocators[g].alloc(n)
                start = len(rc.pages[g])
                rc.pages[g].extend(new)
                self._mark(g, rc.slot, start, start + n, rc.pages[g])

    def slot_mapping(self, rc: RequestCache, group: int, n_new: int) -> list[int]:
        """Flat slots (page * page_size + offset) of the next n_new tokens."""
        ps = self.page_size
        pages = rc.pages[group]
        if n_new <= 16:
            return [pages[p // ps] * ps + p % ps for p in range(rc.num_tokens, rc.num_tokens + n_new)]
        pos = np.arange(rc.num_tokens, rc.num_tokens + n_new, dtype=np.int64)
        first = rc.num_tokens // ps
        held = np.asarray(pages[first:(rc.num_tokens + n_new - 1) // ps + 1], dtype=np.int64)
        return held[pos // ps - first] * ps + pos % ps

    def commit(self, rc: RequestCache, n_new: int) -> None:
        """The step wrote n_new tokens.  Pages of windowed groups that no later
        token can reach are given back."""
        rc.num_tokens += n_new
        ps = self.page_size
        for g, info in enumerate(self.groups):
            w = info.need.window
            if w is None:
                continue
            # the next token sits at position num_tokens and sees positions >= num_tokens - w + 1
            first_needed = max(0, rc.num_tokens - w + 1) // ps
            lo = rc.first_live_page[g]
            if first_needed > lo:
                gone = [p for p in rc.pages[g][lo:first_needed] if p >= 0]
                self.allocators[g].free(gone)
                for i in range(lo, first_needed):
                    rc.pages[g][i] = -1
                self._mark(g, rc.slot, lo, first_needed, rc.pages[g])
                rc.first_live_page[g] = first_needed

    def publish(self, rc: RequestCache, tokens) -> None:
        """Makes the request's completed full pages findable by other requests
        while it is still running (`tokens`: the ids whose keys/values are
        written).  The request keeps holding them.  The reference publishes only
        at finish (ullm/core/kv_cache.py:358-398)."""
        if self.tree is None:
            return
        ps = self.page_size
        full = min(rc.num_tokens, len(tokens)) // ps
        while len(rc.prefix_nodes) < full:
            i = len(rc.prefix_nodes)
            parent = rc.prefix_nodes[-1] if rc.prefix_nodes else None
            node = self.tree.adopt(parent, tuple(tokens[i * ps:(i + 1) * ps]), rc.pages[0][i])
            if node is None:
                break  # someone else published this content first; ours stays private until release
            rc.prefix_nodes.append(node)

    def release(self, rc: RequestCache, tokens=None) -> None:
        """The request ends (finished, aborted or preempted): its slot and pages
        are given back.  With `tokens` (the ids whose keys/values are written)
        and a prefix tree, its full pages stay findable in the tree."""
        if self.requests.get(rc.request_id) is not rc:
            raise ValueError(f"request {rc.request_id!r} is not live (released twice?)")
        for g in range(len(self.groups)):
            pages = rc.pages[g]
            if g == 0 and self.tree is not None:
                held = len(rc.prefix_nodes)
                private = pages[held:]
                if tokens is not None:
                    full = min(rc.num_tokens, len(tokens)) // self.page_size
                    full = max(full, held)
                    dup = self.tree.insert(tokens, pages[:full], rc.prefix_nodes)
                    self.allocators[g].free(dup + pages[full:])
                else:
                    self.allocators[g].free(private)
                self.tree.release(rc.prefix_nodes)
            else:
                self.allocators[g].free([p for p in pages if p >= 0])
            self._mark(g, rc.slot, 0, len(pages), [-1] * len(pages))
        self.slots.free(rc.slot)
        del self.requests[rc.request_id]
        rc.pages = [[] for _ in self.groups]
        rc.prefix_nodes = []

    # -- device block tables -------------------------------------------------------
    def _mark(self, g: int, slot: int, a: int, b: int, pages: list[int]) -> None:
        if self.device is None or b <= a:
            return
        self.block_tables_host[g][slot, a:b] = torch.tensor(pages[a:b], dtype=torch.int32)
        self._dirty[g].append((slot, a, b))

    def flush_block_tables(self) -> None:
        """Copies the table rows that changed since the last call to the device
        (stream-ordered).  The copies read a pinned SNAPSHOT of the changed
        spans taken now, not the host mirror itself: `commit` and `release`
        write -1 into the mirror right after a step is launched, possibly
        before that step's copies have run, and the step must still see the
        table as it was when it was prepared.  A snapshot buffer is reused only
        after the copies that read it have run (its event)."""
        if self.device is None or not any(self._dirty):
            return
        k = self._flush_next
        self._flush_next = (k + 1) % len(self._flush_ring)
        if self._flush_events[k] is not None:
            self._flush_events[k].synchronize()
        snap = self._flush_ring[k]
        off = 0
        for g, dirty in enumerate(self._dirty):
            if not dirty:
                continue
            spans: dict[int, tuple[int, int]] = {}
            for slot, a, b in dirty:
                lo, hi = spans.get(slot, (a, b))
                spans[slot] = (min(lo, a), max(hi, b))
            for slot, (a, b) in spans.items():
                n = b - a
                snap[off:off + n] = self.block_tables_host[g][slot, a:b]
                self.block_tables[g][slot, a:b].copy_(snap[off:off + n], non_blocking=True)
                off += n
            dirty.clear()
        if self._flush_events[k] is not None:
            self._flush_events[k].record()

    # -- views for the model --------------------------------------------------------
    def layer_caches(self, group_steps) -> list[LayerCache]:
        out = []
        for i, (need, _state, cache_of) in enumerate(self.needs):
            w = self.where[i]
            st = self.states.get(i)
            if w is None:
                out.append(LayerCache(None, None, None, False, st))
                continue
            g, j = w
            out.append(LayerCache(self.k_pools[g][j], self.v_pools[g][j], group_steps[g], cache_of is None, st))
        return out

    # -- accounting, for tests -------------------------------------------------------
    def check_invariants(self) -> None:
        """Every page of every group is exactly one of: free, in the prefix tree,
        private to one live request."""
        for g, alloc in enumerate(self.allocators):
            owners: dict[int, str] = {}
            tree_pages = set(self.tree.pages()) if (self.tree is not None and g == 0) else set()
            if len(tree_pages) != (self.tree.num_pages if (self.tree is not None and g == 0) else 0):
                raise AssertionError("prefix tree holds a page twice")
            if self.tree is not None and g == 0 and self.tree.num_evictable() != self.tree.count_evictable_by_walk():
                raise AssertionError(f"prefix tree counts {self.tree.num_evictable()} evictable pages, a walk finds "
                                     f"{self.tree.count_evictable_by_walk()}")
            for p in tree_pages:
                owners[p] = "tree"
            for rc in self.requests.values():
                held = len(rc.prefix_nodes) if g == 0 else 0
                for i, p in enumerate(rc.pages[g]):
                    if p < 0:
                        continue
                    if i < held:
                        if p not in tree_pages:
                            raise AssertionError(f"request {rc.request_id}: shared page {p} is not in the tree")
                        continue
                    if p in owners:
                        raise AssertionError(f"page {p} of group {g} held twice ({owners[p]} and {rc.request_id})")
                    owners[p] = rc.request_id
            for p in owners:
                if not alloc.is_held(p):
                    raise AssertionError(f"page {p} of group {g} is owned by {owners[p]} but on the free list")
            if alloc.num_free + len(owners) != alloc.num_pages:
                raise AssertionError(
                    f"group {g}: {alloc.num_free} free + {len(owners)} owned != {alloc.num_pages} pages (a page is lost)")
