"""The cache manager: pages of keys and values with a block table per request, one pool
per group of layers with the same need, and slots for per-request state of fixed size.

What the reference has (crates/sglang-srt/src/cache.rs:340-473): fixed-size pages handed
out whole, so that two requests never share a partly filled page (:397-447); a request's
tail page is filled before a new one is taken (:406-414); an allocation that cannot be
met consumes nothing and says how much was asked and how much was free (:417-422); pages
that come back are used again before pages that were never used (:464-466).  State slots
follow crates/sglang-srt/src/recurrent_state.rs:23-101 (a free list of slot ids, a slot
zeroed when it is assigned, given back when the request ends).

Here a page is the unit (not a token slot), pages are reference-counted so that a prefix
tree can share full pages between requests, and layers are grouped by need: all layers
that keep every key share one block table per request; layers that keep only a window
share another, whose pages are given back as soon as the window has passed them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, PagedKV, RequestState

GroupKey = Hashable        # ("kv", window) with window None for "all keys"


class OutOfPages(RuntimeError):
    def __init__(self, group: GroupKey, requested: int, available: int):
        self.group, self.requested, self.available = group, requested, available
        super().__init__(f"cache group {group}: {requested} pages requested, {available} free")


class OutOfStateSlots(RuntimeError):
    pass


class PageAllocator:
    """Reference-counted pages of one group.  The free list is a stack: a page that was
    just given back is the next one handed out."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() yields 0, 1, 2, ...
        self._refs: List[int] = [0] * self.num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self, count: int, group: GroupKey = None) -> List[int]:
        if count > len(self._free):
            raise OutOfPages(group, count, len(self._free))
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            self._refs[page] = 1
        return pages

    def retain(self, page: int) -> None:
        if self._refs[page] <= 0:
            raise RuntimeError(f"page {page} is free and cannot be shared")
        self._refs[page] += 1

    def release(self, page: int) -> bool:
        """Drops one reference; True if the page went back to the free list."""
        if not 0 <= page < self.num_pages or self._refs[page] <= 0:
            raise RuntimeError(f"page {page} is freed twice or was never handed out")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False

    def refcount(self, page: int) -> int:
        return self._refs[page]


class StateSlotPool:
    """Slots for per-request state of fixed size; capacity = the most requests that run."""

    def __init__(self, capacity: int):
        self.capacity = int(capacity)
        self._free: List[int] = list(range(self.capacity - 1, -1, -1))
        self._used: set = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    def assign(self) -> int:
        if not self._free:
            raise OutOfStateSlots(f"all {self.capacity} state slots are in use")
        slot = self._free.pop()
        self._used.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._used:
            raise RuntimeError(f"state slot {slot} is freed twice or was never assigned")
        self._used.remove(slot)
        self._free.append(slot)


@dataclass
class PagedLayerCache:
    """What a mixer with a :class:`PagedKV` need is handed for one layer call."""
    group: GroupKey
    k_pool: Optional[torch.Tensor]      # [pages, kv_heads, page_size, head_dim]
    v_pool: Optional[torch.Tensor]
    writable: bool = True

    def read_only(self) -> "PagedLayerCache":
        return PagedLayerCache(self.group, self.k_pool, self.v_pool, False)


@dataclass
class StateLayerCache:
    """What a mixer with a :class:`RequestState` need is handed: ``state[slot]`` is the
    request's state; the step's ``state_slots`` gives each request's slot."""
    state: Optional[torch.Tensor]       # [slots, *shape]
    writable: bool = True

    def read_only(self) -> "StateLayerCache":
        return StateLayerCache(self.state, False)


@dataclass
class RequestCache:
    """A live request's hold on the cache."""
    request_id: Hashable
    length: int = 0                                   # tokens whose keys and values are stored
    tables: Dict[GroupKey, List[int]] = field(default_factory=dict)   # logical page -> page id, -1 = given back
    state_slot: int = -1
    shared_prefix_pages: int = 0                      # leading pages that came from the prefix tree
    closed: bool = False


def group_key(need: PagedKV) -> GroupKey:
    return ("kv", need.window)


class CacheManager:
    #: pages freed at once when cached prefixes have to make room
    EVICT_AHEAD = 32

    def __init__(self, needs: Sequence[CacheNeed], *, page_size: int, max_tokens: int, max_requests: int,
                 device=None, dtype: torch.dtype = torch.bfloat16,
                 pages_per_group: Optional[Dict[GroupKey, int]] = None):
        """``needs``: one entry per layer call of the model's program (None: no cache).
        ``max_tokens``: tokens the live requests may hold together; every paged group gets
        ``ceil(max_tokens / page_size)`` pages unless ``pages_per_group`` says otherwise.
        ``device`` None keeps the books only (no storage), for host-side tests."""
        if page_size <= 0:
            raise ValueError("page size must be positive")
        self.page_size, self.max_requests = int(page_size), int(max_requests)
        self.device, self.dtype = device, dtype
        self.needs = list(needs)
        default_pages = max(1, -(-int(max_tokens) // self.page_size))
        self.allocators: Dict[GroupKey, PageAllocator] = {}
        self.windows: Dict[GroupKey, Optional[int]] = {}
        for need in self.needs:
            if isinstance(need, PagedKV):
                key = group_key(need)
                if key not in self.allocators:
                    count = (pages_per_group or {}).get(key, default_pages)
                    self.allocators[key] = PageAllocator(count)
                    self.windows[key] = need.window
        self.state_pool = StateSlotPool(self.max_requests)
        self.has_state = any(isinstance(need, RequestState) for need in self.needs)
        self.layer_caches: List[object] = []
        for need in self.needs:
            if isinstance(need, PagedKV):
                key = group_key(need)
                pools = (None, None)
                if device is not None:
                    # one page more than the allocator owns: rows that pad a captured step write there
                    shape = (self.allocators[key].num_pages + 1, need.num_kv_heads, self.page_size, need.head_dim)
                    pools = (torch.zeros(shape, dtype=dtype, device=device),
                             torch.zeros(shape, dtype=dtype, device=device))
                self.layer_caches.append(PagedLayerCache(key, *pools))
            elif isinstance(need, RequestState):
                state = None
                if device is not None:
                    state = torch.zeros((self.max_requests, *need.shape), dtype=need.dtype or dtype, device=device)
                self.layer_caches.append(StateLayerCache(state))
            elif need is None:
                self.layer_caches.append(None)
            else:
                raise TypeError(f"unknown cache need {need!r}")
        self.live: Dict[Hashable, RequestCache] = {}
        self.prefix_tree = None

    # ------------------------------------------------------------------ prefix reuse
    def prefix_reuse_possible(self) -> bool:
        """Full pages can be shared only if every layer keeps all its keys in pages: a window
        gives pages back, and state of fixed size cannot be rebuilt from shared pages (the
        reference switches its prefix cache off for such models,
        crates/sglang-srt/src/models/mod.rs:508-516)."""
        return (not self.has_state and list(self.allocators) == [("kv", None)])

    def enable_prefix_reuse(self):
        from .radix import PrefixTree
        if not self.prefix_reuse_possible():
            raise ValueError("this model's cache cannot share prefixes")
        key = ("kv", None)
        self.prefix_tree = PrefixTree(self.page_size, self.allocators[key])
        return self.prefix_tree

    def _reclaim(self, key: GroupKey, shortfall: int) -> None:
        if self.prefix_tree is not None and key == ("kv", None) and shortfall > 0:
            # a search of the tree costs as much for one page as for many: take some ahead
            self.prefix_tree.evict(max(shortfall, self.EVICT_AHEAD))

    def _reclaimable(self, key: GroupKey) -> int:
        return self.prefix_tree.evictable() if self.prefix_tree is not None and key == ("kv", None) else 0

    # ------------------------------------------------------------------ requests
    def open(self, request_id: Hashable) -> RequestCache:
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        if len(self.live) >= self.max_requests:
            raise OutOfStateSlots(f"{self.max_requests} requests are live already")
        handle = RequestCache(request_id, tables={key: [] for key in self.allocators})
        handle.state_slot = self.state_pool.assign()
        if self.has_state and self.device is not None:
            for cache in self.layer_caches:
                if isinstance(cache, StateLayerCache):
                    cache.state[handle.state_slot].zero_()       # a new request starts from zero state
        self.live[request_id] = handle
        return handle

    def first_kept_position(self, key: GroupKey, length: int) -> int:
        """The first position whose key a query at position >= ``length`` can still see."""
        window = self.windows[key]
        return 0 if window is None else max(0, length - window + 1)

    def pages_needed(self, handle: RequestCache, tokens: int) -> Dict[GroupKey, int]:
        need = -(-(handle.length + tokens) // self.page_size)
        return {key: max(0, need - len(table)) for key, table in handle.tables.items()}

    def can_reserve(self, handle: RequestCache, tokens: int, spare: Optional[Dict[GroupKey, int]] = None) -> bool:
        spare = spare or {}
        for key, count in self.pages_needed(handle, tokens).items():
            free = self.allocators[key].free_count - spare.get(key, 0)
            if count > free and count > free + self._reclaimable(key):
                return False
        return True

    def reserve(self, handle: RequestCache, tokens: int) -> None:
        """Makes room for ``tokens`` more tokens in every group, or changes nothing and
        raises :class:`OutOfPages`."""
        if handle.closed:
            raise RuntimeError(f"request {handle.request_id!r} has ended")
        needed = self.pages_needed(handle, tokens)
        for key, count in needed.items():
            if count > self.allocators[key].free_count:
                self._reclaim(key, count - self.allocators[key].free_count)     # pages only the prefix tree holds
            if count > self.allocators[key].free_count:
                raise OutOfPages(key, count, self.allocators[key].free_count)
        for key, count in needed.items():
            handle.tables[key].extend(self.allocators[key].allocate(count, key))

    def trim_reservation(self, handle: RequestCache) -> None:
        """Gives back pages that were reserved beyond what the stored tokens need (a step
        that did not run)."""
        keep = -(-handle.length // self.page_size)
        for key, table in handle.tables.items():
            while len(table) > keep:
                page = table.pop()
                if page >= 0:
                    self.allocators[key].release(page)

    def commit(self, handle: RequestCache, tokens: int) -> None:
        """``tokens`` more tokens are stored; pages a window has passed are given back."""
        handle.length += tokens
        if handle.length > self.capacity(handle):
            raise RuntimeError("more tokens were stored than pages were reserved for")
        for key, table in handle.tables.items():
            first = self.first_kept_position(key, handle.length)
            for logical in range(min(len(table), first // self.page_size)):
                if table[logical] >= 0:
                    self.allocators[key].release(table[logical])
                    table[logical] = -1

    def capacity(self, handle: RequestCache) -> int:
        return min((len(table) * self.page_size for table in handle.tables.values()), default=1 << 62)

    def close(self, handle: RequestCache) -> None:
        if handle.closed:
            raise RuntimeError(f"request {handle.request_id!r} is ended twice")
        for key, table in handle.tables.items():
            for page in table:
                if page >= 0:
                    self.allocators[key].release(page)
            table.clear()
        self.state_pool.release(handle.state_slot)
        handle.closed = True
        del self.live[handle.request_id]

    # ------------------------------------------------------------------ sharing (prefix tree)
    def adopt_prefix(self, handle: RequestCache, key: GroupKey, pages: Sequence[int]) -> None:
        """Starts a new request on full pages that another owner already holds."""
        if handle.length or handle.tables[key]:
            raise RuntimeError("a prefix can only be adopted by a request that holds nothing yet")
        for page in pages:
            self.allocators[key].retain(page)
        handle.tables[key].extend(pages)
        handle.shared_prefix_pages = len(pages)
        handle.length = len(pages) * self.page_size

    # ------------------------------------------------------------------ step support
    def slot_of(self, handle: RequestCache, key: GroupKey, position: int) -> int:
        page = handle.tables[key][position // self.page_size]
        if page < 0:
            raise RuntimeError(f"position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def free_pages(self) -> Dict[GroupKey, int]:
        """Pages that can be had now: free ones and those only the prefix tree holds."""
        return {key: allocator.free_count + self._reclaimable(key) for key, allocator in self.allocators.items()}

    def layer_cache(self, call_index: int):
        return self.layer_caches[call_index]

    # ------------------------------------------------------------------ checks
    def check_invariants(self, extra_holders: Optional[Dict[GroupKey, Sequence[int]]] = None) -> None:
        """No page lost, none held more often than counted, none both free and held."""
        for key, allocator in self.allocators.items():
            held: Dict[int, int] = {}
            for handle in self.live.values():
                for page in handle.tables[key]:
                    if page >= 0:
                        held[page] = held.get(page, 0) + 1
            for page in (extra_holders or {}).get(key, ()):
                held[page] = held.get(page, 0) + 1
            if self.prefix_tree is not None and key == ("kv", None):
                for page in self.prefix_tree.pages():
                    held[page] = held.get(page, 0) + 1
            free = list(allocator._free)
            if len(set(free)) != len(free):
                raise AssertionError(f"group {key}: a page is on the free list twice")
            for page in free:
                if page in held:
                    raise AssertionError(f"group {key}: page {page} is free and held")
                if allocator.refcount(page) != 0:
                    raise AssertionError(f"group {key}: free page {page} has references")
            for page, count in held.items():
                if allocator.refcount(page) != count:
                    raise AssertionError(f"group {key}: page {page} held {count} times, counted {allocator.refcount(page)}")
            if len(free) + len(held) != allocator.num_pages:
                raise AssertionError(f"group {key}: {allocator.num_pages - len(free) - len(held)} pages are lost")
        slots = [handle.state_slot for handle in self.live.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("a state slot is held by two requests")
        if len(slots) + self.state_pool.free_count != self.state_pool.capacity:
            raise AssertionError("a state slot is lost")
