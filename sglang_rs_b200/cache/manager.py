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

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..parts.base import CacheNeed, PagedKV, RequestState

GroupKey = Hashable        # ("kv", window) with window None for "all keys"


class OutOfPages(RuntimeError):
    def __init__(self, group: GroupKey, requested: int, available: int):
        self.group, self.requested, self.available = group, requested, available
        super().__init__(f"cache group {group}: {requested} pages requested, {available} free")


class OutOfStateSlots(RuntimeError):
    pass


def _core_library():
    """The C++ books (csrc/host_core.cu), built at first use like the kernels."""
    global _library
    if _library is None:
        from ..csrc.build import load_library
        lib = load_library("host_core")
        lib.hc_create.restype = ctypes.c_void_p
        lib.hc_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        lib.hc_destroy.argtypes = [ctypes.c_void_p]
        for name in ("hc_free_count", "hc_allocate", "hc_retain", "hc_release", "hc_refcount", "hc_free_list", "hc_open",
                     "hc_close", "hc_live_count", "hc_free_state_count", "hc_length", "hc_state_slot", "hc_table_length",
                     "hc_table", "hc_pages_needed", "hc_reserve", "hc_trim", "hc_capacity", "hc_commit",
                     "hc_adopt_prefix", "hc_check", "hc_fill_group", "hc_fill_decode"):
            getattr(lib, name).restype = ctypes.c_int
        _library = lib
    return _library


_library = None


def _ints(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


def _pointer(array: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(array.ctypes.data)


def _message(lib) -> str:
    return lib.srb_last_error().decode("utf-8", "replace")


class _Core:
    """Owner of one set of C++ books."""

    def __init__(self, page_size: int, windows: Sequence[int], num_pages: Sequence[int], max_requests: int):
        self.lib = _core_library()
        self.page_size = int(page_size)
        w, n = _ints(windows), _ints(num_pages)
        self.pointer = self.lib.hc_create(int(page_size), len(w), _pointer(w), _pointer(n), int(max_requests))
        if not self.pointer:
            raise ValueError("a page pool needs at least one page, a positive page size and room for a request")
        self.pointer = ctypes.c_void_p(self.pointer)

    def __del__(self):
        try:
            if getattr(self, "pointer", None):
                self.lib.hc_destroy(self.pointer)
        except Exception:
            pass


class PageAllocator:
    """Reference-counted pages of one group (kept by the C++ books).  The free list is a stack:
    a page that was just given back is the next one handed out."""

    def __init__(self, num_pages: int, core: Optional[_Core] = None, group: int = 0, key: GroupKey = None):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._core = core if core is not None else _Core(1, [0], [self.num_pages], 1)
        self._group, self._key = int(group), key
        self._lib, self._pointer = self._core.lib, self._core.pointer

    @property
    def free_count(self) -> int:
        return self._lib.hc_free_count(self._pointer, self._group)

    def allocate(self, count: int, group: GroupKey = None) -> List[int]:
        out = np.empty(max(int(count), 1), dtype=np.int32)
        status = self._lib.hc_allocate(self._pointer, self._group, int(count), _pointer(out))
        if status == -2:
            raise OutOfPages(group if group is not None else self._key, count, self.free_count)
        if status < 0:
            raise RuntimeError(_message(self._lib))
        return out[:count].tolist()

    def retain(self, page: int) -> None:
        if self._lib.hc_retain(self._pointer, self._group, int(page)) < 0:
            raise RuntimeError(_message(self._lib))

    def release(self, page: int) -> bool:
        """Drops one reference; True if the page went back to the free list."""
        status = self._lib.hc_release(self._pointer, self._group, int(page))
        if status < 0:
            raise RuntimeError(_message(self._lib))
        return status == 1

    def refcount(self, page: int) -> int:
        return self._lib.hc_refcount(self._pointer, self._group, int(page))

    def free_list(self) -> List[int]:
        out = np.empty(self.num_pages, dtype=np.int32)
        count = self._lib.hc_free_list(self._pointer, self._group, _pointer(out), self.num_pages)
        return out[:count].tolist()


class _StateSlots:
    """What ``CacheManager.state_pool`` shows of the slots in the C++ books."""

    def __init__(self, core: _Core, capacity: int):
        self._core, self.capacity = core, int(capacity)

    @property
    def free_count(self) -> int:
        return self._core.lib.hc_free_state_count(self._core.pointer)


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


class RequestCache:
    """A live request's hold on the cache.  Length, state slot and block tables live in the C++
    books; ``tables`` copies them out (logical page -> page id, -1 = given back)."""

    def __init__(self, request_id: Hashable, manager: "CacheManager", index: int):
        self.request_id, self._manager, self.index = request_id, manager, index
        self.length = 0                                  # tokens whose keys and values are stored
        self.state_slot = manager._lib.hc_state_slot(manager._pointer, index)
        self.shared_prefix_pages = 0                     # leading pages that came from the prefix tree
        self.closed = False

    def table(self, key: GroupKey) -> List[int]:
        manager = self._manager
        if self.closed:
            return []
        g = manager._group_index[key]
        count = manager._lib.hc_table_length(manager._pointer, self.index, g)
        out = np.empty(max(count, 1), dtype=np.int32)
        manager._lib.hc_table(manager._pointer, self.index, g, _pointer(out), count)
        return out[:count].tolist()

    def table_length(self, key: GroupKey) -> int:
        manager = self._manager
        return 0 if self.closed else manager._lib.hc_table_length(manager._pointer, self.index, manager._group_index[key])

    @property
    def tables(self) -> Dict[GroupKey, List[int]]:
        return {key: self.table(key) for key in self._manager.allocators}


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
        self.windows: Dict[GroupKey, Optional[int]] = {}
        counts: Dict[GroupKey, int] = {}
        for need in self.needs:
            if isinstance(need, PagedKV):
                key = group_key(need)
                if key not in counts:
                    counts[key] = (pages_per_group or {}).get(key, default_pages)
                    self.windows[key] = need.window
        for key, count in counts.items():
            if count <= 0:
                raise ValueError("a page pool needs at least one page")
        self._core = _Core(self.page_size, [self.windows[key] or 0 for key in counts], list(counts.values()),
                           self.max_requests)
        self._lib, self._pointer = self._core.lib, self._core.pointer
        self._group_index: Dict[GroupKey, int] = {key: g for g, key in enumerate(counts)}
        self._group_keys: List[GroupKey] = list(counts)
        self.allocators: Dict[GroupKey, PageAllocator] = {
            key: PageAllocator(count, self._core, g, key) for g, (key, count) in enumerate(counts.items())}
        self._needed = np.zeros(max(len(counts), 1), dtype=np.int32)
        self._short_group, self._shortfall = ctypes.c_int(0), ctypes.c_int(0)
        self.state_pool = _StateSlots(self._core, self.max_requests)
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
                    # one slot more than requests can hold: rows that pad a captured step use it
                    state = torch.zeros((self.max_requests + 1, *need.shape), dtype=need.dtype or dtype, device=device)
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
            # some ahead, so that the next pages are there without another call
            self.prefix_tree.evict(max(shortfall, self.EVICT_AHEAD))

    def _reclaimable(self, key: GroupKey) -> int:
        return self.prefix_tree.evictable() if self.prefix_tree is not None and key == ("kv", None) else 0

    # ------------------------------------------------------------------ requests
    def open(self, request_id: Hashable) -> RequestCache:
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        index = self._lib.hc_open(self._pointer)
        if index < 0:
            raise OutOfStateSlots(f"{self.max_requests} requests are live already")
        handle = RequestCache(request_id, self, index)
        if self.has_state and self.device is not None:
            for cache in self.layer_caches:
                if isinstance(cache, StateLayerCache):
                    cache.state[handle.state_slot].zero_()       # a new request starts from zero state
        self.live[request_id] = handle
        return handle

    def attach(self, request_id: Hashable, index: int) -> RequestCache:
        """The handle of a request that the C++ scheduler has opened in the books already."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        handle = RequestCache(request_id, self, index)
        handle.length = self._lib.hc_length(self._pointer, index)
        if self.has_state and self.device is not None:
            for cache in self.layer_caches:
                if isinstance(cache, StateLayerCache):
                    cache.state[handle.state_slot].zero_()       # a new request starts from zero state
        self.live[request_id] = handle
        return handle

    def detach(self, handle: RequestCache) -> None:
        """The C++ scheduler has closed the request in the books: the handle ends too."""
        handle.closed = True
        self.live.pop(handle.request_id, None)

    def first_kept_position(self, key: GroupKey, length: int) -> int:
        """The first position whose key a query at position >= ``length`` can still see."""
        window = self.windows[key]
        return 0 if window is None else max(0, length - window + 1)

    def _live(self, handle: RequestCache) -> None:
        if handle.closed:
            raise RuntimeError(f"request {handle.request_id!r} has ended")

    def pages_needed(self, handle: RequestCache, tokens: int) -> Dict[GroupKey, int]:
        self._live(handle)
        self._lib.hc_pages_needed(self._pointer, handle.index, int(tokens), _pointer(self._needed))
        return {key: int(self._needed[g]) for g, key in enumerate(self._group_keys)}

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
        self._live(handle)
        status = self._lib.hc_reserve(self._pointer, handle.index, int(tokens), ctypes.byref(self._short_group),
                                      ctypes.byref(self._shortfall))
        if status == -2:
            key = self._group_keys[self._short_group.value]
            self._reclaim(key, self._shortfall.value)            # pages only the prefix tree holds
            status = self._lib.hc_reserve(self._pointer, handle.index, int(tokens), ctypes.byref(self._short_group),
                                          ctypes.byref(self._shortfall))
            if status == -2:
                key = self._group_keys[self._short_group.value]
                free = self.allocators[key].free_count
                raise OutOfPages(key, free + self._shortfall.value, free)
        if status < 0:
            raise RuntimeError(_message(self._lib))

    def trim_reservation(self, handle: RequestCache) -> None:
        """Gives back pages that were reserved beyond what the stored tokens need (a step
        that did not run)."""
        if handle.closed:
            return
        if self._lib.hc_trim(self._pointer, handle.index) < 0:
            raise RuntimeError(_message(self._lib))

    def commit(self, handle: RequestCache, tokens: int) -> None:
        """``tokens`` more tokens are stored; pages a window has passed are given back."""
        self._live(handle)
        length = self._lib.hc_commit(self._pointer, handle.index, int(tokens))
        if length < 0:
            raise RuntimeError(_message(self._lib))
        handle.length = length

    def capacity(self, handle: RequestCache) -> int:
        self._live(handle)
        return self._lib.hc_capacity(self._pointer, handle.index)

    def close(self, handle: RequestCache) -> None:
        if handle.closed:
            raise RuntimeError(f"request {handle.request_id!r} is ended twice")
        if self._lib.hc_close(self._pointer, handle.index) < 0:
            raise RuntimeError(_message(self._lib))
        handle.closed = True
        del self.live[handle.request_id]

    # ------------------------------------------------------------------ sharing (prefix tree)
    def adopt_prefix(self, handle: RequestCache, key: GroupKey, pages: Sequence[int]) -> None:
        """Starts a new request on full pages that another owner already holds."""
        self._live(handle)
        array = _ints(list(pages))
        length = self._lib.hc_adopt_prefix(self._pointer, handle.index, self._group_index[key], _pointer(array), len(array))
        if length < 0:
            raise RuntimeError(_message(self._lib))
        handle.shared_prefix_pages = len(array)
        handle.length = length

    # ------------------------------------------------------------------ step support
    def slot_of(self, handle: RequestCache, key: GroupKey, position: int) -> int:
        page = handle.table(key)[position // self.page_size]
        if page < 0:
            raise RuntimeError(f"position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def free_pages(self) -> Dict[GroupKey, int]:
        """Pages that can be had now: free ones and those only the prefix tree holds."""
        return {key: allocator.free_count + self._reclaimable(key) for key, allocator in self.allocators.items()}

    def can_take(self, count: int) -> bool:
        """True if every group could hand out ``count`` pages now.  The prefix tree is only searched
        for pages it could give up when the free ones do not do."""
        for key, allocator in self.allocators.items():
            free = allocator.free_count
            if free < count and free + self._reclaimable(key) < count:
                return False
        return True

    def layer_cache(self, call_index: int):
        return self.layer_caches[call_index]

    # ------------------------------------------------------------------ checks
    def check_invariants(self, extra_holders: Optional[Dict[GroupKey, Sequence[int]]] = None) -> None:
        """No page lost, none held more often than counted, none both free and held."""
        pairs: List[int] = []
        for key, pages in (extra_holders or {}).items():
            for page in pages:
                pairs += [self._group_index[key], int(page)]
        if self.prefix_tree is not None:
            for page in self.prefix_tree.pages():
                pairs += [self._group_index[("kv", None)], int(page)]
        array = _ints(pairs if pairs else [0])
        if self._lib.hc_check(self._pointer, _pointer(array), len(pairs) // 2) < 0:
            raise AssertionError(_message(self._lib))
        if self.prefix_tree is not None:
            self.prefix_tree.check()
        if len(self.live) != self._lib.hc_live_count(self._pointer):
            raise AssertionError("the live requests of the books and of the manager differ")

    # ------------------------------------------------------------------ index arrays of a step
    def fill_group(self, key: GroupKey, handles: Sequence[RequestCache], counts: Sequence[int], stride: int):
        """Block tables [requests, stride] and write slots [rows] of one group for a step whose
        request i brings ``counts[i]`` rows at its next positions."""
        requests, rows = _ints([h.index for h in handles]), _ints(list(counts))
        table = np.empty((len(requests), stride), dtype=np.int32)
        slots = np.empty(max(int(rows.sum()), 1), dtype=np.int32)
        status = self._lib.hc_fill_group(self._pointer, self._group_index[key], _pointer(requests), _pointer(rows),
                                         len(requests), int(stride), _pointer(table), _pointer(slots))
        if status < 0:
            raise RuntimeError(_message(self._lib))
        return table, slots[:status]

    def fill_decode(self, handles: Sequence[RequestCache], tokens: Sequence[int], token_from: Sequence[int], bucket: int,
                    stride: int, offsets: Sequence[int], buffer: np.ndarray) -> None:
        """The static buffer of a captured decode step (one row per request, padded to
        ``bucket`` rows whose writes go to each pool's spare page)."""
        # the arrays stay referenced until the call has returned
        requests = _ints([h.index for h in handles])
        spare = _ints([self.allocators[key].num_pages for key in self._group_keys] or [0])
        token_ids, sources, starts = _ints(list(tokens)), _ints(list(token_from)), _ints(list(offsets))
        status = self._lib.hc_fill_decode(self._pointer, _pointer(requests), _pointer(token_ids), _pointer(sources),
                                          len(requests), int(bucket), int(stride), _pointer(spare), _pointer(starts),
                                          ctypes.c_void_p(buffer.ctypes.data))
        if status < 0:
            raise RuntimeError(_message(self._lib))
