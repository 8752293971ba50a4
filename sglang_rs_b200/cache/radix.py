"""Prefix reuse: a tree over full pages of tokens.

The reference keeps a per-token trie and floors a match to whole pages
(crates/sglang-srt/src/cache.rs:475-547; only whole pages are reused, :532-540), un-matches
the last token of a prompt that is cached entirely so that logits exist
(crates/sglang-srt/src/scheduler.rs:547-563), publishes prompt pages after a prefill step
(:849-892) and never evicts.  Here an edge is one page of tokens, a node holds the page id,
the tree holds one reference on every page it knows (so a finished request's prompt pages
stay until they are evicted), and pages nobody else holds are given back, least recently
used leaves first, when the pool runs short.

A match never covers the whole sequence: at most ``(len - 1) // page_size`` pages, so at
least one token is computed, into a page of the request's own.

The tree itself lives in the C++ books beside the pages it refers to (csrc/host_core.cu);
this class is its Python face.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import numpy as np

from .manager import PageAllocator, _core_library, _message, _pointer


class PrefixTree:
    def __init__(self, page_size: int, allocator: PageAllocator):
        self.page_size, self.allocator = int(page_size), allocator
        self._lib = _core_library()
        for name in ("hc_tree_match", "hc_tree_insert", "hc_tree_evictable", "hc_tree_evict", "hc_tree_pages_held",
                     "hc_tree_pages", "hc_tree_clear", "hc_tree_counters", "hc_tree_check"):
            getattr(self._lib, name).restype = ctypes.c_int
        self._lib.hc_tree_create.restype = ctypes.c_void_p
        self._lib.hc_tree_create.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        self._lib.hc_tree_destroy.argtypes = [ctypes.c_void_p]
        self._core = allocator._core                     # the books outlive the tree
        pointer = self._lib.hc_tree_create(self._core.pointer, allocator._group, self.page_size)
        if not pointer:
            raise ValueError("the prefix tree could not be made for this group of pages")
        self._pointer = ctypes.c_void_p(pointer)

    def __del__(self):
        try:
            if getattr(self, "_pointer", None):
                self._lib.hc_tree_destroy(self._pointer)
        except Exception:
            pass

    def _counters(self):
        out = np.zeros(2, dtype=np.int64)
        self._lib.hc_tree_counters(self._pointer, _pointer(out))
        return int(out[0]), int(out[1])

    @property
    def lookups(self) -> int:
        """Prefix look-ups so far, the scheduler's among them."""
        return self._counters()[0]

    @property
    def hits(self) -> int:
        return self._counters()[1]

    @property
    def pages_held(self) -> int:
        return self._lib.hc_tree_pages_held(self._pointer)

    def match(self, tokens: Sequence[int]) -> List[int]:
        """Page ids of the longest known prefix of ``tokens``, leaving at least one token out."""
        array = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty(max(len(array) // self.page_size, 1), dtype=np.int32)
        found = self._lib.hc_tree_match(self._pointer, _pointer(array), len(array), _pointer(out))
        if found < 0:
            raise RuntimeError(_message(self._lib))
        return out[:found].tolist()

    def insert(self, tokens: Sequence[int], pages: Sequence[int]) -> int:
        """Makes the full pages ``pages[i]`` holding ``tokens[i*P:(i+1)*P]`` known.  Pages that are
        new to the tree get one more reference; a page whose tokens are known already under
        another page id is left to its request.  Returns the number of pages adopted."""
        token_array = np.ascontiguousarray(tokens, dtype=np.int32)
        page_array = np.ascontiguousarray(list(pages) or [0], dtype=np.int32)
        adopted = self._lib.hc_tree_insert(self._pointer, _pointer(token_array), len(token_array), _pointer(page_array),
                                           len(pages))
        if adopted < 0:
            raise RuntimeError(_message(self._lib))
        return adopted

    def evictable(self) -> int:
        """Pages that only the tree holds and that could be freed (leaves first, then their parents).  The
        tree keeps the count up to date as holders of its pages come and go; asking costs nothing."""
        return self._lib.hc_tree_evictable(self._pointer)

    def check(self) -> None:
        """The count of evictable pages that the tree keeps up to date equals a walk over the whole tree."""
        if self._lib.hc_tree_check(self._pointer) < 0:
            raise AssertionError(_message(self._lib))

    def evict(self, pages: int) -> int:
        """Frees up to ``pages`` pages that nobody but the tree holds, least recently used leaves first."""
        freed = self._lib.hc_tree_evict(self._pointer, int(pages))
        if freed < 0:
            raise RuntimeError(_message(self._lib))
        return freed

    def pages(self) -> List[int]:
        out = np.empty(max(self.pages_held, 1), dtype=np.int32)
        count = self._lib.hc_tree_pages(self._pointer, _pointer(out), len(out))
        return out[:count].tolist()

    def clear(self) -> None:
        if self._lib.hc_tree_clear(self._pointer) < 0:
            raise RuntimeError(_message(self._lib))
