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
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Tuple

from .manager import PageAllocator


class _Node:
    __slots__ = ("key", "page", "parent", "children", "stamp")

    def __init__(self, key, page, parent):
        self.key, self.page, self.parent = key, page, parent
        self.children: Dict[Tuple[int, ...], "_Node"] = {}
        self.stamp = 0


class PrefixTree:
    def __init__(self, page_size: int, allocator: PageAllocator):
        self.page_size, self.allocator = int(page_size), allocator
        self.root = _Node((), -1, None)
        self._clock = itertools.count(1)
        self.pages_held = 0
        self.hits = self.lookups = 0

    def _walk(self, tokens: Sequence[int], max_pages: int) -> List[_Node]:
        path, node = [], self.root
        for i in range(max_pages):
            child = node.children.get(tuple(tokens[i * self.page_size:(i + 1) * self.page_size]))
            if child is None:
                break
            path.append(child)
            node = child
        return path

    def match(self, tokens: Sequence[int]) -> List[int]:
        """Page ids of the longest known prefix of ``tokens``, leaving at least one token out."""
        self.lookups += 1
        path = self._walk(tokens, (len(tokens) - 1) // self.page_size)
        stamp = next(self._clock)
        for node in path:
            node.stamp = stamp
        self.hits += bool(path)
        return [node.page for node in path]

    def insert(self, tokens: Sequence[int], pages: Sequence[int]) -> int:
        """Makes the full pages ``pages[i]`` holding ``tokens[i*P:(i+1)*P]`` known.  Pages that are
        new to the tree get one more reference; a page whose tokens are known already under
        another page id is left to its request.  Returns the number of pages adopted."""
        count = min(len(pages), len(tokens) // self.page_size)
        node, adopted, stamp = self.root, 0, next(self._clock)
        for i in range(count):
            key = tuple(tokens[i * self.page_size:(i + 1) * self.page_size])
            child = node.children.get(key)
            if child is None:
                if pages[i] < 0:
                    break
                child = _Node(key, pages[i], node)
                node.children[key] = child
                self.allocator.retain(pages[i])
                self.pages_held += 1
                adopted += 1
            child.stamp = stamp
            node = child
        return adopted

    def evictable(self) -> int:
        """Pages that only the tree holds and that could be freed (leaves first, then their parents)."""
        def count(node) -> Tuple[int, bool]:
            total, all_free = 0, True
            for child in node.children.values():
                sub, free = count(child)
                total += sub
                all_free &= free
            if node is self.root:
                return total, False
            mine = all_free and self.allocator.refcount(node.page) == 1
            return total + int(mine), mine
        return count(self.root)[0]

    def evict(self, pages: int) -> int:
        """Frees up to ``pages`` pages that nobody but the tree holds, least recently used leaves first."""
        freed = 0
        while freed < pages:
            leaves = [n for n in self._leaves() if self.allocator.refcount(n.page) == 1]
            if not leaves:
                break
            for node in sorted(leaves, key=lambda n: n.stamp):
                del node.parent.children[node.key]
                self.allocator.release(node.page)
                self.pages_held -= 1
                freed += 1
                if freed >= pages:
                    break
        return freed

    def _leaves(self):
        stack = list(self.root.children.values())
        while stack:
            node = stack.pop()
            if node.children:
                stack.extend(node.children.values())
            else:
                yield node

    def pages(self) -> List[int]:
        out, stack = [], list(self.root.children.values())
        while stack:
            node = stack.pop()
            out.append(node.page)
            stack.extend(node.children.values())
        return out

    def clear(self) -> None:
        for page in self.pages():
            self.allocator.release(page)
        self.root.children.clear()
        self.pages_held = 0
