"""Python face of the native prefix cache (``include/b200kv_prefix_cache.h``).

The exact-prompt table and the block table with its parent-fingerprint chain live in C++
inside ``libb200kv.so``; this class marshals token and page ids as int64 arrays and hands the
caller the reference-count changes a store asks for.  It replaces the two ``OrderedDict``
caches of the reference executor (``lite_llama/executor/model_executor.py:293-303``) and the
loops over them (``:547-683``).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib


def _tokens(prompt_tokens: Sequence[int]) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(prompt_tokens, dtype=np.int64).reshape(-1))


class NativePrefixCache:
    """LRU exact-prompt table + LRU block table; never touches the page pool itself."""

    def __init__(self, page_size: int, max_exact_entries: int = 128, max_block_entries: int = 4096):
        self._lib = _lib.lib()
        self._h = self._lib.b200kv_prefix_cache_create(int(page_size), int(max_exact_entries),
                                                       int(max_block_entries))
        if not self._h:
            raise ValueError("page_size and the table capacities must be positive")
        self.page_size = int(page_size)
        self._pages = np.empty(64, dtype=np.int64)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.b200kv_prefix_cache_destroy(h)

    def _room(self, n: int) -> np.ndarray:
        if self._pages.shape[0] < n:
            self._pages = np.empty(max(n, 2 * self._pages.shape[0]), dtype=np.int64)
        return self._pages

    @property
    def exact_entries(self) -> int:
        return int(self._lib.b200kv_prefix_cache_entries(self._h, 0))

    @property
    def block_entries(self) -> int:
        return int(self._lib.b200kv_prefix_cache_entries(self._h, 1))

    def lookup_exact(self, prompt_tokens) -> Optional[tuple[np.ndarray, int, int]]:
        """``(pages, token count, first generated token)`` of a stored prompt, or ``None``."""
        t = _tokens(prompt_tokens)
        num, first = ctypes.c_int64(0), ctypes.c_int64(0)
        while True:
            buf = self._pages
            n = self._lib.b200kv_prefix_cache_lookup_exact(self._h, t.ctypes.data, t.shape[0], buf.ctypes.data,
                                                           buf.shape[0], ctypes.byref(num), ctypes.byref(first))
            if n != -2:
                break
            self._room(2 * buf.shape[0])
        if n == -1:
            return None
        if n < 0:
            raise ValueError("bad argument to the prefix cache")
        return buf[:n].copy(), int(num.value), int(first.value)

    def lookup_blocks(self, prompt_tokens) -> tuple[np.ndarray, int]:
        """``(pages, matched tokens)`` of the longest cached page-aligned prefix (possibly empty)."""
        t = _tokens(prompt_tokens)
        buf = self._room(t.shape[0] // self.page_size + 1)
        matched = ctypes.c_int64(0)
        n = self._lib.b200kv_prefix_cache_lookup_blocks(self._h, t.ctypes.data, t.shape[0], buf.ctypes.data,
                                                        buf.shape[0], ctypes.byref(matched))
        if n < 0:
            raise ValueError("bad argument to the prefix cache")
        return buf[:n].copy(), int(matched.value)

    def _ops(self, n: int) -> list[tuple[int, np.ndarray]]:
        """The recorded reference changes as runs of equal sign: ``[(+1 | -1, pages), ...]``."""
        if n <= 0:
            return []
        pages = np.empty(n, dtype=np.int64)
        delta = np.empty(n, dtype=np.int32)
        got = self._lib.b200kv_prefix_cache_ref_ops(self._h, pages.ctypes.data, delta.ctypes.data, n)
        if got != n:
            raise RuntimeError("prefix cache: reference operations changed underneath the caller")
        cuts = np.flatnonzero(np.diff(delta)) + 1
        return [(int(delta[s]), pages[s:e]) for s, e in zip(np.r_[0, cuts], np.r_[cuts, n])]

    def store(self, prompt_tokens, pages, num_tokens: int, first_token_id: int) -> list[tuple[int, np.ndarray]]:
        """Remember a prompt and its pages.  Returns the reference changes to apply to the page
        pool, in order, as runs ``(+1 | -1, pages)``; empty when the prompt was already stored."""
        t = _tokens(prompt_tokens)
        p = np.ascontiguousarray(np.asarray(pages, dtype=np.int64).reshape(-1))
        n = self._lib.b200kv_prefix_cache_store(self._h, t.ctypes.data, t.shape[0], p.ctypes.data, p.shape[0],
                                                int(num_tokens), int(first_token_id))
        if n < 0:
            raise ValueError("bad argument to the prefix cache")
        return self._ops(int(n))

    def clear(self) -> list[tuple[int, np.ndarray]]:
        """Forget everything; returns the references to drop."""
        return self._ops(int(self._lib.b200kv_prefix_cache_clear(self._h)))
