"""Host side of the paged KV cache: page pool, refcounts and per-request tables.

Same classes, methods, attributes and return conventions as the reference's
``lite_llama/executor/paged_attention.py`` (``PagedKVCacheManager`` :19-147,
``PagedReqTokensManager`` :153-384) so ``ModelExecutor`` can use them unchanged:
capacity problems return ``False`` / ``None``, misuse raises ``ValueError``, an
unknown request raises ``KeyError``.  Pages are handed out lowest id first, as
there, so page ids are identical for identical call sequences.

What is different underneath (B200-first):

* free pages live in a min-heap, so ``alloc`` costs O(n log P) instead of a scan
  of the whole free mask per call;
* besides the reference's token table (``b_req_tokens_table``, one int32 per
  token) a **block table** (``b_req_block_table``, one int32 per page) is kept,
  which is what the CUDA kernels prefer to walk;
* both device tables are written lazily: mutations go to a pinned host mirror and
  are pushed to the device in one batched copy the next time a device table (or
  ``batch_metadata``) is asked for, instead of one small copy per request per step.
"""

from __future__ import annotations

import bisect
import heapq
from typing import List, Optional, Tuple

import numpy as np
import torch


class PagedKVCacheManager:
    """Fixed-size page pool: one ``[num_pages*page_size, 2*kv_heads, head_dim]`` tensor per
    layer (K heads first, then V heads, inside a token row) plus host refcounts."""

    def __init__(
        self,
        num_layers: int,
        num_kv_heads: int,
        head_dim: int,
        num_pages: int,
        page_size: int = 16,
        dtype: torch.dtype = torch.float16,
        device: str = "cuda:0",
    ):
        self.num_layers = num_layers
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.num_pages = num_pages
        self.page_size = page_size
        self.dtype = dtype
        self.device = device

        self.max_tokens = num_pages * page_size
        self.max_num_tokens = self.max_tokens
        self.gpu_kv_buffer = [
            torch.empty((self.max_tokens, 2 * num_kv_heads, head_dim), dtype=dtype, device=device)
            for _ in range(num_layers)
        ]

        # Ownership is scheduler metadata and stays on the host.
        self.page_free = torch.ones(num_pages, dtype=torch.bool, device="cpu")
        self.page_refcount = torch.zeros(num_pages, dtype=torch.int32, device="cpu")
        self.num_free_pages = num_pages
        self._free_heap: list[int] = list(range(num_pages))  # already a valid min-heap
        self._free_np = self.page_free.numpy()          # views of the two tensors above
        self._refcount_np = self.page_refcount.numpy()

    # -- allocation ---------------------------------------------------------
    def alloc(self, num_tokens: int) -> Optional[torch.Tensor]:
        """Pages for ``num_tokens`` tokens (lowest free ids, ascending) or ``None``."""
        num_needed = (num_tokens + self.page_size - 1) // self.page_size
        if num_needed > self.num_free_pages:
            return None
        ids = [heapq.heappop(self._free_heap) for _ in range(num_needed)]
        pages = torch.tensor(ids, dtype=torch.long)
        self.page_free[pages] = False
        self.page_refcount[pages] = 1
        self.num_free_pages -= num_needed
        return pages

    def alloc_one(self) -> Optional[int]:
        """The lowest free page id (one reference taken) or ``None``: ``alloc(page_size)`` without
        building a tensor, for the decode step that crosses a page boundary."""
        if self.num_free_pages < 1:
            return None
        page = heapq.heappop(self._free_heap)
        self._free_np[page] = False
        self._refcount_np[page] = 1
        self.num_free_pages -= 1
        return page

    def add_ref(self, page_indices: torch.Tensor):
        """One more owner for pages that are already allocated."""
        if len(page_indices) == 0:
            return
        page_indices = page_indices.to(device="cpu", dtype=torch.long)
        if torch.any(self.page_refcount[page_indices] <= 0):
            raise ValueError("cannot add ref to a free KV page")
        self.page_refcount[page_indices] += 1

    def free(self, page_indices: torch.Tensor):
        """Drop one reference; pages whose count reaches zero return to the pool."""
        if len(page_indices) == 0:
            return
        page_indices = page_indices.to(device="cpu", dtype=torch.long)
        if torch.any(self.page_refcount[page_indices] <= 0):
            raise ValueError("KV page refcount would become negative")
        self.page_refcount[page_indices] -= 1
        released = page_indices[self.page_refcount[page_indices] == 0]
        if len(released) > 0:
            released = torch.unique(released)
            self.page_free[released] = True
            self.num_free_pages += int(len(released))
            for page_id in released.tolist():
                heapq.heappush(self._free_heap, page_id)

    def free_all(self):
        self.page_free[:] = True
        self.page_refcount[:] = 0
        self.num_free_pages = self.num_pages
        self._free_heap = list(range(self.num_pages))

    # -- logical -> physical mapping ------------------------------------------
    def build_token_table(
        self, page_indices: torch.Tensor, num_tokens: int, token_table: torch.Tensor, req_idx: int,
    ) -> int:
        """``token_table[req_idx, t] = page_indices[t // page_size] * page_size + t % page_size``
        for ``t < num_tokens`` (bounded by the pages given).  Returns the tokens mapped."""
        mapped = min(int(num_tokens), len(page_indices) * self.page_size)
        if mapped <= 0:
            return 0
        pos = torch.arange(mapped, dtype=torch.long)
        pages = page_indices.to(device="cpu", dtype=torch.long)
        slots = pages[pos // self.page_size] * self.page_size + pos % self.page_size
        token_table[req_idx, :mapped] = slots.to(device=token_table.device, dtype=token_table.dtype)
        return mapped


class PagedReqTokensManager:
    """Request -> pages bookkeeping and the device tables the attention kernels read."""

    def __init__(
        self, max_requests: int, max_seq_len: int, page_manager: PagedKVCacheManager,
        device: str = "cuda:0",
    ):
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.page_mgr = page_manager
        self.device = device
        self.max_pages_per_req = (max_seq_len + page_manager.page_size - 1) // page_manager.page_size

        on_gpu = torch.device(device).type == "cuda"
        self._lazy = on_gpu
        # Host mirrors (pinned when a device copy exists); on CPU they ARE the tables.
        self._host_tokens = torch.zeros((max_requests, max_seq_len), dtype=torch.int32,
                                        pin_memory=on_gpu)
        self._host_blocks = torch.zeros((max_requests, self.max_pages_per_req), dtype=torch.int32,
                                        pin_memory=on_gpu)
        if on_gpu:
            self._dev_tokens = torch.zeros((max_requests, max_seq_len), dtype=torch.int32, device=device)
            self._dev_blocks = torch.zeros((max_requests, self.max_pages_per_req), dtype=torch.int32,
                                           device=device)
        else:
            self._dev_tokens = self._host_tokens
            self._dev_blocks = self._host_blocks
        # pages present per table row (what the device-side metadata kernel checks against)
        self._host_page_counts = torch.zeros(max_requests, dtype=torch.int32, pin_memory=on_gpu)
        self._dev_page_counts = (torch.zeros(max_requests, dtype=torch.int32, device=device)
                                 if on_gpu else self._host_page_counts)
        self._dirty_counts = False
        self._dirty_count_rows: set[int] = set()
        self._dirty_tokens: list[tuple[int, int, int]] = []  # (row, start, end) token spans
        self._dirty_blocks: list[tuple[int, int, int]] = []  # (row, start, end) page spans

        # numpy views of the host mirrors, and per-row arrays behind the two dictionaries below:
        # the decode step reads and advances whole batches of rows through these, not through
        # per-request dictionary lookups
        self._tokens_np = self._host_tokens.numpy()
        self._blocks_np = self._host_blocks.numpy()
        self._counts_np = self._host_page_counts.numpy()
        self._len_np = np.zeros(max_requests, dtype=np.int64)
        self._pages64 = torch.zeros((max_requests, self.max_pages_per_req), dtype=torch.long)
        self._pages64_np = self._pages64.numpy()
        self._batch_rows = None      # (request ids, the same as an int64 array, as a list)

        # request id -> its pages in logical order (a view of a row of _pages64) / its token count
        self.req_page_table: dict[int, torch.Tensor] = {}
        self.req_token_count: dict[int, int] = {}
        self.req_active = torch.zeros(max_requests, dtype=torch.bool, device="cpu")
        self.free_req_indices = list(range(max_requests))

    # -- device tables --------------------------------------------------------
    @property
    def b_req_tokens_table(self) -> torch.Tensor:
        """int32 ``[max_requests, max_seq_len]``: physical slot of each logical token."""
        self.flush()
        return self._dev_tokens

    @property
    def b_req_block_table(self) -> torch.Tensor:
        """int32 ``[max_requests, ceil(max_seq_len/page_size)]``: physical page of each logical page."""
        self.flush()
        return self._dev_blocks

    @property
    def page_counts(self) -> torch.Tensor:
        """int32 ``[max_requests]`` on the device: pages present in each block-table row."""
        self.flush()
        return self._dev_page_counts

    def flush(self) -> None:
        """Push pending table edits to the device: one index buffer, one value buffer per table."""
        if not self._lazy:
            self._dirty_tokens.clear()
            self._dirty_blocks.clear()
            self._dirty_counts = False
            self._dirty_count_rows.clear()
            return
        n_dirty = sum(e - s for _, s, e in self._dirty_tokens) + sum(e - s for _, s, e in self._dirty_blocks)
        if n_dirty <= self._PATCH_LIMIT:
            self._flush_small()
            return
        if self._dirty_counts:
            self._dev_page_counts.copy_(self._host_page_counts, non_blocking=True)
            self._dirty_counts = False
            self._dirty_count_rows.clear()
        for dirty, host, dev in (
            (self._dirty_tokens, self._host_tokens, self._dev_tokens),
            (self._dirty_blocks, self._host_blocks, self._dev_blocks),
        ):
            if not dirty:
                continue
            width = host.shape[1]
            idx = torch.cat([torch.arange(row * width + s, row * width + e, dtype=torch.long)
                             for row, s, e in dirty])
            vals = host.view(-1)[idx]
            dev.view(-1).index_copy_(
                0,
                idx.pin_memory().to(dev.device, non_blocking=True),
                vals.pin_memory().to(dev.device, non_blocking=True),
            )
            dirty.clear()

    _PATCH_LIMIT = 192   # table entries up to which edits travel as launch arguments

    def _flush_small(self) -> None:
        """A few edited entries (the usual decode step: some sequences crossed a page boundary):
        one small launch per edited table with the (offset, value) pairs as its arguments."""
        from . import kernels

        for dirty, host_np, dev in ((self._dirty_tokens, self._tokens_np, self._dev_tokens),
                                    (self._dirty_blocks, self._blocks_np, self._dev_blocks)):
            if not dirty:
                continue
            width = host_np.shape[1]
            off = np.fromiter((row * width + t for row, s, e in dirty for t in range(s, e)), dtype=np.int64)
            kernels.patch_table(dev, off, host_np.reshape(-1)[off])
            dirty.clear()
        if self._dirty_counts:
            if self._dirty_count_rows and len(self._dirty_count_rows) <= self._PATCH_LIMIT:
                rows = np.fromiter(self._dirty_count_rows, dtype=np.int64, count=len(self._dirty_count_rows))
                kernels.patch_table(self._dev_page_counts, rows, self._counts_np[rows])
            else:
                self._dev_page_counts.copy_(self._host_page_counts, non_blocking=True)
            self._dirty_count_rows.clear()
            self._dirty_counts = False

    def _set_pages(self, req_idx: int, have: int, extra: torch.Tensor) -> None:
        """Pages ``have ...`` of a request become ``extra``; its page list is a view of its row."""
        n = have + len(extra)
        self._pages64[req_idx, have:n] = extra
        self.req_page_table[req_idx] = self._pages64[req_idx, :n]

    def _write_pages(self, req_idx: int, first_page: int) -> None:
        pages = self.req_page_table[req_idx]
        if first_page < len(pages):
            self._host_blocks[req_idx, first_page:len(pages)] = pages[first_page:].to(torch.int32)
            self._dirty_blocks.append((req_idx, first_page, len(pages)))
        self._host_page_counts[req_idx] = len(pages)
        self._dirty_counts = True
        self._dirty_count_rows.add(req_idx)

    def _write_tokens(self, req_idx: int, start: int, end: int) -> None:
        if end <= start:
            return
        ps = self.page_mgr.page_size
        pos = torch.arange(start, end, dtype=torch.long)
        slots = self.req_page_table[req_idx][pos // ps] * ps + pos % ps
        self._host_tokens[req_idx, start:end] = slots.to(torch.int32)
        self._dirty_tokens.append((req_idx, start, end))

    # -- request lifecycle ------------------------------------------------------
    def alloc_req(self, req_idx: int, num_tokens: int, reserved_tokens: int | None = None) -> bool:
        """Give request id ``req_idx`` pages for ``reserved_tokens`` (default ``num_tokens``)
        tokens and expose ``num_tokens`` of them as its logical length."""
        if req_idx not in self.free_req_indices:
            return False
        num_tokens = int(num_tokens)
        capacity = int(reserved_tokens) if reserved_tokens is not None else num_tokens
        if num_tokens < 1 or capacity < num_tokens or capacity > self.max_seq_len:
            return False
        pages = self.page_mgr.alloc(capacity)
        if pages is None:
            return False
        self._adopt(req_idx, pages, num_tokens)
        return True

    def _adopt(self, req_idx: int, pages: torch.Tensor, num_tokens: int) -> None:
        self.free_req_indices.remove(req_idx)
        self._set_pages(req_idx, 0, pages)
        self.req_token_count[req_idx] = num_tokens
        self._len_np[req_idx] = num_tokens
        self.req_active[req_idx] = True
        mapped = self.page_mgr.build_token_table(pages, num_tokens, self._host_tokens, req_idx)
        if mapped:
            self._dirty_tokens.append((req_idx, 0, mapped))
        self._write_pages(req_idx, 0)

    def reserve_req(self, num_tokens: int, reserved_tokens: int | None = None) -> Optional[int]:
        """Lowest free request id with freshly allocated pages, or ``None``."""
        if not self.free_req_indices:
            return None
        req_idx = self.free_req_indices[0]
        if not self.alloc_req(req_idx, num_tokens, reserved_tokens):
            return None
        return req_idx

    def ensure_req_capacity(self, req_idx: int, total_tokens: int) -> bool:
        """Make sure pages exist for ``total_tokens``; the logical length is unchanged."""
        if req_idx not in self.req_page_table:
            return False
        total_tokens = int(total_tokens)
        if total_tokens < self.req_token_count[req_idx]:
            return True
        if total_tokens > self.max_seq_len:
            return False
        ps = self.page_mgr.page_size
        have = len(self.req_page_table[req_idx])
        need = (total_tokens + ps - 1) // ps
        if need <= have:
            return True
        extra = self.page_mgr.alloc((need - have) * ps)
        if extra is None:
            return False
        self._set_pages(req_idx, have, extra)
        self._write_pages(req_idx, have)
        return True

    def share_req_from_pages(self, req_idx: int, page_indices: torch.Tensor, num_tokens: int) -> bool:
        """Map a new request onto existing pages (prefix sharing) and take a reference on each."""
        if req_idx not in self.free_req_indices:
            return False
        num_tokens = int(num_tokens)
        if num_tokens < 1 or num_tokens > self.max_seq_len:
            return False
        ps = self.page_mgr.page_size
        need = (num_tokens + ps - 1) // ps
        if len(page_indices) < need:
            return False
        pages = page_indices[:need].to(device="cpu", dtype=torch.long)
        self.page_mgr.add_ref(pages)
        self._adopt(req_idx, pages, num_tokens)
        return True

    def reserve_shared_req(self, page_indices: torch.Tensor, num_tokens: int) -> Optional[int]:
        if not self.free_req_indices:
            return None
        req_idx = self.free_req_indices[0]
        if not self.share_req_from_pages(req_idx, page_indices, num_tokens):
            return None
        return req_idx

    def batch_metadata(self, req_indices: List[int]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(req_ids int32, seq_lens int64, last_slot int32)`` on the device for a decode batch,
        built from host state and shipped in a single host-to-device copy."""
        if not req_indices:
            raise ValueError("req_indices must not be empty")
        for req_idx in req_indices:
            if req_idx not in self.req_token_count:
                raise KeyError(f"request {req_idx} is not allocated")
        n = len(req_indices)
        lens = [self.req_token_count[r] for r in req_indices]
        rows = torch.tensor(req_indices, dtype=torch.long)
        last = self._host_tokens[rows, torch.tensor(lens, dtype=torch.long) - 1]
        # int64 lengths first keeps them 8-byte aligned inside the packed int32 buffer.
        packed = torch.empty(4 * n, dtype=torch.int32, pin_memory=self._lazy)
        packed[: 2 * n].view(torch.int64).copy_(torch.tensor(lens, dtype=torch.int64))
        packed[2 * n: 3 * n] = rows.to(torch.int32)
        packed[3 * n:] = last
        dev = packed.to(self.device, non_blocking=True) if self._lazy else packed
        self.flush()
        return dev[2 * n: 3 * n], dev[: 2 * n].view(torch.int64), dev[3 * n:]

    def extend_req(self, req_idx: int, num_new_tokens: int) -> bool:
        """Grow a request's logical length, allocating pages only when a page boundary is
        crossed and appending only the new table entries."""
        if num_new_tokens <= 0:
            return True
        cur = self.req_token_count[req_idx]
        new_total = cur + num_new_tokens
        if new_total > self.max_seq_len:
            return False
        ps = self.page_mgr.page_size
        need = (new_total + ps - 1) // ps
        have = len(self.req_page_table[req_idx])
        if need > have:
            extra = self.page_mgr.alloc((need - have) * ps)
            if extra is None:
                return False
            self._set_pages(req_idx, have, extra)
            self._write_pages(req_idx, have)
        self._write_tokens(req_idx, cur, new_total)
        self.req_token_count[req_idx] = new_total
        self._len_np[req_idx] = new_total
        return True

    def extend_batch_for_device(self, req_indices) -> Optional[int]:
        """Host half of a device-side decode step: grow every request by one token, allocating a
        page only where a page boundary is crossed, WITHOUT queueing per-token table writes (the
        metadata kernel writes the device token table itself).  The host mirror of the token table
        is kept exact with one vectorised write.  Returns ``None`` on success or the request id
        whose extension failed (earlier requests of the batch stay extended, as with
        ``extend_req`` in a loop)."""
        ps = self.page_mgr.page_size
        cached = self._batch_rows
        if cached is None or (cached[0] is not req_indices and cached[0] != tuple(req_indices)):
            key = tuple(int(r) for r in req_indices)
            cached = self._batch_rows = (key, np.array(key, dtype=np.int64), list(key))
        _, rows, row_list = cached
        cur = self._len_np[rows]
        failed = None
        # the rare cases, in batch order: a row at its maximum length, or one that needs a page
        special = np.flatnonzero((cur >= self.max_seq_len) | (cur // ps >= self._counts_np[rows]))
        for i in special.tolist():
            req_idx = row_list[i]
            if cur[i] + 1 > self.max_seq_len:
                failed = i
                break
            page = self.page_mgr.alloc_one()
            if page is None:
                failed = i
                break
            have = int(self._counts_np[req_idx])
            self._pages64_np[req_idx, have] = page
            self._blocks_np[req_idx, have] = page
            self._counts_np[req_idx] = have + 1
            self.req_page_table[req_idx] = self._pages64[req_idx, : have + 1]
            self._dirty_blocks.append((req_idx, have, have + 1))
            self._dirty_counts = True
            self._dirty_count_rows.add(req_idx)
        if failed is not None:
            rows, cur, row_list = rows[:failed], cur[:failed], row_list[:failed]
        self._len_np[rows] = cur + 1
        counts = self.req_token_count
        for r in row_list:
            counts[r] += 1
        self._tokens_np[rows, cur] = self._blocks_np[rows, cur // ps] * ps + cur % ps
        return None if failed is None else int(req_indices[failed])

    def get_token_indices(self, req_idx: int, num_tokens: Optional[int] = None) -> torch.Tensor:
        """Device view of the physical slots of a request's first ``num_tokens`` tokens."""
        if num_tokens is None:
            num_tokens = self.req_token_count[req_idx]
        return self.b_req_tokens_table[req_idx, :num_tokens]

    def free_req(self, req_idx: int):
        if req_idx in self.req_page_table:
            self.page_mgr.free(self.req_page_table[req_idx])
            del self.req_page_table[req_idx]
            del self.req_token_count[req_idx]
            self._len_np[req_idx] = 0
            self._host_page_counts[req_idx] = 0
            self._dirty_counts = True
            self._dirty_count_rows.add(req_idx)
        self.req_active[req_idx] = False
        if req_idx not in self.free_req_indices:
            bisect.insort(self.free_req_indices, req_idx)

    def request_pages(self, req_idx: int) -> Tuple[int, ...]:
        if req_idx not in self.req_page_table:
            raise KeyError(f"request {req_idx} is not allocated")
        return tuple(int(p) for p in self.req_page_table[req_idx].tolist())
