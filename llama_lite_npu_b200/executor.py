"""The caller's side of the paged-KV path: request bookkeeping, prefix cache and the
per-batch attention metadata, plus the two attention call sequences.

Mirrors the paged-KV methods of the reference's ``ModelExecutor``
(``lite_llama/executor/model_executor.py:496-941``) with the same names, arguments, return
values and error messages, and the mutable ``AttentionInfo`` bag the models read
(``lite_llama/executor/executor_struct.py:30-40``), so a scheduler written against the reference
executor (``reserve_paged_requests``, ``activate_paged_*``, ``extend_paged_requests``,
``release_paged_request_ids``, ``share_*`` / ``store_*``) drives this object unchanged.  Model
loading, weights and graphs are out of scope: ``context_forward`` / ``token_forward`` here are the
attention call sequences of ``Attention.context_forward`` / ``token_forward``
(``lite_llama/models/qwen3.py:20-75``) on the CUDA operators of this package.

What differs underneath: all metadata of a batch is computed on the host from the managers'
page lists (no device gathers, no per-request device reads) and reaches the device in one
copy per tensor; the block table is published next to the token table.
"""

from __future__ import annotations

from typing import Optional

import torch

from .paged_attention import PagedKVCacheManager, PagedReqTokensManager
from .prefix_cache import NativePrefixCache


class AttentionInfo:
    """Per-forward attention metadata (same field names as the reference's dataclass)."""

    def __init__(self):
        self.kv_buffer = []
        self.cur_select_index = torch.empty((0,), dtype=torch.int32)
        self.b_req_tokens_table = None
        self.b_req_block_table = None
        self.b_start_loc = None
        self.b_req_idx = None
        self.b_seq_len = None
        self.max_actual_seq_len = 0
        self.is_paged_chunk_prefill = False
        self.chunk_context_len = None
        self.chunk_q_seq_len = None
        self.max_actual_q_seq_len = None
        self.page_size = 16
        # the device half of a staged decode step that has not run yet (see PendingAdvance)
        self.pending_advance = None


class PendingAdvance:
    """The device half of a staged decode step: every sequence of the active batch grows by one
    token — lengths + 1, the new tokens' slots, their token-table entries — in one small kernel on
    the tensors of the ``AttentionInfo`` it is run on.  The host half (page allocation, mirrors,
    the new block-table entry of a sequence that crossed a page boundary) has already happened
    when this object exists.  A graph runner records ``run`` as the first node of the step's
    graph; everybody else calls it once before the layer steps."""

    def __init__(self, executor: "PagedKVExecutor"):
        self._ex = executor

    def run(self, info) -> None:
        from . import kernels

        ex = self._ex
        kernels.advance_decode_metadata(
            info.b_seq_len, info.cur_select_index, info.b_req_block_table, ex.page_size,
            ex.kv_mem_manager.num_pages, b_req_idx=info.b_req_idx,
            page_counts=ex.req_tokens_manager.page_counts, b_req_tokens_table=info.b_req_tokens_table)


class PagedKVExecutor:
    """Owns the page pool, the request tables, the prefix caches and ``atten_info``."""

    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, num_pages: int,
                 max_requests: int, max_seq_len: int, page_size: int = 16,
                 dtype: torch.dtype = torch.float16, device: str = "cuda:0",
                 prefix_cache_entries: int = 128, prefix_cache_block_entries: int = 4096):
        self.device = device
        self.page_size = page_size
        self.num_kv_heads = num_kv_heads
        self.use_paged_attn = True
        self.kv_mem_manager = PagedKVCacheManager(num_layers, num_kv_heads, head_dim, num_pages,
                                                  page_size, dtype, device)
        self.req_tokens_manager = PagedReqTokensManager(max_requests, max_seq_len,
                                                        self.kv_mem_manager, device)
        self.atten_info = AttentionInfo()
        self.atten_info.page_size = page_size
        self.atten_info.kv_buffer = self.kv_mem_manager.gpu_kv_buffer
        self._paged_request_ids: tuple[int, ...] = ()
        # exact-prompt table: prompt -> (pages, tokens, first generated token); block table:
        # (fingerprint of the blocks before, block tokens) -> (page, tokens up to and including
        # the block); capacities as in the reference executor (model_executor.py:296,303)
        self._paged_prefix_cache_max_entries = prefix_cache_entries
        self._paged_block_prefix_cache_max_entries = prefix_cache_block_entries
        self._prefix_cache = NativePrefixCache(page_size, prefix_cache_entries, prefix_cache_block_entries)

    # ------------------------------------------------------------------ helpers
    def _dev(self, values, dtype) -> torch.Tensor:
        t = torch.tensor(values, dtype=dtype)
        if torch.device(self.device).type == "cuda":
            return t.pin_memory().to(self.device, non_blocking=True)
        return t

    def _slots(self, req_idx: int, start: int, end: int) -> torch.Tensor:
        """Physical slots of logical tokens [start, end) of a request, from the host page list."""
        ps = self.page_size
        pos = torch.arange(start, end, dtype=torch.long)
        pages = self.req_tokens_manager.req_page_table[int(req_idx)]
        return (pages[pos // ps] * ps + pos % ps).to(torch.int32)

    def _publish_tables(self) -> None:
        self.atten_info.b_req_tokens_table = self.req_tokens_manager.b_req_tokens_table
        self.atten_info.b_req_block_table = self.req_tokens_manager.b_req_block_table

    def _reset_paged_chunk_prefill_metadata(self) -> None:
        self.atten_info.is_paged_chunk_prefill = False
        self.atten_info.chunk_context_len = None
        self.atten_info.chunk_q_seq_len = None
        self.atten_info.max_actual_q_seq_len = None

    # ------------------------------------------------------------------ request lifecycle
    def reserve_paged_requests(self, prompt_lengths, reserved_lengths=None) -> tuple[int, ...]:
        """Reserve one request id (and its pages) per prompt; all or nothing."""
        if reserved_lengths is not None and len(reserved_lengths) != len(prompt_lengths):
            raise ValueError("reserved_lengths must match prompt_lengths")
        request_ids: list[int] = []
        try:
            for index, prompt_length in enumerate(prompt_lengths):
                reserved = None if reserved_lengths is None else int(reserved_lengths[index])
                req_idx = self.req_tokens_manager.reserve_req(int(prompt_length), reserved)
                if req_idx is None:
                    raise RuntimeError("Paged KV request or page capacity is exhausted")
                request_ids.append(req_idx)
        except BaseException:
            for req_idx in request_ids:
                self.req_tokens_manager.free_req(req_idx)
            raise
        return tuple(request_ids)

    def ensure_paged_request_capacity(self, req_idx: int, total_tokens: int) -> None:
        if not self.req_tokens_manager.ensure_req_capacity(req_idx, total_tokens):
            raise RuntimeError(f"Paged KV capacity reservation failed for request {req_idx}")

    def release_paged_request_ids(self, request_ids: tuple[int, ...]) -> None:
        for req_idx in request_ids:
            self.req_tokens_manager.free_req(req_idx)
        if tuple(request_ids) == self._paged_request_ids:
            self._paged_request_ids = ()

    def release_paged_requests(self) -> None:
        self.release_paged_request_ids(self._paged_request_ids)

    # ------------------------------------------------------------------ prefix cache
    # The tables themselves (exact prompts, blocks chained by parent fingerprint, both LRU) are
    # native code (prefix_cache.NativePrefixCache); these methods keep the reference's names,
    # arguments and return values (model_executor.py:547-683) and apply the reference changes the
    # cache asks for to the page pool.
    def _apply_ref_ops(self, ops) -> None:
        pool = self.req_tokens_manager.page_mgr
        for delta, pages in ops:
            # a run may name a page twice (the prompt's reference and a block's); the pool's
            # vectorised update counts an index once per call, so cut the run at every repeat
            start, seen = 0, set()
            for i, page in enumerate(pages.tolist() + [None]):
                if page is None or page in seen:
                    t = torch.from_numpy(pages[start:i])
                    if delta > 0:
                        pool.add_ref(t)
                    else:
                        pool.free(t)
                    start, seen = i, set()
                if page is not None:
                    seen.add(page)

    def _share(self, pages, num_tokens: int) -> Optional[int]:
        return self.req_tokens_manager.reserve_shared_req(torch.from_numpy(pages), int(num_tokens))

    def share_paged_request_from_cache(self, prompt_tokens) -> Optional[tuple[int, int]]:
        """Exact full-prompt hit: ``(request_id, first generated token)`` or ``None``."""
        hit = self._prefix_cache.lookup_exact(prompt_tokens)
        if hit is None:
            return None
        pages, num_tokens, first_token_id = hit
        req_idx = self._share(pages, num_tokens)
        return None if req_idx is None else (int(req_idx), first_token_id)

    def share_paged_prefix_from_cache(self, prompt_tokens) -> Optional[tuple[int, int, Optional[int]]]:
        """Longest cached page-aligned prefix: ``(request_id, matched_tokens, first_token_id)``;
        ``first_token_id`` is ``None`` for a partial hit (the caller prefills the suffix)."""
        n = len(prompt_tokens)
        if n == 0:
            return None
        hit = self._prefix_cache.lookup_exact(prompt_tokens)
        if hit is not None:
            pages, num_tokens, first_token_id = hit
            req_idx = self._share(pages, num_tokens)
            return None if req_idx is None else (int(req_idx), n, first_token_id)
        pages, matched_tokens = self._prefix_cache.lookup_blocks(prompt_tokens)
        if pages.shape[0] == 0 or matched_tokens <= 0:
            return None
        req_idx = self._share(pages, matched_tokens)
        return None if req_idx is None else (int(req_idx), matched_tokens, None)

    def store_paged_request_prefix(self, prompt_tokens, req_idx: int, first_token_id: int) -> None:
        """Keep a finished prompt's pages alive for reuse: one reference per page for the whole
        prompt, one more per full block that the block table did not know yet; entries evicted to
        make room give theirs back."""
        mgr = self.req_tokens_manager
        if req_idx not in mgr.req_page_table:
            return
        pages = mgr.req_page_table[int(req_idx)]
        ops = self._prefix_cache.store(prompt_tokens, pages.numpy(), mgr.req_token_count[int(req_idx)],
                                       first_token_id)
        self._apply_ref_ops(ops)

    def clear_paged_prefix_cache(self) -> None:
        """Forget every cached prefix and drop the references the cache held."""
        self._apply_ref_ops(self._prefix_cache.clear())

    # ------------------------------------------------------------------ batch activation
    def activate_paged_prefill_batch(self, request_ids: tuple[int, ...], prompt_length: int) -> None:
        """Equal-length prefill group."""
        self._reset_paged_chunk_prefill_metadata()
        if not request_ids:
            raise ValueError("request_ids must not be empty")
        for req_idx in request_ids:
            actual = self.req_tokens_manager.req_token_count[req_idx]
            if actual != prompt_length:
                raise ValueError(
                    "continuous prefill groups must have equal prompt "
                    f"lengths: expected={prompt_length}, request={req_idx}, actual={actual}")
        self.activate_paged_packed_prefill_batch(request_ids, [prompt_length] * len(request_ids))

    def activate_paged_packed_prefill_batch(self, request_ids, prompt_lengths):
        """Mixed-length no-padding prefill: returns ``(position_ids, last-token indices)``."""
        self._reset_paged_chunk_prefill_metadata()
        if not request_ids:
            raise ValueError("request_ids must not be empty")
        if len(request_ids) != len(prompt_lengths):
            raise ValueError("request_ids and prompt_lengths must have same length")
        lengths = tuple(int(n) for n in prompt_lengths)
        if any(n <= 0 for n in lengths):
            raise ValueError("prompt_lengths must be positive")
        for req_idx, n in zip(request_ids, lengths):
            actual = self.req_tokens_manager.req_token_count[int(req_idx)]
            if actual != n:
                raise ValueError("packed prefill request length mismatch: "
                                 f"request={req_idx}, expected={n}, actual={actual}")
        return self._activate_prefill(tuple(int(r) for r in request_ids), (0,) * len(lengths), lengths, False)

    def activate_paged_chunk_prefill_batch(self, request_ids, context_lengths, chunk_lengths):
        """Later chunks / prefix-hit suffixes: extends each request by its chunk, then publishes the
        chunk's slot_mapping and the (context, chunk) lengths for paged chunk attention."""
        if not request_ids:
            raise ValueError("request_ids must not be empty")
        if len(request_ids) != len(context_lengths) or len(request_ids) != len(chunk_lengths):
            raise ValueError("request_ids, context_lengths and chunk_lengths must have same length")
        request_ids = tuple(int(r) for r in request_ids)
        contexts = tuple(int(n) for n in context_lengths)
        chunks = tuple(int(n) for n in chunk_lengths)
        if any(n < 0 for n in contexts):
            raise ValueError("context_lengths must be non-negative")
        if any(n <= 0 for n in chunks):
            raise ValueError("chunk_lengths must be positive")
        mgr = self.req_tokens_manager
        for req_idx, ctx, chunk in zip(request_ids, contexts, chunks):
            actual = mgr.req_token_count[req_idx]
            if actual != ctx:
                raise ValueError("paged chunk prefill context length mismatch: "
                                 f"request={req_idx}, expected={ctx}, actual={actual}")
            if not mgr.extend_req(req_idx, chunk):
                raise RuntimeError(
                    "Paged KV allocation failed for chunked prefill request "
                    f"{req_idx}: context_tokens={ctx}, chunk_tokens={chunk}, "
                    f"current_tokens={mgr.req_token_count.get(req_idx, 'unknown')}, "
                    f"max_seq_len={mgr.max_seq_len}, free_pages={mgr.page_mgr.num_free_pages}")
        return self._activate_prefill(request_ids, contexts, chunks, True)

    def _activate_prefill(self, request_ids, contexts, chunks, chunked: bool):
        starts, sample, positions, slots = [], [], [], []
        cursor = 0
        for req_idx, ctx, n in zip(request_ids, contexts, chunks):
            starts.append(cursor)
            sample.append(cursor + n - 1)
            positions.extend(range(ctx, ctx + n))
            slots.append(self._slots(req_idx, ctx, ctx + n))
            cursor += n
        totals = tuple(c + n for c, n in zip(contexts, chunks))
        info = self.atten_info
        self._paged_request_ids = request_ids
        info.b_req_idx = self._dev(request_ids, torch.int32)
        info.b_seq_len = self._dev(totals, torch.long)
        info.cur_select_index = self._dev(torch.cat(slots).tolist(), torch.int32)
        info.b_start_loc = self._dev(starts, torch.int32)
        info.max_actual_seq_len = max(totals)
        if chunked:
            info.max_actual_q_seq_len = max(chunks)
            info.chunk_context_len = self._dev(contexts, torch.long)
            info.chunk_q_seq_len = self._dev(chunks, torch.long)
            info.is_paged_chunk_prefill = True
        self._publish_tables()
        return self._dev(positions, torch.long), self._dev(sample, torch.long)

    def activate_paged_decode_batch(self, request_ids: tuple[int, ...]) -> None:
        self._reset_paged_chunk_prefill_metadata()
        req_ids, seq_lens, last = self.req_tokens_manager.batch_metadata(list(request_ids))
        info = self.atten_info
        self._paged_request_ids = tuple(request_ids)
        info.b_req_idx = req_ids
        info.b_seq_len = seq_lens
        info.cur_select_index = last
        info.b_start_loc = torch.zeros(len(request_ids), dtype=torch.int32, device=self.device)
        info.max_actual_seq_len = max(self.req_tokens_manager.req_token_count[r] for r in request_ids)
        self._publish_tables()

    def extend_paged_requests(self, request_ids: tuple[int, ...]) -> None:
        """Allocate the slot the next decode token will be written to, then re-activate."""
        mgr = self.req_tokens_manager
        for req_idx in request_ids:
            if not mgr.extend_req(req_idx, 1):
                raise RuntimeError(
                    "Paged KV allocation failed for request "
                    f"{req_idx}: current_tokens={mgr.req_token_count.get(req_idx, 'unknown')}, "
                    f"max_seq_len={mgr.max_seq_len}, free_pages={mgr.page_mgr.num_free_pages}")
        self.activate_paged_decode_batch(request_ids)

    def stage_paged_decode_step(self, request_ids: tuple[int, ...]) -> None:
        """Host half of one decode step of the active batch; the device half stays pending.

        When the batch is the one that is already active: pages are allocated for sequences that
        cross a page boundary (only then does anything cross PCIe: the new block-table entry), the
        host mirrors advance, and ``atten_info.pending_advance`` is set to the kernel launch that
        will advance ``b_seq_len`` / ``cur_select_index`` / the token table in place.  The tensors
        keep their addresses, so a graph that holds that launch and the layer steps can be
        replayed as is (``cuda_graph.CudaGraphRunner`` does exactly this).  Any other batch goes
        through the host path once (nothing stays pending), which also makes it the active one."""
        info = self.atten_info
        if info.pending_advance is not None:
            raise RuntimeError("the previous decode step was staged but its device half never ran")
        if tuple(request_ids) != self._paged_request_ids or info.b_seq_len is None:
            self.extend_paged_requests(request_ids)
            return
        mgr = self.req_tokens_manager
        failed = mgr.extend_batch_for_device(request_ids)
        if failed is not None:
            raise RuntimeError(
                "Paged KV allocation failed for request "
                f"{failed}: current_tokens={mgr.req_token_count.get(failed, 'unknown')}, "
                f"max_seq_len={mgr.max_seq_len}, free_pages={mgr.page_mgr.num_free_pages}")
        self._publish_tables()                                   # flushes a new page entry, if any
        info.max_actual_seq_len += 1
        info.pending_advance = PendingAdvance(self)

    def extend_paged_requests_on_device(self, request_ids: tuple[int, ...]) -> None:
        """``extend_paged_requests`` with the per-step metadata produced on the device:
        ``stage_paged_decode_step`` followed at once by its device half."""
        self.stage_paged_decode_step(request_ids)
        info = self.atten_info
        if info.pending_advance is not None:
            info.pending_advance.run(info)
            info.pending_advance = None

    # ------------------------------------------------------------------ attention call sequences
    def context_forward(self, xq, xk, xv, layer_index: int, qk_scale: float) -> torch.Tensor:
        """Prefill attention of one layer: append the chunk's K/V, then attend.  ``qk_scale`` is the
        softmax scale times log2(e).  Always goes through the paged kernel: a first chunk is the
        same computation with zero history."""
        from . import kernels

        info, kh = self.atten_info, self.num_kv_heads
        pool = info.kv_buffer[layer_index]
        kernels.update_kv_buffer_split(xk, xv, info.cur_select_index, pool)
        if info.is_paged_chunk_prefill:
            ctx, qlen, max_q = info.chunk_context_len, info.chunk_q_seq_len, info.max_actual_q_seq_len
        else:
            ctx, qlen, max_q = torch.zeros_like(info.b_seq_len), info.b_seq_len, info.max_actual_seq_len
        return kernels.paged_chunk_flash_attention(
            xq, pool[:, :kh, :], pool[:, kh:, :], qk_scale, info.b_req_block_table, info.b_req_idx,
            info.b_start_loc, ctx, qlen, max_q, table_kind="block")

    def token_forward(self, xq, xk, xv, layer_index: int, qk_scale: float) -> torch.Tensor:
        """Decode attention of one layer: append the new token's K/V, then attend.  Table rows are
        selected by ``b_req_idx``, so batches with gaps or reordered request ids are correct."""
        from . import kernels

        info = self.atten_info
        # one launch: append + decode.  The first layer's launch may directly follow the kernel or
        # copy that produced the step's lengths, so it gives up its overlap with its predecessor.
        return kernels.append_flash_decoding_split(
            xk, xv, info.cur_select_index, info.kv_buffer[layer_index], xq, qk_scale, info.b_req_block_table,
            info.b_seq_len, info.max_actual_seq_len, b_req_idx=info.b_req_idx, table_kind="block",
            metadata_fresh=(layer_index == 0))

    # ------------------------------------------------------------------ fused prologue variants
    def fused_token_forward(self, xq, xkv, q_norm_weight, k_norm_weight, eps: float, cos, sin,
                            layer_index: int, qk_scale: float) -> torch.Tensor:
        """Decode attention of one layer from the raw projections: QK-RMSNorm, rotary embedding
        and the KV append in one launch, then paged decode.  ``xq`` is rewritten in place;
        ``xkv`` is the kv_proj output ``[batch, 2*kv_heads*head_dim]``.  Same result as
        normalising and rotating first and calling ``token_forward``
        (``lite_llama/models/qwen3.py:109-130`` followed by ``:53-75``)."""
        from . import kernels

        info, kh = self.atten_info, self.num_kv_heads
        pool = info.kv_buffer[layer_index]
        kernels.fused_qk_norm_rope_append(xq, xkv, q_norm_weight, k_norm_weight, eps, cos, sin,
                                          info.cur_select_index, pool)
        return kernels.flash_decoding(
            xq, pool[:, :kh, :], pool[:, kh:, :], qk_scale, info.b_req_block_table, info.b_seq_len,
            info.max_actual_seq_len, b_req_idx=info.b_req_idx, table_kind="block")

    def fused_context_forward(self, xq, xkv, q_norm_weight, k_norm_weight, eps: float, cos, sin,
                              layer_index: int, qk_scale: float) -> torch.Tensor:
        """Prefill attention of one layer from the raw projections (see ``fused_token_forward``);
        ``qk_scale`` is the softmax scale times log2(e) as for ``context_forward``."""
        from . import kernels

        info, kh = self.atten_info, self.num_kv_heads
        pool = info.kv_buffer[layer_index]
        kernels.fused_qk_norm_rope_append(xq, xkv, q_norm_weight, k_norm_weight, eps, cos, sin,
                                          info.cur_select_index, pool)
        if info.is_paged_chunk_prefill:
            ctx, qlen, max_q = info.chunk_context_len, info.chunk_q_seq_len, info.max_actual_q_seq_len
        else:
            ctx, qlen, max_q = torch.zeros_like(info.b_seq_len), info.b_seq_len, info.max_actual_seq_len
        return kernels.paged_chunk_flash_attention(
            xq, pool[:, :kh, :], pool[:, kh:, :], qk_scale, info.b_req_block_table, info.b_req_idx,
            info.b_start_loc, ctx, qlen, max_q, table_kind="block")
