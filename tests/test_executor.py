"""The caller side of the path (request lifecycle, prefix cache, batch metadata) on CPU, and one
end-to-end serving scenario on the GPU checked step by step against the oracle."""

import math

import numpy as np
import pytest
import torch

from llama_lite_npu_b200 import workloads as W
from llama_lite_npu_b200.executor import PagedKVExecutor
from oracle import paged_kv_oracle as O

SCALE = 1.0 / math.sqrt(128)
LOG2E = 1.4426950408889634


def _ex(device="cpu", pages=32, ps=4, max_req=4, max_len=32, kvh=1, layers=1):
    return PagedKVExecutor(layers, kvh, 128, pages, max_req, max_len, page_size=ps, device=device)


def test_reserve_is_all_or_nothing_and_messages():
    ex = _ex(pages=4)
    with pytest.raises(RuntimeError, match="capacity is exhausted"):
        ex.reserve_paged_requests([8, 8, 8])
    assert ex.kv_mem_manager.num_free_pages == 4 and ex.req_tokens_manager.free_req_indices == [0, 1, 2, 3]
    ids = ex.reserve_paged_requests([5, 3], reserved_lengths=[8, 4])
    assert ids == (0, 1) and ex.kv_mem_manager.num_free_pages == 1
    with pytest.raises(ValueError):
        ex.reserve_paged_requests([1], reserved_lengths=[1, 2])
    with pytest.raises(RuntimeError, match="Paged KV capacity reservation failed"):
        ex.ensure_paged_request_capacity(0, 99)


def test_packed_prefill_metadata():
    ex = _ex()
    ids = ex.reserve_paged_requests([5, 2, 7])
    pos, sample = ex.activate_paged_packed_prefill_batch(ids, [5, 2, 7])
    info = ex.atten_info
    assert pos.tolist() == [0, 1, 2, 3, 4, 0, 1, 0, 1, 2, 3, 4, 5, 6] and sample.tolist() == [4, 6, 13]
    assert info.b_start_loc.tolist() == [0, 5, 7] and info.b_seq_len.tolist() == [5, 2, 7]
    assert info.b_seq_len.dtype == torch.int64 and info.cur_select_index.dtype == torch.int32
    want = torch.cat([ex.req_tokens_manager.get_token_indices(r, n) for r, n in zip(ids, [5, 2, 7])])
    assert info.cur_select_index.tolist() == want.tolist()
    assert info.max_actual_seq_len == 7 and not info.is_paged_chunk_prefill
    with pytest.raises(ValueError, match="length mismatch"):
        ex.activate_paged_packed_prefill_batch(ids, [5, 2, 6])
    with pytest.raises(ValueError):
        ex.activate_paged_packed_prefill_batch((), [])


def test_chunk_prefill_and_decode_metadata():
    ex = _ex()
    (r,) = ex.reserve_paged_requests([1], reserved_lengths=[12])
    ex.req_tokens_manager.extend_req(r, 3)                      # context of 4 tokens
    pos, sample = ex.activate_paged_chunk_prefill_batch((r,), [4], [6])
    info = ex.atten_info
    assert info.is_paged_chunk_prefill and info.chunk_context_len.tolist() == [4] and info.chunk_q_seq_len.tolist() == [6]
    assert pos.tolist() == list(range(4, 10)) and sample.tolist() == [5] and info.max_actual_q_seq_len == 6
    assert info.cur_select_index.tolist() == ex.req_tokens_manager.get_token_indices(r, 10)[4:].tolist()
    assert info.b_seq_len.tolist() == [10]
    with pytest.raises(ValueError, match="context length mismatch"):
        ex.activate_paged_chunk_prefill_batch((r,), [4], [1])
    ex.extend_paged_requests((r,))
    assert not info.is_paged_chunk_prefill and info.b_seq_len.tolist() == [11]
    assert info.cur_select_index.tolist() == [ex.req_tokens_manager.b_req_tokens_table[r, 10].item()]
    assert info.b_req_block_table[r, :3].tolist() == list(ex.req_tokens_manager.request_pages(r))
    with pytest.raises(RuntimeError, match="Paged KV allocation failed for request"):
        for _ in range(40):
            ex.extend_paged_requests((r,))
    ex.release_paged_requests()
    assert ex.kv_mem_manager.num_free_pages == 32


def test_prefix_cache_exact_and_block_hits_and_refcounts():
    ex = _ex(pages=16)
    prompt = tuple(range(100, 110))                              # 10 tokens = 2 full pages + 2
    (r,) = ex.reserve_paged_requests([10])
    pages = ex.req_tokens_manager.request_pages(r)
    ex.store_paged_request_prefix(prompt, r, first_token_id=7)
    pm = ex.kv_mem_manager
    assert pm.page_refcount[list(pages)].tolist() == [3, 3, 2]  # request + exact entry (+ block entry)
    ex.release_paged_request_ids((r,))
    assert pm.page_refcount[list(pages)].tolist() == [2, 2, 1] and pm.num_free_pages == 13
    hit = ex.share_paged_prefix_from_cache(prompt)               # exact hit: all pages, cached token
    assert hit is not None and hit[1:] == (10, 7)
    assert ex.req_tokens_manager.request_pages(hit[0]) == pages
    assert ex.share_paged_request_from_cache(prompt)[1] == 7
    part = ex.share_paged_prefix_from_cache(prompt[:8] + (1, 2, 3, 4, 5))   # block hit: 2 full pages
    assert part is not None and part[1:] == (8, None)
    assert ex.req_tokens_manager.request_pages(part[0]) == pages[:2]
    assert ex.share_paged_prefix_from_cache((9, 9, 9, 9, 9)) is None
    assert ex.share_paged_prefix_from_cache(prompt[:3]) is None  # shorter than one page
    assert ex.share_paged_prefix_from_cache((100, 101, 102, 103) + (5, 5, 5, 5))[1] == 4


@pytest.mark.gpu
def test_serving_scenario_on_gpu_matches_oracle():
    """Packed prefill of three prompts, a prefix-cache hit whose suffix is prefilled with history,
    then decode steps of a batch with a gap in its request ids: every attention output equals the
    oracle evaluated on a CPU copy of the pool and tables."""
    dev, kvh, heads, layers = "cuda:0", 2, 8, 2
    ex = PagedKVExecutor(layers, kvh, 128, 256, 8, 512, page_size=16, device=dev)
    for buf in ex.kv_mem_manager.gpu_kv_buffer:
        buf.fill_(float("nan"))                                  # unwritten slots must never matter
    prompts = [list(range(1000, 1000 + n)) for n in (70, 33, 150)]

    def rand(n, h, stream):
        return W.hash_normal_fp16(99, (n, h, 128), stream).to(dev)

    def oracle_attend(xq, layer, req_ids, starts, ctx, qlen):
        pool = ex.kv_mem_manager.gpu_kv_buffer[layer].cpu()
        table = ex.req_tokens_manager.b_req_tokens_table.cpu()
        return O.paged_attention(xq.cpu(), pool[:, :kvh], pool[:, kvh:], SCALE, table, torch.tensor(req_ids),
                                 torch.tensor(starts), torch.tensor(ctx), torch.tensor(qlen))

    def check(got, want):
        assert not bool(torch.isnan(got).any())
        assert float((got.cpu().float() - want.float()).abs().max()) <= 2e-3

    ids = ex.reserve_paged_requests([len(p) for p in prompts])
    ex.activate_paged_packed_prefill_batch(ids, [len(p) for p in prompts])
    total = sum(len(p) for p in prompts)
    for layer in range(layers):
        xq, xk, xv = rand(total, heads, 10 + layer), rand(total, kvh, 20 + layer), rand(total, kvh, 30 + layer)
        got = ex.context_forward(xq, xk, xv, layer, SCALE * LOG2E)
        check(got, oracle_attend(xq, layer, list(ids), [0, 70, 103], [0, 0, 0], [70, 33, 150]))
    ex.store_paged_request_prefix(prompts[2], ids[2], first_token_id=5)
    ex.release_paged_request_ids((ids[1],))                      # leaves a gap in the id space

    # a new prompt sharing 9 full pages (144 tokens) with prompt 2, then 40 new tokens
    new_prompt = prompts[2][:144] + list(range(5000, 5040))
    rid, matched, first = ex.share_paged_prefix_from_cache(new_prompt)
    assert (matched, first) == (144, None) and rid == ids[1]    # lowest free id is reused
    ex.activate_paged_chunk_prefill_batch((rid,), [144], [40])
    for layer in range(layers):
        xq, xk, xv = rand(40, heads, 40 + layer), rand(40, kvh, 50 + layer), rand(40, kvh, 60 + layer)
        got = ex.context_forward(xq, xk, xv, layer, SCALE * LOG2E)
        check(got, oracle_attend(xq, layer, [rid], [0], [144], [40]))
    shared = ex.req_tokens_manager.request_pages(ids[2])[:9]
    assert ex.kv_mem_manager.page_refcount[list(shared)].min().item() >= 3

    batch = (ids[2], ids[0], rid)                                # out of order, as a scheduler may
    for step in range(3):
        ex.extend_paged_requests(batch)
        lens = [ex.req_tokens_manager.req_token_count[r] for r in batch]
        for layer in range(layers):
            xq, xk, xv = rand(3, heads, 70 + step), rand(3, kvh, 80 + step), rand(3, kvh, 90 + step)
            got = ex.token_forward(xq, xk, xv, layer, SCALE)
            want = oracle_attend(xq, layer, list(batch), [0, 1, 2], [n - 1 for n in lens], [1, 1, 1])
            check(got, want)
    ex.release_paged_request_ids(batch)


@pytest.mark.gpu
def test_steady_decode_step_never_synchronises_with_the_host():
    """The reference pins 'no device -> host conversion in the decode step' with a source-text
    check (tests/test_decode_p0.py:272-289).  Here the property itself is checked: with torch's
    synchronisation debug mode set to raise, a steady decode step (metadata advanced on the
    device, append + paged decode, and the fused-prologue form) must run to completion, page
    boundaries included."""
    dev = "cuda:0"
    ex = PagedKVExecutor(1, 2, 128, 128, 8, 512, page_size=16, device=dev)
    ids = ex.reserve_paged_requests([30, 47, 5])
    ex.extend_paged_requests(ids)                              # host path once: activates the batch
    xq = torch.zeros(3, 8, 128, dtype=torch.float16, device=dev)
    xk = torch.zeros(3, 2, 128, dtype=torch.float16, device=dev)
    xkv = torch.zeros(3, 2 * 2 * 128, dtype=torch.float16, device=dev)
    w = torch.ones(128, dtype=torch.float16, device=dev)
    cos = torch.ones(3, 128, dtype=torch.float16, device=dev)
    ex.token_forward(xq, xk, xk, 0, SCALE)                     # warm-up: workspace, status word
    ex.fused_token_forward(xq, xkv, w, w, 1e-6, cos, cos, 0, SCALE)
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        for _ in range(20):
            ex.extend_paged_requests_on_device(ids)
            ex.token_forward(xq, xk, xk, 0, SCALE)
            ex.fused_token_forward(xq, xkv, w, w, 1e-6, cos, cos, 0, SCALE)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()
    from llama_lite_npu_b200 import kernels
    kernels.check_status(0)
    assert ex.req_tokens_manager.req_token_count[ids[0]] == 30 + 1 + 20
