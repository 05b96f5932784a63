"""Host page-pool / metadata classes: identical observable behaviour to the reference's,
checked against a state log recorded from the reference classes (tests/golden/host_golden.json)
and against the expectations of the reference's own host tests."""

from unittest.mock import patch

import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200 import kv_engine, paged_attention


def test_scripted_state_log_matches_reference(golden):
    got = G.host_script(paged_attention, kv_engine)
    ref = golden["host"]
    assert sorted(got) == sorted(ref)
    for key in ref:
        assert got[key] == ref[key], key


def _managers(num_pages=4, page_size=4, max_requests=2, max_seq_len=16):
    pm = paged_attention.PagedKVCacheManager(1, 1, 8, num_pages, page_size, device="cpu")
    rm = paged_attention.PagedReqTokensManager(max_requests, max_seq_len, pm, device="cpu")
    return pm, rm


def test_shared_page_released_at_last_reference():
    pm, _ = _managers()
    pages = pm.alloc(4)
    assert pm.num_free_pages == 3
    pm.add_ref(pages)
    assert int(pm.page_refcount[pages[0]]) == 2
    pm.free(pages)
    assert pm.num_free_pages == 3 and not bool(pm.page_free[pages[0]])
    pm.free(pages)
    assert pm.num_free_pages == 4 and bool(pm.page_free[pages[0]])
    with pytest.raises(ValueError):
        pm.free(pages)
    with pytest.raises(ValueError):
        pm.add_ref(pages)


def test_lowest_page_ids_first_and_reuse():
    pm, _ = _managers(num_pages=8)
    a = pm.alloc(9)   # 3 pages
    b = pm.alloc(4)
    assert a.tolist() == [0, 1, 2] and b.tolist() == [3]
    pm.free(a[1:2])
    assert pm.alloc(8).tolist() == [1, 4]
    assert pm.alloc(4 * 4) is None
    pm.free_all()
    assert pm.num_free_pages == 8 and pm.alloc(4).tolist() == [0]


def test_reserved_capacity_keeps_logical_length():
    pm, rm = _managers()
    req = rm.reserve_req(num_tokens=1, reserved_tokens=9)
    assert req == 0 and rm.req_token_count[0] == 1
    assert len(rm.req_page_table[0]) == 3 and pm.num_free_pages == 1
    assert rm.extend_req(0, 8)
    assert rm.req_token_count[0] == 9 and len(rm.req_page_table[0]) == 3 and pm.num_free_pages == 1
    assert rm.get_token_indices(0, 9).tolist() == list(range(9))


def test_extend_appends_only_new_entries():
    pm, rm = _managers(max_requests=1)
    assert rm.alloc_req(0, 3)
    with patch.object(pm, "build_token_table", side_effect=AssertionError("full rebuild")):
        assert rm.extend_req(0, 1)
        assert rm.extend_req(0, 1)   # crosses into a second page
    assert rm.req_token_count[0] == 5 and len(rm.req_page_table[0]) == 2
    assert rm.b_req_tokens_table[0, :5].tolist() == [0, 1, 2, 3, 4]
    assert rm.b_req_block_table[0, :2].tolist() == [0, 1]


def test_share_and_request_ids():
    pm, rm = _managers()
    assert rm.alloc_req(0, 5)
    pages = rm.req_page_table[0]
    assert rm.share_req_from_pages(1, pages, 5)
    assert rm.get_token_indices(1, 5).tolist() == [0, 1, 2, 3, 4]
    assert int(pm.page_refcount[pages[0]]) == 2
    rm.free_req(0)
    assert not bool(pm.page_free[pages[0]])
    rm.free_req(1)
    assert bool(pm.page_free[pages[0]])
    assert rm.free_req_indices == [0, 1]
    assert rm.reserve_req(3) == 0
    assert all(isinstance(p, int) for p in rm.request_pages(0))


def test_capacity_failures_return_false_or_none():
    pm, rm = _managers(num_pages=2)
    assert rm.alloc_req(0, 8)
    assert not rm.alloc_req(0, 1)          # id in use
    assert not rm.alloc_req(1, 1)          # pool exhausted
    assert rm.reserve_req(1) is None
    assert not rm.extend_req(0, 1)         # needs a page that does not exist
    assert not rm.extend_req(0, 100)       # beyond max_seq_len
    assert rm.extend_req(0, 0)
    assert not rm.alloc_req(1, 0) and not rm.alloc_req(1, 5, reserved_tokens=4)
    with pytest.raises(KeyError):
        rm.extend_req(1, 1)
    with pytest.raises(KeyError):
        rm.batch_metadata([1])
    with pytest.raises(ValueError):
        rm.batch_metadata([])


def test_batch_metadata_dtypes_and_values():
    pm, rm = _managers(num_pages=8)
    assert rm.alloc_req(0, 3) and rm.alloc_req(1, 5)
    ids, lens, last = rm.batch_metadata([1, 0])
    assert ids.dtype == torch.int32 and lens.dtype == torch.int64 and last.dtype == torch.int32
    assert ids.tolist() == [1, 0] and lens.tolist() == [5, 3]
    assert last.tolist() == [rm.b_req_tokens_table[1, 4].item(), rm.b_req_tokens_table[0, 2].item()]


def test_kv_engine_expectations():
    refs = kv_engine.KVBlockRefCounter(total_blocks=4)
    assert refs.acquire(2) == (0, 1) and refs.refcount(0) == 1 and refs.available_count == 2
    refs.add_ref((0,))
    refs.release((0, 1))
    assert refs.refcount(0) == 1 and refs.refcount(1) == 0 and refs.available_count == 3
    with pytest.raises(ValueError):
        kv_engine.KVBlockRefCounter(1).release((0,))
    with pytest.raises(ValueError):
        kv_engine.KVBlockRefCounter(0)
    cache = kv_engine.PrefixCache(block_size=4)
    cache.put((1, 2, 3, 4, 5, 6, 7, 8), (10, 11))
    m = cache.match((1, 2, 3, 4, 5, 6, 9, 9))
    assert (m.matched_tokens, m.block_ids) == (4, (10,))
    cache2 = kv_engine.PrefixCache(block_size=4)
    cache2.put((1, 2, 3), (10,))
    assert cache2.match((1, 2, 3, 4)).matched_tokens == 0
    with pytest.raises(ValueError):
        cache.put((1, 2, 3, 4, 5, 6, 7, 8), (1,))
    chunks = kv_engine.ChunkedPrefillPlanner(chunk_size=4).plan(prompt_length=10)
    assert [(c.start, c.end) for c in chunks] == [(0, 4), (4, 8), (8, 10)]
    with pytest.raises(ValueError):
        kv_engine.ChunkedPrefillPlanner(chunk_size=0)
    plan = kv_engine.MixedLengthPrefillPacker().pack(((10, 11), (20,), (30, 31, 32)))
    assert plan.flat_token_ids == (10, 11, 20, 30, 31, 32)
    assert plan.flat_position_ids == (0, 1, 0, 0, 1, 2)
    assert [(r.request_index, r.start, r.length, r.end) for r in plan.requests] == \
        [(0, 0, 2, 2), (1, 2, 1, 3), (2, 3, 3, 6)]
    assert plan.total_tokens == 6 and plan.start_locs == (0, 2, 3) and plan.seq_lens == (2, 1, 3)
