"""Decode-step batch metadata: the oracle against the reference classes' recorded behaviour, the
host half of the device path against the host path, and (GPU) the kernel against both.  Integer
work: everything here is bit-exact."""

import json

import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200.executor import PagedKVExecutor
from llama_lite_npu_b200.paged_attention import PagedKVCacheManager, PagedReqTokensManager
from oracle import paged_kv_oracle as O


@pytest.fixture(scope="module")
def recorded():
    return json.loads((G.GOLDEN_DIR / "decode_metadata_golden.json").read_text())


def _tables(recorded, rows=8):
    ps = G.METADATA_SCRIPT["page_size"]
    block = torch.zeros(rows, recorded["max_pages"], dtype=torch.int32)
    tokens = torch.zeros(rows, G.METADATA_SCRIPT["max_seq_len"], dtype=torch.int32)
    for r, pages, row in zip(recorded["batch"], recorded["pages_per_request"], recorded["token_rows"]):
        block[r, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
    for r, start, row in zip(recorded["batch"], recorded["start_lens"], recorded["token_rows"]):
        tokens[r, :start] = torch.tensor(row[:start], dtype=torch.int32)
    return ps, block, tokens


def test_oracle_reproduces_reference_decode_metadata(recorded):
    ps, block, tokens = _tables(recorded)
    lens = torch.tensor(recorded["start_lens"], dtype=torch.int64)
    req = torch.tensor(recorded["batch"], dtype=torch.int32)
    for step in recorded["steps"]:
        slots = O.decode_advance(lens, block, ps, req, tokens)
        assert lens.tolist() == step["seq_lens"] and slots.tolist() == step["slots"]
        assert req.tolist() == step["req_ids"]
    for r, row in zip(recorded["batch"], recorded["token_rows"]):
        assert tokens[r, : len(row)].tolist() == row


def _twin_managers():
    sc = G.METADATA_SCRIPT
    out = []
    for _ in range(2):
        pm = PagedKVCacheManager(1, 1, 8, sc["num_pages"], sc["page_size"], torch.float16, "cpu")
        rm = PagedReqTokensManager(sc["max_requests"], sc["max_seq_len"], pm, device="cpu")
        ids = [rm.reserve_req(n) for n in sc["prompt_lengths"]]
        rm.free_req(ids[sc["drop"]])
        out.append((pm, rm, [ids[i] for i in sc["batch_order"]]))
    return out


def test_host_half_of_device_path_matches_host_path_and_reference(recorded):
    (pm_a, rm_a, batch), (pm_b, rm_b, _) = _twin_managers()
    assert batch == recorded["batch"]
    for step in recorded["steps"]:
        for r in batch:
            assert rm_a.extend_req(r, 1)
        assert rm_b.extend_batch_for_device(batch) is None
        assert rm_a.req_token_count == rm_b.req_token_count
        assert torch.equal(rm_a._host_tokens, rm_b._host_tokens)
        assert torch.equal(rm_a._host_blocks, rm_b._host_blocks)
        assert [rm_b.req_token_count[r] for r in batch] == step["seq_lens"]
    assert pm_a.num_free_pages == pm_b.num_free_pages
    assert rm_b._host_page_counts.tolist() == [len(rm_b.req_page_table.get(r, ())) for r in range(8)]
    rm_b.free_req(batch[0])
    assert rm_b._host_page_counts[batch[0]] == 0


def test_host_half_reports_the_request_that_cannot_grow():
    pm = PagedKVCacheManager(1, 1, 8, 3, 4, torch.float16, "cpu")
    rm = PagedReqTokensManager(4, 16, pm, device="cpu")
    a, b = rm.reserve_req(4), rm.reserve_req(8)            # all three pages taken, both rows full pages
    assert rm.extend_batch_for_device([a, b]) == a          # no free page for a's fifth token
    assert rm.req_token_count[a] == 4 and rm.req_token_count[b] == 8
    rm.free_req(b)
    assert rm.extend_batch_for_device([a]) is None and rm.req_token_count[a] == 5


@pytest.mark.gpu
def test_kernel_reproduces_reference_decode_metadata(recorded, built_lib):
    from llama_lite_npu_b200 import kernels

    ps, block, tokens = _tables(recorded)
    dev = "cuda:0"
    for dtype in (torch.int64, torch.int32):
        lens = torch.tensor(recorded["start_lens"], dtype=dtype, device=dev)
        req = torch.tensor(recorded["batch"], dtype=torch.int32, device=dev)
        slots = torch.full((len(recorded["batch"]),), -1, dtype=torch.int32, device=dev)
        d_block, d_tokens = block.to(dev), tokens.to(dev)
        counts = torch.zeros(8, dtype=torch.int32, device=dev)
        for r, pages in zip(recorded["batch"], recorded["pages_per_request"]):
            counts[r] = len(pages)
        for step in recorded["steps"]:
            kernels.advance_decode_metadata(lens, slots, d_block, ps, G.METADATA_SCRIPT["num_pages"],
                                            b_req_idx=req, page_counts=counts, b_req_tokens_table=d_tokens)
            assert lens.tolist() == step["seq_lens"] and slots.tolist() == step["slots"]
        for r, row in zip(recorded["batch"], recorded["token_rows"]):
            assert d_tokens[r, : len(row)].tolist() == row
        kernels.check_status(0)
    # a sequence whose next page is not in the table: refused; its slot becomes -1 (the append skips
    # negative slots) instead of keeping the previous step's slot
    lens = torch.tensor([4, 3], dtype=torch.int32, device=dev)
    slots = torch.full((2,), 77, dtype=torch.int32, device=dev)    # stale slots of the previous step
    tbl = torch.tensor([[5, 0], [6, 0]], dtype=torch.int32, device=dev)
    kernels.advance_decode_metadata(lens, slots, tbl, 4, 8, page_counts=torch.tensor([1, 1], dtype=torch.int32, device=dev))
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    assert lens.tolist() == [4, 4] and slots.tolist() == [-1, 27]


@pytest.mark.gpu
def test_executor_device_extend_equals_host_extend(built_lib):
    dev = "cuda:0"
    twins = [PagedKVExecutor(1, 2, 128, 64, 8, 256, page_size=16, device=dev) for _ in range(2)]
    batches = []
    for ex in twins:
        ids = ex.reserve_paged_requests([30, 16, 47, 1, 9])
        ex.release_paged_request_ids((ids[1],))
        batches.append((ids[3], ids[0], ids[4], ids[2]))
    host, devp = twins
    host.extend_paged_requests(batches[0])
    devp.extend_paged_requests_on_device(batches[1])             # first call: host path, activates
    ptrs = (devp.atten_info.b_seq_len.data_ptr(), devp.atten_info.cur_select_index.data_ptr())
    for _ in range(40):                                          # crosses page boundaries on every row
        host.extend_paged_requests(batches[0])
        devp.extend_paged_requests_on_device(batches[1])
        a, b = host.atten_info, devp.atten_info
        assert torch.equal(a.b_seq_len, b.b_seq_len) and torch.equal(a.cur_select_index, b.cur_select_index)
        assert torch.equal(a.b_req_idx, b.b_req_idx) and a.max_actual_seq_len == b.max_actual_seq_len
        assert torch.equal(a.b_req_block_table, b.b_req_block_table)
        assert torch.equal(a.b_req_tokens_table, b.b_req_tokens_table)
    assert ptrs == (devp.atten_info.b_seq_len.data_ptr(), devp.atten_info.cur_select_index.data_ptr())
    assert host.req_tokens_manager.req_token_count == devp.req_tokens_manager.req_token_count
    # a different batch falls back to the host path and becomes the active one
    devp.extend_paged_requests_on_device(batches[1][:2])
    host.extend_paged_requests(batches[0][:2])
    assert torch.equal(host.atten_info.b_seq_len, devp.atten_info.b_seq_len)
    from llama_lite_npu_b200 import kernels
    kernels.check_status(0)


@pytest.mark.gpu
def test_update_kv_index_matches_statement(built_lib):
    from llama_lite_npu_b200 import kernels, workloads as W

    dev = "cuda:0"
    table = torch.from_numpy(W.hash_randint(4, 16 * 300, 0, 1 << 20, 1).astype("int32")).view(16, 300)
    req = torch.from_numpy(W.hash_permutation(4, 16, 2)[:11].astype("int32"))
    lens = torch.from_numpy(W.hash_randint(4, 11, 1, 301, 3))
    sel = torch.from_numpy(W.hash_randint(4, 11, 0, 1 << 20, 4).astype("int32"))
    for dtype in (torch.int32, torch.int64):
        want = table.clone()
        O.update_kv_index(want, req, lens.to(dtype), sel)
        got = table.to(dev)
        kernels.update_kv_index(got, req.to(dev), lens.to(dtype).to(dev), sel.to(dev))
        assert torch.equal(got.cpu(), want)
    view = table.to(dev).t().contiguous().t()                       # column-major strides
    kernels.update_kv_index(view, req.to(dev), lens.to(dev), sel.to(dev))
    assert torch.equal(view.cpu(), want)
    kernels.check_status(0)
    kernels.update_kv_index(got, req[:1].to(dev), torch.tensor([0], device=dev), sel[:1].to(dev))
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    assert torch.equal(got.cpu(), want)


@pytest.mark.gpu
def test_table_patch_writes_exactly_the_named_entries(built_lib):
    import numpy as np

    from llama_lite_npu_b200 import kernels

    dev = "cuda:0"
    table = torch.arange(7 * 300, dtype=torch.int32).view(7, 300)
    want = table.clone()
    rng = np.random.default_rng(3)
    for n in (1, 5, 96, 97, 250):                       # one launch holds 96 entries
        off = rng.choice(table.numel(), size=n, replace=False).astype(np.int64)
        val = rng.integers(-5, 1 << 30, size=n).astype(np.int32)
        got = want.to(dev)
        kernels.patch_table(got, off, val)
        want.view(-1)[torch.from_numpy(off)] = torch.from_numpy(val)
        assert torch.equal(got.cpu(), want)
    kernels.patch_table(got, np.zeros(0, np.int64), np.zeros(0, np.int32))     # nothing to do
    with pytest.raises(ValueError):                                               # offset outside the table
        kernels.patch_table(got, np.array([table.numel()], np.int64), np.array([1], np.int32))
    assert torch.equal(got.cpu(), want)
    kernels.check_status(0)
