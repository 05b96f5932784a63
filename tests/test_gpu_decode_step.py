"""The one-launch decode step (KV append + paged decode + merge of the split partials) against
the CPU oracle, and the device-side checks of the decode entry points.

Tolerances: pool rows written by the fused append bit-exact; attention max-abs-error <= 2e-3."""

import math

import numpy as np
import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200 import kernels, workloads as W
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3
SCALE = 1.0 / math.sqrt(128)
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _lib_loaded(built_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    kernels.check_status(0)


def _maxdiff(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def _counters_are_zero():
    ws = kernels._workspace.get(0)
    return ws is None or int(ws[: kernels.DECODE_COUNTER_BYTES].view(torch.int32).abs().sum()) == 0


def _oracle_step(c):
    pool = c.pool.clone()
    O.kv_append(c.new_kv, c.slots, pool)
    kvh = c.cfg.kv_heads
    out = O.paged_decode(c.q, pool[:, :kvh], pool[:, kvh:], SCALE, c.token_table, c.seq_lens_t)
    return pool, out


def _fused_gpu(c, table_kind="block", **kw):
    pool = c.pool.to(DEV)
    tbl = (c.block_table if table_kind == "block" else c.token_table).to(DEV)
    out = kernels.append_flash_decoding(c.new_kv.to(DEV), c.slots.to(DEV), pool, c.q.to(DEV), SCALE, tbl,
                                        c.seq_lens_t.to(DEV), c.max_len, table_kind=table_kind, **kw)
    return pool, out


STEP_CASES = {
    "c1": lambda: W.make_decode_case(W.C1, fill="hash"),
    "gqa8_small": lambda: G.build_decode("decode_gqa8_small"),
    "edges": lambda: G.build_decode("decode_gqa4_edges"),
    "page_boundaries": lambda: W.make_decode_case(
        W.DecodeConfig("pb", 9, 8, 1, 256, 1, 1, seed=91), fill="hash",
        lengths=np.array([1, 16, 17, 32, 33, 48, 64, 65, 129])),
    "many_short_all_whole": lambda: W.make_decode_case(
        W.DecodeConfig("short", 300, 8, 2, 400, 1, 16, seed=92), fill="hash"),
    "one_long_many_pieces": lambda: W.make_decode_case(
        W.DecodeConfig("long", 1, 8, 1, 1400, 1, 1, seed=93), fill="hash", lengths=np.array([21003])),
    "gqa16_two_long": lambda: W.make_decode_case(
        W.DecodeConfig("g16", 2, 32, 2, 700, 1, 1, seed=94), fill="hash", lengths=np.array([5000, 4999])),
    "mixed_with_empty": lambda: W.make_decode_case(
        W.DecodeConfig("mix", 7, 16, 2, 512, 1, 1, seed=95), fill="hash",
        lengths=np.array([0, 5, 0, 2000, 1, 0, 333])),
}


@pytest.mark.parametrize("name", list(STEP_CASES))
@pytest.mark.parametrize("table_kind", ["block", "token"])
def test_fused_step_equals_append_then_decode(name, table_kind):
    c = STEP_CASES[name]()
    want_pool, want = _oracle_step(c)
    if (c.seq_lens == 0).any():
        # a sequence without tokens appends nothing: its slot entry is not used
        keep = torch.from_numpy(c.seq_lens > 0)
        want_pool = c.pool.clone()
        O.kv_append(c.new_kv[keep], c.slots[keep], want_pool)
        kvh = c.cfg.kv_heads
        want = O.paged_decode(c.q, want_pool[:, :kvh], want_pool[:, kvh:], SCALE, c.token_table, c.seq_lens_t)
    pool, out = _fused_gpu(c, table_kind)
    torch.cuda.synchronize()
    kernels.check_status(0)
    assert torch.equal(pool.cpu(), want_pool), "the fused append is not bit-exact"
    assert _maxdiff(out, want) <= ATTN_TOL
    assert _counters_are_zero(), "arrival counters must be back at zero after a launch"
    # and the same through the separate operators
    pool2 = c.pool.to(DEV)
    keep = torch.from_numpy(c.seq_lens > 0).to(DEV)
    kernels.update_kv_buffer(c.new_kv.to(DEV)[keep], c.slots.to(DEV)[keep], pool2)
    kvh = c.cfg.kv_heads
    tbl = (c.block_table if table_kind == "block" else c.token_table).to(DEV)
    out2 = kernels.flash_decoding(c.q.to(DEV), pool2[:, :kvh], pool2[:, kvh:], SCALE, tbl,
                                  c.seq_lens_t.to(DEV), c.max_len, table_kind=table_kind)
    assert torch.equal(pool2, pool)
    assert _maxdiff(out2, out) <= ATTN_TOL


def test_fused_step_c2_shard_full_size():
    """One KV head of the Qwen3-32B shape at full size (the 8-GPU shard): pool rows bit-exact,
    sampled sequences against the oracle."""
    cfg = W.shard_kv_heads(W.C2, 8, 0)
    c = W.make_decode_case(cfg, device=DEV, fill="randn")
    before = c.pool.clone()
    out = kernels.append_flash_decoding(c.new_kv, c.slots, c.pool, c.q, SCALE, c.block_table, c.seq_lens_t,
                                        c.max_len, table_kind="block")
    torch.cuda.synchronize()
    kernels.check_status(0)
    before[c.slots.long()] = c.new_kv
    assert torch.equal(before, c.pool)
    for b in (0, 13, 31):
        L = int(c.seq_lens[b])
        sl = c.token_table[b, :L].long()
        want = O.paged_decode(c.q[b: b + 1].cpu(), c.k_cache[sl].cpu(), c.v_cache[sl].cpu(), SCALE,
                              torch.arange(L, dtype=torch.int32)[None], torch.tensor([L]))
        assert _maxdiff(out[b: b + 1], want) <= ATTN_TOL
    assert _counters_are_zero()


def test_fused_step_flags_a_slot_that_is_not_the_last_position():
    c = G.build_decode("decode_gqa8_small")
    slots = c.slots.clone()
    slots[2] = slots[2] - 1          # the previous token's slot: inside the pool, but not position L-1
    pool = c.pool.to(DEV)
    kernels.append_flash_decoding(c.new_kv.to(DEV), slots.to(DEV), pool, c.q.to(DEV), SCALE,
                                  c.block_table.to(DEV), c.seq_lens_t.to(DEV), c.max_len, table_kind="block")
    with pytest.raises(RuntimeError, match="slot"):
        kernels.check_status(0)
    slots[2] = 10 ** 8               # outside the pool: skipped, reported
    pool = c.pool.to(DEV)
    kernels.append_flash_decoding(c.new_kv.to(DEV), slots.to(DEV), pool, c.q.to(DEV), SCALE,
                                  c.block_table.to(DEV), c.seq_lens_t.to(DEV), c.max_len, table_kind="block")
    with pytest.raises(RuntimeError, match="slot"):
        kernels.check_status(0)
    want = c.pool.clone()
    keep = torch.tensor([True, True, False, True, True])
    O.kv_append(c.new_kv[keep], c.slots[keep], want)
    assert torch.equal(pool.cpu(), want)


def test_decode_row_id_outside_the_table_is_skipped_and_reported():
    c = G.build_decode("decode_gqa8_small")
    rows = torch.arange(5, dtype=torch.int32)
    rows[1] = 5                      # the table has rows 0..4
    rows[3] = -2
    got = kernels.flash_decoding(c.q.to(DEV), c.pool.to(DEV)[:, :2], c.pool.to(DEV)[:, 2:], SCALE,
                                 c.block_table.to(DEV), c.seq_lens_t.to(DEV), c.max_len,
                                 b_req_idx=rows.to(DEV), table_kind="block")
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    want = O.paged_decode(c.q, c.k_cache, c.v_cache, SCALE, c.token_table, c.seq_lens_t)
    good = torch.tensor([0, 2, 4])
    assert _maxdiff(got[good], want[good]) <= ATTN_TOL
    assert float(got[1].abs().sum()) == 0.0 and float(got[3].abs().sum()) == 0.0
    assert _counters_are_zero()


def test_decode_length_above_the_stated_maximum_is_clamped_and_reported():
    c = G.build_decode("decode_gqa8_small")
    lens = c.seq_lens_t.clone()
    lens[0] = 10 ** 7                # stale / corrupt length; max_len stays the true bound (300)
    got = kernels.flash_decoding(c.q.to(DEV), c.pool.to(DEV)[:, :2], c.pool.to(DEV)[:, 2:], SCALE,
                                 c.block_table.to(DEV), lens.to(DEV), c.max_len, table_kind="block")
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    want = O.paged_decode(c.q, c.k_cache, c.v_cache, SCALE, c.token_table, c.seq_lens_t)
    assert _maxdiff(got, want) <= ATTN_TOL          # sequence 0 has exactly max_len tokens


def test_advance_then_decode_back_to_back_with_fresh_metadata():
    """decode_advance writes the lengths and slots that the very next launch plans from: with
    metadata_fresh=True the decode launch is fully ordered after it.  Six steps, each against the
    oracle's advance + append + decode."""
    cfg = W.DecodeConfig("chain", 6, 16, 2, 128, 1, 1, seed=96)
    c = W.make_decode_case(cfg, fill="hash", lengths=np.array([14, 15, 16, 31, 200, 1]))
    # the case holds L tokens per sequence; start one step earlier: L-1 in the pool, then advance
    spare = torch.cat([c.block_table, torch.zeros(cfg.batch, 2, dtype=torch.int32)], dim=1)
    used = set(int(x) for p in c.pages for x in p)
    free = [p for p in range(cfg.num_pages) if p not in used]
    for b in range(cfg.batch):       # every row gets a spare page for the steps that cross a boundary
        spare[b, len(c.pages[b])] = free.pop()
    lens_h = c.seq_lens_t.clone()
    pool_h = c.pool.clone()
    lens_d, pool_d, tbl_d = lens_h.to(DEV), pool_h.to(DEV), spare.to(DEV)
    slots_d = torch.zeros(cfg.batch, dtype=torch.int32, device=DEV)
    tok_h = torch.zeros(cfg.batch, spare.shape[1] * 16, dtype=torch.int32)
    tok_h[:, : c.token_table.shape[1]] = c.token_table
    for step in range(6):
        new_kv = W.hash_normal_fp16(400 + step, (cfg.batch, 4, 128), 1)
        q = W.hash_normal_fp16(400 + step, (cfg.batch, 16, 128), 2)
        slots_h = O.decode_advance(lens_h, spare, 16, token_table=tok_h)
        O.kv_append(new_kv, slots_h, pool_h)
        want = O.paged_decode(q, pool_h[:, :2], pool_h[:, 2:], SCALE, tok_h, lens_h)
        kernels.advance_decode_metadata(lens_d, slots_d, tbl_d, 16, cfg.num_pages)
        got = kernels.append_flash_decoding(new_kv.to(DEV), slots_d, pool_d, q.to(DEV), SCALE, tbl_d, lens_d,
                                            int(lens_h.max()), table_kind="block", metadata_fresh=True)
        assert torch.equal(lens_d.cpu(), lens_h) and torch.equal(slots_d.cpu(), slots_h)
        assert _maxdiff(got, want) <= ATTN_TOL, step
    assert torch.equal(pool_d.cpu(), pool_h)
    kernels.check_status(0)


def test_captured_chain_of_whole_sequence_steps():
    """A batch of one-page sequences (every piece is a whole sequence, no partial is ever
    written) stepped through advance -> fused append + decode inside ONE captured graph, two
    layers per step; replayed several times and compared with the oracle after every replay."""
    cfg = W.DecodeConfig("graph_chain", 40, 8, 1, 64, 1, 1, seed=97)
    lens0 = np.full(cfg.batch, 3)
    c = W.make_decode_case(cfg, fill="hash", lengths=lens0)
    layers = 2
    pools_h = [c.pool.clone(), W.hash_normal_fp16(98, tuple(c.pool.shape), 1)]
    pools_d = [p.to(DEV) for p in pools_h]
    tbl_h = c.block_table.clone()
    tbl_d = tbl_h.to(DEV)
    lens_h = c.seq_lens_t.clone()
    lens_d = lens_h.to(DEV)
    slots_d = torch.zeros(cfg.batch, dtype=torch.int32, device=DEV)
    new_kv_d = torch.zeros(cfg.batch, 2, 128, dtype=torch.float16, device=DEV)
    q_d = torch.zeros(cfg.batch, 8, 128, dtype=torch.float16, device=DEV)
    outs_d = [torch.zeros_like(q_d) for _ in range(layers)]
    tok_h = torch.zeros(cfg.batch, 16, dtype=torch.int32)
    tok_h[:, : c.token_table.shape[1]] = c.token_table

    def step():
        kernels.advance_decode_metadata(lens_d, slots_d, tbl_d, 16, cfg.num_pages)
        for li in range(layers):
            kernels.append_flash_decoding(new_kv_d, slots_d, pools_d[li], q_d, SCALE, tbl_d, lens_d, 16,
                                          table_kind="block", out=outs_d[li], metadata_fresh=(li == 0))

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        lens_d.copy_(lens_h)
        step()                                   # warm-up (also sizes the workspace)
        stream.synchronize()
        lens_d.copy_(lens_h)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        lens_d.copy_(lens_h)
        for pd, ph in zip(pools_d, pools_h):
            pd.copy_(ph)
        for it in range(8):                      # stays inside the first page (3 + 8 <= 16)
            new_kv = W.hash_normal_fp16(500 + it, (cfg.batch, 2, 128), 1)
            q = W.hash_normal_fp16(500 + it, (cfg.batch, 8, 128), 2)
            new_kv_d.copy_(new_kv)
            q_d.copy_(q)
            graph.replay()
            stream.synchronize()
            slots_h = O.decode_advance(lens_h, tbl_h, 16, token_table=tok_h)
            for li in range(layers):
                O.kv_append(new_kv, slots_h, pools_h[li])
                want = O.paged_decode(q, pools_h[li][:, :1], pools_h[li][:, 1:], SCALE, tok_h, lens_h)
                assert _maxdiff(outs_d[li], want) <= ATTN_TOL, (it, li)
            assert torch.equal(lens_d.cpu(), lens_h)
    kernels.check_status(0)
    assert _counters_are_zero()


def test_debug_mode_checks_index_tensors_on_the_host_before_launch():
    """Debug mode: an out-of-range slot, two tokens aimed at one slot with different rows, a
    length beyond the stated maximum and a request id outside the table are all refused on the
    host; two tokens that write the same row to one slot (a shared partial page) are allowed."""
    src, slots, pool = G.build_append("append_prefill")
    src, slots, pool = src.to(DEV), slots.to(DEV), pool.to(DEV)
    kernels.set_debug(True)
    try:
        kernels.update_kv_buffer(src, slots, pool)                       # clean input passes
        dup = slots.clone()
        dup[7] = dup[3]
        with pytest.raises(ValueError, match="different K/V rows"):
            kernels.update_kv_buffer(src, dup, pool)
        same = src.clone()
        same[7] = same[3]
        before = pool.clone()
        kernels.update_kv_buffer(same, dup, pool)                        # identical payloads: fine
        before[dup.long()] = same
        assert torch.equal(pool, before)
        far = slots.clone()
        far[0] = pool.shape[0]
        with pytest.raises(ValueError, match="outside the pool"):
            kernels.update_kv_buffer(src, far, pool)
        rows = src.shape[1]
        with pytest.raises(ValueError, match="different K/V rows"):
            kernels.update_kv_buffer_split(src[:, : rows // 2].contiguous(), src[:, rows // 2:].contiguous(), dup, pool)
        c = G.build_decode("decode_gqa8_small")
        lens = c.seq_lens_t.clone()
        lens[1] = c.max_len + 1
        with pytest.raises(ValueError, match="length"):
            kernels.flash_decoding(c.q.to(DEV), c.pool.to(DEV)[:, :2], c.pool.to(DEV)[:, 2:], SCALE,
                                   c.block_table.to(DEV), lens.to(DEV), c.max_len, table_kind="block")
        with pytest.raises(ValueError, match="request id"):
            kernels.flash_decoding(c.q.to(DEV), c.pool.to(DEV)[:, :2], c.pool.to(DEV)[:, 2:], SCALE,
                                   c.block_table.to(DEV), c.seq_lens_t.to(DEV), c.max_len, table_kind="block",
                                   b_req_idx=torch.tensor([0, 1, 2, 3, 9], dtype=torch.int32, device=DEV))
    finally:
        kernels.set_debug(False)
    kernels.check_status(0)


def test_prefill_request_outside_the_table_is_skipped_and_reported():
    """A request id outside the table, or a context + chunk length beyond the table's width, must
    not become a table read: that request is skipped and reported, the others are computed."""
    c = G.build_prefill("prefill_hist_gqa2")
    kvh = c.cfg.kv_heads
    pool = c.pool.clone()
    O.kv_append(c.new_kv, c.slots, pool)
    want = O.paged_attention(c.q, pool[:, :kvh], pool[:, kvh:], SCALE, c.token_table, c.req_ids, c.q_start,
                             c.ctx_lens_t, c.q_lens_t)
    pool_d = pool.to(DEV)
    args = dict(table_kind="block")

    def run(req_ids, ctx):
        return kernels.paged_chunk_flash_attention(
            c.q.to(DEV), pool_d[:, :kvh], pool_d[:, kvh:], SCALE * 1.4426950408889634, c.block_table.to(DEV),
            req_ids.to(DEV), c.q_start.to(DEV), ctx.to(DEV), c.q_lens_t.to(DEV), c.max_q_len, **args)

    def rows(r):
        s0 = int(c.q_start[r])
        return slice(s0, s0 + int(c.q_lens[r]))

    bad_ids = c.req_ids.clone()
    bad_ids[1] = c.block_table.shape[0] + 3
    got = run(bad_ids, c.ctx_lens_t)
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    for r in (0, 2):
        assert _maxdiff(got[rows(r)], want[rows(r)]) <= ATTN_TOL
    bad_ctx = c.ctx_lens_t.clone()
    bad_ctx[2] = c.block_table.shape[1] * 16                      # context alone fills the table: ctx + q overflows it
    got = run(c.req_ids, bad_ctx)
    with pytest.raises(RuntimeError, match="length"):
        kernels.check_status(0)
    for r in (0, 1):
        assert _maxdiff(got[rows(r)], want[rows(r)]) <= ATTN_TOL


@pytest.mark.parametrize("batch,kvh,length", [(64, 4, 290), (32, 8, 333), (74, 8, 160), (64, 8, 129), (37, 8, 33),
                                                (16, 8, 500), (8, 4, 600), (5, 8, 300), (3, 1, 2000)])
def test_uniform_lengths_take_whole_sequences_per_team(batch, kvh, length):
    """Batches of one length are cut at sequence boundaries (one team per sequence, or per group of
    k sequences; with few sequences the general cut applies): same numbers as ever.  With one odd sequence in the batch the general cut, with
    its partial pieces and merges, is back."""
    pages = batch * ((length + 17 + 15) // 16) + 8
    for seed, odd in ((97, False), (98, True)):
        lens = np.full(batch, length)
        if odd:
            lens[batch // 2] = length + 17
        cfg = W.DecodeConfig("uniform", batch, 2 * kvh, kvh, pages, 1, 1, seed=seed)
        c = W.make_decode_case(cfg, fill="hash", lengths=lens)
        want_pool, want = _oracle_step(c)
        for table_kind in ("block", "token"):
            pool, out = _fused_gpu(c, table_kind)
            torch.cuda.synchronize()
            kernels.check_status(0)
            assert torch.equal(pool.cpu(), want_pool)
            assert _maxdiff(out, want) <= ATTN_TOL
            assert _counters_are_zero()
