"""Decode steps with host buffers (HostDecodeSteps / b200kv_host_steps_*): same results as the
device-tensor operator and the CPU oracle, slots reused in a pipeline, argument checks.

Tolerances: pool rows bit-exact; attention max-abs-error <= 2e-3 against the oracle and bit-equal
to the device-tensor operator (it is the same kernel on the same inputs)."""

import math

import numpy as np
import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200 import kernels, workloads as W
from llama_lite_npu_b200.host_step import HostDecodeSteps
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


def _fill(buf, c):
    kvh = c.cfg.kv_heads
    buf.q[...] = c.q.numpy()
    buf.new_k[...] = c.new_kv[:, :kvh].numpy()
    buf.new_v[...] = c.new_kv[:, kvh:].numpy()
    buf.seq_lens[...] = c.seq_lens.astype(np.int32)
    buf.slots[...] = c.slots.numpy()


def _oracle(c):
    pool = c.pool.clone()
    keep = torch.from_numpy(c.seq_lens > 0)
    O.kv_append(c.new_kv[keep], c.slots[keep], pool)
    kvh = c.cfg.kv_heads
    return pool, O.paged_decode(c.q, pool[:, :kvh], pool[:, kvh:], SCALE, c.token_table, c.seq_lens_t)


CASES = {
    "c1": lambda: W.make_decode_case(W.C1, fill="hash"),
    "gqa8_small": lambda: G.build_decode("decode_gqa8_small"),
    "edges": lambda: G.build_decode("decode_gqa4_edges"),
    "mixed_with_empty": lambda: W.make_decode_case(
        W.DecodeConfig("mix", 7, 16, 2, 512, 1, 1, seed=95), fill="hash",
        lengths=np.array([0, 5, 0, 2000, 1, 0, 333])),
}


@pytest.mark.parametrize("name", list(CASES))
@pytest.mark.parametrize("table_kind", ["block", "token"])
def test_host_step_matches_oracle_and_device_operator(name, table_kind):
    c = CASES[name]()
    batch = c.q.shape[0]
    want_pool, want = _oracle(c)
    steps = HostDecodeSteps(batch, c.cfg.q_heads, c.cfg.kv_heads, 128, depth=2)
    pool = c.pool.to(DEV)
    tbl = (c.block_table if table_kind == "block" else c.token_table).to(DEV)
    torch.cuda.synchronize()
    bound = steps.bind(pool, tbl, qk_scale=SCALE, table_kind=table_kind)
    buf = steps.buffers(1, batch)
    _fill(buf, c)
    steps.submit(1, batch, bound, c.max_len)
    steps.wait(1)
    kernels.check_status(0)
    assert torch.equal(pool.cpu(), want_pool), "the append through host buffers is not bit-exact"
    got = torch.from_numpy(buf.out.copy())
    assert float((got.float() - want.float()).abs().max()) <= ATTN_TOL
    # the device-tensor operator on the same inputs: the very same numbers
    pool2 = c.pool.to(DEV)
    out2 = kernels.append_flash_decoding(c.new_kv.to(DEV), c.slots.to(DEV), pool2, c.q.to(DEV), SCALE, tbl,
                                         c.seq_lens_t.to(DEV), c.max_len, table_kind=table_kind)
    live = torch.from_numpy(c.seq_lens > 0)
    assert torch.equal(out2.cpu()[live], got[live])
    steps.close()


def test_pipeline_of_steps_over_reused_slots():
    """Twelve consecutive decode steps of one batch through two slots: every step appends one
    token per sequence and attends over the grown sequence; the pool and every step's output
    must equal the oracle's replay of the same steps."""
    rng = np.random.default_rng(5)
    cfg = W.DecodeConfig("pipe", 6, 8, 2, 200, 1, 1, seed=77)
    batch, kvh = 6, 2
    n_steps = 12
    first = np.array([1, 15, 16, 17, 100, 31])          # lengths at the first step, new token included
    c = W.make_decode_case(cfg, fill="hash", lengths=first + n_steps - 1)   # tables cover the last step
    pool = c.pool.to(DEV)
    tbl = c.block_table.to(DEV)
    block_table = c.block_table.numpy()
    torch.cuda.synchronize()
    steps = HostDecodeSteps(8, 8, 2, 128, depth=2)     # max_batch above the batch in use
    bound = steps.bind(pool, tbl, qk_scale=SCALE, table_kind="block")

    ref_pool = c.pool.clone()
    lens = first.astype(np.int64) - 1                  # lengths before the first step's token
    inputs, outs = [], [None] * n_steps
    for s in range(n_steps):
        lens = lens + 1
        q = torch.from_numpy(rng.standard_normal((batch, 8, 128)).astype(np.float16))
        new_kv = torch.from_numpy(rng.standard_normal((batch, 2 * kvh, 128)).astype(np.float16))
        pos = lens - 1
        slots = (block_table[np.arange(batch), pos // 16].astype(np.int64) * 16 + pos % 16).astype(np.int32)
        inputs.append((q, new_kv, lens.copy(), slots))

    def collect(s):
        steps.wait(s % 2)
        outs[s] = torch.from_numpy(steps.buffers(s % 2, batch).out.copy())

    for s, (q, new_kv, ln, slots) in enumerate(inputs):
        if s >= 2:
            collect(s - 2)                             # the slot is free once its result is home
        buf = steps.buffers(s % 2, batch)
        buf.q[...] = q.numpy()
        buf.new_k[...] = new_kv[:, :kvh].numpy()
        buf.new_v[...] = new_kv[:, kvh:].numpy()
        buf.seq_lens[...] = ln.astype(np.int32)
        buf.slots[...] = slots
        steps.submit(s % 2, batch, bound, int(ln.max()))
    collect(n_steps - 2)
    collect(n_steps - 1)
    kernels.check_status(0)

    token_table = c.token_table
    for s, (q, new_kv, ln, slots) in enumerate(inputs):
        O.kv_append(new_kv, torch.from_numpy(slots), ref_pool)
        want = O.paged_decode(q, ref_pool[:, :kvh], ref_pool[:, kvh:], SCALE, token_table,
                              torch.from_numpy(ln))
        assert float((outs[s].float() - want.float()).abs().max()) <= ATTN_TOL, f"step {s}"
    assert torch.equal(pool.cpu(), ref_pool)
    steps.close()


def test_host_steps_argument_checks():
    steps = HostDecodeSteps(4, 8, 2, 128, depth=2)
    c = G.build_decode("decode_gqa4_edges")
    pool = c.pool.to(DEV)
    tbl = c.block_table.to(DEV)
    with pytest.raises(ValueError):
        steps.buffers(2, 1)                             # slot outside depth
    with pytest.raises(ValueError):
        steps.buffers(0, 5)                             # batch above max_batch
    if c.cfg.kv_heads != 2:
        with pytest.raises(ValueError):
            steps.bind(pool, tbl, qk_scale=SCALE, table_kind="block")
    with pytest.raises(ValueError):
        HostDecodeSteps(4, 8, 2, 64)                    # head_dim the kernel is not built for
    with pytest.raises(ValueError):
        HostDecodeSteps(4, 8, 2, 128, depth=9)
    with pytest.raises(ValueError):
        steps.bind(pool.cpu(), tbl, qk_scale=SCALE)     # the pool is device state
    steps.close()
    steps.close()                                       # idempotent


def test_unbound_submit_entry_point():
    """b200kv_host_steps_submit (every argument per call) gives what the bound form gives."""
    c = G.build_decode("decode_gqa8_small")
    batch, kvh = c.q.shape[0], c.cfg.kv_heads
    want_pool, want = _oracle(c)
    steps = HostDecodeSteps(batch, c.cfg.q_heads, kvh, 128, depth=2)
    pool = c.pool.to(DEV)
    tbl = c.block_table.to(DEV)
    torch.cuda.synchronize()
    _fill(steps.buffers(0, batch), c)
    k_ptr, v_ptr, tok_stride, head_stride, pool_tokens, _, _ = kernels._pool_geometry(pool)
    rc = steps._lib.b200kv_host_steps_submit(
        steps._handle, 0, batch, k_ptr, v_ptr, tok_stride, head_stride, pool_tokens, tbl.data_ptr(), tbl.stride(0),
        kernels.TABLE_BLOCK, tbl.shape[0], tbl.shape[1], None, 16, SCALE, c.max_len, 0,
        kernels.status_tensor(0).data_ptr())
    assert rc == 0
    steps.flush()
    steps.wait(0)
    kernels.check_status(0)
    assert torch.equal(pool.cpu(), want_pool)
    got = torch.from_numpy(steps.buffers(0, batch).out.copy())
    assert float((got.float() - want.float()).abs().max()) <= ATTN_TOL
    # a slot whose step is still pending cannot take another one
    _fill(steps.buffers(1, batch), c)
    bound = steps.bind(pool, tbl, qk_scale=SCALE, table_kind="block")
    steps.submit(1, batch, bound, c.max_len)
    with pytest.raises(ValueError):
        steps.submit(1, batch, bound, c.max_len)
    steps.wait(1)
    # reset: nothing in flight afterwards, and the next step still gives the same numbers
    steps.submit(0, batch, bound, c.max_len)
    steps.reset()
    got2 = torch.from_numpy(steps.buffers(0, batch).out.copy())
    assert torch.equal(got2, got)
    steps.submit(1, batch, bound, c.max_len)
    steps.wait(1)
    assert torch.equal(torch.from_numpy(steps.buffers(1, batch).out.copy()), got)
    kernels.check_status(0)
    steps.close()
