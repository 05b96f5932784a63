"""Seeded random shapes against the CPU oracle: decode through the fused operator, the separate
operators and the host-buffer steps; packed prefill with prefix history.

The named cases elsewhere pin the edges the reference's tests name; this sweep looks for what
nobody thought of naming: odd group sizes with odd batches, empty sequences between long ones,
lengths one off a page or a tile, single-token prompts after a long shared prefix.

Tolerances: pool rows bit-exact; attention max-abs-error <= 2e-3."""

import math

import numpy as np
import pytest
import torch

from llama_lite_npu_b200 import kernels, workloads as W
from llama_lite_npu_b200.host_step import HostDecodeSteps
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3
SCALE = 1.0 / math.sqrt(128)
LOG2E = 1.4426950408889634
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _lib_loaded(built_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    kernels.check_status(0)


def _maxdiff(a, b):
    return float((a.float().cpu() - b.float().cpu()).abs().max())


def _draw_lengths(rng, batch):
    """A mix of the regimes a serving batch has: empty, one token, page/tile edges, short, long."""
    edges = np.array([1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 255, 256, 257])
    lens = np.empty(batch, dtype=np.int64)
    for i in range(batch):
        kind = rng.integers(0, 10)
        if kind == 0:
            lens[i] = 0
        elif kind <= 3:
            lens[i] = edges[rng.integers(0, len(edges))]
        elif kind <= 7:
            lens[i] = rng.integers(1, 400)
        else:
            lens[i] = rng.integers(400, 3000)
    if not lens.any():
        lens[0] = 33
    return lens


DECODE_SEEDS = list(range(16))


@pytest.mark.parametrize("seed", DECODE_SEEDS)
def test_decode_random_shape(seed):
    rng = np.random.default_rng(1000 + seed)
    kvh = int(rng.choice([1, 2, 4, 8]))
    group = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 12, 16]))
    batch = int(rng.integers(1, 24))
    lens = _draw_lengths(rng, batch)
    pages = int(np.ceil(lens / 16).sum()) + int(rng.integers(1, 64))
    cfg = W.DecodeConfig(f"rnd{seed}", batch, group * kvh, kvh, pages, 1, 1, seed=500 + seed)
    c = W.make_decode_case(cfg, fill="hash", lengths=lens)
    table_kind = "block" if seed % 2 == 0 else "token"
    lens_dtype = torch.int32 if seed % 3 == 0 else torch.int64
    live = torch.from_numpy(lens > 0)

    want_pool = c.pool.clone()
    O.kv_append(c.new_kv[live], c.slots[live], want_pool)
    want = O.paged_decode(c.q, want_pool[:, :kvh], want_pool[:, kvh:], SCALE, c.token_table, c.seq_lens_t)

    tbl = (c.block_table if table_kind == "block" else c.token_table).to(DEV)
    lens_d = c.seq_lens_t.to(lens_dtype).to(DEV)
    # fused operator
    pool = c.pool.to(DEV)
    out = kernels.append_flash_decoding(c.new_kv.to(DEV), c.slots.to(DEV), pool, c.q.to(DEV), SCALE, tbl, lens_d,
                                        c.max_len, table_kind=table_kind)
    torch.cuda.synchronize()
    kernels.check_status(0)
    assert torch.equal(pool.cpu(), want_pool)
    assert _maxdiff(out, want) <= ATTN_TOL
    # separate operators
    pool2 = c.pool.to(DEV)
    kernels.update_kv_buffer(c.new_kv.to(DEV)[live.to(DEV)], c.slots.to(DEV)[live.to(DEV)], pool2)
    out2 = kernels.flash_decoding(c.q.to(DEV), pool2[:, :kvh], pool2[:, kvh:], SCALE, tbl, lens_d, c.max_len,
                                  table_kind=table_kind)
    assert torch.equal(pool2, pool)
    assert _maxdiff(out2, want) <= ATTN_TOL
    # host-buffer steps (int32 lengths by construction)
    pool3 = c.pool.to(DEV)
    torch.cuda.synchronize()
    steps = HostDecodeSteps(batch, group * kvh, kvh, 128, depth=2)
    bound = steps.bind(pool3, tbl, qk_scale=SCALE, table_kind=table_kind)
    buf = steps.buffers(seed % 2, batch)
    buf.q[...] = c.q.numpy()
    buf.new_k[...] = c.new_kv[:, :kvh].numpy()
    buf.new_v[...] = c.new_kv[:, kvh:].numpy()
    buf.seq_lens[...] = lens.astype(np.int32)
    buf.slots[...] = c.slots.numpy()
    steps.submit(seed % 2, batch, bound, c.max_len)
    steps.wait(seed % 2)
    kernels.check_status(0)
    assert torch.equal(pool3.cpu(), want_pool)
    got3 = torch.from_numpy(buf.out.copy())
    assert _maxdiff(got3[live], want[live]) <= ATTN_TOL
    assert torch.equal(got3[live], out.cpu()[live]), "same kernel, same inputs: same bits"
    steps.close()


PREFILL_SEEDS = list(range(10))


@pytest.mark.parametrize("seed", PREFILL_SEEDS)
def test_prefill_random_shape(seed):
    rng = np.random.default_rng(2000 + seed)
    kvh = int(rng.choice([1, 2, 4]))
    group = int(rng.choice([1, 2, 3, 4, 7, 8, 16]))
    batch = int(rng.integers(1, 7))
    edges = np.array([1, 2, 16, 17, 64, 127, 128, 129, 255, 256, 257, 300])
    prompts = np.array([int(edges[rng.integers(0, len(edges))]) if rng.integers(0, 2) else int(rng.integers(1, 700))
                        for _ in range(batch)])
    shared = np.array([int(rng.integers(0, max(1, (p - 1) // 16 + 1))) if rng.integers(0, 2) else 0 for p in prompts])
    pages = int(np.ceil(prompts / 16).sum()) + int(rng.integers(1, 32))
    cfg = W.PrefillConfig(f"rndp{seed}", batch, group * kvh, kvh, pages, 1, 1, seed=700 + seed)
    c = W.make_prefill_case(cfg, fill="hash", prompt_lens=prompts, shared_pages=shared)
    table_kind = "block" if seed % 2 else "token"

    pool = c.pool.clone()
    O.kv_append(c.new_kv, c.slots, pool)
    want = O.paged_attention(c.q, pool[:, :kvh], pool[:, kvh:], SCALE, c.token_table, c.req_ids, c.q_start,
                             c.ctx_lens_t, c.q_lens_t)

    pool_d = c.pool.to(DEV)
    kernels.update_kv_buffer(c.new_kv.to(DEV), c.slots.to(DEV), pool_d)
    tbl = (c.token_table if table_kind == "token" else c.block_table).to(DEV)
    lens_cast = (lambda t: t.int()) if seed % 3 == 0 else (lambda t: t)
    got = kernels.paged_chunk_flash_attention(
        c.q.to(DEV), pool_d[:, :kvh], pool_d[:, kvh:], SCALE * LOG2E, tbl, c.req_ids.to(DEV), c.q_start.to(DEV),
        lens_cast(c.ctx_lens_t).to(DEV), lens_cast(c.q_lens_t).to(DEV), c.max_q_len, table_kind=table_kind)
    torch.cuda.synchronize()
    kernels.check_status(0)
    assert torch.equal(pool_d.cpu(), pool)
    assert _maxdiff(got, want) <= ATTN_TOL
