"""The allocation-free decode entry point, called straight through the C ABI.

b200kv_paged_decode_static_scratch exists for hosts that cannot obtain device memory at call
time (an arena-managed server, a plug-in, a latency-critical loop): it keeps the arrival counters
and the split-KV partials in a fixed array inside the library instead of a caller-provided
workspace.  The array is shared by all calls and keeps the previous call's contents, so the
check is made on calls in a row with different inputs: each must equal the CPU oracle (and the
golden arrays where the reference produced some) within the attention tolerance, and what the
workspace-taking entry point returns for the same inputs.  The calls must not change the amount
of device memory torch has handed out.  This file is collected last on purpose, so a failure
here cannot hide the result of any other test in a run that stops at the first failure.
"""

import math

import numpy as np
import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200 import _lib, kernels, workloads as W
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3
DEV = "cuda:0"
SCALE = 1.0 / math.sqrt(128)


def _call_static(c, out):
    cfg = c.cfg
    pool = c.pool
    k, v = pool[:, : cfg.kv_heads], pool[:, cfg.kv_heads:]
    rc = _lib.lib().b200kv_paged_decode_static_scratch(
        c.q.data_ptr(), c.q.stride(0), c.q.stride(1),
        k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.shape[0],
        c.block_table.data_ptr(), c.block_table.stride(0), kernels.TABLE_BLOCK,
        c.block_table.shape[0], c.block_table.shape[1], None,
        c.seq_lens_t.data_ptr(), 1,
        cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.page_size,
        SCALE, c.max_len,
        out.data_ptr(), out.stride(0), out.stride(1),
        0, kernels.status_tensor(0).data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc


def _on_device(c):
    want = O.paged_decode(c.q, c.k_cache, c.v_cache, SCALE, c.token_table, c.seq_lens_t)
    for name in ("q", "pool", "block_table", "seq_lens_t"):
        setattr(c, name, getattr(c, name).to(DEV))
    return c, want


def _cases():
    # (name, case): golden shapes, a group of 16 query heads per KV head (the other template
    # instantiation), and one long sequence that is cut into many more than four pieces
    yield "decode_gqa8_small", G.build_decode("decode_gqa8_small")
    yield "decode_c1_shape", G.build_decode("decode_c1_shape")
    g16 = W.DecodeConfig("static_gqa16", 3, 32, 2, 160, 1, 1, seed=71)
    yield "gqa16", W.make_decode_case(g16, fill="hash", lengths=np.array([700, 90, 1500]))
    long1 = W.DecodeConfig("static_one_long", 1, 8, 1, 700, 1, 1, seed=72)
    yield "one_long", W.make_decode_case(long1, fill="hash", lengths=np.array([11000]))
    yield "decode_gqa8_small_again", G.build_decode("decode_gqa8_small")


def test_static_scratch_matches_oracle_and_workspace_entry_point(built_lib, golden):
    assert torch.cuda.is_available()
    # warm both paths up first: the first call per device resolves the array's address, and the
    # workspace-taking operator allocates its workspace once
    c0, _ = _on_device(G.build_decode("decode_gqa8_small"))
    assert _call_static(c0, torch.empty_like(c0.q)) == 0
    torch.cuda.synchronize()
    # different problems back to back: each runs on scratch the previous one left dirty
    for name, case in _cases():
        c, want = _on_device(case)
        kvh = c.cfg.kv_heads
        via_ws = kernels.flash_decoding(c.q, c.pool[:, :kvh], c.pool[:, kvh:], SCALE,
                                        c.block_table, c.seq_lens_t, c.max_len, table_kind="block")
        got = torch.empty_like(c.q)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert _call_static(c, got) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, "the static-scratch call allocated device memory"
        kernels.check_status(0)
        assert float((got.float().cpu() - want.float()).abs().max()) <= ATTN_TOL, name
        assert float((got.float() - via_ws.float()).abs().max()) <= ATTN_TOL, name
        key = name.replace("_again", "")
        if key in golden["arrays"]:
            ref = torch.from_numpy(golden["arrays"][key]).float()
            assert float((got.float().cpu() - ref).abs().max()) <= ATTN_TOL, name


def test_static_scratch_refuses_oversized_batch(built_lib):
    """A batch whose partials would not fit the fixed array is rejected before any launch."""
    assert torch.cuda.is_available()
    need = built_lib.b200kv_decode_workspace_bytes(4096, 16, 16, 128)
    assert need > (8 << 20)
    q = torch.zeros(4096, 16, 128, dtype=torch.float16, device=DEV)
    pool = torch.zeros(64, 32, 128, dtype=torch.float16, device=DEV)
    table = torch.zeros(4096, 1, dtype=torch.int32, device=DEV)
    lens = torch.ones(4096, dtype=torch.int64, device=DEV)
    out = torch.empty_like(q)
    rc = built_lib.b200kv_paged_decode_static_scratch(
        q.data_ptr(), q.stride(0), q.stride(1), pool[:, :16].data_ptr(), pool[:, 16:].data_ptr(),
        pool.stride(0), pool.stride(1), 64, table.data_ptr(), 1, kernels.TABLE_BLOCK, 4096, 1, None,
        lens.data_ptr(), 1, 4096, 16, 16, 128, 16, 0.1, 16, out.data_ptr(), out.stride(0),
        out.stride(1), 0, None, None)
    assert rc == 6
    assert b"maximum" in built_lib.b200kv_strerror(rc)
