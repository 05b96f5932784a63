"""Pin the CPU oracle to outputs of the reference's own torch code (tests/golden/)."""

import hashlib
import math

import numpy as np
import torch

import golden_cases as G
from oracle import paged_kv_oracle as O


def _digest(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _maxdiff(a, b):
    return float((a.float() - b.float()).abs().max())


# The oracle restates the reference's arithmetic operation by operation; the only freedom left
# is the summation order inside matmul, worth at most one fp16 rounding step of an O(1) output.
PIN_TOL = 1e-3


def test_inputs_are_reproducible(golden):
    for name in G.DECODE_CASES:
        c = G.build_decode(name)
        assert _digest(c.q) == golden["meta"][name]["q_sha256"]
        assert _digest(c.pool) == golden["meta"][name]["pool_sha256"]
        assert c.seq_lens.tolist() == golden["meta"][name]["seq_lens"]


def test_append_bit_exact(golden):
    for name in G.APPEND_CASES:
        src, slots, pool = G.build_append(name)
        assert _digest(src) == golden["meta"][name]["src_sha256"]
        O.kv_append(src, slots, pool)
        assert _digest(pool) == golden["meta"][name]["pool_sha256"]


def test_paged_decode_matches_reference(golden):
    for name in G.DECODE_CASES:
        c = G.build_decode(name)
        got = O.paged_decode(c.q, c.k_cache, c.v_cache, 1.0 / math.sqrt(128), c.token_table, c.seq_lens_t)
        ref = torch.from_numpy(golden["arrays"][name])
        assert _maxdiff(got, ref) <= PIN_TOL, name


def test_decode_kernel_math_agrees_with_torch_statement(golden):
    """The Triton decode kernels keep P in float32; the torch statement rounds P to fp16.
    Both must sit well inside the 2e-3 parity budget of each other."""
    for name in ("decode_gqa4_edges", "decode_gqa8_small", "decode_mha"):
        c = G.build_decode(name)
        got = O.flash_decoding_kernel_math(c.q, c.k_cache, c.v_cache, 1.0 / math.sqrt(128),
                                           c.token_table, c.seq_lens_t)
        ref = torch.from_numpy(golden["arrays"][name])
        assert _maxdiff(got, ref) <= 1e-3, name


def test_contiguous_mha_decode_reference(golden):
    """torch_attention_with_kvcache (fp16 scores) vs the paged oracle on an identity table."""
    for name in G.MHA_DECODE_CASES:
        q, k, v, start, lens = G.build_mha_decode(name)
        width = int(lens.max())
        table = (start[:, None] + torch.arange(width)[None, :]).int()
        got = O.paged_decode(q, k, v, 1.0 / math.sqrt(128), table, lens)
        ref = torch.from_numpy(golden["arrays"][name])
        # that reference path rounds the scores to fp16 before the softmax: looser agreement
        assert _maxdiff(got, ref) <= 4e-3, name


def test_prefill_with_history_matches_reference(golden):
    for name in G.PREFILL_CASES:
        c = G.build_prefill(name)
        pool = c.pool.clone()
        O.kv_append(c.new_kv, c.slots, pool)
        kh = c.cfg.kv_heads
        got = O.paged_attention(c.q, pool[:, :kh], pool[:, kh:], 1.0 / math.sqrt(128), c.token_table,
                                c.req_ids, c.q_start, c.ctx_lens_t, c.q_lens_t)
        ref = torch.from_numpy(golden["arrays"][name])
        assert _maxdiff(got, ref) <= PIN_TOL, name
        assert golden["meta"][name]["ctx"] == c.ctx_lens.tolist()


def test_nopad_prefill_matches_reference(golden):
    for name in G.NOPAD_CASES:
        q, k, v, start, lens = G.build_nopad(name)
        got = O.nopad_prefill(q, k, v, start, lens)
        ref = torch.from_numpy(golden["arrays"][name])
        assert _maxdiff(got, ref) <= PIN_TOL, name
        # and the paged statement with zero history agrees within fp16-score rounding
        width = int(lens.max())
        table = (start[:, None] + torch.arange(width)[None, :]).int()
        got2 = O.paged_attention(q, k, v, 1.0 / math.sqrt(128), table,
                                 torch.arange(len(lens)), start, torch.zeros_like(lens), lens)
        assert _maxdiff(got2, ref) <= 4e-3, name


def test_token_table_expansion():
    bt = torch.tensor([[3, 7, 12]], dtype=torch.int32)
    tt = O.token_table_from_block_table(bt, 4)
    assert tt[0, :10].tolist() == [12, 13, 14, 15, 28, 29, 30, 31, 48, 49]


def test_attention_prologue_matches_reference_statements():
    """QK-RMSNorm + rotary embedding + scatter against the reference's torch statements.

    Those statements work in fp16 throughout (the mean of squares and every product are rounded
    to fp16) whereas the reference's kernels, and the oracle, keep float32 statistics; the
    agreement is therefore a few fp16 units in the last place: 2e-3 absolute + 3e-3 relative.
    V rows, and hence the scatter, are bit-exact."""
    g = np.load(G.GOLDEN_DIR / "qk_prologue_golden.npz")
    for name in G.PROLOGUE_CASES:
        xq, xkv, wq, wk, cos, sin, slots, pool = G.build_prologue(name)
        before = pool.clone()
        q = O.qk_norm_rope_append(xq, xkv, wq, wk, G.PROLOGUE_EPS, cos, sin, slots, pool)
        kvh = pool.shape[1] // 2
        rows = pool[slots.long()]
        want_q, want_rows = torch.from_numpy(g[f"{name}.q"]), torch.from_numpy(g[f"{name}.pool_rows"])
        assert torch.allclose(q.float(), want_q.float(), atol=2e-3, rtol=3e-3), name
        assert torch.allclose(rows[:, :kvh].float(), want_rows[:, :kvh].float(), atol=2e-3, rtol=3e-3), name
        assert torch.equal(rows[:, kvh:], want_rows[:, kvh:]), name
        untouched = torch.ones(pool.shape[0], dtype=torch.bool)
        untouched[slots.long()] = False
        assert torch.equal(pool[untouched], before[untouched]), name


def test_rotation_preserves_norm_and_identity_angle():
    """Two properties of the rotary statement: zero angle is the identity, and a rotation keeps
    the length of every (x1[i], x2[i]) pair."""
    x = G.W.hash_normal_fp16(7, (9, 3, 128), 1)
    one, zero = torch.ones(9, 128, dtype=torch.float16), torch.zeros(9, 128, dtype=torch.float16)
    assert torch.equal(O.rotate_halves(x, one, zero), x)
    ang = 2.0 * G.W.hash_normal_fp16(7, (9, 64), 2).float()
    emb = torch.cat([ang, ang], dim=-1)
    y = O.rotate_halves(x, emb.cos().half(), emb.sin().half()).float()
    xf = x.float()
    r_in = xf[..., :64] ** 2 + xf[..., 64:] ** 2
    r_out = y[..., :64] ** 2 + y[..., 64:] ** 2
    assert torch.allclose(r_in, r_out, atol=2e-2, rtol=1e-2)
