"""Parity of the fused attention prologue (QK-RMSNorm + rotary embedding + KV append) with the
oracle, through the C ABI.

Tolerances: V rows and every slot not named bit-exact; Q and K within 1e-3 absolute + 1e-3
relative of the oracle (one fp16 unit in the last place: the kernel takes the reciprocal square
root with the fast-math approximation, which can move a value that sits on a rounding boundary)."""

import math

import numpy as np
import pytest
import torch

import golden_cases as G
from llama_lite_npu_b200 import kernels, workloads as W
from oracle import paged_kv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _lib_loaded(built_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    kernels.check_status(0)


def _dev(*ts):
    return [None if t is None else t.to(DEV) for t in ts]


def _check(q_got, pool_got, q_want, pool_want, slots, kvh):
    rows_got, rows_want = pool_got[slots.long()], pool_want[slots.long()]
    assert torch.allclose(q_got.float(), q_want.float(), atol=1e-3, rtol=1e-3)
    assert torch.allclose(rows_got[:, :kvh].float(), rows_want[:, :kvh].float(), atol=1e-3, rtol=1e-3)
    assert torch.equal(rows_got[:, kvh:], rows_want[:, kvh:])
    untouched = torch.ones(pool_got.shape[0], dtype=torch.bool)
    untouched[slots.long()] = False
    assert torch.equal(pool_got[untouched], pool_want[untouched])


@pytest.mark.parametrize("name", list(G.PROLOGUE_CASES))
def test_prologue_matches_oracle_and_reference_golden(name):
    xq, xkv, wq, wk, cos, sin, slots, pool = G.build_prologue(name)
    want_pool = pool.clone()
    want_q = O.qk_norm_rope_append(xq, xkv, wq, wk, G.PROLOGUE_EPS, cos, sin, slots, want_pool)
    dq, dkv, dwq, dwk, dcos, dsin, dslots, dpool = _dev(xq, xkv, wq, wk, cos, sin, slots, pool)
    src = dq.clone()
    got = kernels.fused_qk_norm_rope_append(dq, dkv, dwq, dwk, G.PROLOGUE_EPS, dcos, dsin, dslots, dpool)
    assert got.data_ptr() == dq.data_ptr()                       # in place
    kvh = pool.shape[1] // 2
    _check(got.cpu(), dpool.cpu(), want_q, want_pool, slots, kvh)
    # out-of-place leaves the source alone and gives the same bits
    dpool2, out = pool.to(DEV), torch.empty_like(src)
    keep = src.clone()
    kernels.fused_qk_norm_rope_append(src, dkv, dwq, dwk, G.PROLOGUE_EPS, dcos, dsin, dslots, dpool2, out=out)
    assert torch.equal(src, keep) and torch.equal(out, got) and torch.equal(dpool2, dpool)
    # and the reference's own fp16 statements, at the tolerance the oracle is pinned with
    g = np.load(G.GOLDEN_DIR / "qk_prologue_golden.npz")
    assert torch.allclose(got.cpu().float(), torch.from_numpy(g[f"{name}.q"]).float(), atol=2e-3, rtol=3e-3)


def test_prologue_half_width_cos_and_strided_inputs():
    """cos / sin given as [n, D/2]; Q a slice of a fused qkv projection (token stride larger than
    q_heads * D); the kv_proj output likewise a column slice."""
    n, qh, kvh, d = 19, 6, 2, 128
    fused = W.hash_normal_fp16(3, (n, (qh + 2 * kvh) * d + 64), 1).to(DEV)
    xq = fused[:, : qh * d].view(n, qh, d)
    xkv = fused[:, qh * d: (qh + 2 * kvh) * d]
    ang = 2.0 * W.hash_normal_fp16(3, (n, d // 2), 2).float()
    cos, sin = ang.cos().half(), ang.sin().half()
    w = (1.0 + 0.1 * W.hash_normal_fp16(3, (d,), 3).float()).half()
    pool = W.hash_normal_fp16(3, (96, 2 * kvh, d), 4)
    slots = torch.from_numpy(W.hash_permutation(3, 96, 5)[:n].astype(np.int32))
    want_pool = pool.clone()
    want_q = O.qk_norm_rope_append(xq.cpu().contiguous(), xkv.cpu().contiguous(), w, w, 1e-6, cos, sin,
                                   slots, want_pool)
    dpool = pool.to(DEV)
    tail = fused[:, (qh + 2 * kvh) * d:].clone()
    got = kernels.fused_qk_norm_rope_append(xq, xkv, w.to(DEV), w.to(DEV), 1e-6, cos.to(DEV), sin.to(DEV),
                                            slots.to(DEV), dpool)
    _check(got.cpu(), dpool.cpu(), want_q, want_pool, slots, kvh)
    assert torch.equal(fused[:, (qh + 2 * kvh) * d:], tail)      # nothing written past the Q columns


def test_prologue_identity_angle_without_norm_is_the_plain_append():
    n, qh, kvh, d = 40, 4, 4, 128
    xq = W.hash_normal_fp16(5, (n, qh, d), 1).to(DEV)
    xkv = W.hash_normal_fp16(5, (n, 2 * kvh * d), 2).to(DEV)
    pool = W.hash_normal_fp16(5, (128, 2 * kvh, d), 3).to(DEV)
    slots = torch.from_numpy(W.hash_permutation(5, 128, 4)[:n].astype(np.int32)).to(DEV)
    one = torch.ones(n, d, dtype=torch.float16, device=DEV)
    want_pool, q0 = pool.clone(), xq.clone()
    kernels.update_kv_buffer(xkv.view(n, 2 * kvh, d), slots, want_pool)
    kernels.fused_qk_norm_rope_append(xq, xkv, None, None, 0.0, one, torch.zeros_like(one), slots, pool)
    assert torch.equal(pool, want_pool) and torch.equal(xq, q0)


def test_prologue_empty_bad_slot_and_bad_arguments():
    d, kvh = 128, 2
    pool = torch.zeros(32, 2 * kvh, d, dtype=torch.float16, device=DEV)
    e = lambda *shape: torch.zeros(*shape, dtype=torch.float16, device=DEV)  # noqa: E731
    none_slots = torch.zeros(0, dtype=torch.int32, device=DEV)
    out = kernels.fused_qk_norm_rope_append(e(0, 4, d), e(0, 2 * kvh * d), None, None, 1e-6, e(0, d), e(0, d),
                                            none_slots, pool)
    assert out.shape == (0, 4, d)
    # a slot outside the pool: nothing is written for that token, the device status says why
    xq, xkv = W.hash_normal_fp16(8, (3, 4, d), 1).to(DEV), W.hash_normal_fp16(8, (3, 2 * kvh * d), 2).to(DEV)
    slots = torch.tensor([1, 32, 5], dtype=torch.int32, device=DEV)
    one = torch.ones(3, d, dtype=torch.float16, device=DEV)
    kernels.fused_qk_norm_rope_append(xq, xkv, None, None, 0.0, one, torch.zeros_like(one), slots, pool)
    with pytest.raises(RuntimeError, match="slot_mapping"):
        kernels.check_status(0)
    assert torch.equal(pool[1].view(-1), xkv[0]) and torch.equal(pool[5].view(-1), xkv[2])
    assert int(pool.ne(0).any(dim=-1).any(dim=-1).sum()) == 2
    with pytest.raises(ValueError):
        kernels.fused_qk_norm_rope_append(e(3, 4, 96), e(3, 2 * kvh * 96), None, None, 0.0, e(3, 96), e(3, 96),
                                          slots, torch.zeros(32, 2 * kvh, 96, dtype=torch.float16, device=DEV))
    with pytest.raises(ValueError):
        kernels.fused_qk_norm_rope_append(xq, xkv, None, None, 0.0, one[:2], one[:2], slots, pool)


def test_prologue_prefill_size_against_torch_on_device():
    """8192 packed tokens of the Qwen3-32B per-layer shape (64 Q heads, 8 KV heads): the oracle's
    torch statement evaluated on the device is the checker at this size."""
    n, qh, kvh, d = 8192, 64, 8, 128
    g = torch.Generator(device=DEV).manual_seed(11)
    xq = torch.randn(n, qh, d, device=DEV, dtype=torch.float16, generator=g)
    xkv = torch.randn(n, 2 * kvh * d, device=DEV, dtype=torch.float16, generator=g)
    wq = (1 + 0.2 * torch.randn(d, device=DEV, generator=g)).half()
    wk = (1 + 0.2 * torch.randn(d, device=DEV, generator=g)).half()
    pos = torch.arange(n, device=DEV, dtype=torch.float32)[:, None]
    inv = 1.0 / (1e6 ** (torch.arange(0, d, 2, device=DEV, dtype=torch.float32) / d))
    emb = torch.cat([pos * inv, pos * inv], dim=-1)
    cos, sin = emb.cos().half(), emb.sin().half()
    pool = torch.zeros(n + 64, 2 * kvh, d, device=DEV, dtype=torch.float16)
    slots = torch.randperm(n + 64, device=DEV, generator=g)[:n].to(torch.int32)
    want_pool = pool.clone()
    want_q = O.qk_norm_rope_append(xq, xkv, wq, wk, 1e-6, cos, sin, slots, want_pool)
    got = kernels.fused_qk_norm_rope_append(xq, xkv, wq, wk, 1e-6, cos, sin, slots, pool)
    # Among 7e7 values some normalised ones sit on an fp16 rounding boundary and land on the other
    # side when the sum of squares is added up in another order; the rotation then carries that
    # one unit (up to 2^-8 for |x| in [4, 8)) into an output of any size.  So: an absolute bound of
    # one such unit, and bounds on how often and how much on average the results differ at all.
    for a, b in ((got, want_q), (pool[:, :kvh], want_pool[:, :kvh])):
        diff = (a.float() - b.float()).abs()
        assert float(diff.max()) <= 2.0 ** -8 + 1e-3
        assert float((diff > 0).float().mean()) < 5e-3
        assert float(diff.mean()) < 2e-6
    assert torch.equal(pool[:, kvh:], want_pool[:, kvh:])
    assert math.isfinite(float(got.float().abs().max()))


def test_executor_fused_forward_equals_norm_rope_then_forward():
    """Prefill of two prompts and two decode steps from raw projections through the fused calls,
    against the oracle's norm + rotation followed by the executor's unfused calls on a twin pool."""
    from llama_lite_npu_b200.executor import PagedKVExecutor

    kvh, heads, d, eps = 2, 8, 128, 1e-6
    scale = 1.0 / math.sqrt(d)
    twins = [PagedKVExecutor(1, kvh, d, 64, 4, 256, page_size=16, device=DEV) for _ in range(2)]
    for ex in twins:
        ex.kv_mem_manager.gpu_kv_buffer[0].zero_()           # the pools are compared whole at the end
    wq = (1 + 0.1 * W.hash_normal_fp16(21, (d,), 1).float()).half().to(DEV)
    wk = (1 + 0.1 * W.hash_normal_fp16(21, (d,), 2).float()).half().to(DEV)

    def inputs(n, seed):
        xq = W.hash_normal_fp16(seed, (n, heads, d), 1).to(DEV)
        xkv = W.hash_normal_fp16(seed, (n, 2 * kvh * d), 2).to(DEV)
        ang = W.hash_normal_fp16(seed, (n, d // 2), 3).float()
        emb = torch.cat([ang, ang], dim=-1)
        return xq, xkv, emb.cos().half().to(DEV), emb.sin().half().to(DEV)

    def unfused(ex, xq, xkv, cos, sin, forward, sc):
        n = xq.shape[0]
        kv = xkv.view(n, 2 * kvh, d)
        q = O.rotate_halves(O.head_rmsnorm(xq, wq, eps), cos, sin)
        k = O.rotate_halves(O.head_rmsnorm(kv[:, :kvh], wk, eps), cos, sin)
        return forward(q, k, kv[:, kvh:].contiguous(), 0, sc)

    lens = [37, 50]
    ids = [ex.reserve_paged_requests(lens) for ex in twins]
    for ex, i in zip(twins, ids):
        ex.activate_paged_packed_prefill_batch(i, lens)
    xq, xkv, cos, sin = inputs(sum(lens), 31)
    want = unfused(twins[1], xq, xkv, cos, sin, twins[1].context_forward, scale * 1.4426950408889634)
    got = twins[0].fused_context_forward(xq.clone(), xkv, wq, wk, eps, cos, sin, 0, scale * 1.4426950408889634)
    assert float((got.float() - want.float()).abs().max()) <= 2e-3
    for step in range(2):
        for ex, i in zip(twins, ids):
            ex.extend_paged_requests(i)
        xq, xkv, cos, sin = inputs(2, 40 + step)
        want = unfused(twins[1], xq, xkv, cos, sin, twins[1].token_forward, scale)
        got = twins[0].fused_token_forward(xq.clone(), xkv, wq, wk, eps, cos, sin, 0, scale)
        assert float((got.float() - want.float()).abs().max()) <= 2e-3
    p0, p1 = (ex.kv_mem_manager.gpu_kv_buffer[0] for ex in twins)
    assert torch.allclose(p0.float(), p1.float(), atol=1e-3, rtol=1e-3)
    assert torch.equal(p0[:, kvh:], p1[:, kvh:])
