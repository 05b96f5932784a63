"""CPU oracle of the paged-KV path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A restatement, in plain torch-CPU / numpy, of what the reference (lite_llama,
Python + torch + Triton-Ascend) computes on this path.  It exists only to check
the CUDA kernels and to be timed as the CPU baseline; nothing in the package
``llama_lite_npu_b200`` imports it, and the operators there have no CPU route.

Pinning: every function here is compared, on seeded inputs, with golden outputs
produced by importing and running the reference's own torch code
(``tests/golden/make_golden.py`` -> ``tests/golden/*.npz``); see
``tests/test_oracle_golden.py``.  File:line citations are paths inside the
reference project.

Numerics restated (reference: kernels/paged_chunk_flashattention.py:179-222):
scores and softmax in float32 from fp16 inputs, masked positions filled with
-1.0e8, probabilities rounded to fp16, P@V with fp16 operands, fp16 output.
The natural scale 1/sqrt(head_dim) and base-e softmax are used here; the CUDA
prefill kernel is handed log2(e)/sqrt(head_dim) and uses exp2, the same
mathematics (the reference's Triton kernels follow that convention,
models/qwen3.py:296, kernels/paged_chunk_flashattention.py:145-152).
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

MASK_FILL = -1.0e8  # kernels/paged_chunk_flashattention.py:145,219


def kv_append(kv_values: torch.Tensor, select_index: torch.Tensor, kv_buffer: torch.Tensor) -> None:
    """``kv_buffer[select_index[i]] = kv_values[i]`` in place.

    The reference kernel copies row i of KV_Values to row Select_Index[i] of KV_Buffer
    (kernels/update_kv_buffer.py:7-43); its own torch statement of the same scatter is
    ``dest[dest_loc] = src`` (kernels/update_kv_buffer.py:104-105)."""
    n = select_index.shape[0]
    kv_buffer[select_index.long()] = kv_values[:n]


def _attend_request(q_slice, k, v, scale, context_len, group, head_chunk=8):
    """One request: q_slice [q_len, H, D], k/v [kv_len, KH, D] (already gathered)."""
    q_len, n_heads, _ = q_slice.shape
    kv_len = k.shape[0]
    q_pos = torch.arange(context_len, context_len + q_len)
    k_pos = torch.arange(kv_len)
    causal = q_pos[:, None] >= k_pos[None, :]
    out = torch.empty_like(q_slice)
    kf = k.float().permute(1, 2, 0)   # [KH, D, kv_len]
    vf = v.float().permute(1, 0, 2)   # [KH, kv_len, D]
    for h0 in range(0, n_heads, head_chunk):
        h1 = min(n_heads, h0 + head_chunk)
        heads = torch.arange(h0, h1)
        kvh = heads // group
        qh = q_slice[:, h0:h1, :].float().permute(1, 0, 2)          # [h, q_len, D]
        scores = torch.bmm(qh, kf[kvh]) * float(scale)               # :211-214
        scores = scores.masked_fill(~causal[None], MASK_FILL)        # :219
        probs = torch.softmax(scores, dim=-1).to(torch.float16)      # :220
        # P and V are fp16 operands; products are exact in fp32 and summed in fp32, then the
        # result is rounded to fp16 (what an fp16 matmul with fp32 accumulation yields), :221.
        o = torch.bmm(probs.float(), vf[kvh]).to(torch.float16)
        out[:, h0:h1, :] = o.permute(1, 0, 2)
    return out


def paged_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    sm_scale: float,
    req_token_table: torch.Tensor,
    req_ids: torch.Tensor,
    q_start_loc: torch.Tensor,
    context_lens: torch.Tensor,
    q_seq_lens: torch.Tensor,
) -> torch.Tensor:
    """Causal attention of packed query chunks over paged KV with history.

    Restates ``_paged_chunk_attention_torch_fallback``
    (kernels/paged_chunk_flashattention.py:179-222): for request r, query row i sits at
    logical position ctx_r + i and sees keys ``table[req_id, 0 .. ctx_r + i]``; Q head h uses
    KV head h // (H / KH).  Rows of requests with q_len <= 0 are left untouched (:194-195).
    ``sm_scale`` multiplies the raw scores before a base-e softmax."""
    out = torch.empty_like(q)
    n_heads = q.shape[1]
    group = max(1, n_heads // k_cache.shape[1])                      # :191
    for i in range(int(q_seq_lens.shape[0])):
        req = int(req_ids[i])
        start = int(q_start_loc[i])
        ctx = int(context_lens[i])
        q_len = int(q_seq_lens[i])
        if q_len <= 0:
            continue
        phys = req_token_table[req, : ctx + q_len].long()           # :200
        out[start: start + q_len] = _attend_request(
            q[start: start + q_len], k_cache[phys], v_cache[phys], sm_scale, ctx, group)
    return out


def paged_decode(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    qk_scale: float,
    b_req_tokens_table: torch.Tensor,
    b_seq_len: torch.Tensor,
    b_req_idx: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Decode attention ``[B, H, D]`` = the paged statement above with one query row per
    sequence at position L-1 (q_len = 1, ctx = L-1).  Table rows are batch positions unless
    ``b_req_idx`` is given, as in the reference's flash_decoding (kernels/flashdecoding.py:48,85).
    A sequence of length 0 yields a zero row."""
    batch = q.shape[0]
    rows = torch.arange(batch) if b_req_idx is None else b_req_idx
    lens = b_seq_len.long()
    ctx = torch.clamp(lens - 1, min=0)
    q_lens = (lens > 0).long()
    out = paged_attention(q, k_cache, v_cache, qk_scale, b_req_tokens_table, rows,
                          torch.arange(batch), ctx, q_lens)
    out[lens == 0] = 0
    return out


def flash_decoding_kernel_math(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    qk_scale: float,
    b_req_tokens_table: torch.Tensor,
    b_seq_len: torch.Tensor,
    partition: int = 128,
    block_n: int = 16,
) -> torch.Tensor:
    """The arithmetic of the reference's two Triton decode kernels, step by step in float32.

    Stage 1 (kernels/flashdecoding.py:6-138): per (batch, Q head, 128-token partition) an
    online softmax over blocks of 16 tokens with natural exp: running max m, denominator d,
    accumulator acc; stores acc/d and m + log d.  Stage 2 (:199-267): merges partitions
    with weights exp(lse_p - max).  Everything stays float32 (P is NOT rounded to fp16 on this
    path) and the result is cast to fp16 on the final store (:267, output = empty_like(q))."""
    batch, n_heads, dim = q.shape
    group = n_heads // k_cache.shape[1]
    out = torch.zeros_like(q)
    kvh = torch.arange(n_heads) // group
    for b in range(batch):
        length = int(b_seq_len[b])
        if length == 0:
            continue
        qb = q[b].float()                                            # [H, D]
        nparts = (length + partition - 1) // partition
        mid_o = torch.zeros((n_heads, nparts, dim), dtype=torch.float32)
        mid_lse = torch.zeros((n_heads, nparts), dtype=torch.float32)
        for part in range(nparts):
            lo, hi = part * partition, min(length, (part + 1) * partition)
            m = torch.full((n_heads,), float("-inf"))
            d = torch.zeros(n_heads)
            acc = torch.zeros((n_heads, dim))
            for s in range(lo, hi, block_n):
                e = min(hi, s + block_n)
                loc = b_req_tokens_table[b, s:e].long()              # :85-89, row = batch index
                k = k_cache[loc].float()[:, kvh, :]                  # [n, H, D]
                v = v_cache[loc].float()[:, kvh, :]
                qk = (qb[None] * k).sum(-1).T * qk_scale             # [H, n]  :97-98
                m_new = torch.maximum(m, qk.max(dim=1).values)       # :102-103
                p = torch.exp(qk - m_new[:, None])                   # :104
                alpha = torch.exp(m - m_new)                         # :107
                d = alpha * d + p.sum(1)                             # :108
                acc = alpha[:, None] * acc + torch.einsum("hn,nhd->hd", p, v)   # :111
                m = m_new
            mid_o[:, part] = acc / d[:, None]                        # :137
            mid_lse[:, part] = m + torch.log(d)                      # :138
        m = torch.full((n_heads,), float("-inf"))
        d = torch.zeros(n_heads)
        acc = torch.zeros((n_heads, dim))
        for part in range(nparts):                                   # :242-264
            m_new = torch.maximum(mid_lse[:, part], m)
            alpha = torch.exp(m - m_new)
            p = torch.exp(mid_lse[:, part] - m_new)
            acc = alpha[:, None] * acc + p[:, None] * mid_o[:, part]
            d = alpha * d + p
            m = m_new
        out[b] = (acc / d[:, None]).to(torch.float16)                # :267
    return out


def nopad_prefill(q, k, v, b_start_loc, b_seq_len) -> torch.Tensor:
    """Packed causal prefill over dense K/V with no history.

    Restates ``standard_attention_prefill(..., sdpa=False)`` / ``_naive_attention``
    (kernels/flashattention2_nopad.py:227-274): per segment, fp16 Q@K^T (scores rounded to
    fp16) divided by sqrt(head_dim), a float32 softmax of the scores plus a -1e8 mask above
    the diagonal, probabilities rounded to fp16, fp16 P@V.  K/V must already carry one head
    per Q head (the reference function has no GQA)."""
    out = torch.empty_like(q)
    dim = q.shape[-1]
    for i in range(b_start_loc.shape[0]):
        s = int(b_start_loc[i])
        e = s + int(b_seq_len[i])
        n = e - s
        qi = q[s:e].float().permute(1, 0, 2)
        ki = k[s:e].float().permute(1, 2, 0)
        vi = v[s:e].float().permute(1, 0, 2)
        scores = torch.bmm(qi, ki).to(torch.float16) / np.sqrt(dim)                     # :241
        mask = torch.triu(torch.full((n, n), -100000000.0), diagonal=1)                 # :232-235
        probs = torch.softmax(scores.float() + mask[None], dim=-1).to(torch.float16)    # :242
        out[s:e] = torch.bmm(probs.float(), vi).to(torch.float16).permute(1, 0, 2)      # :243-247
    return out


def token_table_from_block_table(block_table: torch.Tensor, page_size: int) -> torch.Tensor:
    """Expand page ids to per-token slots: slot = page * page_size + offset
    (executor/paged_attention.py:116-147)."""
    rows, width = block_table.shape
    off = torch.arange(page_size, dtype=torch.int64)
    return (block_table.long()[:, :, None] * page_size + off).reshape(rows, width * page_size).int()


def head_rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """Per-head RMSNorm as the reference kernel rounds it (kernels/skip_rmsnorm.py:135-143):
    float32 statistics (``sum(x*x/N)``), ``x * rrms`` rounded to fp16, then the fp16 product with
    the weight.  ``weight is None`` returns ``x`` (models without QK-norm)."""
    if weight is None:
        return x
    xf = x.float()
    var = (xf * xf / x.shape[-1]).sum(dim=-1, keepdim=True)
    rrms = 1.0 / torch.sqrt(var + eps)
    return (xf * rrms).half() * weight.half()


def rotate_halves(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x`` ``[n, heads, D]`` with one ``cos`` / ``sin`` row per token, of
    which the first ``D/2`` entries are used (kernels/rope_emb.py:41-87):
    ``o1 = x1*cos - x2*sin``, ``o2 = x2*cos + x1*sin`` on the two halves of the head.  Evaluated
    in float32 from the fp16 values and rounded once (the reference evaluates it in the dtype of
    ``cos``, which leaves the per-operation rounding to its compiler)."""
    half = x.shape[-1] // 2
    c = cos.reshape(x.shape[0], -1)[:, None, :half].float()
    s = sin.reshape(x.shape[0], -1)[:, None, :half].float()
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).half()


def qk_norm_rope_append(xq, xkv, q_weight, k_weight, eps, cos, sin, select_index, kv_buffer) -> torch.Tensor:
    """The attention prologue of one layer (models/qwen3.py:109-126 then :62-65): QK-RMSNorm,
    rotary embedding, and the scatter of ``cat(xk, xv)`` into ``kv_buffer`` (in place).
    ``xkv`` is the kv_proj output ``[n, 2*KH*D]``.  Returns the rotated Q ``[n, H, D]``."""
    n, _, d = xq.shape
    kvh = kv_buffer.shape[1] // 2
    xk, xv = xkv.reshape(n, 2 * kvh, d)[:, :kvh], xkv.reshape(n, 2 * kvh, d)[:, kvh:]
    q = rotate_halves(head_rmsnorm(xq, q_weight, eps), cos, sin)
    k = rotate_halves(head_rmsnorm(xk, k_weight, eps), cos, sin)
    kv_append(torch.cat([k, xv], dim=-2), select_index, kv_buffer)
    return q


def decode_advance(seq_lens: torch.Tensor, block_table: torch.Tensor, page_size: int,
                   req_ids: Optional[torch.Tensor] = None,
                   token_table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of batch metadata: the new token of sequence b sits at logical position
    ``seq_lens[b]`` of table row ``req_ids[b]``; its slot is ``page * page_size + offset``
    (executor/paged_attention.py:346-358 writes exactly this entry in ``extend_req``), the length
    grows by one, and ``batch_metadata`` (:287-311) reports the new length and that slot.
    ``seq_lens`` and ``token_table`` are updated in place; returns the int32 slots."""
    rows = (req_ids if req_ids is not None else torch.arange(seq_lens.shape[0])).long()
    pos = seq_lens.long()
    slots = (block_table[rows, pos // page_size].long() * page_size + pos % page_size).to(torch.int32)
    if token_table is not None:
        token_table[rows, pos] = slots
    seq_lens += 1
    return slots


def update_kv_index(req_to_token_indexs, b_req_idx, b_seq_len, select_index) -> None:
    """``req_to_token_indexs[b_req_idx[i], b_seq_len[i] - 1] = select_index[i]`` in place
    (kernels/update_kv_index.py:16-36; the reference holds no torch statement or fixture for it,
    so this restates the kernel body)."""
    req_to_token_indexs[b_req_idx.long(), b_seq_len.long() - 1] = select_index.to(req_to_token_indexs.dtype)
