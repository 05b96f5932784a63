"""Operator surface of the paged-KV path, same names and positional arguments as
the reference's ``lite_llama.kernels`` (re-exported there by ``kernels/__init__.py:4-16``
and called from ``Attention.context_forward`` / ``token_forward``,
``lite_llama/models/qwen3.py:20-75``).

Every function validates its tensors on the host, then makes exactly one call
into ``libb200kv.so`` through ctypes with raw device pointers and the current
CUDA stream.  PyTorch is used for memory (outputs, the split-KV workspace) and
streams only.  There is no CPU path: tensors must live on a CUDA device and the
shared library must be present.

Debugging aid: with the environment variable ``B200KV_DEBUG=1`` (or ``set_debug(True)``) every
call first validates its index tensors on the host — slots inside the pool, no two tokens of one
append aimed at the same slot with different payloads, lengths within the stated maximum, table
rows inside the table — raising ``ValueError`` before anything is launched, and is followed by a
device synchronisation and a check of the device status word, raising ``RuntimeError``.  Both
cost a device round trip per call; neither runs otherwise.
"""

from __future__ import annotations

import os
from typing import Optional

import numpy as _np
import torch

from . import _lib

TABLE_BLOCK = 0
TABLE_TOKEN = 1
TABLE_DENSE = 2
DECODE_SERIALIZED = 1          # B200KV_DECODE_SERIALIZED
DECODE_COUNTER_BYTES = 256 << 10
OPT_DECODE_TEAMS = 1
OPT_DECODE_PIECE_COST = 2

_TABLE_KINDS = {"block": TABLE_BLOCK, "token": TABLE_TOKEN, "dense": TABLE_DENSE}

_DEBUG = os.environ.get("B200KV_DEBUG", "0") not in ("", "0")

_status: dict[int, torch.Tensor] = {}
_workspace: dict[int, torch.Tensor] = {}
_retired_workspaces: list[torch.Tensor] = []


def _device_index(t: torch.Tensor) -> int:
    if t.device.type != "cuda":
        raise ValueError(
            f"b200kv operators run on CUDA devices only (got a tensor on {t.device}); "
            "there is no CPU fallback"
        )
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def status_tensor(device_index: int) -> torch.Tensor:
    """The per-device int32 status word kernels record index errors in."""
    st = _status.get(device_index)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=f"cuda:{device_index}")
        _status[device_index] = st
    return st


def check_status(device_index: Optional[int] = None) -> None:
    """Synchronise and raise if a kernel recorded a device-side index error."""
    if device_index is None:
        device_index = torch.cuda.current_device()
    st = status_tensor(device_index)
    code = int(st.item())
    if code != 0:
        st.zero_()
        if code == 104:   # a wait ran out: the decode workspace's arrival counters may be off
            ws = _workspace.get(device_index)
            if ws is not None:
                ws[:DECODE_COUNTER_BYTES].zero_()
        raise RuntimeError(f"b200kv device status {code}: {_lib.strerror(code)}")


def _after_call(device_index: int) -> None:
    if _DEBUG:
        check_status(device_index)


def set_debug(enabled: bool) -> None:
    """Switch the debug mode described in the module docstring on or off."""
    global _DEBUG
    _DEBUG = bool(enabled)


def _debug_check_append(values: torch.Tensor, slots: torch.Tensor, pool_tokens: int) -> None:
    """Host-side look at a slot_mapping before the append is launched (debug mode only).

    Slots must lie inside the pool.  Two tokens may name the same slot only with identical
    payloads (an exact-prompt prefix hit shares its partially filled last page and both owners
    append the same row, ``lite_llama/executor/model_executor.py:547-568``); different payloads
    would make the result depend on which write lands last."""
    n = slots.shape[0]
    if n == 0:
        return
    s = slots.long()
    bad = (s < 0) | (s >= pool_tokens)
    if bool(bad.any()):
        i = int(bad.nonzero()[0])
        raise ValueError(f"slot_mapping[{i}] = {int(s[i])} is outside the pool of {pool_tokens} token slots")
    order = torch.argsort(s, stable=True)
    same = s[order][1:] == s[order][:-1]
    if bool(same.any()):
        a, b = order[:-1][same], order[1:][same]
        rows = values[:n].reshape(n, -1)
        differ = (rows[a] != rows[b]).any(dim=1)
        if bool(differ.any()):
            j = int(differ.nonzero()[0])
            raise ValueError(f"tokens {int(a[j])} and {int(b[j])} are both appended to slot {int(s[a[j]])} "
                             "with different K/V rows")


def _debug_check_lengths(lens: torch.Tensor, max_len: int, rows: Optional[torch.Tensor], table_rows: int,
                         what: str) -> None:
    if lens.numel() and (int(lens.min()) < 0 or int(lens.max()) > max_len):
        raise ValueError(f"{what}: a length lies outside [0, {max_len}]")
    if rows is not None and rows.numel() and (int(rows.min()) < 0 or int(rows.max()) >= table_rows):
        raise ValueError(f"{what}: a request id lies outside the table's {table_rows} rows")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device_index: int) -> int:
    """Handle of torch's current stream on the device (the cheap accessor when torch has it)."""
    if _raw_stream is not None:
        return _raw_stream(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on_device(device_index: int):
    """Context that makes ``device_index`` current; free when it already is (the common case)."""
    if torch.cuda.current_device() == device_index:
        return _NO_SWITCH
    return torch.cuda.device(device_index)


_workspace_need: dict[tuple, int] = {}


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _lens_arg(t: torch.Tensor, name: str) -> tuple[int, int]:
    _require(t.dtype in (torch.int32, torch.int64), f"{name} must be int32 or int64")
    _require(t.dim() == 1 and t.is_contiguous(), f"{name} must be a contiguous 1-D tensor")
    return t.data_ptr(), int(t.dtype == torch.int64)


def _kv_views(k_cache: torch.Tensor, v_cache: torch.Tensor):
    _require(k_cache.dtype == torch.float16 and v_cache.dtype == torch.float16,
             "k_cache / v_cache must be float16")
    _require(k_cache.dim() == 3 and v_cache.shape == k_cache.shape,
             "k_cache / v_cache must be [tokens, kv_heads, head_dim] with equal shapes")
    _require(k_cache.stride() == v_cache.stride() and k_cache.stride(2) == 1,
             "k_cache / v_cache must share strides and be contiguous along head_dim")
    return k_cache.stride(0), k_cache.stride(1), k_cache.shape[0]


def decode_workspace(device_index: int, batch: int, q_heads: int, kv_heads: int, head_dim: int):
    """Per-device scratch for the decode kernel (arrival counters + split-KV partials); grown on
    demand, never shrunk, so its address is stable across calls of the same or a smaller shape."""
    key = (device_index, batch, q_heads, kv_heads, head_dim)
    need = _workspace_need.get(key)
    if need is None:
        with _on_device(device_index):
            need = _lib.lib().b200kv_decode_workspace_bytes(batch, q_heads, kv_heads, head_dim)
        _workspace_need[key] = need
    if need == 0:
        raise ValueError(
            "unsupported decode shape: head_dim must be 128 and q_heads/kv_heads an integer <= 16"
        )
    ws = _workspace.get(device_index)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)   # captured CUDA graphs may still point into it
        # zero-filled: the arrival counters at its start must be zero before the first call, and
        # every call leaves them at zero
        ws = torch.zeros(need, dtype=torch.uint8, device=f"cuda:{device_index}")
        _workspace[device_index] = ws
    return ws


@torch.no_grad()
def update_kv_buffer(KV_Values: torch.Tensor, Select_Index: torch.Tensor, KV_Buffer: torch.Tensor) -> None:
    """``KV_Buffer[Select_Index[i], :, :] = KV_Values[i, :, :]`` in place, bit-exact.

    Same contract as the reference's ``update_kv_buffer``
    (``lite_llama/kernels/update_kv_buffer.py:47-81``): ``KV_Values`` is
    ``[num_tokens, 2*kv_heads, head_dim]`` fp16, ``Select_Index`` the int32
    slot_mapping, ``KV_Buffer`` the ``[pool_tokens, 2*kv_heads, head_dim]`` page pool.
    """
    dev = _device_index(KV_Buffer)
    _require(KV_Values.device == KV_Buffer.device and Select_Index.device == KV_Buffer.device,
             "KV_Values, Select_Index and KV_Buffer must be on the same device")
    _require(KV_Values.dtype == torch.float16 and KV_Buffer.dtype == torch.float16,
             "KV_Values and KV_Buffer must be float16")
    _require(Select_Index.dtype == torch.int32 and Select_Index.dim() == 1,
             "Select_Index must be a 1-D int32 tensor")
    _require(KV_Values.dim() == 3 and KV_Buffer.dim() == 3, "KV_Values and KV_Buffer must be 3-D")
    assert KV_Values.shape[1] == KV_Buffer.shape[1] and KV_Values.shape[2] == KV_Buffer.shape[2]
    n = Select_Index.shape[0]
    _require(KV_Values.shape[0] >= n, "KV_Values has fewer rows than Select_Index")
    if n == 0:
        return
    rows, d = KV_Values.shape[1], KV_Values.shape[2]
    _require(KV_Values.stride(2) == 1 and KV_Values.stride(1) == d,
             "KV_Values must be contiguous inside a token")
    _require(KV_Buffer.stride(2) == 1 and KV_Buffer.stride(1) == d,
             "KV_Buffer must be contiguous inside a token")
    if not Select_Index.is_contiguous():
        Select_Index = Select_Index.contiguous()
    if _DEBUG:
        _debug_check_append(KV_Values, Select_Index, KV_Buffer.shape[0])
    with _on_device(dev):
        rc = _lib.lib().b200kv_kv_append(
            KV_Values.data_ptr(), n, KV_Values.stride(0), Select_Index.data_ptr(),
            KV_Buffer.data_ptr(), KV_Buffer.shape[0], KV_Buffer.stride(0), rows, d,
            status_tensor(dev).data_ptr(), _stream(dev),
        )
    _lib.check(rc)
    _after_call(dev)


@torch.no_grad()
def update_kv_buffer_split(xk: torch.Tensor, xv: torch.Tensor, Select_Index: torch.Tensor,
                           KV_Buffer: torch.Tensor) -> None:
    """Same scatter from separate ``xk`` / ``xv`` ``[num_tokens, kv_heads, head_dim]`` tensors,
    i.e. ``update_kv_buffer(torch.cat([xk, xv], dim=-2), ...)`` without the concatenation
    (the reference concatenates first, ``lite_llama/models/qwen3.py:29,62``)."""
    dev = _device_index(KV_Buffer)
    _require(xk.dtype == torch.float16 and xv.dtype == torch.float16
             and KV_Buffer.dtype == torch.float16, "xk, xv and KV_Buffer must be float16")
    _require(xk.dim() == 3 and xk.shape == xv.shape, "xk and xv must be 3-D with equal shapes")
    _require(Select_Index.dtype == torch.int32 and Select_Index.dim() == 1,
             "Select_Index must be a 1-D int32 tensor")
    kvh, d = xk.shape[1], xk.shape[2]
    _require(KV_Buffer.dim() == 3 and KV_Buffer.shape[1] == 2 * kvh and KV_Buffer.shape[2] == d,
             "KV_Buffer must be [pool_tokens, 2*kv_heads, head_dim]")
    for t, name in ((xk, "xk"), (xv, "xv"), (KV_Buffer, "KV_Buffer")):
        _require(t.stride(2) == 1 and t.stride(1) == d, f"{name} must be contiguous inside a token")
    n = Select_Index.shape[0]
    _require(xk.shape[0] >= n, "xk has fewer rows than Select_Index")
    if n == 0:
        return
    if not Select_Index.is_contiguous():
        Select_Index = Select_Index.contiguous()
    if _DEBUG:
        _debug_check_append(torch.cat([xk[:n], xv[:n]], dim=1), Select_Index, KV_Buffer.shape[0])
    with _on_device(dev):
        rc = _lib.lib().b200kv_kv_append_split(
            xk.data_ptr(), xv.data_ptr(), n, xk.stride(0), xv.stride(0), Select_Index.data_ptr(),
            KV_Buffer.data_ptr(), KV_Buffer.shape[0], KV_Buffer.stride(0), kvh, d,
            status_tensor(dev).data_ptr(), _stream(dev),
        )
    _lib.check(rc)
    _after_call(dev)


@torch.no_grad()
def update_kv_index(req_to_token_indexs: torch.Tensor, b_req_idx: torch.Tensor, b_seq_len: torch.Tensor,
                    select_index: torch.Tensor) -> None:
    """``req_to_token_indexs[b_req_idx[i], b_seq_len[i] - 1] = select_index[i]`` on the device.

    Same signature as the reference operator (``lite_llama/kernels/update_kv_index.py:42-74``)."""
    dev = _device_index(req_to_token_indexs)
    _require(req_to_token_indexs.dtype == torch.int32 and req_to_token_indexs.dim() == 2,
             "req_to_token_indexs must be a 2-D int32 tensor")
    _, i64 = _lens_arg(b_seq_len, "b_seq_len")
    n = b_seq_len.shape[0]
    _require(b_req_idx.shape[0] == n and select_index.shape[0] == n,
             "b_req_idx, b_seq_len and select_index must have the same length")
    for t, name in ((b_req_idx, "b_req_idx"), (select_index, "select_index")):
        _require(t.dtype == torch.int32 and t.dim() == 1 and t.is_contiguous(),
                 f"{name} must be a contiguous 1-D int32 tensor")
    if n == 0:
        return
    t = req_to_token_indexs
    with _on_device(dev):
        rc = _lib.lib().b200kv_update_kv_index(
            t.data_ptr(), t.stride(0), t.stride(1), t.shape[0], t.shape[1], b_req_idx.data_ptr(),
            b_seq_len.data_ptr(), i64, select_index.data_ptr(), n, status_tensor(dev).data_ptr(),
            _stream(dev))
    _lib.check(rc)
    _after_call(dev)


def patch_table(table: torch.Tensor, offsets, values) -> None:
    """``table.view(-1)[offsets[i]] = values[i]``: a few entries of an int32 device table that
    changed on the host, sent as launch arguments (no staging buffer, no separate copy).
    ``offsets`` (int64) and ``values`` (int32) are host numpy arrays."""
    dev = _device_index(table)
    if table.dtype != torch.int32 or not table.is_contiguous():
        raise ValueError("table must be a contiguous int32 tensor")
    off = _np.ascontiguousarray(offsets, dtype=_np.int64)
    val = _np.ascontiguousarray(values, dtype=_np.int32)
    if off.shape != val.shape or off.ndim != 1:
        raise ValueError("offsets and values must be 1-D and equally long")
    if off.shape[0] == 0:
        return
    with _on_device(dev):
        rc = _lib.lib().b200kv_table_patch(table.data_ptr(), table.numel(), off.ctypes.data, val.ctypes.data,
                                           off.shape[0], _stream(dev))
    if rc != 0:
        _lib.check(rc)


def advance_decode_metadata(b_seq_len: torch.Tensor, cur_select_index: torch.Tensor,
                            b_req_block_table: torch.Tensor, page_size: int, num_pages: int, *,
                            b_req_idx: Optional[torch.Tensor] = None,
                            page_counts: Optional[torch.Tensor] = None,
                            b_req_tokens_table: Optional[torch.Tensor] = None) -> None:
    """Advance a decode batch by one token on the device, in place.

    ``b_seq_len[b]`` (int32 or int64) becomes ``b_seq_len[b] + 1`` and ``cur_select_index[b]``
    the slot of the new token, looked up in ``b_req_block_table`` (row ``b_req_idx[b]``, or ``b``);
    ``b_req_tokens_table`` (optional) gets the new entry too.  The device-side form of the
    reference's per-request ``extend_req`` + ``batch_metadata``
    (``lite_llama/executor/paged_attention.py:287-359``); the page of the new token must already
    be in the block table (``page_counts`` lets the kernel check that)."""
    dev = _device_index(b_req_block_table)
    lens_dtype = b_seq_len.dtype
    if (lens_dtype != torch.int64 and lens_dtype != torch.int32) or b_seq_len.dim() != 1 \
            or not b_seq_len.is_contiguous():
        raise ValueError("b_seq_len must be a contiguous 1-D int32 or int64 tensor")
    n = b_seq_len.shape[0]
    if cur_select_index.dtype != torch.int32 or cur_select_index.shape != (n,) or not cur_select_index.is_contiguous():
        raise ValueError("cur_select_index must be int32 [batch], contiguous")
    blk = b_req_block_table
    if blk.dtype != torch.int32 or blk.dim() != 2 or blk.stride(1) != 1:
        raise ValueError("b_req_block_table must be a 2-D int32 tensor")
    blk_rows, blk_cols = blk.shape
    for t, name in ((b_req_idx, "b_req_idx"), (page_counts, "page_counts")):
        if t is not None and (t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous 1-D int32 tensor")
    if b_req_idx is not None and b_req_idx.shape[0] != n:
        raise ValueError("b_req_idx must have one entry per sequence")
    if page_counts is not None and page_counts.shape[0] != blk_rows:
        raise ValueError("page_counts must have one entry per table row")
    tt = b_req_tokens_table
    if tt is not None and (tt.dtype != torch.int32 or tt.dim() != 2 or tt.stride(1) != 1 or tt.shape[0] != blk_rows):
        raise ValueError("b_req_tokens_table must be a 2-D int32 tensor with the block table's rows")
    if n == 0:
        return
    with _on_device(dev):
        rc = _lib.lib().b200kv_decode_advance(
            0 if b_req_idx is None else b_req_idx.data_ptr(), b_seq_len.data_ptr(), lens_dtype == torch.int64,
            cur_select_index.data_ptr(), blk.data_ptr(), blk.stride(0), blk_rows, blk_cols,
            0 if page_counts is None else page_counts.data_ptr(),
            0 if tt is None else tt.data_ptr(), 0 if tt is None else tt.stride(0),
            0 if tt is None else tt.shape[1], n, int(page_size), int(num_pages),
            status_tensor(dev).data_ptr(), _stream(dev),
        )
    if rc != 0:
        _lib.check(rc)
    if _DEBUG:
        check_status(dev)


@torch.no_grad()
def fused_qk_norm_rope_append(xq: torch.Tensor, xkv: torch.Tensor, q_norm_weight: Optional[torch.Tensor],
                              k_norm_weight: Optional[torch.Tensor], eps: float, cos: torch.Tensor,
                              sin: torch.Tensor, Select_Index: torch.Tensor, KV_Buffer: torch.Tensor,
                              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The attention prologue of one layer in one launch.

    Equivalent to ``skip_rmsnorm(xq, None, q_norm_weight, eps)``, ``skip_rmsnorm(xk, None,
    k_norm_weight, eps)``, ``rope_emb_forward(xq, xk, cos, sin, ...)`` and ``update_kv_buffer(
    torch.cat([xk, xv], dim=-2), Select_Index, KV_Buffer)`` (``lite_llama/models/qwen3.py:109-126``
    and ``:62-65``), with ``xk, xv`` the two halves of ``xkv``.

    ``xq`` ``[n, q_heads, head_dim]`` is rewritten in place unless ``out`` is given; ``xkv`` is the
    ``kv_proj`` output ``[n, 2*kv_heads*head_dim]`` (or ``[n, 2*kv_heads, head_dim]``) and is only
    read; ``cos`` / ``sin`` are ``[..., head_dim]`` (or ``head_dim/2``) rows, one per token, as the
    rotary embedding returns them.  A ``None`` weight skips that norm.  Returns the rotated Q.
    """
    dev = _device_index(KV_Buffer)
    _require(xq.dim() == 3 and xq.dtype == torch.float16, "xq must be [n, q_heads, head_dim] float16")
    n, qh, d = xq.shape
    _require(KV_Buffer.dim() == 3 and KV_Buffer.dtype == torch.float16 and KV_Buffer.shape[2] == d
             and KV_Buffer.shape[1] % 2 == 0, "KV_Buffer must be [pool_tokens, 2*kv_heads, head_dim] float16")
    rows = KV_Buffer.shape[1]
    xkv = xkv.reshape(xkv.shape[0], -1) if xkv.dim() != 2 else xkv
    _require(xkv.dtype == torch.float16 and xkv.shape[0] == n and xkv.shape[1] == rows * d
             and xkv.stride(1) == 1, "xkv must be [n, 2*kv_heads*head_dim] float16, contiguous rows")
    out = xq if out is None else out
    _require(out.shape == xq.shape and out.dtype == torch.float16, "out must match xq")
    for t, name in ((xq, "xq"), (out, "out"), (KV_Buffer, "KV_Buffer")):
        _require(t.stride(2) == 1 and t.stride(1) == d, f"{name} must be contiguous inside a token")
    cos2, sin2 = cos.reshape(-1, cos.shape[-1]), sin.reshape(-1, sin.shape[-1])
    _require(cos2.dtype == torch.float16 and sin2.dtype == torch.float16, "cos and sin must be float16")
    _require(cos2.shape == sin2.shape and cos2.shape[0] == n and cos2.shape[1] in (d, d // 2)
             and cos2.stride(1) == 1 and sin2.stride(1) == 1 and cos2.stride(0) == sin2.stride(0),
             "cos and sin must be one row of head_dim (or head_dim/2) per token with equal strides")
    for w, name in ((q_norm_weight, "q_norm_weight"), (k_norm_weight, "k_norm_weight")):
        _require(w is None or (w.dtype == torch.float16 and w.shape == (d,) and w.is_contiguous()),
                 f"{name} must be a contiguous float16 [head_dim] tensor or None")
    _require(Select_Index.dtype == torch.int32 and Select_Index.dim() == 1 and Select_Index.shape[0] == n,
             "Select_Index must be a 1-D int32 tensor with one slot per token")
    if n == 0:
        return out
    if not Select_Index.is_contiguous():
        Select_Index = Select_Index.contiguous()
    with _on_device(dev):
        rc = _lib.lib().b200kv_qk_norm_rope_append(
            xq.data_ptr(), out.data_ptr(), xq.stride(0), out.stride(0), xkv.data_ptr(), xkv.stride(0),
            0 if q_norm_weight is None else q_norm_weight.data_ptr(),
            0 if k_norm_weight is None else k_norm_weight.data_ptr(), float(eps),
            cos2.data_ptr(), sin2.data_ptr(), cos2.stride(0), Select_Index.data_ptr(),
            KV_Buffer.data_ptr(), KV_Buffer.shape[0], KV_Buffer.stride(0), n, qh, rows // 2, d,
            status_tensor(dev).data_ptr(), _stream(dev),
        )
    _lib.check(rc)
    _after_call(dev)
    return out


def _decode_call(new_rows, slots, q, kv, qk_scale, tbl, b_seq_len, max_actual_seq_len,
                 b_req_idx, table_kind, page_size, out, metadata_fresh):
    """Shared body of the decode operators.  ``kv`` is ``(k_ptr, v_ptr, token_stride, head_stride,
    pool_tokens, kv_heads, head_dim)`` of the pool views; ``new_rows`` is ``None`` or ``(k_ptr,
    v_ptr, k_token_stride, v_token_stride)`` of the step's new K/V rows for the fused append.
    This runs once per layer per decode step, so it reads each tensor attribute once and makes
    one library call."""
    dev = _device_index(q)
    if q.dtype != torch.float16 or q.dim() != 3:
        raise ValueError("q must be float16 [batch, heads, head_dim]")
    batch, q_heads, d = q.shape
    q_sb, q_sh, q_sd = q.stride()
    k_ptr, v_ptr, tok_stride, head_stride, pool_tokens, kv_heads, kv_d = kv
    assert d == kv_d
    kind = _TABLE_KINDS[table_kind]
    if q_sd != 1 or kind == TABLE_DENSE:
        raise ValueError("q must be contiguous along head_dim; decode takes a 'token' or 'block' table")
    if tbl.dtype != torch.int32 or tbl.dim() != 2 or tbl.stride(1) != 1:
        raise ValueError("the table must be a 2-D int32 tensor contiguous along its last dimension")
    tbl_rows, tbl_cols = tbl.shape
    lens_dtype = b_seq_len.dtype
    if (lens_dtype != torch.int64 and lens_dtype != torch.int32) or b_seq_len.dim() != 1 \
            or not b_seq_len.is_contiguous() or b_seq_len.shape[0] != batch:
        raise ValueError("b_seq_len must be a contiguous int32 or int64 tensor with one entry per batch row")
    rows_ptr = 0
    if b_req_idx is not None:
        if b_req_idx.dtype != torch.int32 or b_req_idx.shape != (batch,) or not b_req_idx.is_contiguous():
            raise ValueError("b_req_idx must be contiguous int32 [batch]")
        rows_ptr = b_req_idx.data_ptr()
    elif tbl_rows < batch:
        raise ValueError("the table has fewer rows than the batch")
    max_len = int(max_actual_seq_len)
    if not 0 <= max_len <= tbl_cols * (page_size if kind == TABLE_BLOCK else 1):
        raise ValueError("max_actual_seq_len exceeds the table width")
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != torch.float16 or out.stride(2) != 1:
        raise ValueError("out must match q")
    if batch == 0:
        return out
    if _DEBUG:
        _debug_check_lengths(b_seq_len, max_len, b_req_idx, tbl_rows, "decode")
    ws = decode_workspace(dev, batch, q_heads, kv_heads, d)
    flags = DECODE_SERIALIZED if metadata_fresh else 0
    lib = _lib.lib()
    out_sb, out_sh, _ = out.stride()
    with _on_device(dev):
        if new_rows is None:
            rc = lib.b200kv_paged_decode(
                q.data_ptr(), q_sb, q_sh, k_ptr, v_ptr, tok_stride, head_stride, pool_tokens,
                tbl.data_ptr(), tbl.stride(0), kind, tbl_rows, tbl_cols, rows_ptr,
                b_seq_len.data_ptr(), lens_dtype == torch.int64,
                batch, q_heads, kv_heads, d, int(page_size), float(qk_scale), max_len,
                ws.data_ptr(), ws.numel(), out.data_ptr(), out_sb, out_sh,
                flags, status_tensor(dev).data_ptr(), _stream(dev),
            )
        else:
            rc = lib.b200kv_append_paged_decode(
                new_rows[0], new_rows[1], new_rows[2], new_rows[3], slots.data_ptr(),
                q.data_ptr(), q_sb, q_sh, k_ptr, v_ptr, tok_stride, head_stride, pool_tokens,
                tbl.data_ptr(), tbl.stride(0), kind, tbl_rows, tbl_cols, rows_ptr,
                b_seq_len.data_ptr(), lens_dtype == torch.int64,
                batch, q_heads, kv_heads, d, int(page_size), float(qk_scale), max_len,
                ws.data_ptr(), ws.numel(), out.data_ptr(), out_sb, out_sh,
                flags, status_tensor(dev).data_ptr(), _stream(dev),
            )
    if rc != 0:
        _lib.check(rc)
    if _DEBUG:
        check_status(dev)
    return out


def _pool_geometry(KV_Buffer: torch.Tensor):
    """``kv`` tuple of :func:`_decode_call` for a whole pool ``[pool_tokens, 2*kv_heads, head_dim]``,
    without materialising its K and V views."""
    if KV_Buffer.dim() != 3 or KV_Buffer.dtype != torch.float16:
        raise ValueError("KV_Buffer must be [pool_tokens, 2*kv_heads, head_dim] float16")
    pool_tokens, rows, d = KV_Buffer.shape
    s0, s1, s2 = KV_Buffer.stride()
    if rows % 2 != 0 or s2 != 1 or s1 != d:
        raise ValueError("KV_Buffer must hold 2*kv_heads rows per token, contiguous inside a token")
    kvh = rows // 2
    k_ptr = KV_Buffer.data_ptr()
    return (k_ptr, k_ptr + kvh * d * 2, s0, s1, pool_tokens, kvh, d)


def flash_decoding(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    qk_scale: float,
    b_req_tokens_table: torch.Tensor,
    b_seq_len: torch.Tensor,
    max_actual_seq_len: int,
    *,
    b_req_idx: Optional[torch.Tensor] = None,
    table_kind: str = "token",
    page_size: int = 16,
    out: Optional[torch.Tensor] = None,
    metadata_fresh: bool = False,
) -> torch.Tensor:
    """Paged decode attention; returns a new ``[batch, q_heads, head_dim]`` fp16 tensor.

    Positional arguments are those of the reference's ``flash_decoding``
    (``lite_llama/kernels/flashdecoding.py:295-342``): ``k_cache`` / ``v_cache`` are the
    strided K and V views of one layer's pool, ``qk_scale`` the natural softmax scale,
    ``b_req_tokens_table`` the logical-token -> physical-slot table whose row ``i`` belongs to
    batch position ``i`` (the reference indexes rows by batch position, ``:48,85``),
    ``b_seq_len`` int32/int64 lengths, ``max_actual_seq_len`` a host upper bound on them.

    Keyword extensions: ``b_req_idx`` (int32 ``[batch]``) selects table rows explicitly, which
    a continuous batch with gaps needs; ``table_kind="block"`` passes a page-id table
    ``[rows, max_pages]`` instead of a token table; ``metadata_fresh=True`` must be passed when
    ``b_seq_len``, ``b_req_idx`` or the table were written by the kernel launched immediately
    before this call on the same stream (the launch then gives up its overlap with that kernel).
    """
    assert q.shape[-1] == k_cache.shape[-1] == v_cache.shape[-1]
    tok_stride, head_stride, pool_tokens = _kv_views(k_cache, v_cache)
    kv = (k_cache.data_ptr(), v_cache.data_ptr(), tok_stride, head_stride, pool_tokens, k_cache.shape[1],
          k_cache.shape[2])
    return _decode_call(None, None, q, kv, qk_scale, b_req_tokens_table, b_seq_len,
                        max_actual_seq_len, b_req_idx, table_kind, page_size, out, metadata_fresh)


def append_flash_decoding(
    KV_Values: torch.Tensor,
    Select_Index: torch.Tensor,
    KV_Buffer: torch.Tensor,
    q: torch.Tensor,
    qk_scale: float,
    b_req_tokens_table: torch.Tensor,
    b_seq_len: torch.Tensor,
    max_actual_seq_len: int,
    *,
    b_req_idx: Optional[torch.Tensor] = None,
    table_kind: str = "token",
    page_size: int = 16,
    out: Optional[torch.Tensor] = None,
    metadata_fresh: bool = False,
) -> torch.Tensor:
    """One decode step of one layer in one launch: ``update_kv_buffer(KV_Values, Select_Index,
    KV_Buffer)`` followed by ``flash_decoding(q, KV_Buffer[:, :kv_heads], KV_Buffer[:, kv_heads:],
    ...)``, the pair ``Attention.token_forward`` issues (``lite_llama/models/qwen3.py:62-74``).

    ``KV_Values`` is ``[batch, 2*kv_heads, head_dim]``, ``Select_Index[b]`` the slot of sequence
    ``b``'s newest token (position ``b_seq_len[b] - 1``, the lengths already count it).  The pool
    rows are written bit-exactly; the other arguments are those of :func:`flash_decoding`."""
    kv = _pool_geometry(KV_Buffer)
    kvh, d = kv[5], kv[6]
    batch = q.shape[0]
    if KV_Values.dtype != torch.float16 or KV_Values.shape != (batch, 2 * kvh, d) or KV_Values.device != KV_Buffer.device:
        raise ValueError("KV_Values must be float16 [batch, 2*kv_heads, head_dim] on the pool's device")
    v_stride, v_s1, v_s2 = KV_Values.stride()
    if v_s2 != 1 or v_s1 != d:
        raise ValueError("KV_Values must be contiguous inside a token")
    if Select_Index.dtype != torch.int32 or Select_Index.shape != (batch,) or not Select_Index.is_contiguous() \
            or Select_Index.device != KV_Buffer.device:
        raise ValueError("Select_Index must be contiguous int32 [batch] on the pool's device")
    k_ptr = KV_Values.data_ptr()
    return _decode_call((k_ptr, k_ptr + kvh * d * 2, v_stride, v_stride), Select_Index, q, kv, qk_scale,
                        b_req_tokens_table, b_seq_len, max_actual_seq_len, b_req_idx, table_kind,
                        page_size, out, metadata_fresh)


def append_flash_decoding_split(
    xk: torch.Tensor,
    xv: torch.Tensor,
    Select_Index: torch.Tensor,
    KV_Buffer: torch.Tensor,
    q: torch.Tensor,
    qk_scale: float,
    b_req_tokens_table: torch.Tensor,
    b_seq_len: torch.Tensor,
    max_actual_seq_len: int,
    *,
    b_req_idx: Optional[torch.Tensor] = None,
    table_kind: str = "token",
    page_size: int = 16,
    out: Optional[torch.Tensor] = None,
    metadata_fresh: bool = False,
) -> torch.Tensor:
    """:func:`append_flash_decoding` with the new K and V rows given separately
    (``[batch, kv_heads, head_dim]`` each), i.e. without ``torch.cat([xk, xv], dim=-2)``
    (``lite_llama/models/qwen3.py:62``)."""
    kv = _pool_geometry(KV_Buffer)
    kvh, d = kv[5], kv[6]
    batch = q.shape[0]
    for t, name in ((xk, "xk"), (xv, "xv")):
        if t.dtype != torch.float16 or t.shape != (batch, kvh, d) or t.stride(2) != 1 or t.stride(1) != d \
                or t.device != KV_Buffer.device:
            raise ValueError(f"{name} must be float16 [batch, kv_heads, head_dim] on the pool's device, "
                             "contiguous inside a token")
    if Select_Index.dtype != torch.int32 or Select_Index.shape != (batch,) or not Select_Index.is_contiguous() \
            or Select_Index.device != KV_Buffer.device:
        raise ValueError("Select_Index must be contiguous int32 [batch] on the pool's device")
    return _decode_call((xk.data_ptr(), xv.data_ptr(), xk.stride(0), xv.stride(0)), Select_Index, q, kv,
                        qk_scale, b_req_tokens_table, b_seq_len, max_actual_seq_len, b_req_idx, table_kind,
                        page_size, out, metadata_fresh)


def set_decode_option(option: int, value: int) -> None:
    """Tuning override of the decode launch (``OPT_DECODE_TEAMS`` / ``OPT_DECODE_PIECE_COST``);
    0 restores the automatic choice."""
    _lib.check(_lib.lib().b200kv_set_option(int(option), int(value)))


def _prefill_call(q, k_cache, v_cache, scale_log2, tbl_ptr, tbl_stride, kind, tbl_rows, tbl_cols,
                  req_ids_ptr, q_start_loc, ctx_ptr, qlen_ptr, lens_i64, batch, max_q_len, page_size):
    dev = _device_index(q)
    tok_stride, head_stride, pool_tokens = _kv_views(k_cache, v_cache)
    total_q, q_heads, d = q.shape
    kv_heads = k_cache.shape[1]
    output = torch.empty_like(q)
    if q.numel() == 0 or batch == 0:
        return output
    with _on_device(dev):
        rc = _lib.lib().b200kv_paged_prefill(
            q.data_ptr(), q.stride(0), q.stride(1),
            k_cache.data_ptr(), v_cache.data_ptr(), tok_stride, head_stride, pool_tokens,
            tbl_ptr, tbl_stride, kind, tbl_rows, tbl_cols, req_ids_ptr, q_start_loc.data_ptr(),
            ctx_ptr, qlen_ptr, lens_i64, batch, total_q, int(max_q_len),
            q_heads, kv_heads, d, int(page_size), float(scale_log2),
            output.data_ptr(), output.stride(0), output.stride(1),
            status_tensor(dev).data_ptr(), _stream(dev),
        )
    _lib.check(rc)
    _after_call(dev)
    return output


@torch.no_grad()
def paged_chunk_flash_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    sm_scale: float,
    req_token_table: torch.Tensor,
    req_ids: torch.Tensor,
    q_start_loc: torch.Tensor,
    context_lens: torch.Tensor,
    q_seq_lens: torch.Tensor,
    max_q_len: int,
    *,
    table_kind: str = "token",
    page_size: int = 16,
) -> torch.Tensor:
    """Causal attention of a packed query chunk over historical paged KV plus the chunk's own
    KV (already appended to the pool).  Same positional arguments as the reference's
    ``paged_chunk_flash_attention`` (``lite_llama/kernels/paged_chunk_flashattention.py:227-327``);
    ``sm_scale`` is the softmax scale already multiplied by log2(e), as the reference's callers
    pass it (``lite_llama/models/qwen3.py:296``).  Returns a tensor like ``q``."""
    _device_index(q)
    _require(q.dtype == torch.float16 and q.dim() == 3 and q.stride(2) == 1,
             "q must be float16 [tokens, heads, head_dim], contiguous along head_dim")
    kind = _TABLE_KINDS[table_kind]
    _require(kind in (TABLE_BLOCK, TABLE_TOKEN), "paged prefill takes a 'token' or 'block' table")
    tbl = req_token_table
    _require(tbl.dtype == torch.int32 and tbl.dim() == 2 and tbl.stride(1) == 1,
             "the table must be a 2-D int32 tensor contiguous along its last dimension")
    batch = int(q_seq_lens.shape[0])
    _require(req_ids.dtype == torch.int32 and req_ids.shape == (batch,) and req_ids.is_contiguous(),
             "req_ids must be contiguous int32 [batch]")
    _require(q_start_loc.dtype == torch.int32 and q_start_loc.shape == (batch,)
             and q_start_loc.is_contiguous(), "q_start_loc must be contiguous int32 [batch]")
    _require(context_lens.dtype == q_seq_lens.dtype and context_lens.shape == (batch,),
             "context_lens and q_seq_lens must share dtype and shape")
    ctx_ptr, lens_i64 = _lens_arg(context_lens, "context_lens")
    qlen_ptr, _ = _lens_arg(q_seq_lens, "q_seq_lens")
    if _DEBUG:
        width = tbl.shape[1] * (page_size if kind == TABLE_BLOCK else 1)
        _debug_check_lengths(context_lens + q_seq_lens, width, req_ids, tbl.shape[0], "paged prefill")
    return _prefill_call(q, k_cache, v_cache, sm_scale, tbl.data_ptr(), tbl.stride(0), kind,
                         tbl.shape[0], tbl.shape[1], req_ids.data_ptr(), q_start_loc, ctx_ptr, qlen_ptr,
                         lens_i64, batch, max_q_len, page_size)


@torch.no_grad()
def flash_attention2_no_pad(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    b_start_loc: torch.Tensor,
    b_seq_len: torch.Tensor,
    max_seq_len: int,
) -> torch.Tensor:
    """Causal attention inside each packed segment ``[start, start+len)`` of dense ``q``/``k``/``v``
    (``[tokens, heads, head_dim]`` fp16, K/V with the KV head count).  Same positional
    arguments as the reference's ``flash_attention2_no_pad``
    (``lite_llama/kernels/flashattention2_nopad.py:171-221``); ``sm_scale`` already carries
    log2(e).  Runs the paged prefill kernel with zero history and the packed K/V as the pool."""
    _device_index(q)
    _require(q.dtype == torch.float16 and q.dim() == 3 and q.stride(2) == 1,
             "q must be float16 [tokens, heads, head_dim], contiguous along head_dim")
    batch = int(b_seq_len.shape[0])
    _require(b_start_loc.dtype == torch.int32 and b_start_loc.shape == (batch,)
             and b_start_loc.is_contiguous(), "b_start_loc must be contiguous int32 [batch]")
    qlen_ptr, lens_i64 = _lens_arg(b_seq_len, "b_seq_len")
    zeros = torch.zeros_like(b_seq_len)
    return _prefill_call(q, k, v, sm_scale, 0, 0, TABLE_DENSE, 0, 0, 0, b_start_loc,
                         zeros.data_ptr(), qlen_ptr, lens_i64, batch, max_seq_len, 16)


__all__ = [
    "update_kv_buffer",
    "update_kv_buffer_split",
    "flash_decoding",
    "append_flash_decoding",
    "append_flash_decoding_split",
    "paged_chunk_flash_attention",
    "flash_attention2_no_pad",
    "check_status",
    "set_debug",
    "status_tensor",
    "decode_workspace",
]
