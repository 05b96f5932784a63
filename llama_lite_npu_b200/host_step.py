"""Decode steps for a caller whose per-step tensors live in host memory.

``kernels.append_flash_decoding`` takes device tensors, as the reference's decode attention does
(``lite_llama/models/qwen3.py:53-75``).  A serving loop that keeps its activations on the host
pays, per step, a copy in, the launch and a copy out; :class:`HostDecodeSteps` makes that one
library call per step (``include/b200kv_host_step.h``) and overlaps the three across steps: the
object owns ``depth`` slots of pinned staging, three streams and the events between them.

    steps = HostDecodeSteps(max_batch=32, q_heads=64, kv_heads=8, head_dim=128)
    bound = steps.bind(kv_buffer, block_table, table_kind="block", qk_scale=scale)
    buf = steps.buffers(slot, batch)          # numpy views of the slot's pinned memory
    buf.q[...] = ...; buf.new_k[...] = ...; buf.new_v[...] = ...
    buf.seq_lens[...] = ...; buf.slots[...] = ...
    steps.submit(slot, batch, bound, max_actual_seq_len)
    ...                                       # fill and submit the next slot meanwhile
    steps.wait(slot)                          # buf.out now holds the step's attention output

The KV pool and the tables stay device tensors (the engine's resident state).  There is no CPU
fallback: without the CUDA library the constructor raises.
"""

from __future__ import annotations

import ctypes
from collections import namedtuple
from typing import Optional

import numpy as np
import torch

from . import _lib
from .kernels import (DECODE_SERIALIZED, _TABLE_KINDS, TABLE_BLOCK, TABLE_DENSE, _on_device, _pool_geometry,
                      status_tensor)

HostStepBuffers = namedtuple("HostStepBuffers", "q new_k new_v seq_lens slots out")
BoundPool = namedtuple("BoundPool", "index rows width keep")


def _view(ptr: int, shape, dtype) -> np.ndarray:
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    raw = (ctypes.c_uint8 * n).from_address(ptr)
    return np.frombuffer(raw, dtype=dtype).reshape(shape)


class HostDecodeSteps:
    """``depth`` slots of pinned staging around the fused append + paged decode step."""

    def __init__(self, max_batch: int, q_heads: int, kv_heads: int, head_dim: int = 128, depth: int = 2,
                 device: Optional[int] = None):
        self.device = torch.cuda.current_device() if device is None else int(device)
        self.max_batch, self.q_heads, self.kv_heads, self.head_dim = max_batch, q_heads, kv_heads, head_dim
        self.depth = depth
        self._lib = _lib.lib()
        handle = ctypes.c_void_p()
        with _on_device(self.device):
            _lib.check(self._lib.b200kv_host_steps_create(depth, max_batch, q_heads, kv_heads, head_dim,
                                                          ctypes.byref(handle)))
        self._handle = handle
        self._status = status_tensor(self.device)
        self._views: dict[tuple[int, int], HostStepBuffers] = {}
        self._status_ptr = self._status.data_ptr()
        self._bound: list = []            # keeps bound tensors alive as long as the handle
        self._submit = self._lib.b200kv_host_steps_submit_bound
        self._wait = self._lib.b200kv_host_steps_wait

    # ------------------------------------------------------------------ staging
    def buffers(self, slot: int, batch: int) -> HostStepBuffers:
        """Numpy views of the slot's pinned host memory for a step of ``batch`` sequences."""
        got = self._views.get((slot, batch))
        if got is not None:
            return got
        ptrs = [ctypes.c_void_p() for _ in range(6)]
        _lib.check(self._lib.b200kv_host_steps_buffers(self._handle, slot, batch, *[ctypes.byref(p) for p in ptrs]))
        d = self.head_dim
        got = HostStepBuffers(
            q=_view(ptrs[0].value, (batch, self.q_heads, d), np.float16),
            new_k=_view(ptrs[1].value, (batch, self.kv_heads, d), np.float16),
            new_v=_view(ptrs[2].value, (batch, self.kv_heads, d), np.float16),
            seq_lens=_view(ptrs[3].value, (batch,), np.int32),
            slots=_view(ptrs[4].value, (batch,), np.int32),
            out=_view(ptrs[5].value, (batch, self.q_heads, d), np.float16),
        )
        self._views[(slot, batch)] = got
        return got

    # ------------------------------------------------------------------ the resident state
    def bind(self, KV_Buffer: torch.Tensor, table: torch.Tensor, *, qk_scale: float, table_kind: str = "token",
             page_size: int = 16, b_req_idx: Optional[torch.Tensor] = None) -> BoundPool:
        """Check a pool / table pair once and return what :meth:`submit` passes on for it."""
        k_ptr, v_ptr, tok_stride, head_stride, pool_tokens, kv_heads, d = _pool_geometry(KV_Buffer)
        if KV_Buffer.device.type != "cuda" or KV_Buffer.device.index != self.device:
            raise ValueError("KV_Buffer must live on the device the steps were created on")
        if kv_heads != self.kv_heads or d != self.head_dim:
            raise ValueError("KV_Buffer does not have the head geometry the steps were created with")
        kind = _TABLE_KINDS[table_kind]
        if kind == TABLE_DENSE:
            raise ValueError("decode takes a 'token' or 'block' table")
        if table.dtype != torch.int32 or table.dim() != 2 or table.stride(1) != 1 or table.device != KV_Buffer.device:
            raise ValueError("the table must be a 2-D int32 device tensor contiguous along its last dimension")
        rows_ptr = 0
        if b_req_idx is not None:
            if b_req_idx.dtype != torch.int32 or b_req_idx.dim() != 1 or not b_req_idx.is_contiguous() \
                    or b_req_idx.device != KV_Buffer.device:
                raise ValueError("b_req_idx must be a contiguous int32 device tensor")
            rows_ptr = b_req_idx.data_ptr()
        rows, cols = table.shape
        index = self._lib.b200kv_host_steps_bind(self._handle, k_ptr, v_ptr, tok_stride, head_stride, pool_tokens,
                                                 table.data_ptr(), table.stride(0), kind, rows, cols, rows_ptr,
                                                 int(page_size), float(qk_scale))
        if index < 0:
            _lib.check(-index)
        width = cols * (int(page_size) if kind == TABLE_BLOCK else 1)
        # the tensors are kept alive with the binding: the library holds their addresses
        bound = BoundPool(index, rows, width,
                          (KV_Buffer, table, b_req_idx, None if b_req_idx is None else b_req_idx.shape[0]))
        self._bound.append(bound)
        return bound

    # ------------------------------------------------------------------ steps
    def submit(self, slot: int, batch: int, bound: BoundPool, max_actual_seq_len: int, *,
               metadata_fresh: bool = False) -> None:
        """Enqueue copy-in, the step and copy-out for ``slot``; returns without waiting.  The
        copy-in starts at once; the kernel is launched by the next ``submit`` / ``flush`` /
        ``wait``, when its inputs have landed and it can follow its predecessor directly."""
        max_len = int(max_actual_seq_len)
        if not 0 <= max_len <= bound.width:
            raise ValueError("max_actual_seq_len exceeds the table width")
        n_rows = bound.keep[3]
        if n_rows is None:
            if bound.rows < batch:
                raise ValueError("the table has fewer rows than the batch")
        elif n_rows != batch:
            raise ValueError("b_req_idx must have one entry per batch row")
        rc = self._submit(self._handle, slot, batch, bound.index, max_len,
                          DECODE_SERIALIZED if metadata_fresh else 0, self._status_ptr)
        if rc != 0:
            _lib.check(rc)

    def flush(self) -> None:
        """Launch the step the last :meth:`submit` left pending (with more than one slot a step's
        kernel is launched by the next ``submit``, by ``flush``, by ``wait`` on its slot, or by any ``wait``
        once its inputs have landed)."""
        rc = self._lib.b200kv_host_steps_flush(self._handle)
        if rc != 0:
            _lib.check(rc)

    def wait(self, slot: int) -> None:
        """Block until the slot's result is in ``buffers(slot, batch).out``."""
        rc = self._wait(self._handle, slot)
        if rc != 0:
            _lib.check(rc)

    def reset(self) -> None:
        """Wait for everything in flight and zero the workspace's arrival counters; needed only
        after ``kernels.check_status`` reported a device-side wait that ran out (code 104)."""
        rc = self._lib.b200kv_host_steps_reset(self._handle)
        if rc != 0:
            _lib.check(rc)

    @property
    def stream(self) -> torch.cuda.Stream:
        """The compute stream of the steps, to order other device work against them."""
        ptr = self._lib.b200kv_host_steps_stream(self._handle)
        return torch.cuda.ExternalStream(ptr, device=self.device)

    def close(self) -> None:
        if self._handle is not None and self._handle.value:
            self._views.clear()
            self._lib.b200kv_host_steps_destroy(self._handle)   # waits for the steps in flight
            self._bound.clear()
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
