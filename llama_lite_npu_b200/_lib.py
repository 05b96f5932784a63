"""ctypes binding of libb200kv.so — the only route from Python to the CUDA kernels.

There is deliberately no fallback: if the shared library is missing or a symbol
cannot be resolved, importing this module's :func:`lib` raises, and every
operator in :mod:`llama_lite_npu_b200.kernels` fails with it.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200kv.so"

# name -> (restype, argtypes); mirrors the headers under include/ one to one.
_SIGNATURES = {
    "b200kv_version": (c_int, []),
    "b200kv_strerror": (c_char_p, [c_int]),
    "b200kv_last_cuda_error": (c_char_p, []),
    "b200kv_kv_append": (
        c_int,
        [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
         c_void_p, c_void_p],
    ),
    "b200kv_kv_append_split": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64,
         c_int, c_int, c_void_p, c_void_p],
    ),
    "b200kv_qk_norm_rope_append": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64,   # q, q_out, strides
         c_void_p, c_int64,                      # kv
         c_void_p, c_void_p, c_float,            # norm weights, eps
         c_void_p, c_void_p, c_int64,            # cos, sin
         c_void_p, c_void_p, c_int64, c_int64,   # slots, pool
         c_int64, c_int, c_int, c_int,           # n_tokens, heads, dim
         c_void_p, c_void_p],
    ),
    "b200kv_decode_advance": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p,            # req_ids, seq_lens, slots
         c_void_p, c_int64, c_int, c_int, c_void_p,      # block table, page_counts
         c_void_p, c_int64, c_int,                       # token table
         c_int, c_int, c_int64, c_void_p, c_void_p],
    ),
    "b200kv_table_patch": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "b200kv_update_kv_index": (
        c_int,
        [c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
         c_void_p, c_void_p],
    ),
    "b200kv_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "b200kv_set_option": (c_int, [c_int, c_int64]),
    "b200kv_paged_decode": (
        c_int,
        [c_void_p, c_int64, c_int64,             # q
         c_void_p, c_void_p, c_int64, c_int64, c_int64,   # k, v, strides, pool_tokens
         c_void_p, c_int64, c_int, c_int, c_int64,        # table, row stride, kind, rows, cols
         c_void_p,                               # row_ids
         c_void_p, c_int,                        # seq_lens
         c_int, c_int, c_int, c_int, c_int,      # batch, heads, dims
         c_float, c_int64,                       # scale, max_seq_len
         c_void_p, c_size_t,                     # workspace
         c_void_p, c_int64, c_int64,             # out
         c_int, c_void_p, c_void_p],             # flags, status, stream
    ),
    "b200kv_append_paged_decode": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64, c_void_p,   # new K, new V, their token strides, slots
         c_void_p, c_int64, c_int64,
         c_void_p, c_void_p, c_int64, c_int64, c_int64,
         c_void_p, c_int64, c_int, c_int, c_int64,
         c_void_p,
         c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_int,
         c_float, c_int64,
         c_void_p, c_size_t,
         c_void_p, c_int64, c_int64,
         c_int, c_void_p, c_void_p],
    ),
    "b200kv_paged_decode_static_scratch": (
        c_int,
        [c_void_p, c_int64, c_int64,
         c_void_p, c_void_p, c_int64, c_int64, c_int64,
         c_void_p, c_int64, c_int, c_int, c_int64,
         c_void_p,
         c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_int,
         c_float, c_int64,
         c_void_p, c_int64, c_int64,
         c_int, c_void_p, c_void_p],
    ),
    "b200kv_selftest_bounded_wait": (c_int, [c_uint64, c_void_p, c_void_p, c_void_p]),
    "b200kv_paged_prefill": (
        c_int,
        [c_void_p, c_int64, c_int64,
         c_void_p, c_void_p, c_int64, c_int64, c_int64,
         c_void_p, c_int64, c_int, c_int, c_int64,
         c_void_p, c_void_p,
         c_void_p, c_void_p, c_int,
         c_int, c_int64, c_int64,
         c_int, c_int, c_int, c_int,
         c_float,
         c_void_p, c_int64, c_int64,
         c_void_p, c_void_p],
    ),
    # host-side prefix cache (include/b200kv_prefix_cache.h)
    "b200kv_prefix_cache_create": (c_void_p, [c_int, c_int64, c_int64]),
    "b200kv_prefix_cache_destroy": (None, [c_void_p]),
    "b200kv_prefix_cache_entries": (c_int64, [c_void_p, c_int]),
    "b200kv_prefix_cache_lookup_exact": (
        c_int64, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200kv_prefix_cache_lookup_blocks": (c_int64, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "b200kv_prefix_cache_store": (c_int64, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64]),
    "b200kv_prefix_cache_ref_ops": (c_int64, [c_void_p, c_void_p, c_void_p, c_int64]),
    "b200kv_prefix_cache_clear": (c_int64, [c_void_p]),
    # decode steps with host buffers (include/b200kv_host_step.h)
    "b200kv_host_steps_create": (c_int, [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200kv_host_steps_destroy": (None, [c_void_p]),
    "b200kv_host_steps_buffers": (
        c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200kv_host_steps_submit": (
        c_int,
        [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64,   # slot, batch, pool
         c_void_p, c_int64, c_int, c_int, c_int64, c_void_p,                      # table, row ids
         c_int, c_float, c_int64, c_int, c_void_p],
    ),
    "b200kv_host_steps_bind": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int, c_int, c_int64,
         c_void_p, c_int, c_float],
    ),
    "b200kv_host_steps_submit_bound": (c_int, [c_void_p, c_int, c_int, c_int, c_int64, c_int, c_void_p]),
    "b200kv_host_steps_flush": (c_int, [c_void_p]),
    "b200kv_host_steps_wait": (c_int, [c_void_p, c_int]),
    "b200kv_host_steps_reset": (c_int, [c_void_p]),
    "b200kv_host_steps_stream": (c_void_p, [c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


class B200KVError(RuntimeError):
    """A libb200kv entry point returned a non-zero code."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200kv error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    """Load (once) and return the shared library with typed entry points."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m llama_lite_npu_b200.build` "
            "(there is no CPU or PyTorch fallback for the b200kv operators)"
        )
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return handle


def check(code: int) -> None:
    """Raise for a non-zero return code of an entry point."""
    if code == 0:
        return
    handle = lib()
    msg = handle.b200kv_strerror(code).decode()
    if code == 5:
        msg += " — " + handle.b200kv_last_cuda_error().decode()
    if code in (1, 2, 3, 6):
        raise ValueError(f"b200kv error {code}: {msg}")
    raise B200KVError(code, msg)


def strerror(code: int) -> str:
    return lib().b200kv_strerror(int(code)).decode()
