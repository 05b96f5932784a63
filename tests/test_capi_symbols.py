"""The C-ABI library builds, loads and exports every symbol the headers under include/ declare.
No compute call is made here (no GPU needed)."""

import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(b200kv_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_symbols_are_exported(built_lib):
    names = _declared_symbols()
    assert "b200kv_paged_decode" in names and "b200kv_kv_append" in names
    for name in names:
        assert hasattr(built_lib, name), f"{name} declared in b200kv.h but not exported"


def test_binding_table_covers_header(built_lib):
    from llama_lite_npu_b200 import _lib

    assert sorted(_lib.EXPORTED_SYMBOLS) == _declared_symbols()
    assert built_lib.b200kv_version() == 200
    assert built_lib.b200kv_strerror(0) == b"ok"
    assert b"workspace" in built_lib.b200kv_strerror(4)


def test_host_side_argument_validation_needs_no_gpu(built_lib):
    # n_tokens == 0 is a no-op and a negative count is rejected before any CUDA call
    assert built_lib.b200kv_kv_append(None, 0, 0, None, None, 0, 0, 16, 128, None, None) == 0
    assert built_lib.b200kv_kv_append(None, -1, 0, None, None, 0, 0, 16, 128, None, None) == 1
    assert built_lib.b200kv_kv_append(None, 4, 2048, None, None, 64, 2048, 16, 128, None, None) == 1


def test_operators_refuse_cpu_tensors():
    import torch

    from llama_lite_npu_b200 import kernels

    with pytest.raises(ValueError, match="no CPU fallback"):
        kernels.update_kv_buffer(torch.zeros(1, 2, 128, dtype=torch.float16),
                                 torch.zeros(1, dtype=torch.int32),
                                 torch.zeros(4, 2, 128, dtype=torch.float16))
