"""The operators keep the reference's positional surface: same parameter names in the same
order (recorded from the reference's own functions by tests/golden/make_golden.py), and anything
this package adds is keyword-only with a default, so a call written for the reference binds the
same way here."""

import inspect

import pytest

from llama_lite_npu_b200 import kernels


@pytest.mark.parametrize("name", ["update_kv_buffer", "flash_decoding", "paged_chunk_flash_attention",
                                  "flash_attention2_no_pad", "update_kv_index"])
def test_operator_binds_like_the_reference(name, golden_signatures):
    recorded = golden_signatures[name]
    ours = list(inspect.signature(getattr(kernels, name)).parameters.values())
    assert len(ours) >= len(recorded)
    for prm, (ref_name, ref_has_default, ref_kind) in zip(ours, recorded):
        assert prm.name == ref_name
        assert prm.kind.name == ref_kind
        assert (prm.default is not inspect.Parameter.empty) == ref_has_default
    for extra in ours[len(recorded):]:
        assert extra.kind is inspect.Parameter.KEYWORD_ONLY and extra.default is not inspect.Parameter.empty, \
            f"{name}: added parameter {extra.name!r} must be keyword-only with a default"
