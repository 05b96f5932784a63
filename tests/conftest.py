import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (ROOT, ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    gdir = ROOT / "tests" / "golden"
    arrays = dict(np.load(gdir / "paged_kv_golden.npz"))
    meta = json.loads((gdir / "host_golden.json").read_text())
    return {"arrays": arrays, "meta": meta["meta"], "host": meta["host"]}


@pytest.fixture(scope="session")
def built_lib():
    """Build (if stale) and load the C-ABI library."""
    from llama_lite_npu_b200 import _lib
    from llama_lite_npu_b200.build import build_library

    build_library()
    return _lib.lib()


@pytest.fixture(scope="session")
def golden_signatures():
    import json

    return json.loads((ROOT / "tests" / "golden" / "host_golden.json").read_text())["signatures"]
