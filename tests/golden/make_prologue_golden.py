"""Generate ``qk_prologue_golden.npz`` by RUNNING THE REFERENCE'S OWN torch statements of the
attention prologue on the seeded inputs of ``tests/golden_cases.py``:

* ``python_rmsnorm``      lite_llama/kernels/skip_rmsnorm.py:230-234  (the check of its norm kernel)
* ``torch_rotary_emb``    tests/kernels/test_rope_forward.py:150-170  (the check of its rope kernel)
* the scatter statement   lite_llama/kernels/update_kv_buffer.py:104-105

    python tests/golden/make_prologue_golden.py --reference /path/to/llama_lite_npu

Both statements run in fp16 on the CPU (every operation rounded to fp16), so they agree with the
reference's kernels only to the tolerance the reference's own tests use (1e-3 absolute + relative
for the norm); the oracle is pinned to these outputs at a tolerance stated in
``tests/test_oracle_golden.py``.
"""

from __future__ import annotations

import argparse
import importlib
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parent))

from make_golden import load  # noqa: E402
from golden_cases import PROLOGUE_CASES, PROLOGUE_EPS, build_prologue  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ref = Path(ap.parse_args().reference)
    # skip_rmsnorm.py imports its sibling ``.utils``: give it a bare parent package whose path is
    # the reference's kernels folder (the folder's own __init__ needs the NPU runtime).
    pkg = types.ModuleType("ref_kernels")
    pkg.__path__ = [str(ref / "lite_llama" / "kernels")]
    sys.modules["ref_kernels"] = pkg
    norm = importlib.import_module("ref_kernels.skip_rmsnorm")
    rope = load(ref, "ref_test_rope_forward", "tests/kernels/test_rope_forward.py")
    out: dict[str, np.ndarray] = {}
    for name in PROLOGUE_CASES:
        xq, xkv, wq, wk, cos, sin, slots, pool = build_prologue(name)
        n, _, d = xq.shape
        kvh = pool.shape[1] // 2
        xk, xv = xkv.view(n, 2 * kvh, d)[:, :kvh], xkv.view(n, 2 * kvh, d)[:, kvh:]
        if wq is not None:
            xq = norm.python_rmsnorm(xq, wq, PROLOGUE_EPS)
            xk = norm.python_rmsnorm(xk, wk, PROLOGUE_EPS)
        half = d // 2
        q = rope.torch_rotary_emb(xq, cos[:, :half].contiguous(), sin[:, :half].contiguous())
        k = rope.torch_rotary_emb(xk, cos[:, :half].contiguous(), sin[:, :half].contiguous())
        pool[slots.long()] = torch.cat([k, xv], dim=-2)
        out[f"{name}.q"] = q.numpy()
        out[f"{name}.pool_rows"] = pool[slots.long()].numpy()
    np.savez(HERE / "qk_prologue_golden.npz", **out)
    print("wrote", HERE / "qk_prologue_golden.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
