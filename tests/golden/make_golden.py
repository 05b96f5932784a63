"""Generate the golden vectors in this directory by RUNNING THE REFERENCE'S OWN CODE.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/llama_lite_npu

The reference modules are imported by file path (the package itself needs an NPU
runtime), exactly as the reference's own tests do.  Inputs come from the bit-reproducible
hash generator in ``llama_lite_npu_b200.workloads`` so only seeds, shapes, input digests
and the reference OUTPUTS are stored:

* ``paged_kv_golden.npz``  — attention / append outputs of the reference's torch functions
* ``host_golden.json``     — state of the reference's page-pool classes after scripted calls
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.util
import inspect
import json
import math
import sys
import warnings
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from llama_lite_npu_b200 import workloads as W  # noqa: E402


def load(ref_root: Path, name: str, rel: str):
    spec = importlib.util.spec_from_file_location(name, ref_root / rel)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        spec.loader.exec_module(mod)
    return mod


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


# Case definitions are shared with the tests (tests/golden_cases.py builds the same inputs).
sys.path.insert(0, str(HERE.parent))
from golden_cases import (  # noqa: E402
    DECODE_CASES, PREFILL_CASES, NOPAD_CASES, APPEND_CASES, MHA_DECODE_CASES,
    build_decode, build_prefill, build_nopad, build_append, build_mha_decode, host_script,
)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = Path(args.reference)
    chunk = load(ref, "ref_paged_chunk_fa", "lite_llama/kernels/paged_chunk_flashattention.py")
    nopad = load(ref, "ref_fa2_nopad", "lite_llama/kernels/flashattention2_nopad.py")
    fdec = load(ref, "ref_flashdecoding", "lite_llama/kernels/flashdecoding.py")
    paged = load(ref, "ref_paged_attention", "lite_llama/executor/paged_attention.py")
    kveng = load(ref, "ref_kv_engine", "lite_llama/kv_engine.py")
    torch.set_num_threads(8)

    out: dict[str, np.ndarray] = {}
    meta: dict[str, dict] = {}

    for name in APPEND_CASES:
        src, slots, pool = build_append(name)
        pool[slots.long()] = src  # the reference's torch statement, update_kv_buffer.py:104-105
        meta[name] = {"pool_sha256": digest(pool), "src_sha256": digest(src)}

    for name in DECODE_CASES:
        c = build_decode(name)
        scale = 1.0 / math.sqrt(c.cfg.head_dim)
        b = c.cfg.batch
        res = chunk._paged_chunk_attention_torch_fallback(
            c.q, c.k_cache, c.v_cache, scale, c.token_table,
            torch.arange(b, dtype=torch.int32), torch.arange(b, dtype=torch.int32),
            c.seq_lens_t - 1, torch.ones(b, dtype=torch.long))
        out[name] = res.numpy()
        meta[name] = {"q_sha256": digest(c.q), "pool_sha256": digest(c.pool),
                      "seq_lens": c.seq_lens.tolist()}

    for name in MHA_DECODE_CASES:
        q, k, v, start, lens = build_mha_decode(name)
        res = fdec.torch_attention_with_kvcache(q, k, v, start, lens)
        out[name] = res.numpy()
        meta[name] = {"q_sha256": digest(q)}

    for name in PREFILL_CASES:
        c = build_prefill(name)
        scale = 1.0 / math.sqrt(c.cfg.head_dim)
        pool = c.pool.clone()
        pool[c.slots.long()] = c.new_kv
        kh = c.cfg.kv_heads
        res = chunk._paged_chunk_attention_torch_fallback(
            c.q, pool[:, :kh], pool[:, kh:], scale, c.token_table, c.req_ids, c.q_start,
            c.ctx_lens_t, c.q_lens_t)
        out[name] = res.numpy()
        meta[name] = {"q_sha256": digest(c.q), "ctx": c.ctx_lens.tolist(), "q_lens": c.q_lens.tolist()}

    for name in NOPAD_CASES:
        q, k, v, start, lens = build_nopad(name)
        res = nopad.standard_attention_prefill(q, k, v, start, lens, sdpa=False)
        out[name] = res.numpy()
        meta[name] = {"q_sha256": digest(q)}

    np.savez(HERE / "paged_kv_golden.npz", **out)
    host = host_script(paged, kveng)
    # the positional surface of the reference's operators: parameter names in order, and which
    # of them have defaults; the tests hold this package's operators to it
    upd = load(ref, "ref_update_kv_buffer", "lite_llama/kernels/update_kv_buffer.py")
    upi = load(ref, "ref_update_kv_index", "lite_llama/kernels/update_kv_index.py")
    signatures = {}
    for fn in (upd.update_kv_buffer, fdec.flash_decoding, chunk.paged_chunk_flash_attention,
               nopad.flash_attention2_no_pad, upi.update_kv_index):
        params = inspect.signature(fn).parameters
        signatures[fn.__name__] = [[n, prm.default is not inspect.Parameter.empty, prm.kind.name]
                                   for n, prm in params.items()]
    (HERE / "host_golden.json").write_text(json.dumps({"meta": meta, "host": host, "signatures": signatures},
                                                      indent=1, sort_keys=True))
    print("wrote", HERE / "paged_kv_golden.npz", (HERE / "paged_kv_golden.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
