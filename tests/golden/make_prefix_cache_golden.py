"""Record what the REFERENCE's prefix-cache methods do on a scripted call sequence.

Usage (only where the reference checkout is available; the tests need only the JSON):

    python tests/golden/make_prefix_cache_golden.py --reference /path/to/llama_lite_npu

The methods live on the reference's ``ModelExecutor`` (``lite_llama/executor/model_executor.py``:
``share_paged_request_from_cache`` :547-568, ``share_paged_prefix_from_cache`` :570-620,
``_paged_block_key`` :622-625, ``_store_paged_prompt_blocks`` :627-656,
``store_paged_request_prefix`` :658-683), whose module cannot be imported here (it needs the NPU
runtime and model code).  The script therefore takes the source text of exactly those five
methods out of the reference file at run time, compiles them into a bare holder class and runs
them against the reference's own ``PagedKVCacheManager`` / ``PagedReqTokensManager`` (loaded by
file path).  After every call the return value and the whole observable state of the page pool
go into ``prefix_cache_golden.json``; ``tests/test_prefix_cache.py`` replays the same script on
this repository's executor and native cache and compares call for call.
"""

from __future__ import annotations

import argparse
import ast
import importlib.util
import json
import sys
import textwrap
import warnings
from collections import OrderedDict
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
sys.path.insert(0, str(HERE.parent))

from golden_cases import PREFIX_CACHE_SCRIPT, run_prefix_cache_script  # noqa: E402

METHODS = ("share_paged_request_from_cache", "share_paged_prefix_from_cache", "_paged_block_key",
           "_store_paged_prompt_blocks", "store_paged_request_prefix")


def load(ref_root: Path, name: str, rel: str):
    spec = importlib.util.spec_from_file_location(name, ref_root / rel)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        spec.loader.exec_module(mod)
    return mod


def reference_holder_class(ref_root: Path):
    """A class holding the reference's five prefix-cache methods, compiled from its source file."""
    path = ref_root / "lite_llama/executor/model_executor.py"
    source = path.read_text()
    tree = ast.parse(source)
    cls = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "ModelExecutor")
    lines = source.splitlines()
    body = []
    for node in cls.body:
        if isinstance(node, ast.FunctionDef) and node.name in METHODS:
            start = min([node.lineno] + [d.lineno for d in node.decorator_list])
            body.append(textwrap.dedent("\n".join(lines[start - 1: node.end_lineno])))
    assert len(body) == len(METHODS), "the reference no longer has all five methods"
    text = "class Holder:\n" + textwrap.indent("\n\n".join(body), "    ") + "\n"
    scope = {"torch": torch, "OrderedDict": OrderedDict}
    exec(compile(text, str(path), "exec"), scope)
    return scope["Holder"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = Path(args.reference)
    paged = load(ref, "ref_paged_attention", "lite_llama/executor/paged_attention.py")
    Holder = reference_holder_class(ref)
    sc = PREFIX_CACHE_SCRIPT

    ex = Holder()
    ex.use_paged_attn = True
    ex.page_size = sc["page_size"]
    pm = paged.PagedKVCacheManager(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=sc["num_pages"],
                                   page_size=sc["page_size"], dtype=torch.float16, device="cpu")
    ex.req_tokens_manager = paged.PagedReqTokensManager(max_requests=sc["max_requests"],
                                                        max_seq_len=sc["max_seq_len"], page_manager=pm, device="cpu")
    ex._paged_prefix_cache = OrderedDict()
    ex._paged_prefix_cache_max_entries = sc["max_exact"]
    ex._paged_block_prefix_cache = OrderedDict()
    ex._paged_block_prefix_cache_max_entries = sc["max_block"]
    log = run_prefix_cache_script(
        ex, ex.req_tokens_manager,
        sizes=lambda: (len(ex._paged_prefix_cache), len(ex._paged_block_prefix_cache)))
    out = HERE / "prefix_cache_golden.json"
    out.write_text(json.dumps({"script": sc, "log": log}, indent=1) + "\n")
    print(f"wrote {out} ({len(log)} calls)")


if __name__ == "__main__":
    main()
