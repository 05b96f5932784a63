"""Generate ``decode_metadata_golden.json`` by driving the reference's own page-pool classes
(lite_llama/executor/paged_attention.py) through decode steps on the CPU:

    python tests/golden/make_metadata_golden.py --reference /path/to/llama_lite_npu

For a batch with a gap in its request ids and out-of-order rows, every step calls
``extend_req(r, 1)`` per request and then ``batch_metadata`` exactly as the reference's executor
does (lite_llama/executor/model_executor.py:893-931); the lengths and last-token slots of every
step, and the final block / token tables, are recorded.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
sys.path.insert(0, str(HERE.parent))

from make_golden import load  # noqa: E402
from golden_cases import METADATA_SCRIPT  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ref = Path(ap.parse_args().reference)
    paged = load(ref, "ref_paged_attention", "lite_llama/executor/paged_attention.py")
    sc = METADATA_SCRIPT
    pm = paged.PagedKVCacheManager(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=sc["num_pages"],
                                   page_size=sc["page_size"], dtype=torch.float16, device="cpu")
    rm = paged.PagedReqTokensManager(sc["max_requests"], sc["max_seq_len"], pm, device="cpu")
    ids = [rm.reserve_req(n) for n in sc["prompt_lengths"]]
    rm.free_req(ids[sc["drop"]])                                   # leaves a gap in the id space
    batch = [ids[i] for i in sc["batch_order"]]
    steps = []
    for _ in range(sc["steps"]):
        for r in batch:
            assert rm.extend_req(r, 1)
        req, lens, last = rm.batch_metadata(batch)
        steps.append({"req_ids": req.tolist(), "seq_lens": lens.tolist(), "slots": last.tolist()})
    pages = max(len(rm.req_page_table[r]) for r in batch)
    block = [[int(p) for p in rm.req_page_table[r].tolist()] for r in batch]
    tokens = [rm.b_req_tokens_table[r, : rm.req_token_count[r]].tolist() for r in batch]
    out = {"batch": batch, "start_lens": [steps[0]["seq_lens"][i] - 1 for i in range(len(batch))],
           "steps": steps, "pages_per_request": block, "max_pages": pages, "token_rows": tokens}
    (HERE / "decode_metadata_golden.json").write_text(json.dumps(out, indent=None, sort_keys=True))
    print("wrote decode_metadata_golden.json:", len(steps), "steps, batch", batch)


if __name__ == "__main__":
    main()
