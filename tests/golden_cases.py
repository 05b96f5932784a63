"""Seeded input builders shared by the golden-vector generator and the tests.

Every builder is a pure function of its case name, built on the bit-reproducible hash
generator of ``llama_lite_npu_b200.workloads``, so the generator script (which runs the
reference) and the tests (which run the oracle and the CUDA kernels) see identical inputs.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from llama_lite_npu_b200 import workloads as W

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

# name -> (DecodeConfig, explicit lengths or None)
DECODE_CASES = {
    "decode_gqa4_edges": (W.DecodeConfig("decode_gqa4_edges", 6, 8, 2, 64, 1, 1, seed=11),
                          [1, 15, 16, 17, 64, 203]),
    "decode_gqa8_small": (W.DecodeConfig("decode_gqa8_small", 5, 16, 2, 96, 1, 1, seed=12),
                          [300, 129, 128, 33, 250]),
    "decode_c1_shape": (W.DecodeConfig("decode_c1_shape", 4, 16, 8, 512, 64, 512, seed=1001), None),
    "decode_mha": (W.DecodeConfig("decode_mha", 3, 2, 2, 32, 1, 1, seed=13), [7, 100, 48]),
}

# name -> (PrefillConfig, prompt lengths, shared pages)
PREFILL_CASES = {
    "prefill_hist_gqa2": (W.PrefillConfig("prefill_hist_gqa2", 3, 4, 2, 48, 1, 1, seed=21),
                          [40, 130, 77], [1, 3, 0]),
    "prefill_hist_gqa8_edges": (W.PrefillConfig("prefill_hist_gqa8_edges", 4, 8, 1, 64, 1, 1, seed=22),
                                [17, 129, 128, 1], [1, 4, 7, 0]),
}

# name -> (heads, [segment lengths])
NOPAD_CASES = {
    "nopad_mha": (2, [33, 100, 1, 64]),
}

# name -> (tokens, rows, pool_tokens)
APPEND_CASES = {
    "append_decode": (4, 16, 8192),
    "append_prefill": (333, 4, 1024),
}

# name -> (tokens, q_heads, kv_heads, head_dim, pool_tokens, qk_norm)
PROLOGUE_CASES = {
    "prologue_qwen3_decode": (7, 8, 2, 128, 256, True),
    "prologue_ragged_prefill": (33, 5, 1, 128, 512, True),
    "prologue_d64_no_norm": (5, 4, 4, 64, 128, False),
}
PROLOGUE_EPS = 1e-6

# Decode-step metadata script: five prompts, one released (gap in the ids), batch rows out of order.
METADATA_SCRIPT = {
    "num_pages": 64, "page_size": 4, "max_requests": 8, "max_seq_len": 64,
    "prompt_lengths": [5, 8, 3, 15, 1], "drop": 1, "batch_order": [3, 0, 4, 2], "steps": 21,
}

MHA_DECODE_CASES = {
    "decode_contiguous_mha": (3, 4, [50, 128, 77]),
}


def build_decode(name: str, device="cpu") -> W.DecodeCase:
    cfg, lens = DECODE_CASES[name]
    return W.make_decode_case(cfg, device=device, fill="hash",
                              lengths=None if lens is None else np.array(lens))


def build_prefill(name: str, device="cpu") -> W.PrefillCase:
    cfg, prompts, shared = PREFILL_CASES[name]
    return W.make_prefill_case(cfg, device=device, fill="hash", prompt_lens=np.array(prompts),
                               shared_pages=np.array(shared))


def build_nopad(name: str, device="cpu"):
    heads, lens = NOPAD_CASES[name]
    total = int(sum(lens))
    seed = 31
    q = W.hash_normal_fp16(seed, (total, heads, 128), 1).to(device)
    k = W.hash_normal_fp16(seed, (total, heads, 128), 2).to(device)
    v = W.hash_normal_fp16(seed, (total, heads, 128), 3).to(device)
    start = torch.tensor(np.concatenate([[0], np.cumsum(lens)[:-1]]), dtype=torch.int32, device=device)
    return q, k, v, start, torch.tensor(lens, dtype=torch.int32, device=device)


def build_append(name: str, device="cpu"):
    n, rows, pool_tokens = APPEND_CASES[name]
    seed = 41 + n
    src = W.hash_normal_fp16(seed, (n, rows, 128), 1).to(device)
    pool = W.hash_normal_fp16(seed, (pool_tokens, rows, 128), 2).to(device)
    slots = torch.from_numpy(W.hash_permutation(seed, pool_tokens, 3)[:n].astype(np.int32)).to(device)
    return src, slots, pool


def build_prologue(name: str, device="cpu"):
    """Inputs of one attention prologue: Q, the kv_proj output, norm weights (or None), cos / sin
    rows of full head_dim as the rotary module returns them, slots and the pool."""
    n, qh, kvh, d, pool_tokens, norm = PROLOGUE_CASES[name]
    seed = 61 + n
    xq = W.hash_normal_fp16(seed, (n, qh, d), 1)
    xkv = W.hash_normal_fp16(seed, (n, 2 * kvh * d), 2)
    wq = (1.0 + 0.25 * W.hash_normal_fp16(seed, (d,), 3).float()).half() if norm else None
    wk = (1.0 + 0.25 * W.hash_normal_fp16(seed, (d,), 4).float()).half() if norm else None
    angles = 3.0 * W.hash_normal_fp16(seed, (n, d // 2), 5).float()
    emb = torch.cat([angles, angles], dim=-1)
    cos, sin = emb.cos().half(), emb.sin().half()
    pool = W.hash_normal_fp16(seed, (pool_tokens, 2 * kvh, d), 6)
    slots = torch.from_numpy(W.hash_permutation(seed, pool_tokens, 7)[:n].astype(np.int32))
    mv = lambda t: None if t is None else t.to(device)  # noqa: E731
    return mv(xq), mv(xkv), mv(wq), mv(wk), mv(cos), mv(sin), mv(slots), mv(pool)


def build_mha_decode(name: str, device="cpu"):
    batch, heads, lens = MHA_DECODE_CASES[name]
    seed = 51
    total = int(sum(lens))
    q = W.hash_normal_fp16(seed, (batch, heads, 128), 1).to(device)
    k = W.hash_normal_fp16(seed, (total, heads, 128), 2).to(device)
    v = W.hash_normal_fp16(seed, (total, heads, 128), 3).to(device)
    start = torch.tensor(np.concatenate([[0], np.cumsum(lens)[:-1]]), dtype=torch.int32, device=device)
    return q, k, v, start, torch.tensor(lens, dtype=torch.int32, device=device)


def host_script(paged, kveng) -> dict:
    """Drive the page-pool classes of module ``paged`` and the metadata classes of module
    ``kveng`` through a fixed script and return everything observable as plain data."""
    log: dict = {}
    pm = paged.PagedKVCacheManager(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=12,
                                   page_size=4, dtype=torch.float16, device="cpu")
    rm = paged.PagedReqTokensManager(max_requests=4, max_seq_len=24, page_manager=pm, device="cpu")

    def snap(tag):
        log[tag] = {
            "free": int(pm.num_free_pages),
            "page_free": pm.page_free.int().tolist(),
            "refcount": pm.page_refcount.tolist(),
            "req_pages": {str(k): [int(x) for x in v.tolist()] for k, v in sorted(rm.req_page_table.items())},
            "req_tokens": {str(k): int(v) for k, v in sorted(rm.req_token_count.items())},
            "free_reqs": list(rm.free_req_indices),
            "tables": {str(k): rm.b_req_tokens_table[k, : rm.req_token_count[k]].tolist()
                       for k in sorted(rm.req_token_count)},
        }

    r0 = rm.reserve_req(5)
    r1 = rm.reserve_req(num_tokens=1, reserved_tokens=9)
    log["ids_a"] = [r0, r1]
    snap("after_reserve")
    log["extend_r1_8"] = rm.extend_req(r1, 8)
    log["extend_r0_3"] = rm.extend_req(r0, 3)
    log["extend_r0_1"] = rm.extend_req(r0, 1)
    snap("after_extend")
    r2 = rm.reserve_shared_req(rm.req_page_table[r0], 8)
    log["ids_b"] = [r2]
    snap("after_share")
    ids, lens, last = rm.batch_metadata([r2, r0, r1])
    log["batch_metadata"] = [ids.tolist(), lens.tolist(), last.tolist(),
                             str(ids.dtype), str(lens.dtype), str(last.dtype)]
    log["ensure_r1_16"] = rm.ensure_req_capacity(r1, 16)
    log["ensure_r1_99"] = rm.ensure_req_capacity(r1, 99)
    snap("after_ensure")
    rm.free_req(r0)
    snap("after_free_r0")
    log["too_long"] = rm.reserve_req(25)
    r3 = rm.reserve_req(17)
    log["ids_c"] = [r3]
    log["exhaust"] = rm.reserve_req(16)
    log["extend_over_max"] = rm.extend_req(r3, 8)
    snap("after_r3")
    log["request_pages_r2"] = list(rm.request_pages(r2))
    rm.free_req(r2)
    rm.free_req(r1)
    rm.free_req(r3)
    snap("after_free_all")
    errs = {}
    try:
        pm.free(torch.tensor([0]))
    except ValueError as e:
        errs["free_free_page"] = str(e)
    try:
        pm.add_ref(torch.tensor([1]))
    except ValueError as e:
        errs["addref_free_page"] = str(e)
    try:
        rm.batch_metadata([])
    except ValueError as e:
        errs["empty_batch"] = str(e)
    try:
        rm.batch_metadata([3])
    except KeyError as e:
        errs["unknown_req"] = str(e)
    try:
        rm.request_pages(2)
    except KeyError as e:
        errs["unknown_pages"] = str(e)
    log["errors"] = errs

    refs = kveng.KVBlockRefCounter(total_blocks=6)
    a = refs.acquire(3)
    refs.add_ref((0, 2))
    refs.release((0, 1))
    b = refs.acquire(2)
    k = {"a": list(a), "b": list(b), "avail": refs.available_count,
         "rc": [refs.refcount(i) for i in range(6)]}
    for label, fn, exc in (
        ("neg", lambda: refs.release((5,)), ValueError),
        ("free_ref", lambda: refs.add_ref((5,)), ValueError),
        ("range", lambda: refs.refcount(6), IndexError),
        ("short", lambda: refs.acquire(9), RuntimeError),
        ("zero", lambda: refs.acquire(0), ValueError),
    ):
        try:
            fn()
            k[label] = "no error"
        except exc as e:
            k[label] = type(e).__name__
    log["refcounter"] = k

    cache = kveng.PrefixCache(block_size=4)
    cache.put((1, 2, 3, 4, 5, 6, 7, 8, 9), (10, 11, 12))
    m1 = cache.match((1, 2, 3, 4, 5, 6, 9, 9))
    m2 = cache.match((1, 2, 3, 4, 5, 6, 7, 8, 9, 9, 9, 9))
    m3 = cache.match((5, 6, 7, 8))
    m4 = cache.match((1, 2, 3))
    log["prefix"] = [[m.matched_tokens, list(m.block_ids)] for m in (m1, m2, m3, m4)]
    plan = kveng.ChunkedPrefillPlanner(chunk_size=4).plan(10)
    log["chunks"] = [[c.start, c.end, c.length] for c in plan]
    log["chunks_empty"] = len(kveng.ChunkedPrefillPlanner(chunk_size=3).plan(0))
    pk = kveng.MixedLengthPrefillPacker().pack(((10, 11), (20,), (), (30, 31, 32)))
    log["pack"] = {"tokens": list(pk.flat_token_ids), "pos": list(pk.flat_position_ids),
                   "rows": [[r.request_index, r.start, r.length, r.end] for r in pk.requests],
                   "total": pk.total_tokens, "batch": pk.batch_size}
    return log


# Prefix-cache script: small capacities so that both tables evict; page_size 4.
PREFIX_CACHE_SCRIPT = {
    "page_size": 4, "num_pages": 40, "max_requests": 12, "max_seq_len": 32, "max_exact": 3, "max_block": 6,
}


def run_prefix_cache_script(ex, mgr, sizes) -> list:
    """Drive an executor-like object ``ex`` (prefix-cache methods of the reference's ModelExecutor)
    over request manager ``mgr`` through a fixed call sequence; after every call record the return
    value, the table sizes and the page pool's observable state."""
    pm = mgr.page_mgr
    log = []

    def snap(call, ret):
        log.append({
            "call": call, "ret": ret, "sizes": list(sizes()), "free": int(pm.num_free_pages),
            "refcount": [int(x) for x in pm.page_refcount.tolist()],
            "req_pages": {str(k): [int(x) for x in v.tolist()] for k, v in sorted(mgr.req_page_table.items())},
            "req_tokens": {str(k): int(v) for k, v in sorted(mgr.req_token_count.items())},
        })

    def prompt(seed, n):   # deterministic token ids, distinct per seed, shared 8-token head for seeds < 10
        head = [1000 + i for i in range(8)] if seed < 10 else [2000 + seed * 7 + i for i in range(8)]
        return tuple((head + [seed * 100 + i for i in range(n)])[:n])

    def new_request(tokens):
        return mgr.reserve_req(len(tokens))

    def norm(ret):
        return None if ret is None else [None if x is None else int(x) for x in ret]

    prompts = {
        "a": prompt(1, 13), "b": prompt(2, 16), "c": prompt(3, 9), "d": prompt(11, 12), "e": prompt(12, 8),
        "f": prompt(4, 20), "short": prompt(5, 3),
    }
    live = {}
    # 1. misses on an empty cache
    snap("share_prefix a (empty)", norm(ex.share_paged_prefix_from_cache(prompts["a"])))
    snap("share_exact a (empty)", norm(ex.share_paged_request_from_cache(prompts["a"])))
    snap("share_prefix () ", norm(ex.share_paged_prefix_from_cache(())))
    # 2. store a and b (they share the first two blocks), then hit them
    for name in ("a", "b"):
        live[name] = new_request(prompts[name])
        ex.store_paged_request_prefix(prompts[name], live[name], 500 + len(prompts[name]))
        snap(f"store {name}", None)
    ex.store_paged_request_prefix(prompts["a"], live["a"], 999)          # already stored: no change
    snap("store a again", None)
    ex.store_paged_request_prefix(prompts["c"], 11, 1)                    # unknown request id: ignored
    snap("store unknown request", None)
    r = ex.share_paged_request_from_cache(prompts["a"])
    snap("share_exact a", norm(r))
    live["a2"] = r[0]
    r = ex.share_paged_prefix_from_cache(prompts["b"])
    snap("share_prefix b (exact)", norm(r))
    live["b2"] = r[0]
    r = ex.share_paged_prefix_from_cache(prompts["c"])                    # partial: the shared head blocks
    snap("share_prefix c (partial)", norm(r))
    live["c_part"] = r[0]
    snap("share_prefix short", norm(ex.share_paged_prefix_from_cache(prompts["short"])))
    snap("share_prefix d (miss)", norm(ex.share_paged_prefix_from_cache(prompts["d"])))
    # 3. more stores: the block table (6) and then the exact table (3) evict
    for name in ("d", "e", "f"):
        live[name] = new_request(prompts[name])
        ex.store_paged_request_prefix(prompts[name], live[name], 600 + len(prompts[name]))
        snap(f"store {name}", None)
    snap("share_exact a (evicted?)", norm(ex.share_paged_request_from_cache(prompts["a"])))
    r = ex.share_paged_prefix_from_cache(prompts["f"])
    snap("share_prefix f", norm(r))
    live["f2"] = r[0]
    r = ex.share_paged_prefix_from_cache(prompts["a"])
    snap("share_prefix a (after evictions)", norm(r))
    if r is not None:
        live["a3"] = r[0]
    # 4. release every request: what stays referenced is what the caches hold
    for name in sorted(live):
        mgr.free_req(live[name])
    snap("all requests released", None)
    # 5. a hit with no free request row left
    taken = []
    while True:
        rid = mgr.reserve_req(1)
        if rid is None:
            break
        taken.append(rid)
    snap("rows exhausted", len(taken))
    snap("share_exact f (no row)", norm(ex.share_paged_request_from_cache(prompts["f"])))
    snap("share_prefix e (no row)", norm(ex.share_paged_prefix_from_cache(prompts["e"])))
    for rid in taken:
        mgr.free_req(rid)
    snap("rows returned", None)
    return log
