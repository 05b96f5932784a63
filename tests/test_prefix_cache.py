"""The native prefix cache behind the executor's reference-named methods, call for call against a
log recorded from the REFERENCE's own methods (``tests/golden/make_prefix_cache_golden.py``), plus
the C++ tables on their own.  No GPU needed: the cache is host code."""

import json
from pathlib import Path

import numpy as np
import pytest

import golden_cases as G
from llama_lite_npu_b200.executor import PagedKVExecutor
from llama_lite_npu_b200.prefix_cache import NativePrefixCache

GOLDEN = Path(__file__).resolve().parent / "golden" / "prefix_cache_golden.json"


def test_executor_prefix_cache_replays_the_reference_log(built_lib):
    recorded = json.loads(GOLDEN.read_text())
    sc = recorded["script"]
    assert sc == G.PREFIX_CACHE_SCRIPT, "regenerate the golden log: the script changed"
    ex = PagedKVExecutor(1, 1, 8, sc["num_pages"], sc["max_requests"], sc["max_seq_len"],
                         page_size=sc["page_size"], device="cpu", prefix_cache_entries=sc["max_exact"],
                         prefix_cache_block_entries=sc["max_block"])
    log = G.run_prefix_cache_script(
        ex, ex.req_tokens_manager,
        sizes=lambda: (ex._prefix_cache.exact_entries, ex._prefix_cache.block_entries))
    assert len(log) == len(recorded["log"])
    for got, want in zip(log, recorded["log"]):
        assert got == want, f"diverged at call {want['call']!r}"
    # forgetting everything returns every reference the cache still held
    ex.clear_paged_prefix_cache()
    pm = ex.req_tokens_manager.page_mgr
    assert int(pm.num_free_pages) == sc["num_pages"] and int(pm.page_refcount.sum()) == 0


def test_native_tables_lru_and_fingerprint_chain(built_lib):
    c = NativePrefixCache(page_size=4, max_exact_entries=2, max_block_entries=3)
    # store: +1 on every page (exact entry), +1 per new full block; 9 tokens = 2 full blocks
    ops = c.store(list(range(1, 10)), [10, 11, 12], 9, 77)
    assert [(d, p.tolist()) for d, p in ops] == [(1, [10, 11, 12, 10, 11])]
    assert (c.exact_entries, c.block_entries) == (1, 2)
    pages, n, first = c.lookup_exact(range(1, 10))
    assert pages.tolist() == [10, 11, 12] and (n, first) == (9, 77)
    assert c.lookup_exact([1, 2]) is None
    # the chain: block 2 is only found under the fingerprint of block 1
    pages, matched = c.lookup_blocks([1, 2, 3, 4, 5, 6, 7, 8, 1, 1, 1, 1])
    assert pages.tolist() == [10, 11] and matched == 8
    pages, matched = c.lookup_blocks([5, 6, 7, 8])             # same tokens, no parent: a miss
    assert pages.shape[0] == 0 and matched == 0
    pages, matched = c.lookup_blocks([1, 2, 3])                # no full block
    assert pages.shape[0] == 0
    assert c.store(list(range(1, 10)), [10, 11, 12], 9, 5) == []   # already there: nothing changes
    # a second prompt sharing block 1: only its new block takes a reference
    ops = c.store([1, 2, 3, 4, 9, 9, 9, 9], [20, 21], 8, 5)
    assert [(d, p.tolist()) for d, p in ops] == [(1, [20, 21, 21])]
    assert (c.exact_entries, c.block_entries) == (2, 3)
    # a third prompt: block table evicts its least recently used entry per insert, then the exact
    # table evicts the oldest prompt and hands back all of its pages
    ops = c.store([7, 7, 7, 7, 8, 8, 8, 8], [30, 31], 8, 5)
    flat = [(d, p.tolist()) for d, p in ops]
    assert flat == [(1, [30, 31, 30]), (-1, [11]), (1, [31]), (-1, [10, 10, 11, 12])]
    assert sum(d * len(p) for d, p in flat) == 2 + 2 - 2 - 3      # +2 pages, +2 blocks, -2 blocks, -3 pages
    assert (c.exact_entries, c.block_entries) == (2, 3)
    assert c.lookup_exact(range(1, 10)) is None
    dropped = c.clear()
    assert all(d == -1 for d, _ in dropped) and (c.exact_entries, c.block_entries) == (0, 0)


def test_native_tables_many_prompts_against_a_python_model(built_lib):
    """Random stores and lookups against a direct restatement with ordered dictionaries."""
    from collections import OrderedDict

    rng = np.random.default_rng(5)
    ps, max_e, max_b = 4, 5, 9
    c = NativePrefixCache(ps, max_e, max_b)
    exact, block = OrderedDict(), OrderedDict()
    refs = {}

    def bump(page, d):
        refs[page] = refs.get(page, 0) + d

    next_page = 0
    for step in range(400):
        n = int(rng.integers(1, 14))
        toks = tuple(int(x) for x in rng.integers(0, 3, size=n))     # tiny alphabet: many shared prefixes
        if rng.random() < 0.5:
            pages = list(range(next_page, next_page + (n + ps - 1) // ps))
            next_page += len(pages)
            for d, pg in c.store(toks, pages, n, step):
                for x in pg.tolist():
                    bump(x, d)
            if toks not in exact:
                exact[toks] = (pages, n, step)
                parent = None
                for b in range(n // ps):
                    key = (parent, toks[b * ps: (b + 1) * ps])
                    parent = key
                    if key in block:
                        block.move_to_end(key)
                        continue
                    block[key] = (pages[b], (b + 1) * ps)
                    while len(block) > max_b:
                        block.popitem(last=False)
                while len(exact) > max_e:
                    exact.popitem(last=False)
        else:
            got = c.lookup_exact(toks)
            if toks in exact:
                exact.move_to_end(toks)
                assert got is not None and got[0].tolist() == exact[toks][0] and got[1:] == exact[toks][1:]
            else:
                assert got is None
            pages, matched = c.lookup_blocks(toks)
            want_pages, want_matched, parent = [], 0, None
            for b in range(n // ps):
                key = (parent, toks[b * ps: (b + 1) * ps])
                if key not in block:
                    break
                block.move_to_end(key)
                want_pages.append(block[key][0])
                want_matched = block[key][1]
                parent = key
            assert pages.tolist() == want_pages and matched == want_matched
        assert (c.exact_entries, c.block_entries) == (len(exact), len(block))
    # the references the cache says it holds are exactly those of the surviving entries
    held = {}
    for pages, _, _ in exact.values():
        for x in pages:
            held[x] = held.get(x, 0) + 1
    for page, _ in block.values():
        held[page] = held.get(page, 0) + 1
    assert {k: v for k, v in refs.items() if v} == held
