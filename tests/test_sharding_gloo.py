"""The multi-GPU path on CPU: two gloo ranks each take a shard of one job, run it with the CPU
oracle standing in for the kernels, and the shards must reassemble into the unsharded result
without any data-path collective (all_gather is used here only to CHECK the result)."""

import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import golden_cases as G
from llama_lite_npu_b200 import workloads as W
from oracle import paged_kv_oracle as O

SCALE = 1.0 / math.sqrt(128)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _decode(c):
    pool = c.pool.clone()
    O.kv_append(c.new_kv, c.slots, pool)
    kh = c.cfg.kv_heads
    return O.paged_decode(c.q, pool[:, :kh], pool[:, kh:], SCALE, c.token_table, c.seq_lens_t)


def _worker(rank, world, port, mode, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    try:
        if mode == "kv_heads":
            full = G.build_decode("decode_c1_shape")            # 16 Q / 8 KV heads
            mine = _decode(W.shard_decode_case(full, world, rank))
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            got = torch.cat(parts, dim=1)
        elif mode == "requests":
            full = G.build_decode("decode_gqa4_edges")          # 6 requests, 2 KV heads
            shard = W.shard_decode_requests(full, world, rank)
            mine = _decode(shard)
            got = torch.zeros_like(full.q)
            parts = [None] * world
            dist.all_gather_object(parts, mine)
            for r in range(world):
                got[r::world] = parts[r]
        else:
            full = G.build_prefill("prefill_hist_gqa2")          # 4 Q / 2 KV heads
            sh = W.shard_prefill_case(full, world, rank)
            pool = sh.pool.clone()
            O.kv_append(sh.new_kv, sh.slots, pool)
            kh = sh.cfg.kv_heads
            mine = O.paged_attention(sh.q, pool[:, :kh], pool[:, kh:], SCALE, sh.token_table, sh.req_ids,
                                     sh.q_start, sh.ctx_lens_t, sh.q_lens_t)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            got = torch.cat(parts, dim=1)
        # timing reduction used by the benchmark: the step time of the job is the slowest rank's
        t = torch.tensor([10.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            torch.save({"got": got, "tmax": float(t)}, result_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["kv_heads", "requests", "prefill_kv_heads"])
def test_two_rank_shards_reassemble(mode, tmp_path):
    path = str(tmp_path / "out.pt")
    mp.spawn(_worker, args=(2, _free_port(), mode, path), nprocs=2, join=True)
    res = torch.load(path)
    if mode == "kv_heads":
        want = _decode(G.build_decode("decode_c1_shape"))
    elif mode == "requests":
        want = _decode(G.build_decode("decode_gqa4_edges"))
    else:
        c = G.build_prefill("prefill_hist_gqa2")
        pool = c.pool.clone()
        O.kv_append(c.new_kv, c.slots, pool)
        want = O.paged_attention(c.q, pool[:, :2], pool[:, 2:], SCALE, c.token_table, c.req_ids,
                                 c.q_start, c.ctx_lens_t, c.q_lens_t)
    assert torch.equal(res["got"], want)       # heads / requests never mix: shards are bit-identical
    assert res["tmax"] == 11.0


def test_shard_config_and_slices():
    cfg = W.shard_kv_heads(W.C2, 4, 1)
    assert (cfg.kv_heads, cfg.q_heads, cfg.batch) == (2, 16, 32)
    kv, q = W.head_shard(8, 64, 4, 1)
    assert (kv.start, kv.stop, q.start, q.stop) == (2, 4, 16, 32)
    with pytest.raises(ValueError):
        W.shard_kv_heads(W.C3, 8, 0)           # 4 KV heads do not split over 8 ranks: shard requests
    full = G.build_decode("decode_gqa4_edges")
    parts = [W.shard_decode_requests(full, 4, r) for r in range(4)]
    assert sorted(int(x) for p in parts for x in p.seq_lens) == sorted(int(x) for x in full.seq_lens)


def test_benchmark_partition_choice():
    """KV-head shards where the heads divide, request shards for the 4-KV-head shape on 8 GPUs."""
    cfg, kind = W.shard_config(W.C2, 8, 3)
    assert (cfg.kv_heads, cfg.q_heads, cfg.batch) == (1, 8, 32) and kind.startswith("kv-head")
    parts = [W.shard_config(W.C3, 8, r) for r in range(8)]
    assert all(k.startswith("request") for _, k in parts)
    assert sum(c.batch for c, _ in parts) == W.C3.batch and {c.kv_heads for c, _ in parts} == {W.C3.kv_heads}
    assert len({c.seed for c, _ in parts}) == 8 and sum(c.num_pages for c, _ in parts) == W.C3.num_pages
    assert W.shard_config(W.C2, 1, 0) == (W.C2, "single GPU")
