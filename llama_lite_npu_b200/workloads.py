"""Seeded synthetic workloads for the paged-KV path.

The shapes follow the five benchmark configurations of this project (decode at
Qwen3-0.6B / Qwen3-32B / Qwen3-30B-A3B head shapes, packed prefill with
prefix-cache hits, long mixed-length decode).  They stand in for serving traffic:
fp16 Q/K/V ~ N(0,1), context lengths from the stated distribution, and physical
pages drawn from a shuffled pool so consecutive logical pages are never adjacent.

Two value sources:

* ``fill="hash"`` — a counter-based integer hash (SplitMix64) turned into an
  Irwin-Hall(4) approximation of N(0,1).  Pure integer arithmetic plus one
  float32 multiply, so the same seed gives the same bits on every machine and
  library version; used for tests and committed golden vectors.
* ``fill="randn"`` — ``torch.Tensor.normal_`` on the target device; used for
  benchmark-sized pools (gigabytes) where only speed matters.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

_MASK64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def hash_u64(seed: int, n: int, stream: int = 0) -> np.ndarray:
    """``n`` reproducible 64-bit words for (seed, stream)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed * 1_000_003 + stream], dtype=np.uint64))[0]
        return _splitmix64(np.arange(n, dtype=np.uint64) * np.uint64(0xD1342543DE82EF95) + base)


def hash_normal_fp16(seed: int, shape, stream: int = 0) -> torch.Tensor:
    """fp16 tensor of approximately N(0,1) values, bit-reproducible everywhere."""
    n = int(np.prod(shape))
    w = hash_u64(seed, n, stream)
    s = ((w & np.uint64(0xFFFF)) + ((w >> np.uint64(16)) & np.uint64(0xFFFF))
         + ((w >> np.uint64(32)) & np.uint64(0xFFFF)) + (w >> np.uint64(48))).astype(np.int64)
    # sum of four U{0..65535}: mean 131070, std 65536/sqrt(3)
    v = (s - 131070).astype(np.float32) * np.float32(math.sqrt(3.0) / 65536.0)
    return torch.from_numpy(v.astype(np.float16)).reshape(shape)


def hash_randint(seed: int, n: int, lo: int, hi: int, stream: int = 0) -> np.ndarray:
    """``n`` integers uniform on [lo, hi] (inclusive)."""
    w = hash_u64(seed, n, stream)
    return (lo + (w % np.uint64(hi - lo + 1)).astype(np.int64)).astype(np.int64)


def hash_uniform(seed: int, n: int, stream: int = 0) -> np.ndarray:
    return (hash_u64(seed, n, stream) >> np.uint64(11)).astype(np.float64) / float(1 << 53)


def hash_permutation(seed: int, n: int, stream: int = 0) -> np.ndarray:
    return np.argsort(hash_u64(seed, n, stream), kind="stable").astype(np.int64)


# ---------------------------------------------------------------------------------------------
# The benchmark configurations.
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class DecodeConfig:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    num_pages: int
    len_lo: int
    len_hi: int
    len_dist: str = "uniform"  # "uniform" | "fixed" | "loguniform"
    head_dim: int = 128
    page_size: int = 16
    seed: int = 1000


@dataclass(frozen=True)
class PrefillConfig:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    num_pages: int
    prompt_lo: int
    prompt_hi: int
    shared_frac_hi: float = 0.5
    head_dim: int = 128
    page_size: int = 16
    seed: int = 1004


C1 = DecodeConfig("c1_qwen3_0p6b_decode", 4, 16, 8, 512, 64, 512, seed=1001)
C2 = DecodeConfig("c2_qwen3_32b_decode", 32, 64, 8, 65536, 1024, 4096, seed=1002)
C3 = DecodeConfig("c3_qwen3_30b_a3b_decode", 64, 32, 4, 16384, 2048, 2048, "fixed", seed=1003)
C4 = PrefillConfig("c4_packed_prefill_prefix_hits", 8, 64, 8, 4096, 128, 2048, seed=1004)
C5 = DecodeConfig("c5_long_mixed_decode", 128, 64, 8, 1 << 20, 16, 32768, "loguniform", seed=1005)

CONFIGS = {c.name: c for c in (C1, C2, C3, C4, C5)}


def shard_kv_heads(cfg, world_size: int, rank: int):
    """KV-head shard of a config for one of ``world_size`` GPUs: same sequences, tables and
    lengths, ``kv_heads / world_size`` KV heads and their query groups."""
    if cfg.kv_heads % world_size != 0:
        raise ValueError(f"{cfg.kv_heads} KV heads do not split over {world_size} GPUs")
    kwargs = dict(cfg.__dict__)
    kwargs["kv_heads"] = cfg.kv_heads // world_size
    kwargs["q_heads"] = cfg.q_heads // world_size
    return type(cfg)(**kwargs)


def shard_requests_config(cfg, world_size: int, rank: int):
    """Request shard of a config for one of ``world_size`` GPUs: ``batch / world_size`` of the
    batch's (independently drawn) requests with all heads, in the rank's own pool and tables (the
    partition used when the KV heads are fewer than the GPUs)."""
    if cfg.batch % world_size != 0:
        raise ValueError(f"a batch of {cfg.batch} does not split over {world_size} GPUs")
    kwargs = dict(cfg.__dict__)
    kwargs["batch"] = cfg.batch // world_size
    kwargs["num_pages"] = max(1, cfg.num_pages // world_size)
    kwargs["seed"] = cfg.seed * 131 + rank
    return type(cfg)(**kwargs)


def shard_config(cfg, world_size: int, rank: int):
    """The partition a benchmark configuration names: by request for the 30B-A3B shape (4 KV
    heads, up to 8 GPUs), by KV head otherwise.  Returns ``(config, kind)``."""
    if world_size == 1:
        return cfg, "single GPU"
    if cfg.name.startswith("c3") or cfg.kv_heads % world_size != 0:
        return shard_requests_config(cfg, world_size, rank), f"request shards over {world_size} GPUs, no collective"
    return shard_kv_heads(cfg, world_size, rank), f"kv-head shards over {world_size} GPUs, no collective"


def draw_lengths(cfg: DecodeConfig) -> np.ndarray:
    if cfg.len_dist == "fixed":
        return np.full(cfg.batch, cfg.len_lo, dtype=np.int64)
    if cfg.len_dist == "uniform":
        return hash_randint(cfg.seed, cfg.batch, cfg.len_lo, cfg.len_hi, stream=1)
    if cfg.len_dist == "loguniform":
        u = hash_uniform(cfg.seed, cfg.batch, stream=1)
        v = np.floor(np.exp(math.log(cfg.len_lo) + u * (math.log(cfg.len_hi) - math.log(cfg.len_lo))))
        return np.clip(v.astype(np.int64), cfg.len_lo, cfg.len_hi)
    raise ValueError(cfg.len_dist)


def _fill(t: torch.Tensor, fill: str, seed: int, stream: int) -> torch.Tensor:
    if fill == "hash":
        t.copy_(hash_normal_fp16(seed, tuple(t.shape), stream))
    elif fill == "randn":
        g = torch.Generator(device=t.device)
        g.manual_seed(seed * 131 + stream)
        t.normal_(generator=g)
    else:
        raise ValueError(fill)
    return t


@dataclass
class DecodeCase:
    cfg: DecodeConfig
    seq_lens: np.ndarray                 # lengths INCLUDING the token appended this step
    pages: list                          # per sequence: np.ndarray of physical page ids
    pool: torch.Tensor                   # [num_pages*ps, 2*KH, D] fp16
    token_table: torch.Tensor            # int32 [B, width]
    block_table: torch.Tensor            # int32 [B, width/ps]
    seq_lens_t: torch.Tensor             # int64 [B]
    q: torch.Tensor                      # [B, H, D] fp16
    new_kv: torch.Tensor                 # [B, 2*KH, D] fp16: the row appended this step
    slots: torch.Tensor                  # int32 [B] = token_table[b, L_b - 1]
    max_len: int = 0

    @property
    def k_cache(self) -> torch.Tensor:
        return self.pool[:, : self.cfg.kv_heads, :]

    @property
    def v_cache(self) -> torch.Tensor:
        return self.pool[:, self.cfg.kv_heads:, :]

    def algorithmic_bytes(self) -> int:
        """K and V of every context token once, Q in, O out, one int32 per page walked."""
        c = self.cfg
        kv = int(self.seq_lens.sum()) * c.kv_heads * c.head_dim * 2 * 2
        qo = 2 * c.batch * c.q_heads * c.head_dim * 2
        tbl = int(np.ceil(self.seq_lens / c.page_size).sum()) * 4
        return kv + qo + tbl


def assign_pages(num_pages: int, pages_needed: np.ndarray, seed: int) -> list:
    total = int(pages_needed.sum())
    if total > num_pages:
        raise ValueError(f"workload needs {total} pages, pool has {num_pages}")
    perm = hash_permutation(seed, num_pages, stream=2)
    out, cur = [], 0
    for n in pages_needed.tolist():
        out.append(perm[cur: cur + n].copy())
        cur += n
    return out


def tables_from_pages(pages: list, width_tokens: int, page_size: int):
    """(token_table int32 [B, width], block_table int32 [B, width/ps]); unused entries are 0."""
    width_pages = (width_tokens + page_size - 1) // page_size
    width_tokens = width_pages * page_size
    bt = np.zeros((len(pages), width_pages), dtype=np.int32)
    for i, pg in enumerate(pages):
        bt[i, : len(pg)] = pg
    tt = (bt[:, :, None].astype(np.int64) * page_size + np.arange(page_size)[None, None, :])
    tt = tt.reshape(len(pages), width_tokens).astype(np.int32)
    return torch.from_numpy(tt), torch.from_numpy(bt)


def make_decode_case(cfg: DecodeConfig, device="cpu", fill="hash",
                     lengths: Optional[np.ndarray] = None, fill_pool: bool = True) -> DecodeCase:
    """One decode step: every sequence already has L-1 tokens in the pool, the step appends the
    L-th (``new_kv`` at ``slots``) and then attends over all L."""
    ps = cfg.page_size
    lens = draw_lengths(cfg) if lengths is None else np.asarray(lengths, dtype=np.int64)
    assert len(lens) == cfg.batch
    need = (lens + ps - 1) // ps
    pages = assign_pages(cfg.num_pages, need, cfg.seed)
    max_len = int(lens.max()) if len(lens) else 0
    tt, bt = tables_from_pages(pages, max(max_len, 1), ps)
    pool = torch.empty((cfg.num_pages * ps, 2 * cfg.kv_heads, cfg.head_dim), dtype=torch.float16,
                       device=device)
    if fill_pool:
        _fill(pool, fill, cfg.seed, 3)
    q = _fill(torch.empty((cfg.batch, cfg.q_heads, cfg.head_dim), dtype=torch.float16, device=device),
              fill, cfg.seed, 4)
    new_kv = _fill(torch.empty((cfg.batch, 2 * cfg.kv_heads, cfg.head_dim), dtype=torch.float16,
                               device=device), fill, cfg.seed, 5)
    rows = np.arange(cfg.batch)
    slots = tt.numpy()[rows, np.maximum(lens - 1, 0)].astype(np.int32)
    return DecodeCase(
        cfg=cfg, seq_lens=lens, pages=pages, pool=pool,
        token_table=tt.to(device), block_table=bt.to(device),
        seq_lens_t=torch.from_numpy(lens).to(device), q=q, new_kv=new_kv,
        slots=torch.from_numpy(slots).to(device), max_len=max_len,
    )


@dataclass
class PrefillCase:
    cfg: PrefillConfig
    prompt_lens: np.ndarray
    ctx_lens: np.ndarray                # tokens already in the pool (shared prefix pages)
    q_lens: np.ndarray                  # prompt - ctx, appended then attended
    pages: list
    page_refcount: np.ndarray           # int32 [num_pages]: 2 on shared prefix pages, 1 on own pages
    pool: torch.Tensor
    token_table: torch.Tensor
    block_table: torch.Tensor
    req_ids: torch.Tensor               # int32 [B]
    q_start: torch.Tensor               # int32 [B]
    ctx_lens_t: torch.Tensor            # int64 [B]
    q_lens_t: torch.Tensor              # int64 [B]
    q: torch.Tensor                     # [sum q, H, D]
    new_kv: torch.Tensor                # [sum q, 2*KH, D]
    slots: torch.Tensor                 # int32 [sum q]
    max_q_len: int = 0

    @property
    def k_cache(self) -> torch.Tensor:
        return self.pool[:, : self.cfg.kv_heads, :]

    @property
    def v_cache(self) -> torch.Tensor:
        return self.pool[:, self.cfg.kv_heads:, :]

    def flops(self) -> int:
        """QK^T and PV over causal (query, key) pairs only: 4*D*H*sum(q*ctx + q(q+1)/2)."""
        c = self.cfg
        q = self.q_lens.astype(np.int64)
        pairs = int((q * self.ctx_lens + q * (q + 1) // 2).sum())
        return 4 * c.head_dim * c.q_heads * pairs


def draw_prefill_lengths(cfg: PrefillConfig):
    """(prompt lengths, shared prefix pages) of a prefill configuration, without building it."""
    ps = cfg.page_size
    prompt_lens = hash_randint(cfg.seed, cfg.batch, cfg.prompt_lo, cfg.prompt_hi, stream=1)
    f = hash_uniform(cfg.seed, cfg.batch, stream=6) * cfg.shared_frac_hi
    shared = np.floor(f * ((prompt_lens + ps - 1) // ps)).astype(np.int64)
    return prompt_lens, np.minimum(shared, (prompt_lens - 1) // ps)


def make_prefill_case(cfg: PrefillConfig, device="cpu", fill="hash",
                      prompt_lens: Optional[np.ndarray] = None,
                      shared_pages: Optional[np.ndarray] = None) -> PrefillCase:
    """Packed prefill with prefix-cache hits: the first ``shared_pages`` pages of each prompt are
    already in the pool (and hold a second reference); the rest of the prompt is the query
    chunk whose K/V the step appends before attending."""
    ps = cfg.page_size
    if prompt_lens is None or shared_pages is None:
        drawn_lens, drawn_shared = draw_prefill_lengths(cfg)
        if prompt_lens is None:
            prompt_lens = drawn_lens
            if shared_pages is None:
                shared_pages = drawn_shared
        else:
            prompt_lens = np.asarray(prompt_lens, dtype=np.int64)
            f = hash_uniform(cfg.seed, cfg.batch, stream=6) * cfg.shared_frac_hi
            shared_pages = np.floor(f * ((prompt_lens + ps - 1) // ps)).astype(np.int64)
    prompt_lens = np.asarray(prompt_lens, dtype=np.int64)
    total_pages = (prompt_lens + ps - 1) // ps
    shared_pages = np.minimum(np.asarray(shared_pages, dtype=np.int64), (prompt_lens - 1) // ps)
    ctx = shared_pages * ps
    qn = prompt_lens - ctx
    pages = assign_pages(cfg.num_pages, total_pages, cfg.seed)
    refc = np.zeros(cfg.num_pages, dtype=np.int32)
    for pg, sh in zip(pages, shared_pages.tolist()):
        refc[pg] = 1
        refc[pg[:sh]] = 2
    tt, bt = tables_from_pages(pages, int(prompt_lens.max()), ps)
    pool = _fill(torch.empty((cfg.num_pages * ps, 2 * cfg.kv_heads, cfg.head_dim), dtype=torch.float16,
                             device=device), fill, cfg.seed, 3)
    total_q = int(qn.sum())
    q = _fill(torch.empty((total_q, cfg.q_heads, cfg.head_dim), dtype=torch.float16, device=device),
              fill, cfg.seed, 4)
    new_kv = _fill(torch.empty((total_q, 2 * cfg.kv_heads, cfg.head_dim), dtype=torch.float16,
                               device=device), fill, cfg.seed, 5)
    q_start = np.concatenate([[0], np.cumsum(qn)[:-1]]).astype(np.int32)
    ttn = tt.numpy()
    slots = np.concatenate([ttn[i, ctx[i]: prompt_lens[i]] for i in range(cfg.batch)]).astype(np.int32)
    return PrefillCase(
        cfg=cfg, prompt_lens=prompt_lens, ctx_lens=ctx, q_lens=qn, pages=pages, page_refcount=refc,
        pool=pool, token_table=tt.to(device), block_table=bt.to(device),
        req_ids=torch.arange(cfg.batch, dtype=torch.int32, device=device),
        q_start=torch.from_numpy(q_start).to(device),
        ctx_lens_t=torch.from_numpy(ctx).to(device), q_lens_t=torch.from_numpy(qn).to(device),
        q=q, new_kv=new_kv, slots=torch.from_numpy(slots).to(device), max_q_len=int(qn.max()),
    )


# ---------------------------------------------------------------------------------------------
# Sharding one job over the GPUs of a box (no collective: every shard is self-contained)
# ---------------------------------------------------------------------------------------------
def head_shard(kv_heads: int, q_heads: int, world_size: int, rank: int):
    """(kv head slice, q head slice) owned by ``rank``: a contiguous block of KV heads with the
    query heads of their groups, the layout a tensor-parallel attention layer uses."""
    if kv_heads % world_size != 0:
        raise ValueError(f"{kv_heads} KV heads do not split over {world_size} ranks")
    per = kv_heads // world_size
    group = q_heads // kv_heads
    return slice(rank * per, (rank + 1) * per), slice(rank * per * group, (rank + 1) * per * group)


def _shard_pool(pool: torch.Tensor, kv_heads: int, kv_sl: slice) -> torch.Tensor:
    k = pool[:, :kv_heads][:, kv_sl]
    v = pool[:, kv_heads:][:, kv_sl]
    return torch.cat([k, v], dim=1).contiguous()


def shard_decode_case(case: DecodeCase, world_size: int, rank: int) -> DecodeCase:
    """KV-head shard of a decode step: same sequences, tables, lengths and slots; this rank's
    heads of q, of the pool and of the appended rows.  Concatenating the shards' outputs along
    the head axis gives the unsharded output."""
    cfg = case.cfg
    kv_sl, q_sl = head_shard(cfg.kv_heads, cfg.q_heads, world_size, rank)
    return DecodeCase(
        cfg=shard_kv_heads(cfg, world_size, rank), seq_lens=case.seq_lens, pages=case.pages,
        pool=_shard_pool(case.pool, cfg.kv_heads, kv_sl), token_table=case.token_table,
        block_table=case.block_table, seq_lens_t=case.seq_lens_t, q=case.q[:, q_sl].contiguous(),
        new_kv=_shard_pool(case.new_kv, cfg.kv_heads, kv_sl), slots=case.slots, max_len=case.max_len,
    )


def shard_prefill_case(case: PrefillCase, world_size: int, rank: int) -> PrefillCase:
    cfg = case.cfg
    kv_sl, q_sl = head_shard(cfg.kv_heads, cfg.q_heads, world_size, rank)
    out = PrefillCase(**{**case.__dict__})
    out.cfg = shard_kv_heads(cfg, world_size, rank)
    out.pool = _shard_pool(case.pool, cfg.kv_heads, kv_sl)
    out.new_kv = _shard_pool(case.new_kv, cfg.kv_heads, kv_sl)
    out.q = case.q[:, q_sl].contiguous()
    return out


def shard_decode_requests(case: DecodeCase, world_size: int, rank: int) -> DecodeCase:
    """Request shard (used when KV heads are fewer than ranks): requests rank::world_size with all
    heads; tables keep their page ids, so the rank needs the same pool (or its own copy of the
    pages it references)."""
    idx = np.arange(rank, case.cfg.batch, world_size)
    t = torch.from_numpy(idx)
    kwargs = dict(case.cfg.__dict__)
    kwargs["batch"] = len(idx)
    return DecodeCase(
        cfg=DecodeConfig(**kwargs), seq_lens=case.seq_lens[idx], pages=[case.pages[i] for i in idx],
        pool=case.pool, token_table=case.token_table[t].contiguous(),
        block_table=case.block_table[t].contiguous(), seq_lens_t=case.seq_lens_t[t].contiguous(),
        q=case.q[t].contiguous(), new_kv=case.new_kv[t].contiguous(), slots=case.slots[t].contiguous(),
        max_len=int(case.seq_lens[idx].max()) if len(idx) else 0,
    )
