"""Benchmark of the paged-KV decode step (KV append + paged flash-decoding).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c5|c1|c4] [--impl reference]

A "step" is one decode step of one transformer layer over the whole batch: scatter the
step's new K/V rows into the page pool by slot_mapping, then attend every sequence's single
query token to its paged context (one fused launch).  The default workload is the Qwen3-32B
shape (batch 32, 64 Q / 8 KV heads, head_dim 128, page_size 16, context lengths uniform in
[1024, 4096], 65536-page shuffled pool).  With N > 1 (launched by torchrun, one rank per GPU)
the KV heads are sharded over the ranks — same sequences, 8/N KV heads each — which needs no
collective in the path; torch.distributed is used only for the timing barrier and the
max-over-ranks reduction.

Prints ONE JSON line (rank 0).  ``value`` is algorithmic HBM traffic of the whole job per
second with all inputs resident in HBM (CUDA-graph replay, device-timed); ``e2e`` is the
same metric through the library's host-buffer form of the step (HostDecodeSteps): the step's
inputs are copied from pinned host memory and the result copied back inside the timed region,
every step; ``check`` is the max-abs-error of
a few sequences of the benchmarked run's own output against the CPU oracle (untimed); at one
GPU ``secondary`` carries the other benchmark configurations (30B-A3B decode, the long mixed
decode on its full 2^20-page pool, packed prefill) and the stand-alone KV append at a
prefill-sized token count, timed the same way outside the headline region.  ``--impl reference`` times the CPU torch statement of the same path (the oracle port)
on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

from llama_lite_npu_b200 import workloads as W  # noqa: E402

METRIC = "paged_decode_hbm_throughput"
UNIT = "GB/s"
PREFILL_METRIC = "paged_prefill_tensor_throughput"
L2_BYTES = 126 * 1024 * 1024
GRAPH_STEPS = 64   # layer steps captured per CUDA graph (a 64-layer model's decode pass)
ATTN_TOL = 2e-3
LOG2E = 1.4426950408889634
# "c2s" is the C2 shape on a 1 GiB pool: small enough for multi-pass ncu captures.
C2_SMALL_POOL = W.DecodeConfig("c2_qwen3_32b_decode_smallpool", 32, 64, 8, 16384, 1024, 4096, seed=1002)
WORKLOADS = {"c1": W.C1, "c2": W.C2, "c2s": C2_SMALL_POOL, "c3": W.C3, "c4": W.C4, "c5": W.C5}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, as "workload bytes"
# lines written by the profiling pass
TRAFFIC_FILE = ROOT / "profiles" / "ncu_dram_traffic.txt"


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm": float(d["hbm_gbs"]), "tensor": float(d["bf16_tflops"]),
                    "tensor_sustained": d.get("bf16_tflops_sustained"), "kind": "measured"}
        except Exception:
            pass
    return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "kind": "fallback"}


def ncu_traffic(workload: str, world: int):
    if world != 1 or not TRAFFIC_FILE.exists():
        return None
    for line in TRAFFIC_FILE.read_text().splitlines():
        parts = line.split()
        if len(parts) >= 2 and parts[0] == workload:
            try:
                return float(parts[1])
            except ValueError:
                return None
    return None


# ------------------------------------------------------------------------------------------
# clocks: sampled with NVML while the GPU is busy
# ------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._active = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._period = period_s
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(self._period)

    def __enter__(self):
        self._active.set()
        return self

    def __exit__(self, *exc):
        self._active.clear()

    def close(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self, reset: bool = False):
        if not self.samples:
            out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        else:
            out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                   "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if reset:
            self.samples, self.reasons = [], set()
        return out


# ------------------------------------------------------------------------------------------
# configuration echo: identical in the GPU arm and the CPU arm
# ------------------------------------------------------------------------------------------
def workload_config(cfg):
    if isinstance(cfg, W.PrefillConfig):
        return {
            "workload": cfg.name, "batch": cfg.batch, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads,
            "head_dim": cfg.head_dim, "page_size": cfg.page_size, "num_pages": cfg.num_pages,
            "prompt_lengths": f"uniform[{cfg.prompt_lo},{cfg.prompt_hi}]",
            "shared_prefix_pages": f"0-{int(cfg.shared_frac_hi * 100)}% of each prompt",
            "step": "kv_append(suffix tokens) + paged causal prefill",
            "parallelism": "kv-head shards over the GPUs, no collective",
            "l2": "L2 flushed by the step itself: q + out + new K/V (>200 MB) stream through every step",
        }
    return {
        "workload": cfg.name, "batch": cfg.batch, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads,
        "head_dim": cfg.head_dim, "page_size": cfg.page_size, "num_pages": cfg.num_pages,
        "context_lengths": f"{cfg.len_dist}[{cfg.len_lo},{cfg.len_hi}]",
        "step": "kv_append(1 token/seq) + paged flash-decoding",
        "parallelism": ("request shards over the GPUs, no collective" if cfg.name.startswith("c3")
                        else "kv-head shards over the GPUs, no collective"),
        "l2": (f"inputs larger than L2: consecutive steps visit different layer pools round-robin, at least "
               f"2.5 x {L2_BYTES >> 20} MiB of K/V traffic before a byte repeats"),
    }


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's torch statement, on a bounded sample
# ------------------------------------------------------------------------------------------
def cpu_sample_case(cfg: W.DecodeConfig, n_seqs: int):
    """The first ``n_seqs`` sequences of the workload (same drawn lengths) in a compact pool."""
    lens = W.draw_lengths(cfg)[:n_seqs]
    pages = int(np.ceil(lens / cfg.page_size).sum())
    small = W.DecodeConfig(cfg.name + "_cpu_sample", len(lens), cfg.q_heads, cfg.kv_heads,
                           pages, cfg.len_lo, cfg.len_hi, cfg.len_dist, cfg.head_dim, cfg.page_size,
                           cfg.seed)
    return W.make_decode_case(small, device="cpu", fill="hash", lengths=lens)


def cpu_step(case) -> None:
    from oracle import paged_kv_oracle as O

    O.kv_append(case.new_kv, case.slots, case.pool)
    O.paged_decode(case.q, case.k_cache, case.v_cache, 1.0 / math.sqrt(case.cfg.head_dim),
                   case.token_table, case.seq_lens_t)


def step_bytes(case) -> int:
    """Algorithmic bytes of one step: decode traffic + the append's read, write and slots."""
    c = case.cfg
    append = c.batch * (2 * (2 * c.kv_heads * c.head_dim * 2) + 4)
    return case.algorithmic_bytes() + append


def cpu_decode_baseline(cfg, steps: int, warmup: int, budget_s: float):
    """Time the oracle's decode step on as many of the workload's first sequences as fit the
    budget.  Returns (seconds per sample step, GB/s, sequences used, steps, warm-ups)."""
    probe = cpu_sample_case(cfg, min(2, cfg.batch))
    cpu_step(probe)
    t0 = time.perf_counter()
    cpu_step(probe)
    per_seq = (time.perf_counter() - t0) / probe.cfg.batch
    n = int(max(1, min(cfg.batch, budget_s / max(per_seq, 1e-6) / max(steps + warmup, 1))))
    case = cpu_sample_case(cfg, n)
    for _ in range(warmup):
        cpu_step(case)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(case)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return dt, step_bytes(case) / dt / 1e9, n


def cpu_prefill_case(cfg: W.PrefillConfig, n_req: int):
    """The ``n_req`` shortest requests of the workload (same drawn lengths and prefix hits) in a
    compact pool."""
    lens, shared = W.draw_prefill_lengths(cfg)
    order = np.argsort(lens, kind="stable")[:n_req]
    pages = int(((lens[order] + cfg.page_size - 1) // cfg.page_size).sum())
    sub = W.PrefillConfig(cfg.name + "_cpu_sample", len(order), cfg.q_heads, cfg.kv_heads, pages,
                          cfg.prompt_lo, cfg.prompt_hi, cfg.shared_frac_hi, cfg.head_dim, cfg.page_size, cfg.seed)
    return W.make_prefill_case(sub, device="cpu", fill="hash", prompt_lens=lens[order], shared_pages=shared[order])


def cpu_prefill_step(case) -> None:
    from oracle import paged_kv_oracle as O

    kvh = case.cfg.kv_heads
    O.kv_append(case.new_kv, case.slots, case.pool)
    O.paged_attention(case.q, case.pool[:, :kvh], case.pool[:, kvh:], 1.0 / math.sqrt(case.cfg.head_dim),
                      case.token_table, case.req_ids, case.q_start, case.ctx_lens_t, case.q_lens_t)


def cpu_prefill_baseline(cfg, steps: int, warmup: int, budget_s: float):
    """Oracle prefill on the workload's shortest ``n`` requests that fit the budget.  Returns
    (seconds per sample step, TFLOP/s, requests used)."""
    probe = cpu_prefill_case(cfg, 1)
    t0 = time.perf_counter()
    cpu_prefill_step(probe)
    rate = probe.flops() / max(time.perf_counter() - t0, 1e-6)      # flop/s on the smallest request
    lens, shared = W.draw_prefill_lengths(cfg)
    order = np.argsort(lens, kind="stable")
    ctx = (shared[order] * cfg.page_size).astype(np.int64)
    q = lens[order].astype(np.int64) - ctx
    cum = np.cumsum(4 * cfg.head_dim * cfg.q_heads * (q * ctx + q * (q + 1) // 2))
    allowed = rate * budget_s / max(steps + warmup, 1)
    n = int(max(1, min(cfg.batch, np.searchsorted(cum, allowed, side="right"))))
    case = probe if n == 1 else cpu_prefill_case(cfg, n)
    for _ in range(warmup):
        cpu_prefill_step(case)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_prefill_step(case)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return dt, case.flops() / dt / 1e12, n


def run_reference(args, cfg_full):
    rank, _, world = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    if isinstance(cfg_full, W.PrefillConfig):
        dt, rate, n = cpu_prefill_baseline(cfg_full, steps, warmup, budget_s=150.0)
        metric, unit = PREFILL_METRIC, "TFLOP/s"
        sample = (f"the {n} shortest of {cfg_full.batch} requests, all {cfg_full.q_heads} Q heads, {steps} timed "
                  f"steps after {warmup} warm-up; value = sample flops / sample time")
    else:
        dt, rate, n = cpu_decode_baseline(cfg_full, steps, warmup, budget_s=150.0)
        metric, unit = METRIC, UNIT
        sample = (f"first {n} of {cfg_full.batch} sequences, all {cfg_full.q_heads} Q heads, {steps} timed "
                  f"steps after {warmup} warm-up; value = sample bytes / sample time")
    line = {
        "impl": "reference", "metric": metric, "value": rate, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * cfg_full.batch / n,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(cfg_full),
        "cpu_baseline": {"value": rate, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class Timer:
    """CUDA-graph capture + event timing on one stream, barrier + synchronize on both sides."""

    def __init__(self, stream, barrier):
        self.stream, self.barrier = stream, barrier

    def capture(self, fn, n):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            for i in range(n):
                fn(i)
        return g

    def run(self, fn, k, per_graph=GRAPH_STEPS):
        """Milliseconds for exactly k steps: graphs of up to per_graph consecutive steps."""
        full, rest = divmod(k, per_graph)
        g_full = self.capture(fn, per_graph) if full else None
        g_rest = self.capture(fn, rest) if rest else None
        for g in (g_full, g_rest):     # untimed replay: first-launch upload of the graph
            if g is not None:
                g.replay()
        self.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # A short device-side spin ahead of the start event: the host enqueues the graph launches
        # while it runs, so the events bracket K steps of device work and not the host's launch call.
        spin = getattr(torch.cuda, "_sleep", None)
        if spin is not None:
            with torch.cuda.stream(self.stream):
                spin(60_000)
        t0.record(self.stream)
        for _ in range(full):
            g_full.replay()
        if g_rest is not None:
            g_rest.replay()
        t1.record(self.stream)
        self.barrier()
        return t0.elapsed_time(t1)


def decode_check(case, pool, out, n_seqs=4):
    """Max-abs-error of a few sequences of a benchmarked output against the CPU oracle."""
    from oracle import paged_kv_oracle as O

    b_all = sorted({0, case.cfg.batch // 3, (2 * case.cfg.batch) // 3, case.cfg.batch - 1})[:n_seqs]
    kvh = case.cfg.kv_heads
    worst = 0.0
    for b in b_all:
        L = int(case.seq_lens[b])
        sl = case.token_table[b, :L].long()
        k, v = pool[:, :kvh][sl].cpu(), pool[:, kvh:][sl].cpu()
        want = O.paged_decode(case.q[b: b + 1].cpu(), k, v, 1.0 / math.sqrt(case.cfg.head_dim),
                              torch.arange(L, dtype=torch.int32)[None], torch.tensor([L]))
        worst = max(worst, float((out[b: b + 1].float().cpu() - want.float()).abs().max()))
    return {"max_abs_err": worst, "sequences": len(b_all), "tolerance": ATTN_TOL, "ok": worst <= ATTN_TOL,
            "against": "CPU oracle, on the output of the benchmarked step"}


def decode_bench(cfg, dev, steps, warmup, timer, prologue=False, with_e2e=True):
    """Device-time the decode step of one (sharded) configuration.  Returns a dict of figures."""
    from llama_lite_npu_b200 import kernels

    scale = 1.0 / math.sqrt(cfg.head_dim)
    kvh = cfg.kv_heads
    stream = timer.stream
    # One case gives tables, lengths, q and the new rows; the pool is replicated per "layer".
    case = W.make_decode_case(cfg, device=dev, fill="randn", fill_pool=False)
    bytes_step = step_bytes(case)
    layers = max(2, math.ceil(2.5 * L2_BYTES / bytes_step))
    pool_bytes = case.pool.numel() * 2
    free_b, _ = torch.cuda.mem_get_info()
    layers = max(1, min(layers, int(0.6 * free_b // pool_bytes)))
    pools = [case.pool] + [torch.empty_like(case.pool) for _ in range(layers - 1)]
    for i, p in enumerate(pools):
        g = torch.Generator(device=dev)
        g.manual_seed(cfg.seed * 977 + i)
        p.normal_(generator=g)
    out = torch.empty_like(case.q)
    torch.cuda.synchronize()     # the fills ran on the default stream; the steps run on the timer's own

    if prologue:
        # the step starts from the raw projections: QK-RMSNorm + rotary embedding + append, fused
        g = torch.Generator(device=dev)
        g.manual_seed(cfg.seed + 5)
        d = cfg.head_dim
        raw_q = torch.randn(case.q.shape, device=dev, dtype=torch.float16, generator=g)
        raw_kv = case.new_kv.reshape(case.new_kv.shape[0], -1)
        norm_w = (1 + 0.1 * torch.randn(2, d, device=dev, generator=g)).half()
        ang = torch.rand(case.q.shape[0], d // 2, device=dev, generator=g) * 6.283
        cos, sin = ang.cos().half(), ang.sin().half()

    def step(i):
        pool = pools[i % layers]
        if prologue:
            kernels.fused_qk_norm_rope_append(raw_q, raw_kv, norm_w[0], norm_w[1], 1e-6, cos, sin,
                                              case.slots, pool, out=case.q)
            kernels.flash_decoding(case.q, pool[:, :kvh], pool[:, kvh:], scale, case.block_table,
                                   case.seq_lens_t, case.max_len, table_kind="block", out=out)
        else:
            kernels.append_flash_decoding(case.new_kv, case.slots, pool, case.q, scale, case.block_table,
                                          case.seq_lens_t, case.max_len, table_kind="block", out=out)

    def decode_only(i):
        pool = pools[i % layers]
        kernels.flash_decoding(case.q, pool[:, :kvh], pool[:, kvh:], scale, case.block_table,
                               case.seq_lens_t, case.max_len, table_kind="block", out=out)

    res = {"case": case, "bytes_step": bytes_step, "alg_bytes": case.algorithmic_bytes(), "layers": layers,
           "launches_per_step": 2 if prologue else 1}
    with torch.cuda.stream(stream):
        for i in range(max(warmup, 3)):
            step(i)
        stream.synchronize()
        kernels.check_status(torch.device(dev).index)
        res["check"] = decode_check(case, pools[(max(warmup, 3) - 1) % layers], out)
        # ---- value: K graph-replayed steps, inputs resident in HBM ---------------------------
        res["ms_total"] = timer.run(step, steps)
        # ---- roofline: the decode kernel alone, same events -----------------------------------
        n_k = max(steps, GRAPH_STEPS)
        res["ms_kernel"] = timer.run(decode_only, n_k) / n_k
        if with_e2e:
            # ---- e2e: host buffers in, result out, every step ---------------------------------
            # The library's host-buffer form of the step (HostDecodeSteps): q, the new K/V rows,
            # slot_mapping and lengths sit in pinned staging and cross PCIe in one copy, the result
            # comes back in one copy, one library call per step.  Six slots in flight: step i+1's inputs
            # travel while step i computes, step i's result returns while step i+1 computes.
            # Every step makes both copies inside the timed region, and a slot is only reused
            # after the host has waited for its result.
            from llama_lite_npu_b200.host_step import HostDecodeSteps

            depth = 6
            batch = case.q.shape[0]
            hs = HostDecodeSteps(batch, cfg.q_heads, kvh, cfg.head_dim, depth=depth, device=torch.device(dev).index)
            bound = [hs.bind(p, case.block_table, qk_scale=scale, table_kind="block") for p in pools]
            new_kv_host = case.new_kv.cpu().numpy()
            for k in range(depth):
                buf = hs.buffers(k, batch)
                buf.q[...] = case.q.cpu().numpy()
                buf.new_k[...] = new_kv_host[:, :kvh]
                buf.new_v[...] = new_kv_host[:, kvh:]
                buf.seq_lens[...] = case.seq_lens_t.cpu().numpy()
                buf.slots[...] = case.slots.cpu().numpy()
            buf = hs.buffers(0, batch)
            res["h2d"] = sum(int(a.nbytes) for a in (buf.q, buf.new_k, buf.new_v, buf.seq_lens, buf.slots))
            res["d2h"] = int(buf.out.nbytes)
            hs_stream = hs.stream
            stream.synchronize()

            def e2e_run(n):
                for i in range(n):
                    k = i % depth
                    if i >= depth:
                        hs.wait(k)                     # the result of step i - depth is in host memory
                    hs.submit(k, batch, bound[i % layers], case.max_len)
                hs.flush()                             # the last step is not left waiting for a next submit
                for k in range(depth):
                    hs.wait(k)

            e2e_run(2 * depth)
            timer.barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record(hs_stream)
            e2e_run(steps)
            x1.record(hs_stream)                       # after the host has the last result
            x1.synchronize()
            timer.barrier()
            res["ms_e2e_total"] = x0.elapsed_time(x1)
            # the last step's result in host memory against the device-tensor path on the same pool
            got = torch.from_numpy(hs.buffers((steps - 1) % depth, batch).out.copy())
            step(steps - 1)
            stream.synchronize()
            res["e2e_check"] = float((got.float() - out.float().cpu()).abs().max())
            hs.close()
        kernels.check_status(torch.device(dev).index)
    del pools
    return res


def prefill_bench(cfg, dev, steps, warmup, timer, with_e2e=True):
    from llama_lite_npu_b200 import kernels
    from oracle import paged_kv_oracle as O

    kvh = cfg.kv_heads
    scale_log2 = LOG2E / math.sqrt(cfg.head_dim)
    case = W.make_prefill_case(cfg, device="cpu", fill="hash")
    host_q = case.q
    for name in ("pool", "block_table", "req_ids", "q_start", "ctx_lens_t", "q_lens_t", "q", "new_kv", "slots"):
        setattr(case, name, getattr(case, name).to(dev))
    stream = timer.stream
    torch.cuda.synchronize()     # inputs were copied on the default stream; the steps run on the timer's own

    def attend(_i=0):
        return kernels.paged_chunk_flash_attention(
            case.q, case.pool[:, :kvh], case.pool[:, kvh:], scale_log2, case.block_table, case.req_ids,
            case.q_start, case.ctx_lens_t, case.q_lens_t, case.max_q_len, table_kind="block")

    def step(_i=0):
        kernels.update_kv_buffer(case.new_kv, case.slots, case.pool)
        return attend()

    res = {"case": case, "flops": case.flops()}
    with torch.cuda.stream(stream):
        for _ in range(max(warmup, 3)):
            got = step()
        stream.synchronize()
        kernels.check_status(torch.device(dev).index)
        # check: the shortest request of the benchmarked output against the oracle
        r = int(np.argmin(case.prompt_lens))
        q0, qn, ctx = int(case.q_start[r]), int(case.q_lens[r]), int(case.ctx_lens[r])
        sl = case.token_table[r, : ctx + qn].long()
        pool_c = case.pool[sl.to(dev)].cpu()
        want = O.paged_attention(host_q[q0: q0 + qn], pool_c[:, :kvh], pool_c[:, kvh:], 1.0 / math.sqrt(cfg.head_dim),
                                 torch.arange(ctx + qn, dtype=torch.int32)[None], torch.zeros(1, dtype=torch.int32),
                                 torch.zeros(1, dtype=torch.int32), torch.tensor([ctx]), torch.tensor([qn]))
        err = float((got[q0: q0 + qn].float().cpu() - want.float()).abs().max())
        res["check"] = {"max_abs_err": err, "requests": 1, "tolerance": ATTN_TOL, "ok": err <= ATTN_TOL,
                        "against": "CPU oracle, shortest request of the benchmarked output"}
        res["ms_step"] = timer.run(step, steps, per_graph=1) / steps
        res["ms_kernel"] = timer.run(attend, steps, per_graph=1) / steps
        if with_e2e:
            h_q, h_kv = host_q.pin_memory(), case.new_kv.cpu().pin_memory()
            h_out = torch.empty_like(h_q).pin_memory()
            d_q, d_kv = torch.empty_like(case.q), torch.empty_like(case.new_kv)

            def e2e_step():
                d_q.copy_(h_q, non_blocking=True)
                d_kv.copy_(h_kv, non_blocking=True)
                kernels.update_kv_buffer(d_kv, case.slots, case.pool)
                o = kernels.paged_chunk_flash_attention(
                    d_q, case.pool[:, :kvh], case.pool[:, kvh:], scale_log2, case.block_table, case.req_ids,
                    case.q_start, case.ctx_lens_t, case.q_lens_t, case.max_q_len, table_kind="block")
                h_out.copy_(o, non_blocking=True)

            for _ in range(2):
                e2e_step()
            timer.barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_e2e = max(3, min(steps, 20))
            x0.record(stream)
            for _ in range(n_e2e):
                e2e_step()
            x1.record(stream)
            timer.barrier()
            res["ms_e2e"] = x0.elapsed_time(x1) / n_e2e
            res["h2d"], res["d2h"] = (h_q.numel() + h_kv.numel()) * 2, h_out.numel() * 2
        kernels.check_status(torch.device(dev).index)
    return res


def gpu_setup(args):
    from llama_lite_npu_b200 import _lib

    rank, local_rank, world = dist_env()
    if world != args.gpus and world != 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    _lib.lib()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    dist = None
    if world > 1:
        import torch.distributed as dist

        # The communication library announces its version on stdout when it starts; stdout
        # carries the JSON line only, so that banner goes to stderr.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device(dev))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    return rank, local_rank, world, dev, dist, barrier


def secondary_lines(dev, timer, sampler, peaks):
    """The other benchmark configurations at one GPU, a short device-timed run each."""
    out = {}
    for key, cfg in (("c3", W.C3), ("c5", W.C5)):
        sampler.summary(reset=True)
        with sampler:
            r = decode_bench(cfg, dev, 40, 3, timer, with_e2e=False)
        ach = r["alg_bytes"] / (r["ms_kernel"] * 1e-3) / 1e9
        out[key] = {"workload": cfg.name, "us": r["ms_kernel"] * 1e3, "us_per_step": r["ms_total"] / 40 * 1e3,
                    "achieved": ach, "unit": "GB/s", "frac": ach / peaks["hbm"], "bound": "hbm",
                    "bytes_per_launch": r["alg_bytes"], "num_pages": cfg.num_pages, "check": r["check"],
                    "clocks": sampler.summary(reset=True)}
        del r
        torch.cuda.empty_cache()
    with sampler:
        r = prefill_bench(W.C4, dev, 40, 3, timer, with_e2e=False)
    ach = r["flops"] / (r["ms_kernel"] * 1e-3) / 1e12
    out["c4"] = {"workload": W.C4.name, "us": r["ms_kernel"] * 1e3, "us_per_step": r["ms_step"] * 1e3,
                 "achieved": ach, "unit": "TFLOP/s", "frac": ach / peaks["tensor"], "bound": "tensor",
                 "flops_per_launch": r["flops"], "check": r["check"], "clocks": sampler.summary(reset=True)}
    del r
    torch.cuda.empty_cache()
    with sampler:
        out["append"] = append_bench(dev, timer, peaks)
    out["append"]["clocks"] = sampler.summary(reset=True)
    return out


def append_bench(dev, timer, peaks, tokens=65536, kv_heads=8, steps=20):
    """The stand-alone KV append at a prefill-sized token count (the decode step's one-token
    append rides in the decode launch): scatter `tokens` rows of 2*kv_heads*128 fp16 into a pool
    twice as large by a seeded permutation; two pools alternate so no launch finds its rows in L2."""
    from llama_lite_npu_b200 import kernels

    rows = 2 * kv_heads
    g = torch.Generator(device=dev)
    g.manual_seed(4242)
    src = torch.randn(tokens, rows, 128, device=dev, dtype=torch.float16, generator=g)
    slots = torch.randperm(2 * tokens, device=dev, generator=g)[:tokens].to(torch.int32)
    pools = [torch.zeros(2 * tokens, rows, 128, device=dev, dtype=torch.float16) for _ in range(2)]
    torch.cuda.synchronize()

    def step(i):
        kernels.update_kv_buffer(src, slots, pools[i % 2])

    with torch.cuda.stream(timer.stream):
        for i in range(3):
            step(i)
        timer.stream.synchronize()
        kernels.check_status(torch.device(dev).index)
        ms = timer.run(step, steps) / steps
        exact = all(bool(torch.equal(p[slots.long()], src)) for p in pools)
    nbytes = 2 * src.numel() * 2 + 4 * tokens
    ach = nbytes / (ms * 1e-3) / 1e9
    return {"workload": f"kv_append_{tokens}_tokens_{rows}x128_fp16", "us": ms * 1e3, "achieved": ach, "unit": "GB/s",
            "frac": ach / peaks["hbm"], "bound": "hbm", "bytes_per_launch": nbytes,
            "check": {"bit_exact": exact, "ok": exact, "against": "the rows gathered back from the pool"}}


def run_b200(args, cfg_full):
    rank, local_rank, world, dev, dist, barrier = gpu_setup(args)
    cfg, _ = W.shard_config(cfg_full, world, rank)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    timer = Timer(torch.cuda.Stream(), barrier)
    if sampler:
        sampler.__enter__()
    r = decode_bench(cfg, dev, args.steps, args.warmup, timer, prologue=args.prologue)
    if sampler:
        sampler.__exit__()
    clocks = sampler.summary(reset=True) if sampler else None

    times = torch.tensor([r["ms_total"], r["ms_e2e_total"], r["ms_kernel"]], dtype=torch.float64, device=dev)
    total_bytes = torch.tensor([float(r["bytes_step"])], dtype=torch.float64, device=dev)
    ok = torch.tensor([1.0 if r["check"]["ok"] else 0.0, r["check"]["max_abs_err"]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
        dist.all_reduce(ok, op=dist.ReduceOp.MAX)     # worst error over ranks (and "ok" of rank 0 kept below)
    ms_total, ms_e2e_total, ms_kernel = times.tolist()
    job_bytes = float(total_bytes.item())

    if rank == 0:
        peaks = measured_peaks()
        ms_step = ms_total / args.steps
        value = job_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = job_bytes / (ms_e2e_total / args.steps * 1e-3) / 1e9
        achieved = r["alg_bytes"] / (ms_kernel * 1e-3) / 1e9   # this rank's kernel
        check = dict(r["check"], max_abs_err=float(ok[1].item()), ok=float(ok[1].item()) <= ATTN_TOL)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": workload_config(cfg_full),
            "warmup_run": max(args.warmup, 3), "layer_pools": r["layers"],
            "timing": "CUDA events on the launching stream around exactly K graph-replayed steps, max over "
                      "ranks; a device-side spin precedes the start event so that the host's graph-launch call "
                      "is not inside the region",
            "bytes_per_step": job_bytes,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": achieved / peaks["hbm"], "peak_source": f"of {peaks['kind']}",
                "kernel": "paged_decode_kernel (split-KV walk + merge of the partials, one launch)",
                "us_per_launch": ms_kernel * 1e3, "bytes_per_launch": r["alg_bytes"],
                "traffic": ncu_traffic(cfg_full.name, world),
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": r["h2d"] * world,
                    "d2h_bytes_per_step": r["d2h"] * world, "us_per_step": ms_e2e_total / args.steps * 1e3,
                    "api": "HostDecodeSteps.submit / wait (b200kv_host_steps_*): pinned host buffers in and out, "
                           "6 slots in flight",
                    "max_abs_diff_vs_device_tensor_path": r["e2e_check"]},
            "gpu_launches": r["launches_per_step"] * args.steps,
            "check": check,
            "clocks": clocks,
        }
        if args.prologue:
            line["step_prologue"] = "fused QK-RMSNorm + rotary embedding + KV append, then paged decode"
        del r
        torch.cuda.empty_cache()
        if world == 1 and not args.no_secondary and cfg_full.name == W.C2.name:
            line["secondary"] = secondary_lines(dev, timer, sampler, peaks)
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            cdt, cgbs, n = cpu_decode_baseline(cfg_full, 2, 1, budget_s=15.0)
            line["cpu_baseline"] = {
                "value": cgbs, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"first {n} of {cfg_full.batch} sequences, all Q heads, 2 timed steps after 1 warm-up",
            }
        print(json.dumps(line))
    if sampler:
        sampler.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# Prefill workload (config C4): suffix KV append + packed causal prefill over paged KV
# ------------------------------------------------------------------------------------------
def run_prefill(args, cfg_full):
    rank, local_rank, world, dev, dist, barrier = gpu_setup(args)
    cfg = W.shard_kv_heads(cfg_full, world, rank) if world > 1 else cfg_full
    sampler = ClockSampler(local_rank) if rank == 0 else None
    timer = Timer(torch.cuda.Stream(), barrier)
    if sampler:
        sampler.__enter__()
    r = prefill_bench(cfg, dev, args.steps, args.warmup, timer)
    if sampler:
        sampler.__exit__()
    times = torch.tensor([r["ms_step"], r["ms_e2e"], r["ms_kernel"]], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(r["flops"])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_step, ms_e2e, ms_kernel = times.tolist()
    if rank == 0:
        peaks = measured_peaks()
        sustained = peaks["tensor_sustained"]
        achieved = r["flops"] / (ms_kernel * 1e-3) / 1e12
        line = {
            "metric": PREFILL_METRIC, "value": float(tot.item()) / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": workload_config(cfg_full),
            "total_query_tokens": int(r["case"].q_lens.sum()), "flops_per_step": float(tot.item()),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tensor"], "peak_source": f"of {peaks['kind']} (burst)",
                         "kernel": "paged_prefill_kernel", "us_per_launch": ms_kernel * 1e3,
                         "traffic": ncu_traffic(cfg_full.name, world),
                         # the timed region is seconds of back-to-back tensor work when --steps is
                         # large: the power-capped (sustained) cuBLAS figure is given beside the burst one
                         "peak_sustained": sustained,
                         "frac_of_sustained": (achieved / float(sustained)) if sustained else None},
            "e2e": {"value": float(tot.item()) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": r["h2d"] * world, "d2h_bytes_per_step": r["d2h"] * world},
            "gpu_launches": 2 * args.steps,
            "check": r["check"],
            "clocks": sampler.summary() if sampler else None,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            cdt, ctf, n = cpu_prefill_baseline(cfg_full, 1, 0, budget_s=25.0)
            line["cpu_baseline"] = {
                "value": ctf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"the {n} shortest of {cfg_full.batch} requests, all Q heads, one timed step",
            }
        print(json.dumps(line))
    if sampler:
        sampler.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_append(args):
    """``--workload append``: the stand-alone KV append alone (one GPU), for profiling it."""
    rank, local_rank, world, dev, dist, barrier = gpu_setup(args)
    timer = Timer(torch.cuda.Stream(), barrier)
    peaks = measured_peaks()
    with ClockSampler(local_rank) as sampler:
        line = append_bench(dev, timer, peaks, steps=max(args.steps, 1))
    line = {"metric": "kv_append_hbm_throughput", "value": line["achieved"], "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": line["us"] * 1e-3, "higher_is_better": True,
            "dtype": "f16", "data": "synthetic", "config": {"workload": line["workload"]},
            "roofline": {"bound": "hbm", "achieved": line["achieved"], "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": line["frac"], "peak_source": f"of {peaks['kind']}", "kernel": "kv_append_kernel",
                         "us_per_launch": line["us"], "bytes_per_launch": line["bytes_per_launch"],
                         "traffic": ncu_traffic(line["workload"], 1)},
            "gpu_launches": args.steps, "check": line["check"], "clocks": sampler.summary()}
    if rank == 0:
        print(json.dumps(line))
    sampler.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["append"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the short runs of the other configurations that a one-GPU c2 run appends")
    ap.add_argument("--prologue", action="store_true",
                    help="decode workloads: start each step from raw projections (fused QK-RMSNorm + "
                         "rotary embedding + KV append) instead of the append fused into the decode launch")
    args = ap.parse_args()
    if args.workload == "append":
        run_append(args)
        return
    cfg = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg)
    elif isinstance(cfg, W.PrefillConfig):
        run_prefill(args, cfg)
    else:
        run_b200(args, cfg)


if __name__ == "__main__":
    main()
