"""Benchmark of the paged-KV decode step (KV append + paged flash-decoding).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c5|c1] [--impl reference]

A "step" is one decode step of one transformer layer over the whole batch: scatter the
step's new K/V rows into the page pool by slot_mapping, then attend every sequence's single
query token to its paged context.  The default workload is the Qwen3-32B shape (batch 32, 64
Q / 8 KV heads, head_dim 128, page_size 16, context lengths uniform in [1024, 4096], 65536-page
shuffled pool).  With N > 1 (launched by torchrun, one rank per GPU) the KV heads are sharded
over the ranks — same sequences, 8/N KV heads each — which needs no collective in the path;
torch.distributed is used only for the timing barrier and the max-over-ranks reduction.

Prints ONE JSON line (rank 0).  ``value`` is algorithmic HBM traffic of the whole job per
second with all inputs resident in HBM (CUDA-graph replay, device-timed); ``e2e`` is the
same metric through the Python operator API with the step's inputs copied from pinned host
memory and the result copied back inside the timed region.  ``--impl reference`` times the
CPU torch statement of the same path (the oracle port) on the host cores instead.
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
L2_BYTES = 126 * 1024 * 1024
GRAPH_STEPS = 64   # layer steps captured per CUDA graph (a 64-layer model's decode pass)
# "c2s" is the C2 shape on a 1 GiB pool: small enough for multi-pass ncu captures.
C2_SMALL_POOL = W.DecodeConfig("c2_qwen3_32b_decode_smallpool", 32, 64, 8, 16384, 1024, 4096, seed=1002)
WORKLOADS = {"c1": W.C1, "c2": W.C2, "c2s": C2_SMALL_POOL, "c3": W.C3, "c4": W.C4, "c5": W.C5}


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------
# clocks: sampled with NVML while the GPU is busy
# ------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index: int, period_s: float = 0.01):
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

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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


def time_cpu(case, steps: int, warmup: int):
    for _ in range(warmup):
        cpu_step(case)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(case)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return dt, step_bytes(case) / dt / 1e9


def step_bytes(case) -> int:
    """Algorithmic bytes of one step: decode traffic + the append's read, write and slots."""
    c = case.cfg
    append = c.batch * (2 * (2 * c.kv_heads * c.head_dim * 2) + 4)
    return case.algorithmic_bytes() + append


def cpu_sample_size(cfg) -> int:
    # sized for roughly 10-30 s of CPU work over the few repetitions made
    return {"c2_qwen3_32b_decode": 16, "c3_qwen3_30b_a3b_decode": 16, "c5_long_mixed_decode": 16}.get(
        cfg.name, cfg.batch)


def run_reference(args, cfg_full):
    rank, _, world = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    n = min(cfg_full.batch, cpu_sample_size(cfg_full))
    case = cpu_sample_case(cfg_full, n)
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    dt, gbs = time_cpu(case, steps, warmup)
    sample = (f"first {n} of {cfg_full.batch} sequences, all {cfg_full.q_heads} Q heads, "
              f"{steps} timed steps after {warmup} warm-up; value = sample bytes / sample time")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3 * cfg_full.batch / n,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": workload_config(cfg_full, args.gpus, None),
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(cfg, gpus, layers):
    d = {
        "workload": cfg.name, "batch": cfg.batch, "q_heads": cfg.q_heads, "kv_heads": cfg.kv_heads,
        "head_dim": cfg.head_dim, "page_size": cfg.page_size, "num_pages": cfg.num_pages,
        "context_lengths": f"{cfg.len_dist}[{cfg.len_lo},{cfg.len_hi}]",
        "step": "kv_append(1 token/seq) + paged flash-decoding",
        "parallelism": f"kv-head shards over {gpus} GPU(s), no collective",
    }
    if layers is not None:
        d["l2"] = (f"inputs larger than L2: {layers} layer pools visited round-robin, so no K/V byte "
                   f"is re-read within {L2_BYTES >> 20} MiB of traffic")
    return d


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_b200(args, cfg_full):
    from llama_lite_npu_b200 import _lib, kernels

    rank, local_rank, world = dist_env()
    if world != args.gpus and world != 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    _lib.lib()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg, parallelism = W.shard_config(cfg_full, world, rank)
    scale = 1.0 / math.sqrt(cfg.head_dim)
    kvh = cfg.kv_heads

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

    if args.prologue:
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
        if args.prologue:
            kernels.fused_qk_norm_rope_append(raw_q, raw_kv, norm_w[0], norm_w[1], 1e-6, cos, sin,
                                              case.slots, pool, out=case.q)
        else:
            kernels.update_kv_buffer(case.new_kv, case.slots, pool)
        return kernels.flash_decoding(case.q, pool[:, :kvh], pool[:, kvh:], scale, case.block_table,
                                      case.seq_lens_t, case.max_len, table_kind="block")

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i)
        stream.synchronize()
        kernels.check_status(local_rank)
        # A decode pass of a model is one CUDA graph holding every layer's step back to back, so
        # the timed region is graphs of up to GRAPH_STEPS consecutive steps (layer pools
        # visited round-robin), replayed until exactly K steps have run.
        def capture(fn, n):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(n):
                    fn(i)
            return g

        def plan(k):
            full, rest = divmod(k, GRAPH_STEPS)
            return full, rest

        def timed(fn, k):
            full, rest = plan(k)
            g_full = capture(fn, GRAPH_STEPS) if full else None
            g_rest = capture(fn, rest) if rest else None
            for g in (g_full, g_rest):     # untimed replay: first-launch upload of the graph
                if g is not None:
                    g.replay()
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(full):
                g_full.replay()
            if g_rest is not None:
                g_rest.replay()
            t1.record(stream)
            barrier()
            return t0.elapsed_time(t1)

        # ---- value: K graph-replayed steps, inputs resident in HBM ---------------------------
        if sampler:
            sampler.__enter__()
        ms_total = timed(step, args.steps)

        # ---- roofline: the decode kernels alone (split-KV kernel + its merge), same events ----
        out = torch.empty_like(case.q)

        def decode_only(i):
            pool = pools[i % layers]
            kernels.flash_decoding(case.q, pool[:, :kvh], pool[:, kvh:], scale, case.block_table,
                                   case.seq_lens_t, case.max_len, table_kind="block", out=out)

        n_k = max(args.steps, GRAPH_STEPS)
        ms_kernel = timed(decode_only, n_k) / n_k

        # ---- e2e: operator API, host inputs in, result out, every step -----------------------
        # The step's host inputs (q, the new K/V rows, slot_mapping, lengths) sit in ONE pinned
        # staging buffer and cross PCIe in one copy; the result comes back in one copy.
        parts = [("q", case.q), ("kv", case.new_kv), ("lens", case.seq_lens_t), ("slots", case.slots)]
        offs, cur = {}, 0
        for name, t in parts:
            cur = (cur + 15) // 16 * 16
            offs[name] = (cur, t.numel() * t.element_size())
            cur += t.numel() * t.element_size()
        h_in = torch.empty(cur, dtype=torch.uint8).pin_memory()
        d_in = torch.empty(cur, dtype=torch.uint8, device=dev)

        def view(buf, name, like):
            o, n = offs[name]
            return buf[o:o + n].view(like.dtype).view(like.shape)

        for name, t in parts:
            view(h_in, name, t).copy_(t.cpu())
        d_q, d_kv = view(d_in, "q", case.q), view(d_in, "kv", case.new_kv)
        d_lens, d_slots = view(d_in, "lens", case.seq_lens_t), view(d_in, "slots", case.slots)
        h_out = torch.empty(case.q.shape, dtype=case.q.dtype).pin_memory()
        h2d = cur
        d2h = h_out.numel() * h_out.element_size()

        def e2e_step(i):
            pool = pools[i % layers]
            d_in.copy_(h_in, non_blocking=True)
            kernels.update_kv_buffer(d_kv, d_slots, pool)
            o = kernels.flash_decoding(d_q, pool[:, :kvh], pool[:, kvh:], scale, case.block_table,
                                       d_lens, case.max_len, table_kind="block")
            h_out.copy_(o, non_blocking=True)

        for i in range(3):
            e2e_step(i)
        barrier()
        x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        x0.record(stream)
        for i in range(args.steps):
            e2e_step(i)
        x1.record(stream)
        barrier()
        ms_e2e_total = x0.elapsed_time(x1)
        if sampler:
            sampler.__exit__()
        kernels.check_status(local_rank)

    times = torch.tensor([ms_total, ms_e2e_total, ms_kernel], dtype=torch.float64, device=dev)
    total_bytes = torch.tensor([float(bytes_step)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total_bytes, op=dist.ReduceOp.SUM)
    ms_total, ms_e2e_total, ms_kernel = times.tolist()
    job_bytes = float(total_bytes.item())

    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_step = ms_total / args.steps
        value = job_bytes / (ms_step * 1e-3) / 1e9
        e2e_value = job_bytes / (ms_e2e_total / args.steps * 1e-3) / 1e9
        achieved = case.algorithmic_bytes() / (ms_kernel * 1e-3) / 1e9   # this rank's kernel
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "us_per_step": ms_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": dict(workload_config(cfg_full, world, layers), parallelism=parallelism,
                           **({"step_prologue": "fused QK-RMSNorm + rotary embedding + KV append"}
                              if args.prologue else {})),
            "bytes_per_step": job_bytes,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                "kernel": "paged_decode_split_kernel (+ decode_combine_kernel, timed together)",
                "us_per_launch": ms_kernel * 1e3, "bytes_per_launch": case.algorithmic_bytes(),
                "traffic": ncu_traffic(cfg_full.name, world),
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "us_per_step": ms_e2e_total / args.steps * 1e3},
            "gpu_launches": 3 * args.steps,
            "clocks": sampler.summary() if sampler else None,
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            n = min(cfg_full.batch, cpu_sample_size(cfg_full))
            cdt, cgbs = time_cpu(cpu_sample_case(cfg_full, n), 2, 1)
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


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel from
# the ncu captures summarised under profiles/.  The decode capture ran on the small-pool twin of
# the Qwen3-32B workload (identical sequences and lengths, so identical traffic).
NCU_TRAFFIC_BYTES = {
    "c2_qwen3_32b_decode": 345.7e6,
    "c2_qwen3_32b_decode_smallpool": 345.7e6,
}


def ncu_traffic(workload: str, world: int):
    return NCU_TRAFFIC_BYTES.get(workload) if world == 1 else None


# ------------------------------------------------------------------------------------------
# Prefill workload (config C4): suffix KV append + packed causal prefill over paged KV
# ------------------------------------------------------------------------------------------
def run_prefill(args, cfg_full):
    from llama_lite_npu_b200 import _lib, kernels

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    _lib.lib()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg = W.shard_kv_heads(cfg_full, world, rank) if world > 1 else cfg_full
    kvh = cfg.kv_heads
    scale_log2 = 1.4426950408889634 / math.sqrt(cfg.head_dim)
    case = W.make_prefill_case(cfg, device="cpu", fill="hash")
    for name in ("pool", "block_table", "req_ids", "q_start", "ctx_lens_t", "q_lens_t", "q", "new_kv", "slots"):
        setattr(case, name, getattr(case, name).to(dev))
    flops = case.flops()
    stream = torch.cuda.Stream()

    def attend():
        return kernels.paged_chunk_flash_attention(
            case.q, case.pool[:, :kvh], case.pool[:, kvh:], scale_log2, case.block_table, case.req_ids,
            case.q_start, case.ctx_lens_t, case.q_lens_t, case.max_q_len, table_kind="block")

    def step(_i=0):
        kernels.update_kv_buffer(case.new_kv, case.slots, case.pool)
        return attend()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        kernels.check_status(local_rank)

        def timed(fn, k):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            g.replay()
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(k):
                g.replay()
            t1.record(stream)
            barrier()
            return t0.elapsed_time(t1) / k

        if sampler:
            sampler.__enter__()
        ms_step = timed(step, args.steps)
        ms_kernel = timed(attend, args.steps)
        h_q, h_kv = case.q.cpu().pin_memory(), case.new_kv.cpu().pin_memory()
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
        barrier()
        x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 20))
        x0.record(stream)
        for _ in range(n_e2e):
            e2e_step()
        x1.record(stream)
        barrier()
        ms_e2e = x0.elapsed_time(x1) / n_e2e
        if sampler:
            sampler.__exit__()
        kernels.check_status(local_rank)

    times = torch.tensor([ms_step, ms_e2e, ms_kernel], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(flops)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms_step, ms_e2e, ms_kernel = times.tolist()
    if rank == 0:
        peak_file = ROOT / "MEASURED_PEAKS.json"
        peak, kind = 1590.0, "fallback"
        sustained = None
        if peak_file.exists():
            peaks = json.loads(peak_file.read_text())
            peak, kind = float(peaks["bf16_tflops"]), "measured (burst)"
            sustained = peaks.get("bf16_tflops_sustained")
        achieved = flops / (ms_kernel * 1e-3) / 1e12
        line = {
            "metric": "paged_prefill_tensor_throughput", "value": float(tot.item()) / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": cfg_full.name, "batch": cfg_full.batch, "q_heads": cfg_full.q_heads,
                       "kv_heads": cfg_full.kv_heads, "head_dim": 128, "page_size": 16,
                       "prompt_lengths": f"uniform[{cfg_full.prompt_lo},{cfg_full.prompt_hi}]",
                       "shared_prefix_pages": "0-50% of each prompt", "total_query_tokens": int(case.q_lens.sum()),
                       "step": "kv_append(suffix tokens) + paged causal prefill",
                       "l2": "L2 flushed by the step itself: q + out + new K/V (>200 MB) stream through every step"},
            "flops_per_step": float(tot.item()),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "peak_source": f"of {kind}",
                         "kernel": "paged_prefill_kernel", "us_per_launch": ms_kernel * 1e3, "traffic": None,
                         # the timed region is seconds of back-to-back tensor work when --steps is
                         # large: the power-capped (sustained) cuBLAS figure is given beside the burst one
                         "peak_sustained": sustained,
                         "frac_of_sustained": (achieved / float(sustained)) if sustained else None},
            "e2e": {"value": float(tot.item()) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (h_q.numel() + h_kv.numel()) * 2 * world,
                    "d2h_bytes_per_step": h_out.numel() * 2 * world},
            "gpu_launches": 2 * args.steps,
            "clocks": sampler.summary() if sampler else None,
        }
        print(json.dumps(line))
    if sampler:
        sampler.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prologue", action="store_true",
                    help="decode workloads: start each step from raw projections (fused QK-RMSNorm + "
                         "rotary embedding + KV append) instead of the plain KV append")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if isinstance(cfg, W.PrefillConfig):
        if args.impl == "reference":
            raise SystemExit("--impl reference times the decode workloads; see tests for the prefill oracle")
        run_prefill(args, cfg)
    elif args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_b200(args, cfg)


if __name__ == "__main__":
    main()
