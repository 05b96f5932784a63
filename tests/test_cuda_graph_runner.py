"""Decode graph runner: control flow on CPU with a fake graph API (as the reference tests its
runner with a fake torch.npu), and real capture/replay of the paged decode step on the GPU."""

import math
from contextlib import contextmanager
from types import SimpleNamespace

import pytest
import torch

from llama_lite_npu_b200 import workloads as W
from llama_lite_npu_b200.cuda_graph import CudaGraphRunner
from llama_lite_npu_b200.executor import PagedKVExecutor


class FakeGraph:
    def __init__(self):
        self.replays = 0
        self.fn = None

    def replay(self):
        self.replays += 1
        self.fn()


class FakeApi:
    """Records the captured call and re-runs it on replay (what a graph does, minus the GPU)."""

    fail_next = False
    current = None

    @staticmethod
    def available():
        return True

    @staticmethod
    def new_graph():
        return FakeGraph()

    @staticmethod
    @contextmanager
    def capture(graph, pool):
        if FakeApi.fail_next:
            FakeApi.fail_next = False
            raise RuntimeError("capture refused")
        FakeApi.current = graph
        yield
        FakeApi.current = None

    @staticmethod
    def pool_handle():
        return object()

    @staticmethod
    def synchronize():
        pass


class FakeModel:
    """forward = lengths + select index, written into a persistent output when under capture."""

    def __init__(self):
        self.calls = 0

    def forward(self, input_ids, position_ids, info):
        self.calls += 1
        out = torch.empty(input_ids.shape[0], dtype=torch.float32)

        def run():
            out.copy_(info.b_seq_len.float() + info.cur_select_index.float() + input_ids[:, 0].float())

        run()
        if FakeApi.current is not None:
            FakeApi.current.fn = run
        return out


def _info(lens, slots):
    return SimpleNamespace(b_seq_len=torch.tensor(lens), cur_select_index=torch.tensor(slots, dtype=torch.int32),
                           b_req_idx=torch.arange(len(lens), dtype=torch.int32), max_actual_seq_len=max(lens))


def test_bucket_keys():
    assert CudaGraphRunner.sequence_bucket(1) == 128 and CudaGraphRunner.sequence_bucket(128) == 128
    assert CudaGraphRunner.sequence_bucket(129) == 256 and CudaGraphRunner.sequence_bucket(0) == 128
    r = CudaGraphRunner(FakeModel(), graph_api=FakeApi)
    assert r.graph_key(torch.zeros(4, 1), 300) == (4, 384)


def test_capture_once_per_bucket_and_replay_sees_new_metadata():
    model = FakeModel()
    r = CudaGraphRunner(model, "qwen3", graph_api=FakeApi)
    ids, pos = torch.tensor([[1], [2]]), torch.zeros(2, 1, dtype=torch.long)
    out = r(ids, pos, _info([100, 90], [5, 6]))
    assert out.tolist() == [106.0, 98.0] and (r.capture_count, r.replay_count, r.fallback_count) == (1, 1, 0)
    calls = model.calls
    out = r(torch.tensor([[3], [4]]), pos, _info([101, 91], [7, 8]))       # same bucket: replay only
    assert out.tolist() == [111.0, 103.0] and model.calls == calls and r.capture_count == 1
    r(ids, pos, _info([129, 91], [7, 8]))                                   # next bucket: new capture
    assert r.capture_count == 2 and r.captured


def test_failed_capture_falls_back_and_is_not_retried():
    model = FakeModel()
    r = CudaGraphRunner(model, graph_api=FakeApi)
    FakeApi.fail_next = True
    ids, pos = torch.tensor([[1]]), torch.zeros(1, 1, dtype=torch.long)
    out = r(ids, pos, _info([10], [3]))
    assert out.tolist() == [14.0] and (r.capture_count, r.fallback_count, r.capture_attempt_count) == (0, 1, 1)
    r(ids, pos, _info([11], [3]))
    assert r.capture_attempt_count == 1 and r.fallback_count == 2


def test_replay_copies_nothing_when_the_caller_passes_the_recorded_tensors():
    """Address-stable inputs are read in place: only tensors that moved are refreshed."""
    model = FakeModel()
    r = CudaGraphRunner(model, graph_api=FakeApi)
    ids, pos = torch.tensor([[1], [2]]), torch.zeros(2, 1, dtype=torch.long)
    info = _info([100, 90], [5, 6])
    r(ids, pos, info)                                   # records private copies, refreshes all five
    assert r.refresh_copy_count == 5
    rec = r._graphs[(2, 128)]
    # hand the runner its own recorded tensors back (what a pointer-stable executor amounts to)
    stable = SimpleNamespace(b_seq_len=rec.inputs["b_seq_len"], cur_select_index=rec.inputs["cur_select_index"],
                             b_req_idx=rec.inputs["b_req_idx"], max_actual_seq_len=100)
    stable.b_seq_len += 1                               # "the device advanced them in place"
    out = r(rec.inputs["input_ids"], rec.inputs["position_ids"], stable)
    assert out.tolist() == [107.0, 99.0] and r.refresh_copy_count == 5 and r.replay_count == 2
    stable.cur_select_index = torch.tensor([9, 9], dtype=torch.int32)     # one tensor moved: one copy
    out = r(rec.inputs["input_ids"], rec.inputs["position_ids"], stable)
    assert out.tolist() == [111.0, 102.0] and r.refresh_copy_count == 6


class FakePending:
    """Device half of a staged step: lengths + 1 on whatever info it is run on."""

    def __init__(self):
        self.runs = 0

    def run(self, info):
        self.runs += 1
        lens = info.b_seq_len

        def advance():
            lens.add_(1)

        if FakeApi.current is not None:      # under capture nothing executes: it is only recorded
            FakeApi.current.advance = advance
        else:
            advance()


class FakeGraphWithAdvance(FakeGraph):
    def replay(self):
        self.replays += 1
        if getattr(self, "advance", None) is not None:
            self.advance()
        self.fn()


def test_staged_step_is_advanced_exactly_once_by_the_graph_and_rebinds_on_a_new_batch():
    class Api(FakeApi):
        @staticmethod
        def new_graph():
            return FakeGraphWithAdvance()

    model = FakeModel()
    r = CudaGraphRunner(model, graph_api=Api)
    ids, pos = torch.tensor([[1], [2]]), torch.zeros(2, 1, dtype=torch.long)
    info = _info([100, 90], [5, 6])
    for step in range(3):
        info.pending_advance = FakePending()
        info.max_actual_seq_len += 1
        out = r(ids, pos, info)
        # lengths advanced once per step, on the live tensor, and the model saw the advanced value
        assert info.b_seq_len.tolist() == [101 + step, 91 + step]
        assert out.tolist() == [101.0 + step + 5 + 1, 91.0 + step + 6 + 2]
        assert info.pending_advance is None
    assert (r.capture_count, r.replay_count, r.fallback_count, r.refresh_copy_count) == (1, 3, 0, 0)
    # the batch changed: new metadata tensors -> the old graph is dropped and a new one recorded
    info2 = _info([50, 60], [1, 2])
    info2.pending_advance = FakePending()
    info2.max_actual_seq_len += 1
    out = r(ids, pos, info2)
    assert info2.b_seq_len.tolist() == [51, 61] and out.tolist() == [53.0, 65.0]
    assert (r.capture_count, r.rebind_count, r.refresh_copy_count) == (2, 1, 0)
    # a step that was advanced eagerly (nothing pending) cannot use the advancing graph
    info2.b_seq_len += 1
    out = r(ids, pos, info2)
    assert out.tolist() == [54.0, 66.0] and info2.b_seq_len.tolist() == [52, 62] and r.rebind_count == 2


def test_last_bucket_of_a_narrow_table_still_captures():
    """A table 1000 tokens wide: the 1024 bucket is recorded with the bound clamped to 1000."""
    seen = []

    class Model(FakeModel):
        def forward(self, input_ids, position_ids, info):
            if info.max_actual_seq_len > info.b_req_tokens_table.shape[1]:
                raise ValueError("max_actual_seq_len exceeds the table width")
            seen.append(info.max_actual_seq_len)
            return super().forward(input_ids, position_ids, info)

    r = CudaGraphRunner(Model(), graph_api=FakeApi)
    info = _info([990], [3])
    info.b_req_tokens_table = torch.zeros(4, 1000, dtype=torch.int32)
    ids, pos = torch.tensor([[1]]), torch.zeros(1, 1, dtype=torch.long)
    r(ids, pos, info)
    assert (r.capture_count, r.fallback_count) == (1, 0) and set(seen) == {1000}
    assert not r._failed_keys


@pytest.mark.gpu
@pytest.mark.parametrize("extend", ["extend_paged_requests", "extend_paged_requests_on_device",
                                    "stage_paged_decode_step"])
def test_paged_decode_step_replays_in_cuda_graph(extend, monkeypatch):
    """Two 'layers' of (append + paged decode) captured once, replayed over several steps while
    the requests keep growing.  Metadata comes from the host path (new tensors every step: the
    runner refreshes its recorded copies), from the device path run eagerly, or from a staged
    step whose device half is the graph's first node: then the graph reads the live tensors and
    the runner issues no copy at all between replays.  Every replay equals an eager
    twin driven through the host path."""
    dev, kvh, heads, layers = "cuda:0", 2, 16, 2
    twins = [PagedKVExecutor(layers, kvh, 128, 512, 8, 1024, page_size=16, device=dev) for _ in range(2)]
    for ex in twins:
        for li, buf in enumerate(ex.kv_mem_manager.gpu_kv_buffer):
            buf.copy_(W.hash_normal_fp16(5 + li, tuple(buf.shape), 1))
    ex, ref = twins
    ids = ex.reserve_paged_requests([37, 100, 64, 5])
    assert ref.reserve_paged_requests([37, 100, 64, 5]) == ids
    scale = 1.0 / math.sqrt(128)

    def model_on(executor):
        class Model:
            def forward(self, input_ids, position_ids, info):
                saved, executor.atten_info = executor.atten_info, info
                try:
                    x = xq
                    for layer in range(layers):
                        x = executor.token_forward(x, xk, xv, layer, scale)
                    return x
                finally:
                    executor.atten_info = saved
        return Model()

    runner = CudaGraphRunner(model_on(ex), "harness")
    eager = model_on(ref)
    xq = torch.empty(4, heads, 128, dtype=torch.float16, device=dev)      # static graph inputs
    xk = torch.empty(4, kvh, 128, dtype=torch.float16, device=dev)
    xv = torch.empty(4, kvh, 128, dtype=torch.float16, device=dev)
    inp = torch.zeros(4, 1, dtype=torch.long, device=dev)
    copies = {"n": 0}
    real_copy = torch.Tensor.copy_

    def counting_copy(self, *a, **k):
        copies["n"] += 1
        return real_copy(self, *a, **k)

    steady_copies = 0
    for step in range(20):                                   # every row crosses a page boundary
        getattr(ex, extend)(ids)
        ref.extend_paged_requests(ids)
        xq.copy_(W.hash_normal_fp16(50 + step, (4, heads, 128), 1))
        xk.copy_(W.hash_normal_fp16(50 + step, (4, kvh, 128), 2))
        xv.copy_(W.hash_normal_fp16(50 + step, (4, kvh, 128), 3))
        want = eager.forward(inp, inp, ref.atten_info).clone()
        copies["n"] = 0
        with monkeypatch.context() as m:
            m.setattr(torch.Tensor, "copy_", counting_copy)
            got = runner(inp, inp, ex.atten_info)
        if step >= 2:
            steady_copies += copies["n"]
        torch.cuda.synchronize()
        # the bucketed length bound may split the page line differently from the exact one
        assert float((got.float() - want.float()).abs().max()) <= 2e-3, step
        assert torch.equal(ex.atten_info.b_seq_len.cpu(), ref.atten_info.b_seq_len.cpu())
    for a, b in zip(ex.kv_mem_manager.gpu_kv_buffer, ref.kv_mem_manager.gpu_kv_buffer):
        assert torch.equal(a, b)
    assert (runner.replay_count, runner.fallback_count) == (20, 0)
    if extend != "stage_paged_decode_step":
        # recorded on private copies, as the reference does: ids, positions and the three metadata
        # tensors are refreshed before every replay
        assert runner.capture_count == 1 and steady_copies == 18 * 5 and runner.refresh_copy_count == 20 * 5
    else:
        # step 1: host path (activates the batch), graph without advance; step 2: first staged step,
        # that graph is replaced by one that advances; from then on no copy of any kind
        assert runner.capture_count == 2 and runner.rebind_count == 1 and steady_copies == 0
    from llama_lite_npu_b200 import kernels
    kernels.check_status(0)
