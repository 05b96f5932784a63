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


@pytest.mark.gpu
@pytest.mark.parametrize("extend", ["extend_paged_requests", "extend_paged_requests_on_device"])
def test_paged_decode_step_replays_in_cuda_graph(extend):
    """Two 'layers' of (append + paged decode) captured once, replayed over several steps while
    the requests keep growing (metadata from the host, or advanced on the device); every replay
    equals the eager result."""
    dev, kvh, heads, layers = "cuda:0", 2, 16, 2
    ex = PagedKVExecutor(layers, kvh, 128, 512, 8, 1024, page_size=16, device=dev)
    for buf in ex.kv_mem_manager.gpu_kv_buffer:
        buf.copy_(W.hash_normal_fp16(5, tuple(buf.shape), 1))
    ids = ex.reserve_paged_requests([37, 100, 64, 5])
    scale = 1.0 / math.sqrt(128)

    class Model:
        def forward(self, input_ids, position_ids, info):
            saved, ex.atten_info = ex.atten_info, info
            try:
                x = xq
                for layer in range(layers):
                    x = ex.token_forward(x, xk, xv, layer, scale)
                return x
            finally:
                ex.atten_info = saved

    runner = CudaGraphRunner(Model(), "harness")
    eager = Model()
    xq = torch.empty(4, heads, 128, dtype=torch.float16, device=dev)      # static graph inputs
    xk = torch.empty(4, kvh, 128, dtype=torch.float16, device=dev)
    xv = torch.empty(4, kvh, 128, dtype=torch.float16, device=dev)
    inp = torch.zeros(4, 1, dtype=torch.long, device=dev)
    for step in range(20):                                   # every row crosses a page boundary
        getattr(ex, extend)(ids)
        xq.copy_(W.hash_normal_fp16(50 + step, (4, heads, 128), 1))
        xk.copy_(W.hash_normal_fp16(50 + step, (4, kvh, 128), 2))
        xv.copy_(W.hash_normal_fp16(50 + step, (4, kvh, 128), 3))
        want = eager.forward(inp, inp, ex.atten_info).clone()
        got = runner(inp, inp, ex.atten_info)
        torch.cuda.synchronize()
        # the bucketed length bound may split the page line differently from the exact one
        assert float((got.float() - want.float()).abs().max()) <= 2e-3, step
    assert (runner.capture_count, runner.replay_count, runner.fallback_count) == (1, 20, 0)
    from llama_lite_npu_b200 import kernels
    kernels.check_status(0)
