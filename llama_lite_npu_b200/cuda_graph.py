"""Capture-and-replay of the decode step in CUDA graphs, keyed by (batch, length bucket).

Same contract as the reference's ``NpuGraphRunner``
(``lite_llama/executor/npu_graph.py:66-217``): ``runner(input_ids, position_ids, atten_info)``
replays a graph captured for the batch size and the 128-token bucket of
``atten_info.max_actual_seq_len`` after copying the step's dynamic metadata
(``cur_select_index``, ``b_seq_len``, ``b_req_idx``) into the tensors the graph was captured
with; a key whose capture failed is remembered and runs eagerly from then on; counters
``capture_count`` / ``replay_count`` / ``fallback_count`` have the same meaning.

Why the paged-KV operators of this package are capturable: lengths, slot_mapping and tables are
read on the device at replay time (no host sync), the split-KV workspace and the tables have
stable addresses, outputs come from the graph's private memory pool, and the bucketed
``max_actual_seq_len`` only sizes the launch.

The graph API is injectable (``graph_api``) so the control flow is testable without a GPU.
"""

from __future__ import annotations

import copy
import logging
from dataclasses import dataclass
from typing import Optional

import torch

logger = logging.getLogger(__name__)


class _TorchCudaGraphs:
    """The real backend: ``torch.cuda`` graphs."""

    @staticmethod
    def available() -> bool:
        return torch.cuda.is_available()

    @staticmethod
    def new_graph():
        return torch.cuda.CUDAGraph()

    @staticmethod
    def capture(graph, pool):
        return torch.cuda.graph(graph, pool=pool)

    @staticmethod
    def pool_handle():
        return torch.cuda.graph_pool_handle()

    @staticmethod
    def synchronize():
        torch.cuda.synchronize()


@dataclass
class _CapturedGraph:
    graph: object
    output: torch.Tensor
    input_ids: torch.Tensor
    position_ids: torch.Tensor
    cur_select_index: Optional[torch.Tensor]
    b_seq_len: Optional[torch.Tensor]
    b_req_idx: Optional[torch.Tensor]


class CudaGraphRunner:
    """Cache and replay decode graphs using 128-token length buckets."""

    PARTITION_SIZE = 128

    def __init__(self, model, model_type: str = "unknown", graph_api=None):
        self.model = model
        self.model_type = model_type
        self._api = graph_api if graph_api is not None else _TorchCudaGraphs
        self._graphs: dict[tuple[int, int], _CapturedGraph] = {}
        self._failed_keys: set[tuple[int, int]] = set()
        self._pool = self._api.pool_handle() if self._api.available() else None
        self.capture_count = 0
        self.capture_attempt_count = 0
        self.replay_count = 0
        self.fallback_count = 0

    @property
    def available(self) -> bool:
        return self._api.available()

    @property
    def captured(self) -> bool:
        return bool(self._graphs)

    @classmethod
    def sequence_bucket(cls, sequence_length: int) -> int:
        sequence_length = max(1, int(sequence_length))
        return -(-sequence_length // cls.PARTITION_SIZE) * cls.PARTITION_SIZE

    def graph_key(self, input_ids: torch.Tensor, sequence_length: int) -> tuple[int, int]:
        return input_ids.shape[0], self.sequence_bucket(sequence_length)

    def capture(self, input_ids, position_ids, atten_info) -> bool:
        """Capture one graph for the current batch size and sequence bucket."""
        if not self.available:
            return False
        key = self.graph_key(input_ids, atten_info.max_actual_seq_len)
        if key in self._graphs:
            return True
        if key in self._failed_keys:
            return False
        self.capture_attempt_count += 1
        try:
            # The live AttentionInfo is rewritten after every step, so the graph gets its own
            # copies of the per-step tensors and shares the pool and the request tables.
            ids, pos = input_ids.clone(), position_ids.clone()
            info = copy.copy(atten_info)
            info.cur_select_index = atten_info.cur_select_index.clone()
            info.b_seq_len = atten_info.b_seq_len.clone()
            req = getattr(atten_info, "b_req_idx", None)
            info.b_req_idx = req.clone() if req is not None else None
            info.max_actual_seq_len = key[1]
            _ = self.model.forward(ids, pos, info)          # warm-up: workspaces, attributes
            self._api.synchronize()
            graph = self._api.new_graph()
            with self._api.capture(graph, self._pool):
                out = self.model.forward(ids, pos, info)
            self._graphs[key] = _CapturedGraph(graph, out, ids, pos, info.cur_select_index,
                                               info.b_seq_len, info.b_req_idx)
            self.capture_count += 1
            logger.info("Captured CUDA decode graph for model=%s batch=%d bucket=%d", self.model_type, *key)
            return True
        except Exception as exc:  # a shape that cannot be captured must not be retried every token
            self._failed_keys.add(key)
            logger.warning("CUDA graph capture failed for model=%s batch=%d bucket=%d; using eager "
                           "execution: %s", self.model_type, key[0], key[1], exc)
            return False

    def replay(self, input_ids, position_ids, atten_info) -> Optional[torch.Tensor]:
        """Replay the captured bucket after refreshing its dynamic inputs; ``None`` if not captured."""
        captured = self._graphs.get(self.graph_key(input_ids, atten_info.max_actual_seq_len))
        if captured is None:
            return None
        captured.input_ids.copy_(input_ids)
        captured.position_ids.copy_(position_ids)
        if captured.cur_select_index is not None:
            captured.cur_select_index.copy_(atten_info.cur_select_index)
        if captured.b_seq_len is not None:
            captured.b_seq_len.copy_(atten_info.b_seq_len)
        if captured.b_req_idx is not None:
            captured.b_req_idx.copy_(atten_info.b_req_idx)
        captured.graph.replay()
        self.replay_count += 1
        return captured.output

    def __call__(self, input_ids, position_ids, atten_info):
        if not self.available:
            self.fallback_count += 1
            return self.model.forward(input_ids, position_ids, atten_info)
        key = self.graph_key(input_ids, atten_info.max_actual_seq_len)
        if key not in self._graphs and key not in self._failed_keys:
            self.capture(input_ids, position_ids, atten_info)
        result = self.replay(input_ids, position_ids, atten_info)
        if result is None:
            self.fallback_count += 1
            return self.model.forward(input_ids, position_ids, atten_info)
        return result
