"""Decode steps in CUDA graphs, keyed by (batch, 128-token length bucket).

The calling contract is the reference's ``NpuGraphRunner``
(``lite_llama/executor/npu_graph.py:66-217``): ``runner(input_ids, position_ids, atten_info)``
returns the model's output for one decode step, from a graph when one exists for the batch size
and the bucket of ``atten_info.max_actual_seq_len``, capturing it on first use; a key whose
capture failed is remembered and runs eagerly from then on; ``capture_count`` /
``capture_attempt_count`` / ``replay_count`` / ``fallback_count`` mean what they mean there.

What is built differently here, around two things this package has and the reference lacks —
per-batch metadata tensors that keep their addresses, and a kernel that advances them on the
device:

* **Bound replay.**  A graph reads ``cur_select_index`` / ``b_seq_len`` / ``b_req_idx`` (and the
  input tensors) through whatever tensors it was recorded with.  The reference always records
  private copies and refreshes all five before every replay.  Here a replay first compares the
  caller's tensors with the recorded ones by address: identical ones are left alone, the others
  are refreshed with one ``copy_`` each (``refresh_copy_count`` counts them).  With the executor's
  device path the metadata never moves, so a steady replay copies nothing.
* **The advance is part of the graph.**  When the step was staged with
  ``PagedKVExecutor.stage_paged_decode_step`` the device half of the step (lengths + 1, new
  slots, token-table entries: one small kernel) is still pending in
  ``atten_info.pending_advance``; the runner records it as the graph's first node, directly on
  the live tensors.  A steady decode step is then: host page bookkeeping, one graph launch.  Such
  a graph is only valid for the tensors it advances; when the batch changes (new tensors) it is
  dropped and recorded again (``rebind_count``).
* The length bound recorded into the graph is the bucket, clamped to what the request table can
  hold, so the last bucket of a table whose width is not a multiple of 128 still captures.

The graph API is injectable (``graph_api``) so the control flow is testable without a GPU.
"""

from __future__ import annotations

import copy
import logging
from typing import Optional

import torch

logger = logging.getLogger(__name__)

_METADATA = ("cur_select_index", "b_seq_len", "b_req_idx")


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


def _same_memory(a: Optional[torch.Tensor], b: Optional[torch.Tensor]) -> bool:
    if a is None or b is None:
        return a is b
    return a is b or (a.data_ptr() == b.data_ptr() and a.shape == b.shape and a.dtype == b.dtype
                      and a.stride() == b.stride())


class _Recording:
    """One captured graph and the tensors it reads its per-step inputs from."""

    def __init__(self, graph, output, inputs: dict, advances: bool):
        self.graph = graph
        self.output = output
        self.inputs = inputs          # name -> tensor recorded into the graph (None: absent)
        self.advances = advances      # the graph's first node advances the metadata in place

    def reads(self, live: dict) -> bool:
        """True when every per-step tensor of the caller IS the recorded one."""
        return all(_same_memory(self.inputs[name], live[name]) for name in self.inputs)

    def refresh(self, live: dict) -> int:
        """Bring the recorded tensors up to date; returns the number of copies that took."""
        copies = 0
        for name, recorded in self.inputs.items():
            src = live[name]
            if recorded is None or src is None or _same_memory(recorded, src):
                continue
            recorded.copy_(src)
            copies += 1
        return copies


class CudaGraphRunner:
    """Cache and replay decode graphs using 128-token length buckets."""

    PARTITION_SIZE = 128

    def __init__(self, model, model_type: str = "unknown", graph_api=None):
        self.model = model
        self.model_type = model_type
        self._api = graph_api if graph_api is not None else _TorchCudaGraphs
        self._graphs: dict[tuple[int, int], _Recording] = {}
        self._failed_keys: set[tuple[int, int]] = set()
        self._retired: list[_Recording] = []
        self._pool = self._api.pool_handle() if self._api.available() else None
        self.capture_count = 0
        self.capture_attempt_count = 0
        self.replay_count = 0
        self.fallback_count = 0
        self.refresh_copy_count = 0   # copy_ calls made to refresh recorded inputs
        self.rebind_count = 0         # graphs dropped because their tensors were no longer the batch's

    # ------------------------------------------------------------------ contract
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

    # ------------------------------------------------------------------ pieces
    @staticmethod
    def _live(input_ids, position_ids, atten_info) -> dict:
        live = {"input_ids": input_ids, "position_ids": position_ids}
        for name in _METADATA:
            live[name] = getattr(atten_info, name, None)
        return live

    @staticmethod
    def _length_bound(atten_info, bucket: int) -> int:
        """The bucket, but never more than the request table can address."""
        widths = []
        table = getattr(atten_info, "b_req_tokens_table", None)
        if table is not None:
            widths.append(int(table.shape[1]))
        blocks = getattr(atten_info, "b_req_block_table", None)
        if blocks is not None:
            widths.append(int(blocks.shape[1]) * int(getattr(atten_info, "page_size", 16)))
        return min([bucket] + widths)

    @staticmethod
    def _take_pending(atten_info):
        return getattr(atten_info, "pending_advance", None)

    def _eager(self, input_ids, position_ids, atten_info):
        pending = self._take_pending(atten_info)
        if pending is not None:
            pending.run(atten_info)
            atten_info.pending_advance = None
        return self.model.forward(input_ids, position_ids, atten_info)

    # ------------------------------------------------------------------ capture
    def capture(self, input_ids, position_ids, atten_info) -> bool:
        """Record one graph for the current batch size and sequence bucket."""
        if not self.available:
            return False
        key = self.graph_key(input_ids, atten_info.max_actual_seq_len)
        if key in self._graphs:
            return True
        if key in self._failed_keys:
            return False
        self.capture_attempt_count += 1
        pending = self._take_pending(atten_info)
        try:
            bound = self._length_bound(atten_info, key[1])
            live = self._live(input_ids, position_ids, atten_info)
            # Private copies of the step's inputs: the rehearsal below runs on them, so that it can
            # size workspaces and load code without moving the live state (the pending advance, if
            # any, must happen exactly once on the live tensors: in the replay that follows).
            private = {name: (None if t is None else t.clone()) for name, t in live.items()}
            shadow = copy.copy(atten_info)
            for name in _METADATA:
                setattr(shadow, name, private[name])
            shadow.max_actual_seq_len = bound
            if pending is not None:
                pending.run(shadow)
            self.model.forward(private["input_ids"], private["position_ids"], shadow)
            self._api.synchronize()

            if pending is not None:
                # record on the live tensors themselves: the graph advances them in place
                recorded, view = live, copy.copy(atten_info)
                view.max_actual_seq_len = bound
            else:
                # record on the private copies (refreshed before each replay unless the caller
                # passes these very tensors); undo nothing: without an advance the rehearsal left
                # them as the caller's values
                recorded, view = private, shadow
            graph = self._api.new_graph()
            with self._api.capture(graph, self._pool):
                if pending is not None:
                    pending.run(view)
                output = self.model.forward(recorded["input_ids"], recorded["position_ids"], view)
            self._graphs[key] = _Recording(graph, output, recorded, advances=pending is not None)
            self.capture_count += 1
            logger.info("Captured CUDA decode graph for model=%s batch=%d bucket=%d%s", self.model_type, key[0],
                        key[1], " (advance recorded)" if pending is not None else "")
            return True
        except Exception as exc:  # a shape that cannot be captured must not be retried every token
            self._failed_keys.add(key)
            logger.warning("CUDA graph capture failed for model=%s batch=%d bucket=%d; using eager "
                           "execution: %s", self.model_type, key[0], key[1], exc)
            return False

    # ------------------------------------------------------------------ replay
    def _usable(self, key, recording: _Recording, live: dict, pending) -> bool:
        """A graph that advances can only serve the tensors it advances, and only a staged step;
        a graph that does not advance cannot serve a staged step."""
        if recording.advances:
            return pending is not None and recording.reads(live)
        return pending is None

    def replay(self, input_ids, position_ids, atten_info) -> Optional[torch.Tensor]:
        """Launch the graph of this step's key with its inputs in place; ``None`` if there is none
        (or the one there was belonged to another batch and has been dropped)."""
        key = self.graph_key(input_ids, atten_info.max_actual_seq_len)
        recording = self._graphs.get(key)
        if recording is None:
            return None
        live = self._live(input_ids, position_ids, atten_info)
        pending = self._take_pending(atten_info)
        if not self._usable(key, recording, live, pending):
            # retired, not destroyed: the graphs share one memory pool, which must not lose its
            # last user while further captures into it are to come
            self._retired.append(self._graphs.pop(key))
            self.rebind_count += 1
            return None
        self.refresh_copy_count += recording.refresh(live)
        recording.graph.replay()
        self.replay_count += 1
        if recording.advances:
            atten_info.pending_advance = None   # it ran as the graph's first node
        return recording.output

    def __call__(self, input_ids, position_ids, atten_info):
        if not self.available:
            self.fallback_count += 1
            return self._eager(input_ids, position_ids, atten_info)
        key = self.graph_key(input_ids, atten_info.max_actual_seq_len)
        for _ in range(2):      # second round: the graph found belonged to another batch
            if key not in self._graphs and key not in self._failed_keys:
                self.capture(input_ids, position_ids, atten_info)
            result = self.replay(input_ids, position_ids, atten_info)
            if result is not None:
                return result
            if key in self._failed_keys or key in self._graphs:
                break
        self.fallback_count += 1
        return self._eager(input_ids, position_ids, atten_info)
