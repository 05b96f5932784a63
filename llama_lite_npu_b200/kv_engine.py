"""CPU-side KV scheduling metadata: block refcounts, block-aligned prefix cache,
mixed-length prefill packing and chunk planning.

Same public types and behaviour as the reference's ``lite_llama/kv_engine.py``
(``PrefixCacheMatch`` :14, ``PrefillChunk`` :20, ``PackedPrefillRequest`` :30,
``PackedPrefillPlan`` :43, ``MixedLengthPrefillPacker`` :62-89,
``KVBlockRefCounter`` :92-147, ``PrefixCache`` :150-194,
``ChunkedPrefillPlanner`` :197-215).  These objects own no device memory.

The only difference is internal: free blocks sit in a min-heap (the reference
rescans every refcount per ``acquire`` / ``available_count``); ids still come out
lowest first, so results are identical call for call.
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import Iterable, Sequence


@dataclass(frozen=True)
class PrefixCacheMatch:
    matched_tokens: int
    block_ids: tuple[int, ...]


@dataclass(frozen=True)
class PrefillChunk:
    start: int
    end: int

    @property
    def length(self) -> int:
        return self.end - self.start


@dataclass(frozen=True)
class PackedPrefillRequest:
    """Where one request's tokens sit inside a packed (no-padding) prefill batch."""

    request_index: int
    start: int
    length: int

    @property
    def end(self) -> int:
        return self.start + self.length


@dataclass(frozen=True)
class PackedPrefillPlan:
    """Flattened tokens / positions of a mixed-length prefill plus per-request rows."""

    flat_token_ids: tuple[int, ...]
    flat_position_ids: tuple[int, ...]
    requests: tuple[PackedPrefillRequest, ...]

    @property
    def total_tokens(self) -> int:
        return len(self.flat_token_ids)

    @property
    def batch_size(self) -> int:
        return len(self.requests)

    @property
    def start_locs(self) -> tuple[int, ...]:
        """Packed start offset of every request (``b_start_loc`` of the attention kernels)."""
        return tuple(r.start for r in self.requests)

    @property
    def seq_lens(self) -> tuple[int, ...]:
        return tuple(r.length for r in self.requests)


class MixedLengthPrefillPacker:
    """Concatenate prompts of different lengths without padding."""

    def pack(self, prompt_token_ids: Sequence[Sequence[int]]) -> PackedPrefillPlan:
        tokens: list[int] = []
        positions: list[int] = []
        rows: list[PackedPrefillRequest] = []
        for index, prompt in enumerate(prompt_token_ids):
            ids = [int(t) for t in prompt]
            rows.append(PackedPrefillRequest(request_index=index, start=len(tokens), length=len(ids)))
            tokens += ids
            positions += range(len(ids))
        return PackedPrefillPlan(tuple(tokens), tuple(positions), tuple(rows))


class KVBlockRefCounter:
    """Reference counts of logical KV blocks; free blocks are handed out lowest id first."""

    def __init__(self, total_blocks: int) -> None:
        total_blocks = int(total_blocks)
        if total_blocks < 1:
            raise ValueError("total_blocks must be positive")
        self._refcounts = [0] * total_blocks
        self._free = list(range(total_blocks))  # min-heap of blocks with refcount 0

    @property
    def total_blocks(self) -> int:
        return len(self._refcounts)

    @property
    def available_count(self) -> int:
        return len(self._free)

    def refcount(self, block_id: int) -> int:
        return self._refcounts[self._check_block_id(block_id)]

    def acquire(self, count: int) -> tuple[int, ...]:
        count = int(count)
        if count < 1:
            raise ValueError("count must be positive")
        if count > len(self._free):
            raise RuntimeError(f"insufficient KV blocks: need {count}, available {len(self._free)}")
        blocks = tuple(heapq.heappop(self._free) for _ in range(count))
        for block_id in blocks:
            self._refcounts[block_id] = 1
        return blocks

    def add_ref(self, block_ids: Iterable[int]) -> None:
        for block_id in block_ids:
            checked = self._check_block_id(block_id)
            if self._refcounts[checked] == 0:
                raise ValueError(f"cannot add ref to free KV block {checked}")
            self._refcounts[checked] += 1

    def release(self, block_ids: Iterable[int]) -> None:
        for block_id in block_ids:
            checked = self._check_block_id(block_id)
            if self._refcounts[checked] == 0:
                raise ValueError(f"KV block {checked} refcount would become negative")
            self._refcounts[checked] -= 1
            if self._refcounts[checked] == 0:
                heapq.heappush(self._free, checked)

    def _check_block_id(self, block_id: int) -> int:
        block_id = int(block_id)
        if block_id < 0 or block_id >= len(self._refcounts):
            raise IndexError(f"KV block id out of range: {block_id}")
        return block_id


class PrefixCache:
    """Block-aligned prefix cache: token blocks -> logical KV block ids.

    Only full blocks are stored or matched, and matching stops at the first miss.
    As in the reference, a block is keyed by its own tokens alone, not by what
    precedes it; callers that need position-dependent reuse chain the keys themselves.
    """

    def __init__(self, block_size: int) -> None:
        block_size = int(block_size)
        if block_size < 1:
            raise ValueError("block_size must be positive")
        self.block_size = block_size
        self._block_to_id: dict[tuple[int, ...], int] = {}

    def _blocks(self, token_ids: Sequence[int]):
        size = self.block_size
        for index in range(len(token_ids) // size):
            yield index, tuple(int(t) for t in token_ids[index * size:(index + 1) * size])

    def put(self, token_ids: Sequence[int], block_ids: Sequence[int]) -> None:
        full = len(token_ids) // self.block_size
        if full == 0:
            return
        if len(block_ids) < full:
            raise ValueError("not enough block ids for full token blocks")
        for index, key in self._blocks(token_ids):
            self._block_to_id[key] = int(block_ids[index])

    def match(self, token_ids: Sequence[int]) -> PrefixCacheMatch:
        found: list[int] = []
        for _, key in self._blocks(token_ids):
            block_id = self._block_to_id.get(key)
            if block_id is None:
                break
            found.append(block_id)
        return PrefixCacheMatch(matched_tokens=len(found) * self.block_size, block_ids=tuple(found))


class ChunkedPrefillPlanner:
    """Cut a prompt into consecutive chunks of at most ``chunk_size`` tokens."""

    def __init__(self, chunk_size: int) -> None:
        chunk_size = int(chunk_size)
        if chunk_size < 1:
            raise ValueError("chunk_size must be positive")
        self.chunk_size = chunk_size

    def plan(self, prompt_length: int) -> tuple[PrefillChunk, ...]:
        prompt_length = int(prompt_length)
        if prompt_length < 0:
            raise ValueError("prompt_length must be non-negative")
        return tuple(
            PrefillChunk(start=s, end=min(s + self.chunk_size, prompt_length))
            for s in range(0, prompt_length, self.chunk_size)
        )
