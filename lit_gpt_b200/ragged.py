"""What a step over several sequences is made of: the device-side description of its rows (``RaggedBatch``) and the allocator
of cache / state slots (``SlotAllocator``).  A step packs the new tokens of several sequences into one (n, d) matrix; each
sequence lives in one slot of every layer's cache or state and continues at its own position."""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Iterator, List, Optional, Sequence, Tuple

import torch


@dataclass
class RaggedBatch:
    """Device-side description of one step.  n rows (tokens) of S sequences."""

    row_pos: torch.Tensor            # int32 (n,)   position of each row in its sequence
    row_slot: torch.Tensor           # int32 (n,)   cache slot of each row
    cache_rows: torch.Tensor         # int64 (n,)   slot * max_seq + position: where the row's latent is stored
    decode: bool                     # every sequence brings exactly one row
    context_hint: int                # upper bound of any row's position + 1 (sizes the decode split)
    seqs: Optional[torch.Tensor] = None        # int32 (S, 4): first row, rows, first position, first row of its context in ctx_rows
    ctx_rows: Optional[torch.Tensor] = None    # int64 (m,)   cache rows of every sequence's whole context, sequence after sequence
    max_q_len: int = 1
    seq_state: Optional[torch.Tensor] = None   # int32 (S, 4): first row, rows, first position, state slot (models with per-slot states)
    row_seq: Optional[torch.Tensor] = None     # int32 (n,)   index of each row's sequence in seq_state
    identity_ctx: bool = False       # every sequence starts at position 0: the context rows ARE the step's rows, in order


def state_batch(seqs: Sequence[Tuple[int, int, int]], device: torch.device, extra: Sequence[int] = (),
                positions: bool = False) -> Tuple[RaggedBatch, torch.Tensor]:
    """The description of a step for models that keep a state per slot.  `seqs`: per sequence (state slot, position of its first
    new row, number of new rows), rows packed in this order.  One host-to-device copy carries the table, the row map, with
    `positions` every row's position, and `extra` (e.g. the step's token ids), which comes back as the second result."""
    meta: List[int] = []
    row_seq: List[int] = []
    row_pos: List[int] = []
    first = 0
    for i, (slot, start, length) in enumerate(seqs):
        meta.extend((first, length, start, slot))
        row_seq.extend([i] * length)
        if positions:
            row_pos.extend(range(start, start + length))
        first += length
    S = len(seqs)
    i32 = torch.tensor(meta + row_seq + row_pos + [int(v) for v in extra], dtype=torch.int32).to(device, non_blocking=True)
    rest = 4 * S + first + len(row_pos)
    batch = RaggedBatch(row_pos=i32[4 * S + first : rest] if positions else None, row_slot=None, cache_rows=None, decode=all(s[2] == 1 for s in seqs),
                        context_hint=max(s[1] + s[2] for s in seqs), max_q_len=max(s[2] for s in seqs),
                        seq_state=i32[: 4 * S].view(S, 4), row_seq=i32[4 * S : 4 * S + first], identity_ctx=all(s[1] == 0 for s in seqs))
    return batch, i32[rest:]


class SlotAllocator:
    """Hands out cache slots (rows of the latent caches) to live sequences; a released slot is reused, lowest first."""

    def __init__(self, slots: int) -> None:
        self.capacity = slots
        self._free = list(range(slots))

    def acquire(self) -> int:
        if not self._free:
            raise RuntimeError(f"all {self.capacity} cache slots are in use")
        self._free.sort()
        return self._free.pop(0)

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.capacity or slot in self._free:
            raise ValueError(f"slot {slot} is not in use")
        self._free.append(slot)

    @property
    def in_use(self) -> int:
        return self.capacity - len(self._free)


class SlotServed:
    """What the generation entry points and ``generate.serve.Session`` use of a model that keeps its sequences in slots: the
    sequence-length bound, dtype / device, the true-fp32 matrix-product mode, and the invalidation of captured decode graphs.
    The model provides ``embed`` (a parameter), ``config.block_size``, ``slots`` (a SlotAllocator or None),
    ``set_kv_cache`` / ``clear_kv_cache`` and ``state_tensors()`` (every per-slot buffer, slot first)."""

    supports_prefill_graph = False   # a prompt's extent is read on the host
    repeatable_steps = True          # running a step twice at the same position leaves the same cache (false for recurrent states)
    tp_world_size = 1

    @property
    def max_seq_length(self) -> int:
        return self._max_seq_length

    @max_seq_length.setter
    def max_seq_length(self, value: int) -> None:
        if value > self.config.block_size:
            raise ValueError(f"Cannot attend to {value}, block size is only {self.config.block_size}")
        self._max_seq_length = value

    @property
    def dtype(self) -> torch.dtype:
        return self.embed.dtype

    @property
    def device(self) -> torch.device:
        return self.embed.device

    def _drop_graphs(self) -> None:
        self.__dict__.pop("_decode_graphs", None)   # captured graphs pin the cache buffers
        self.__dict__.pop("_const", None)

    def fused_decode_ready(self, idx: Optional[torch.Tensor] = None) -> bool:
        """True when a decode step is made of capturable launches only (CUDA, caches set)."""
        if idx is not None and not idx.is_cuda:
            return False
        return self.embed.is_cuda and self.slots is not None and self.dtype in (torch.bfloat16, torch.float32)

    def spans_devices(self) -> bool:
        return False

    def graph_key(self):
        return (self.max_seq_length, tuple(t.data_ptr() for t in self.state_tensors()), self.embed.data_ptr(), self.head.data_ptr())

    @contextlib.contextmanager
    def _true_fp32(self) -> Iterator[None]:
        """fp32 models multiply in fp32: no TF32 inside the vendor GEMM, whatever the process-wide setting is."""
        if self.dtype != torch.float32:
            yield
            return
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            yield
        finally:
            torch.backends.cuda.matmul.allow_tf32 = old
