"""The description of one step's work, on the host and on the device.

Rows of all sequences are packed without padding: sequence s brings
`n_new[s]` tokens, which become rows `row0[s] .. row0[s] + n_new[s]` at
positions `start[s] ..`.  Every kernel reads a row's position and slot from
device arrays, so the same launch set serves any mix of lengths and a captured
graph can be replayed with new contents.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepBatch:
    # host side
    slots: List[int]
    starts: List[int]          # positions already in the cache per sequence
    new_counts: List[int]
    row0: List[int]            # first row of each sequence; len S + 1
    want_rows_host: List[int]  # packed row indices whose logits are wanted
    # device side (int32)
    tokens: torch.Tensor       # [R]
    row_pos: torch.Tensor      # [R]
    row_slot: torch.Tensor     # [R]
    seq_slot: torch.Tensor     # [S]
    seq_start: torch.Tensor    # [S]
    seq_new: torch.Tensor      # [S]
    seq_row0: torch.Tensor     # [S + 1]
    want_rows: torch.Tensor    # [n_want]
    # decode steps: the longest context rounded up to its bucket
    # (`decode_context_bucket`), so that kernels which size their launches by it
    # make the same choice in an eager step and in every replay of a captured one
    context_hint: Optional[int] = None

    @property
    def n_rows(self) -> int:
        return self.row0[-1]

    @property
    def n_seqs(self) -> int:
        return len(self.slots)

    @property
    def is_decode(self) -> bool:
        return all(n == 1 for n in self.new_counts)

    @property
    def max_new(self) -> int:
        return max(self.new_counts)

    @property
    def max_context(self) -> int:
        if self.context_hint is not None:
            return self.context_hint
        return max(s + n for s, n in zip(self.starts, self.new_counts))


def decode_context_bucket(max_context: int, page_tokens: int = 64) -> int:
    """The longest context of a decode step, rounded up to where its launch set
    may change: steps of 4 pages up to 32 pages, then powers of two."""
    pages = -(-max_context // page_tokens)
    bucket = -(-pages // 4) * 4 if pages <= 32 else 1 << (pages - 1).bit_length()
    return bucket * page_tokens


def layout(n_rows: int, n_seqs: int, n_want: int):
    """Offsets of the fields inside one int32 buffer."""
    o = {}
    p = 0
    for name, n in (("tokens", n_rows), ("row_pos", n_rows), ("row_slot", n_rows),
                    ("seq_slot", n_seqs), ("seq_start", n_seqs), ("seq_new", n_seqs),
                    ("seq_row0", n_seqs + 1), ("want_rows", n_want)):
        o[name] = (p, n)
        p += (n + 3) // 4 * 4  # 16-byte aligned fields
    return o, p


def pack_host(tokens: Sequence[Sequence[int]], slots: Sequence[int], starts: Sequence[int],
              want: Sequence[Sequence[int]]):
    """Flatten a step into the int32 words of `layout` (a NumPy array), plus the
    host lists.  Array operations throughout: a step's cost on the host does
    not grow with a Python loop over its rows."""
    S = len(tokens)
    counts = np.fromiter((len(t) for t in tokens), dtype=np.int64, count=S)
    row0 = np.zeros(S + 1, dtype=np.int64)
    np.cumsum(counts, out=row0[1:])
    R = int(row0[-1])
    starts_a = np.asarray(starts, dtype=np.int64)
    slots_a = np.asarray(slots, dtype=np.int64)
    if R == S:  # one token a sequence: the decode step
        flat = np.fromiter((t[0] for t in tokens), dtype=np.int64, count=S)
        row_pos, row_slot = starts_a, slots_a
    else:
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens])
        first = np.repeat(row0[:-1], counts)
        row_pos = np.repeat(starts_a, counts) + (np.arange(R, dtype=np.int64) - first)
        row_slot = np.repeat(slots_a, counts)
    want_rows = [int(row0[i]) + w for i, ws in enumerate(want) for w in ws]
    offs, total = layout(R, S, len(want_rows))
    words = np.zeros(total, dtype=np.int32)

    def put(name, values):
        p, n = offs[name]
        words[p:p + n] = values

    put("tokens", flat)
    put("row_pos", row_pos)
    put("row_slot", row_slot)
    put("seq_slot", slots_a)
    put("seq_start", starts_a)
    put("seq_new", counts)
    put("seq_row0", row0)
    put("want_rows", want_rows)
    return words, offs, counts.tolist(), row0.tolist(), want_rows


class Staging:
    """Pinned host memory for the steps' descriptors: a small ring of buffers,
    each with the event of the copy that last read it, so that a step never
    overwrites words a copy still in flight has to read."""

    def __init__(self, device, depth: int = 4):
        self.device = torch.device(device)
        self.depth = depth
        self.buffers: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.next = 0

    def copy(self, words, dev: torch.Tensor) -> None:
        """words -> pinned buffer -> `dev` (device int32, at least as long), on
        the current stream, without blocking the host."""
        i = self.next
        self.next = (i + 1) % self.depth
        if self.events[i] is not None:
            self.events[i].synchronize()
        n = len(words)
        if self.buffers[i] is None or self.buffers[i].numel() < n:
            self.buffers[i] = torch.empty((max(n, 256),), dtype=torch.int32, pin_memory=True)
        host = self.buffers[i][:n]
        host.copy_(torch.from_numpy(words))
        dev[:n].copy_(host, non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


def make_batch(tokens, slots, starts, want, device, buffer: Optional[torch.Tensor] = None,
               staging: Optional[Staging] = None) -> StepBatch:
    """Build the step's descriptors with one host-to-device copy (from pinned
    memory when a `staging` ring is given).  With `buffer` (a device int32
    tensor large enough) the words are copied into it, so a captured graph that
    reads the buffer sees the new step."""
    words, offs, new_counts, row0, want_rows = pack_host(tokens, slots, starts, want)
    if buffer is None:
        from ..ops.workspace import new

        dev = new((len(words),), torch.int32, device, keep=True)  # lives for the step
    else:
        dev = buffer[: len(words)]
    if staging is not None:
        staging.copy(words, dev)
    else:
        dev.copy_(torch.from_numpy(words))

    def f(name):
        p, n = offs[name]
        return dev[p:p + n]

    hint = None
    if all(n == 1 for n in new_counts):
        hint = decode_context_bucket(max(starts) + 1)
    return StepBatch(
        slots=list(slots), starts=list(starts), new_counts=new_counts, row0=row0,
        want_rows_host=want_rows, tokens=f("tokens"), row_pos=f("row_pos"), row_slot=f("row_slot"),
        seq_slot=f("seq_slot"), seq_start=f("seq_start"), seq_new=f("seq_new"),
        seq_row0=f("seq_row0"), want_rows=f("want_rows"), context_hint=hint)
