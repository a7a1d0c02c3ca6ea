"""The step's working memory: allocated once, handed out by bumping an offset.

Every kernel face in `ops` takes the memory for its result from `new()`.
Outside a step that is `torch.empty`; inside one (`with workspace.use(ws)`)
it is a view into the engine's `Workspace`, so a step allocates nothing: no
call into an allocator per op, which the reference removed from its decode
step for the same reason (src/model/decode_step.rs:60-115, ~390 allocations a
step before, docs/design/decode-speed.md:153-166).

A workspace has three regions.  `keep` holds what lives for the whole step
(the residual stream).  Two phase regions take turns, one per layer run: a run
starts by rewinding its own region, which frees what the run before the last
one made, while the other region still holds what the last run handed on (its
pending delta).  So the memory a step needs is that of two layers, not of all.

A region that is too small for a request hands out `torch.empty` memory for
the rest of the step and remembers how much would have been needed; `settle()`
(after the step, outside graph capture) then grows it.  A captured graph keeps
the buffers it was captured with alive, so growing never pulls memory from
under a replay.
"""

from __future__ import annotations

import contextlib
from typing import List, Optional

import torch

_ALIGN = 256
_ITEM = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.uint8: 1, torch.float16: 2,
         torch.int64: 8, torch.float64: 8}


class _Region:
    def __init__(self, device):
        self.device = device
        self.buf: Optional[torch.Tensor] = None
        self.offset = 0
        self.need = 0  # bytes this region would have needed so far (its high-water mark)

    def rewind(self) -> None:
        self.offset = 0

    def take(self, shape, dtype) -> Optional[torch.Tensor]:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * _ITEM[dtype]
        base = 0 if self.buf is None else self.buf.data_ptr() % _ALIGN  # results start on 256 bytes
        start = (self.offset + base + _ALIGN - 1) // _ALIGN * _ALIGN - base
        end = start + nbytes
        self.offset = end
        self.need = max(self.need, end)
        if self.buf is None or end > self.buf.numel():
            return None
        return self.buf[start:end].view(dtype).view(tuple(int(s) for s in shape))

    def settle(self) -> None:
        if self.need > (0 if self.buf is None else self.buf.numel()):
            self.buf = torch.empty((self.need * 5 // 4 + _ALIGN,), dtype=torch.uint8, device=self.device)


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self.keep = _Region(self.device)
        self.phases = [_Region(self.device), _Region(self.device)]
        self.phase = 0
        self.misses = 0  # requests served by torch.empty because a region was too small

    def begin_step(self) -> None:
        self.keep.rewind()
        for p in self.phases:
            p.rewind()
        self.phase = 0

    def next_phase(self) -> None:
        """A new layer run: its region is rewound (what the run before the last
        made is dead); the other still holds what the last run handed on."""
        self.phase ^= 1
        self.phases[self.phase].rewind()

    def take(self, shape, dtype, keep: bool = False) -> torch.Tensor:
        region = self.keep if keep else self.phases[self.phase]
        t = region.take(shape, dtype)
        if t is None:
            self.misses += 1
            t = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        return t

    def settle(self) -> None:
        """Grow the regions to what the steps so far needed (not during capture)."""
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return
        self.keep.settle()
        for p in self.phases:
            p.settle()

    def buffers(self) -> List[Optional[torch.Tensor]]:
        """The regions' current memory (a captured graph keeps a reference)."""
        return [self.keep.buf] + [p.buf for p in self.phases]

    @property
    def nbytes(self) -> int:
        return sum(0 if b is None else b.numel() for b in self.buffers())


_ACTIVE: Optional[Workspace] = None


@contextlib.contextmanager
def use(ws: Optional[Workspace]):
    """Results of `ops` calls inside the block come from `ws`."""
    global _ACTIVE
    prev = _ACTIVE
    _ACTIVE = ws
    if ws is not None:
        ws.begin_step()
    try:
        yield ws
    finally:
        _ACTIVE = prev


def active() -> Optional[Workspace]:
    return _ACTIVE


def next_phase() -> None:
    if _ACTIVE is not None:
        _ACTIVE.next_phase()


def new(shape, dtype, device, keep: bool = False, own: bool = False) -> torch.Tensor:
    """Uninitialised memory for a result.  `keep`: lives for the whole step.
    `own`: memory of its own that outlives the step (what a step returns)."""
    ws = _ACTIVE
    if own or ws is None or ws.device != torch.device(device):
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    return ws.take(shape, dtype, keep=keep)
