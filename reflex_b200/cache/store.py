"""The cache: a slot for each live sequence, keys and values for each caching
layer run, each sequence with its own length; and per-sequence state of fixed
size beside it.

Storage is grouped by need.  All cache entries whose mixers ask for the same
`KVSpec` share a *group*: one pool of pages of `PAGE_TOKENS` positions, one
page table [slots, pages-per-sequence], and tensors
K, V [entries, pages, kv heads, PAGE_TOKENS, head_dim], so a (page, head) tile
is one contiguous block.  A group with a window gives a sequence's pages back
as soon as no later query can see them.  Entries that ask for a `StateSpec`
share a state group, [entries, slots, *shape], zeroed when a slot is taken.
The reference allocates fresh flat K/V buffers per request
(src/model/dense.rs:1823-1845, src/model/kv_cache.rs:204-312) and keeps
fixed-size state per layer for its recurrent architectures
(src/model/hybrid.rs:131-140); slots, pages and groups are this library's own.

Slots are given back when a sequence ends and are used again without
clearing: a sequence never reads a position it has not written.

The size is given in tokens: `max_tokens` is the most tokens live sequences
hold at any time when each sequence's count is rounded up to `PAGE_TOKENS`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from ..errors import CacheError, ContextOverflow, InvalidInput, OutOfMemory
from .pool import IdPool
from .specs import KVSpec, StateSpec

PAGE_TOKENS = 64


@dataclass
class KVView:
    """What a kernel needs to read and write one cache entry."""

    k_pages: torch.Tensor  # [pages, kv heads, PAGE_TOKENS, head_dim]
    v_pages: torch.Tensor  # [pages, kv heads, PAGE_TOKENS, value_dim]
    page_table: torch.Tensor  # int32 [slots, pages per sequence]
    page_size: int
    spec: KVSpec


class KVGroup:
    def __init__(self, spec: KVSpec, entries: Sequence[int], n_pages: int, max_slots: int,
                 pages_per_seq: int, dtype: torch.dtype, device):
        self.spec = spec
        self.entries = list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.n_pages = n_pages
        self.pages_per_seq = pages_per_seq
        self.pool = IdPool(n_pages, "page")
        shape = (len(self.entries), n_pages, spec.n_kv_heads, PAGE_TOKENS, spec.head_dim)
        v_shape = shape[:-1] + (spec.value_dim,)
        self.device = device
        if device is not None:
            self.k = torch.empty(shape, dtype=dtype, device=device)
            self.v = torch.empty(v_shape, dtype=dtype, device=device)
            self.table_dev = torch.zeros((max_slots, pages_per_seq), dtype=torch.int32, device=device)
        else:  # bookkeeping only (host tests)
            self.k = self.v = self.table_dev = None
        # the host's copy of the page table; pinned beside a GPU so that `flush` can
        # copy from it without making the host wait for the device
        pin = device is not None and torch.device(device).type == "cuda"
        self.table_host = torch.zeros((max_slots, pages_per_seq), dtype=torch.int32, pin_memory=pin)
        # per slot: first page index still held, one past the last page index held
        self.first: Dict[int, int] = {}
        self.end: Dict[int, int] = {}
        self._dirty: Dict[int, Tuple[int, int]] = {}

    # --- bookkeeping --------------------------------------------------
    def open(self, slot: int) -> None:
        self.first[slot] = 0
        self.end[slot] = 0

    def pages_needed(self, slot: int, new_len: int) -> int:
        want_end = (new_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        return max(0, want_end - self.end[slot])

    def grow(self, slot: int, new_len: int) -> None:
        want_end = (new_len + PAGE_TOKENS - 1) // PAGE_TOKENS
        have = self.end[slot]
        if want_end <= have:
            return
        if want_end > self.pages_per_seq:
            raise ContextOverflow(new_len, self.pages_per_seq * PAGE_TOKENS)
        pages = self.pool.take(want_end - have)
        row = self.table_host[slot]
        for i, p in enumerate(pages):
            row[have + i] = p
        self.end[slot] = want_end
        lo, hi = self._dirty.get(slot, (have, want_end))
        self._dirty[slot] = (min(lo, have), max(hi, want_end))

    def shrink_to(self, slot: int, end_pages: int) -> None:
        """Undo a `grow` (a step that failed before it ran)."""
        have = self.end[slot]
        if end_pages >= have:
            return
        row = self.table_host[slot]
        self.pool.give(int(row[i]) for i in range(end_pages, have))
        self.end[slot] = end_pages

    def trim(self, slot: int, length: int) -> None:
        """Give back pages that no query at a position >= `length` can see."""
        w = self.spec.window
        if not w:
            return
        first_visible = max(0, length - w + 1)
        keep_from = min(first_visible // PAGE_TOKENS, self.end[slot])
        have = self.first[slot]
        if keep_from > have:
            row = self.table_host[slot]
            self.pool.give(int(row[i]) for i in range(have, keep_from))
            self.first[slot] = keep_from

    def close(self, slot: int) -> None:
        row = self.table_host[slot]
        self.pool.give(int(row[i]) for i in range(self.first[slot], self.end[slot]))
        del self.first[slot], self.end[slot]
        self._dirty.pop(slot, None)

    def flush(self) -> None:
        """Bring the device's page table up to date: one copy of the block of rows
        that holds every changed row, enqueued on the stream without waiting for
        the device.  The copy reads the pinned host table when the stream reaches
        it; an entry the host has changed again by then belongs to a position no
        kernel enqueued before the copy reads (a sequence's later pages, or a slot's
        next sequence, which starts only after its last step has come back), so
        the newer value does no harm."""
        if self.table_dev is not None and self._dirty:
            lo, hi = min(self._dirty), max(self._dirty) + 1
            self.table_dev[lo:hi].copy_(self.table_host[lo:hi], non_blocking=True)
        self._dirty.clear()

    def view(self, entry: int) -> KVView:
        i = self.index[entry]
        return KVView(self.k[i], self.v[i], self.table_dev, PAGE_TOKENS, self.spec)


class StateGroup:
    def __init__(self, spec: StateSpec, entries: Sequence[int], max_slots: int, device):
        self.spec = spec
        self.entries = list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        dtype = getattr(torch, spec.dtype)
        self.data = (
            torch.zeros((len(self.entries), max_slots) + tuple(spec.shape), dtype=dtype, device=device)
            if device is not None
            else None
        )

    def open(self, slot: int) -> None:
        if self.data is not None:
            self.data[:, slot].zero_()

    def view(self, entry: int) -> torch.Tensor:
        """[slots, *shape]; a mixer indexes it by a sequence's slot: on the host
        (`batch.slots`), or with the step's device-side indices
        (`batch.seq_slot`, `batch.row_slot`; `index_select` / `index_copy_`), which
        keeps its launches free of host values so that they can be captured."""
        return self.data[self.index[entry]]

    def snapshot(self, slots: Sequence[int]):
        """The state of the given slots, copied aside before a step runs: fixed-size
        state is overwritten in place and cannot be rewound any other way
        (src/model/mod.rs:1026-1030)."""
        if self.data is None:
            return None
        idx = torch.tensor(list(slots), dtype=torch.int64, device=self.data.device)
        return idx, self.data.index_select(1, idx)

    def restore(self, saved) -> None:
        if saved is not None:
            idx, data = saved
            self.data.index_copy_(1, idx, data)


class Cache:
    """`entry_specs`: cache entry id -> KVSpec | StateSpec | None."""

    def __init__(self, entry_specs: Dict[int, Union[KVSpec, StateSpec, None]], max_tokens: int,
                 max_positions: int, dtype: torch.dtype, device, max_slots: Optional[int] = None):
        if max_tokens <= 0:
            raise InvalidInput("max_tokens must be positive")
        n_pages = (max_tokens + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.max_tokens = n_pages * PAGE_TOKENS
        self.max_positions = max_positions
        self.max_slots = max_slots if max_slots is not None else n_pages
        if self.max_slots <= 0:
            raise InvalidInput("max_slots must be positive")
        pages_per_seq = min(n_pages, (max_positions + PAGE_TOKENS - 1) // PAGE_TOKENS)
        self.slots = IdPool(self.max_slots, "slot")
        self.lengths: Dict[int, int] = {}
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._where: Dict[int, Tuple[str, int]] = {}
        by_spec: Dict[Union[KVSpec, StateSpec], List[int]] = {}
        for entry in sorted(entry_specs):
            spec = entry_specs[entry]
            if spec is None:
                continue
            by_spec.setdefault(spec, []).append(entry)
        for spec, entries in by_spec.items():
            if isinstance(spec, KVSpec):
                g = KVGroup(spec, entries, n_pages, self.max_slots, pages_per_seq, dtype, device)
                for e in entries:
                    self._where[e] = ("kv", len(self.kv_groups))
                self.kv_groups.append(g)
            elif isinstance(spec, StateSpec):
                g = StateGroup(spec, entries, self.max_slots, device)
                for e in entries:
                    self._where[e] = ("state", len(self.state_groups))
                self.state_groups.append(g)
            else:
                raise InvalidInput(f"cache entry spec {spec!r} is neither KVSpec nor StateSpec")

    # --- slots ----------------------------------------------------------
    def take_slot(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for g in self.kv_groups:
            g.open(slot)
        for g in self.state_groups:
            g.open(slot)
        return slot

    def give_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheError(f"slot {slot} is not held (freed twice or never taken)")
        for g in self.kv_groups:
            g.close(slot)
        del self.lengths[slot]
        self.slots.give([slot])

    def length(self, slot: int) -> int:
        try:
            return self.lengths[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not held") from None

    # --- a step's side effects -------------------------------------------
    def reserve(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Make room for `n_new` more positions in each `(slot, n_new)`; all or
        nothing.  Does not change lengths."""
        need = [0] * len(self.kv_groups)
        for slot, n_new in growth:
            new_len = self.length(slot) + n_new
            if n_new <= 0:
                raise InvalidInput("a step must bring at least one token per sequence")
            if new_len > self.max_positions:
                raise ContextOverflow(new_len, self.max_positions)
            for gi, g in enumerate(self.kv_groups):
                if (new_len + PAGE_TOKENS - 1) // PAGE_TOKENS > g.pages_per_seq:
                    # within the model's positions, so it is the cache that is too small
                    raise OutOfMemory(
                        f"cache is out of pages: one sequence of {new_len} tokens needs more than "
                        f"the cache's {g.pages_per_seq * PAGE_TOKENS} tokens")
                need[gi] += g.pages_needed(slot, new_len)
        for gi, g in enumerate(self.kv_groups):
            if need[gi] > g.pool.free_count:
                raise OutOfMemory(
                    f"cache is out of pages: the step needs {need[gi]} more pages of "
                    f"{PAGE_TOKENS} tokens, {g.pool.free_count} of {g.n_pages} are free"
                )
        for slot, n_new in growth:
            for g in self.kv_groups:
                g.grow(slot, self.lengths[slot] + n_new)
        for g in self.kv_groups:
            g.flush()

    def snapshot_state(self, slots: Sequence[int]):
        """What `restore_state` needs to put the slots' fixed-size state back as it
        is now; None when the model keeps no such state (then nothing is copied)."""
        if not self.state_groups:
            return None
        return [g.snapshot(slots) for g in self.state_groups]

    def restore_state(self, saved) -> None:
        if saved is not None:
            for g, s in zip(self.state_groups, saved):
                g.restore(s)

    def commit(self, growth: Sequence[Tuple[int, int]]) -> None:
        for slot, n_new in growth:
            self.lengths[slot] += n_new
            for g in self.kv_groups:
                g.trim(slot, self.lengths[slot])

    # --- views ------------------------------------------------------------
    def kv(self, entry: int) -> KVView:
        kind, gi = self._where[entry]
        if kind != "kv":
            raise CacheError(f"cache entry {entry} holds state, not keys and values")
        return self.kv_groups[gi].view(entry)

    def state(self, entry: int) -> torch.Tensor:
        kind, gi = self._where[entry]
        if kind != "state":
            raise CacheError(f"cache entry {entry} holds keys and values, not state")
        return self.state_groups[gi].view(entry)

    def has(self, entry: int) -> Optional[str]:
        return self._where.get(entry, (None, 0))[0]

    def tokens_held(self) -> int:
        """Most pages any group holds, in tokens."""
        return max((g.pool.held_count for g in self.kv_groups), default=0) * PAGE_TOKENS
