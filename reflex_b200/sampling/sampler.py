"""Picking next tokens on the device from float32 logits [B, V]."""

from __future__ import annotations

import os
import sys
from typing import List, Optional, Sequence

import torch

from .. import ops
from .params import SamplingParams, fresh_seed, uniform


# Pick buffers (device ids, scratch, pinned host ids, event) by (device, batch
# size), kept for the life of the process: pinned allocations take milliseconds
# and synchronise the device, far too much for every generation call.
_RINGS: dict = {}


# `REFLEX_TOP2_TRACE=1`: a numerics probe that prints, to stderr, the two
# highest logits of every picked position (src/sampling.rs:166-191); comparing
# two runs' traces gives the margin a greedy choice had where they part.
TOP2_TRACE = os.environ.get("REFLEX_TOP2_TRACE", "") not in ("", "0")


def trace_top2(logits: torch.Tensor, requests: Sequence[int]) -> None:
    top = torch.topk(logits, 2, dim=1)
    for r, ids, vals in zip(requests, top.indices.tolist(), top.values.tolist()):
        print(f"REFLEX_TOP2 request={r} top1_id={ids[0]} top1_logit={vals[0]} top2_id={ids[1]} "
              f"top2_logit={vals[1]}", file=sys.stderr)


class PendingIds:
    """Ids picked on the device and on their way to the host: `dev` (int32 [n])
    can feed the next step at once; `wait()` gives the host list.  The device's
    error word travels with them, so reading a step's ids also tells whether a
    kernel up to that step reported an error, without a wait of its own."""

    def __init__(self, dev: torch.Tensor, host: torch.Tensor, event, err_host=None, err_dev=None):
        self.dev, self.host, self.event = dev, host, event
        self.err_host, self.err_dev = err_host, err_dev

    def wait(self) -> List[int]:
        self.event.synchronize()
        if self.err_host is not None:
            code = int(self.err_host[0])
            if code:
                from ..errors import CudaError

                self.err_dev.zero_()
                raise CudaError(f"a kernel reported an error (code {code}: a bounded wait that ran out, or a "
                                f"token id outside the vocabulary); the step's results are not valid")
        return self.host.tolist()


class Sampler:
    """One generation call's chooser: greedy argmax, or temperature / top-k /
    top-p with counter-based uniforms keyed by (seed, request, step)."""

    def __init__(self, params: SamplingParams, device):
        params.validate()
        self.params = params
        self.device = device
        self.seed = params.seed if params.seed is not None else fresh_seed()
        self._const = {}
        self._scratch = None
        self._work = None
        self._uniforms = {}

    def _constants(self, n: int):
        if n not in self._const:
            p = self.params
            t = torch.full((n,), float(p.temperature), dtype=torch.float32, device=self.device)
            k = torch.full((n,), int(p.top_k), dtype=torch.int32, device=self.device) if p.top_k else None
            tp = (torch.full((n,), float(p.top_p), dtype=torch.float32, device=self.device)
                  if p.top_p is not None else None)
            self._const[n] = (t, k, tp)
        return self._const[n]

    RING = 3  # picks in flight at most: the one being read and the one feeding the next step

    def _slot(self, n: int):
        """(ids on the device, argmax scratch, pinned host ids, event, pinned error word) for the
        next pick of n rows, from a small ring per batch size."""
        ring = _RINGS.setdefault((str(self.device), n), {"next": 0, "slots": [None] * self.RING})
        i = ring["next"]
        ring["next"] = (i + 1) % self.RING
        if ring["slots"][i] is None:
            ring["slots"][i] = (torch.empty((n,), dtype=torch.int32, device=self.device),
                                torch.empty((n * 128,), dtype=torch.float32, device=self.device),
                                torch.empty((n,), dtype=torch.int32, pin_memory=True),
                                torch.cuda.Event(),
                                torch.zeros((1,), dtype=torch.int32, pin_memory=True))
        return ring["slots"][i]

    def _upload_uniforms(self, values: List[float]) -> torch.Tensor:
        """The step's uniform numbers on the device, through pinned buffers that
        take turns (a pick may still be in flight when the next is prepared)."""
        n = len(values)
        ring = self._uniforms.setdefault(n, {"next": 0, "slots": [None] * self.RING})
        i = ring["next"]
        ring["next"] = (i + 1) % self.RING
        if ring["slots"][i] is None:
            ring["slots"][i] = (torch.empty((n,), dtype=torch.float32, pin_memory=True),
                                torch.empty((n,), dtype=torch.float32, device=self.device),
                                torch.cuda.Event())
        host, dev, copied = ring["slots"][i]
        copied.synchronize()  # the copy that last read this pinned buffer is done
        for j, v in enumerate(values):
            host[j] = v
        dev.copy_(host, non_blocking=True)
        copied.record()
        return dev

    def pick_async(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int]) -> PendingIds:
        """As `pick`, without waiting: the ids stay on the device for the next
        step and travel to the host behind an event."""
        n, V = logits.shape
        dev, scratch, host, event, err_host = self._slot(n)
        if TOP2_TRACE:
            trace_top2(logits, requests)
        if self.params.is_greedy():
            ops.argmax(logits, out=dev, scratch=scratch)
        else:
            u = self._upload_uniforms([uniform(self.seed, r, s) for r, s in zip(requests, steps)])
            t, k, tp = self._constants(n)
            if self._scratch is None or self._scratch.shape[0] < n or self._scratch.shape[1] != V:
                self._scratch = torch.empty((n, V), dtype=torch.float32, device=self.device)
                self._work = torch.empty((ops.sample_work_bytes(n, V),), dtype=torch.uint8, device=self.device)
            ops.sample(logits, t, u, top_k=k, top_p=tp, scratch=self._scratch[:n], out=dev, work=self._work)
        host.copy_(dev, non_blocking=True)
        err_dev = ops.device_error_word(self.device)
        err_host.copy_(err_dev, non_blocking=True)
        event.record()
        return PendingIds(dev, host, event, err_host, err_dev)

    def pick(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int]) -> List[int]:
        """logits [n, V] for the given requests, each at its own step count;
        returns the chosen ids on the host."""
        return self.pick_async(logits, requests, steps).wait()
