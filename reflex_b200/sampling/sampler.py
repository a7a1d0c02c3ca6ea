"""Picking next tokens on the device from float32 logits [B, V]."""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .params import SamplingParams, fresh_seed, uniform


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
        self._greedy = {}  # batch size -> (ids, scratch) reused by every greedy pick

    def _constants(self, n: int):
        if n not in self._const:
            p = self.params
            t = torch.full((n,), float(p.temperature), dtype=torch.float32, device=self.device)
            k = torch.full((n,), int(p.top_k), dtype=torch.int32, device=self.device) if p.top_k else None
            tp = (torch.full((n,), float(p.top_p), dtype=torch.float32, device=self.device)
                  if p.top_p is not None else None)
            self._const[n] = (t, k, tp)
        return self._const[n]

    def pick(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int]) -> List[int]:
        """logits [n, V] for the given requests, each at its own step count;
        returns the chosen ids on the host."""
        n, V = logits.shape
        if self.params.is_greedy():
            if n not in self._greedy:
                self._greedy[n] = (torch.empty((n,), dtype=torch.int32, device=self.device),
                                   torch.empty((n * 128,), dtype=torch.float32, device=self.device))
            out, scratch = self._greedy[n]
            return ops.argmax(logits, out=out, scratch=scratch).tolist()
        u = torch.tensor([uniform(self.seed, r, s) for r, s in zip(requests, steps)],
                         dtype=torch.float32).to(self.device)
        t, k, tp = self._constants(n)
        if self._scratch is None or self._scratch.shape[0] < n or self._scratch.shape[1] != V:
            self._scratch = torch.empty((n, V), dtype=torch.float32, device=self.device)
        return ops.sample(logits, t, u, top_k=k, top_p=tp, scratch=self._scratch[:n]).tolist()
