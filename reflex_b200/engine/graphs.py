"""Decode steps replayed as CUDA graphs.

A decode step is a fixed set of launches whose sizes depend only on the number
of sequences; positions, slots and tokens are read from device memory.  So one
graph per batch size is captured at its first use and replayed afterwards with
new contents copied into the same descriptor buffer.  (The reference's attempt
failed because positions were kernel arguments that changed each step:
docs/design/decode-speed.md:189-207.)
"""

from __future__ import annotations

import torch

from .batch import layout, make_batch


class DecodeGraph:
    WARMUP = 2

    def __init__(self, engine, n_seqs: int, context_hint: int):
        self.engine = engine
        self.n = n_seqs
        # kernels that size themselves by the longest context see this bucket's
        # upper end, so that the captured launches fit every step that uses it
        self.context_hint = context_hint
        _, total = layout(n_seqs, n_seqs, n_seqs)
        self.buffer = torch.zeros((total,), dtype=torch.int32, device=engine.device)
        self.graph = None
        self.logits = None
        self.calls = 0
        self.kernels = 0

    def run(self, tokens, slots, starts, want, tokens_dev=None) -> torch.Tensor:
        """`tokens_dev` (int32 [n] on the device), when given, takes the place of
        the host `tokens`: it is copied over the descriptor's token field on the
        stream, after the descriptor itself."""
        eng = self.engine
        batch = make_batch(tokens, slots, starts, want, eng.device, buffer=self.buffer, staging=eng.staging)
        if tokens_dev is not None:
            batch.tokens.copy_(tokens_dev)
        batch.context_hint = self.context_hint
        if self.graph is None:
            # the first decode steps of a batch size run eagerly: they size every
            # lazily allocated buffer; later graphs of that size capture at once
            done = eng._eager_decodes.get(self.n, 0)
            if done < self.WARMUP:
                eng._eager_decodes[self.n] = done + 1
                return eng.model.forward(batch, eng.cache)
            # capture: the eager call above has already sized every lazy buffer
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            from .. import ops

            before = ops.launch_count()
            with torch.cuda.graph(g):
                self.logits = eng.model.forward(batch, eng.cache)
            self.kernels = ops.launch_count() - before  # this library's kernels in the graph
            self.graph = g
        self.graph.replay()
        return self.logits
