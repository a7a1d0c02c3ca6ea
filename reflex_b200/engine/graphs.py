"""Decode steps replayed as CUDA graphs.

A decode step is a fixed set of launches whose sizes depend only on the number
of sequences; positions, slots and tokens are read from device memory.  So one
graph per (batch size, context bucket) is captured at its first use and
replayed afterwards with new contents copied into the same descriptor buffer.
(The reference's attempt failed because positions were kernel arguments that
changed each step: docs/design/decode-speed.md:189-207.)

All graphs of an engine allocate from one memory pool: only one of them runs at
a time, so they share their intermediate buffers and a batch that shrinks
through many sizes does not grow the device memory with every size.  Their
results therefore live in shared storage too, and `run` hands out a copy unless
the caller asks to borrow the graph's own buffer.  Only the engine's very first
decode step runs eagerly (it sizes the lazily made buffers), and the first step
of a batch size above what the library's own products take (it lets the
vendor's product load its kernel for that shape); every other (size, bucket)
captures at its first use.  The engine keeps at most
`Engine.max_graphs` graphs and drops the least recently used.
"""

from __future__ import annotations

import torch

from .batch import layout, make_batch


class DecodeGraph:
    WARMUP = 1  # eager decode steps per engine before the first capture

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

    def run(self, tokens, slots, starts, want, tokens_dev=None, borrow: bool = False) -> torch.Tensor:
        """`tokens_dev` (int32 [n] on the device), when given, takes the place of
        the host `tokens`: it is copied over the descriptor's token field on the
        stream, after the descriptor itself.  The logits are a copy of the
        graph's result; with `borrow` they are the graph's own buffer, valid
        only until the engine's next step."""
        eng = self.engine
        batch = make_batch(tokens, slots, starts, want, eng.device, buffer=self.buffer, staging=eng.staging)
        if tokens_dev is not None:
            batch.tokens.copy_(tokens_dev)
        batch.context_hint = self.context_hint
        if self.graph is None:
            # the first decode steps of a batch size run eagerly: they size every
            # lazily allocated buffer; later graphs of that size capture at once
            from .. import ops

            # Beyond the rows the library's own products take, the step calls the
            # vendor's matrix product, which picks (and loads) a kernel per shape the
            # first time it sees it, and loading inside a capture invalidates it: such
            # a batch size runs eagerly once before it is captured.
            first_of_size = self.n > ops.GEMV_MAX_ROWS and self.n not in eng._eager_sizes
            if eng._eager_decodes < self.WARMUP or first_of_size:
                eng._eager_decodes += 1
                eng._eager_sizes.add(self.n)
                return eng.model.forward(batch, eng.cache)
            # capture: the eager call above has already sized every lazy buffer
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g, pool=eng.graph_pool()):
                self.logits = eng.model.forward(batch, eng.cache)
            self.kernels = ops.launch_count() - before  # this library's kernels in the graph
            self.graph = g
            # the captured launches point into the workspace as it is now: keep that
            # memory alive, whatever the workspace grows to later
            self.workspace_memory = eng.workspace.buffers() if eng.workspace is not None else None
        self.graph.replay()
        return self.logits if borrow else self.logits.clone()
