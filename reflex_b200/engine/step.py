"""The step function: the one way tokens go through the model.

`Engine.step(entries)` takes, for each sequence of the batch, its next tokens
(a whole prompt, a chunk of one, or a single decoded token) and the places
among them whose logits are wanted.  It runs exactly those tokens as one packed
batch against the cache that earlier steps left, writes their keys and values,
and returns float32 logits [wanted, vocab] that belong to the caller (a later
step never overwrites them; `borrow=True` spares the copy of a replayed decode
step's logits, which are then valid only until the next step).  There is no
padding: a row's result depends only on its own sequence.  The reference has the two special
cases, a whole-prompt prefill of one sequence and a one-token step
(src/model/dense.rs:1930-1985, src/model/decode_step.rs:139-329); batches and
mixed steps are this library's own.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.store import PAGE_TOKENS, Cache
from ..errors import CacheError, InvalidInput
from .batch import Staging, StepBatch, decode_context_bucket, make_batch
from .model import CausalLM
from ..ops.workspace import Workspace, use as use_workspace

StepEntry = Tuple[int, Sequence[int], Sequence[int]]  # (sequence, tokens, wanted places)


def ops_profile_on() -> bool:
    from .. import ops

    return ops.PROFILE


class Engine:
    lends_logits = True  # `step(..., borrow=True)` is understood

    def __init__(self, model: CausalLM, max_tokens: int, max_slots: Optional[int] = None,
                 use_graphs: bool = True, max_graphs: int = 48):
        self.model = model
        self.device = model.device
        self.cache = Cache(model.cache_entry_specs(), max_tokens, model.spec.max_positions,
                           model.dtype, model.device, max_slots=max_slots)
        self.vocab_size = model.spec.vocab_size
        # decode steps are captured into CUDA graphs when every part of the model
        # says that its launches may be (`CausalLM.capturable`) and the path is
        # the serving one; the 32-bit path always runs eagerly
        self.use_graphs = bool(use_graphs and model.dtype == torch.bfloat16 and model.capturable
                               and torch.device(self.device).type == "cuda")
        self.max_graphs = max(1, int(max_graphs))
        self._graphs: Dict[Tuple[int, int], "object"] = {}  # insertion order = least recently used first
        self._graph_pool = None
        self._eager_decodes = 0  # eager decode steps run so far
        self._eager_sizes: set = set()  # batch sizes that have run eagerly once
        self.steps_run = 0
        on_gpu = torch.device(self.device).type == "cuda"
        self.staging = Staging(self.device) if on_gpu else None
        # the steps' working memory: every op's result is a view into it, so a step
        # allocates nothing; it grows to what the largest step so far needed
        self.workspace = Workspace(self.device) if on_gpu else None

    # --- sequences ----------------------------------------------------------
    def open(self) -> int:
        """Start a sequence: takes a cache slot, returns its handle."""
        return self.cache.take_slot()

    def close(self, seq: int) -> None:
        """End a sequence: its slot and pages go back to the cache."""
        self.cache.give_slot(seq)

    def length(self, seq: int) -> int:
        return self.cache.length(seq)

    def check_errors(self) -> None:
        """Raises `CudaError` if a kernel of an earlier step gave up a bounded
        wait (its results are then not valid).  Synchronises: callers use it
        where they wait for the device anyway."""
        from .. import ops

        ops.check_device_errors(self.device)

    def graph_pool(self):
        """The one memory pool all of this engine's decode graphs allocate from."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    # --- the step -------------------------------------------------------------
    def _check(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise InvalidInput("a step needs at least one sequence")
        seen = set()
        V = self.vocab_size
        for seq, tokens, want in entries:
            if seq in seen:
                raise InvalidInput(f"sequence {seq} appears twice in one step")
            seen.add(seq)
            if len(tokens) == 0:
                raise InvalidInput(f"sequence {seq}: a step must bring at least one token")
            for t in tokens:
                if not (0 <= int(t) < V):
                    raise InvalidInput(f"sequence {seq}: token id {t} is outside the vocabulary [0, {V})")
            for w in want:
                if not (0 <= int(w) < len(tokens)):
                    raise InvalidInput(
                        f"sequence {seq}: wanted place {w} is outside this step's {len(tokens)} tokens")

    def step(self, entries: Sequence[StepEntry], borrow: bool = False) -> torch.Tensor:
        return self._run(entries, None, borrow)

    def _run(self, entries: Sequence[StepEntry], head=None, borrow: bool = False) -> torch.Tensor:
        """Checks, reserves cache, runs, commits.  `head(batch)`, when given, takes
        the place of the full-vocabulary logits."""
        self._check(entries)
        cache = self.cache
        slots = [int(e[0]) for e in entries]
        starts = [cache.length(s) for s in slots]
        tokens = [[int(t) for t in e[1]] for e in entries]
        want = [[int(w) for w in e[2]] for e in entries]
        growth = [(s, len(t)) for s, t in zip(slots, tokens)]
        before = [[g.end[s] for s in slots] for g in cache.kv_groups]
        cache.reserve(growth)
        saved_state = cache.snapshot_state(slots)
        try:
            n_want = sum(len(w) for w in want)
            # the captured step has one token and one wanted row, that token's, per sequence
            with use_workspace(self.workspace):
                if (head is None and self.use_graphs and all(len(t) == 1 for t in tokens)
                        and all(w == [0] for w in want)):
                    logits = self._decode_graphed(tokens, slots, starts, want, borrow=borrow)
                else:
                    batch = make_batch(tokens, slots, starts, want, self.device, staging=self.staging)
                    if head is not None:
                        logits = head(batch)
                    elif n_want:
                        logits = self.model.forward(batch, cache)
                    else:
                        self.model.hidden_states(batch, cache)
                        logits = torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            if self.workspace is not None:
                self.workspace.settle()
        except Exception:
            # the cache as it was: pages given back, fixed-size state put back
            for g, ends in zip(cache.kv_groups, before):
                for s, e in zip(slots, ends):
                    g.shrink_to(s, e)
            cache.restore_state(saved_state)
            raise
        cache.commit(growth)
        self.steps_run += 1
        if ops_profile_on():
            from .. import ops

            ops.prof_report(f"{self.steps_run - 1}:rows={sum(len(t) for t in tokens)}")
        return logits

    def step_scores(self, entries: Sequence[Tuple[int, Sequence[int], Sequence[int], Sequence[int]]]) -> torch.Tensor:
        """A step that returns, instead of whole rows of logits, the logit of one
        given token id at each wanted place: entries are (sequence, tokens,
        wanted places, ids), one id per place; float32 [wanted] comes back.
        The head's rows of those ids alone are read.  The ids need not be among
        the step's tokens (a continuation's last token is only ever scored), so
        they are checked here."""
        V = self.vocab_size
        for seq, _t, want, ids in entries:
            if len(ids) != len(want):
                raise InvalidInput(f"sequence {seq}: one token id per wanted place is needed")
            for t in ids:
                if not (0 <= int(t) < V):
                    raise InvalidInput(f"sequence {seq}: token id {t} is outside the vocabulary [0, {V})")
        flat = [int(t) for e in entries for t in e[3]]
        if not flat:
            raise InvalidInput("step_scores needs at least one wanted place")

        def head(batch):
            ids = torch.tensor(flat, dtype=torch.int32).to(self.device, non_blocking=True)
            return self.model.scores(batch, self.cache, ids)

        return self._run([(e[0], e[1], e[2]) for e in entries], head)

    def step_decode(self, seqs: Sequence[int], tokens_dev: torch.Tensor, borrow: bool = False) -> torch.Tensor:
        """One decode step whose tokens are already on the device: sequence
        `seqs[i]` goes on by token `tokens_dev[i]` (int32), and the logits of
        every row come back, float32 [len(seqs), vocab].  Nothing waits for the
        host, so a caller can enqueue the step while it is still reading the
        ids that feed it (the generation loop does).  The ids must be valid
        token ids: ids picked from this model's logits are (an id outside the
        vocabulary gives a zero embedding row and is reported by
        `check_errors`).  `borrow` as in `step`."""
        n = len(seqs)
        if n == 0:
            raise InvalidInput("a step needs at least one sequence")
        if len(set(int(s) for s in seqs)) != n:
            raise InvalidInput("a sequence appears twice in one step")
        if tokens_dev.dtype != torch.int32 or tokens_dev.numel() != n or not tokens_dev.is_cuda:
            raise InvalidInput(f"step_decode needs {n} int32 token ids on the device")
        cache = self.cache
        slots = [int(s) for s in seqs]
        starts = [cache.length(s) for s in slots]
        tokens = [[0]] * n  # placeholders: the token field is overwritten on the device
        want = [[0]] * n
        growth = [(s, 1) for s in slots]
        before = [[g.end[s] for s in slots] for g in cache.kv_groups]
        cache.reserve(growth)
        saved_state = cache.snapshot_state(slots)
        try:
            with use_workspace(self.workspace):
                if self.use_graphs:
                    logits = self._decode_graphed(tokens, slots, starts, want, tokens_dev=tokens_dev, borrow=borrow)
                else:
                    batch = make_batch(tokens, slots, starts, want, self.device, staging=self.staging)
                    batch.tokens.copy_(tokens_dev)
                    logits = self.model.forward(batch, cache)
            if self.workspace is not None:
                self.workspace.settle()
        except Exception:
            # the cache as it was: pages given back, fixed-size state put back
            for g, ends in zip(cache.kv_groups, before):
                for s, e in zip(slots, ends):
                    g.shrink_to(s, e)
            cache.restore_state(saved_state)
            raise
        cache.commit(growth)
        self.steps_run += 1
        return logits

    # --- decode steps as CUDA graphs -----------------------------------------
    def _decode_graphed(self, tokens, slots, starts, want, tokens_dev=None, borrow=False) -> torch.Tensor:
        from .graphs import DecodeGraph

        n = len(tokens)
        # the launch set depends on the batch size and, through the attention
        # kernel's key splits, on how long the longest context is: one graph per
        # (batch size, context bucket)
        bucket = decode_context_bucket(max(starts) + 1, PAGE_TOKENS)
        key = (n, bucket)
        g = self._graphs.pop(key, None)
        if g is None:
            g = DecodeGraph(self, n, bucket)
            while len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))  # the least recently used
        self._graphs[key] = g  # most recently used last
        return g.run(tokens, slots, starts, want, tokens_dev=tokens_dev, borrow=borrow)

    def launches_per_decode_step(self, n_seqs: int) -> int:
        """This library's kernels in one decode step of `n_seqs` sequences
        (counted when the step's graph was captured; 0 if it never ran)."""
        best = 0
        for (n, _bucket), g in self._graphs.items():
            if n == n_seqs:
                best = max(best, g.kernels)
        return best
