"""The generation loop above the step function.

Requests are taken in order, as many to a batch as the cache and the batch
limit allow.  A batch starts together: step 0 runs every prompt whole and
picks each request's first token from its last row; every later step feeds
each live request's last token.  A request ends when it has `max_new_tokens`
tokens or picks a stop token, which is kept (src/model/dense.rs:2036,
src/sampling.rs:120-125); it then leaves the batch, its slot goes back to the
cache, and the others go on unchanged.  When a batch is empty the next one
starts in the freed slots.  The reference runs one request at a time
(src/model/dense.rs:2002-2062); batching is this library's own.

The decisions are host logic over an object with `open/close/step` and a
`pick(logits, requests, steps)` function, so they can be tested without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.store import PAGE_TOKENS
from ..errors import ContextOverflow, InvalidInput


def _round_up(n: int) -> int:
    return (n + PAGE_TOKENS - 1) // PAGE_TOKENS * PAGE_TOKENS


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_tokens: int,
                 max_batch: int) -> List[List[int]]:
    """Request indices grouped into batches, in order: a batch takes requests
    while their worst-case token counts (prompt + max_new_tokens, each rounded
    up to a page) fit the cache and the batch limit."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lengths):
        need = _round_up(n + max_new_tokens)
        if need > max_tokens:
            raise ContextOverflow(n + max_new_tokens, max_tokens, "cache tokens")
        if cur and (used + need > max_tokens or len(cur) >= max_batch):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


@dataclass
class GenerationStats:
    prefill_tokens: int = 0
    decode_steps: int = 0
    decode_tokens: int = 0
    batches: int = 0


def generate(engine, prompts: Sequence[Sequence[int]], max_new_tokens: int,
             pick: Callable[[object, Sequence[int], Sequence[int]], List[int]],
             stop_token_ids: Sequence[int] = (), max_batch: int = 64,
             on_token: Optional[Callable[[int, int], None]] = None,
             stats: Optional[GenerationStats] = None,
             pick_async: Optional[Callable] = None) -> List[List[int]]:
    """Generated ids per prompt (the prompt itself is not repeated).

    With `pick_async` (a pick that leaves the ids on the device and hands back
    an object with `.dev` and `.wait()`) and an engine that has `step_decode`,
    the loop runs one step ahead of the host: see `_decode_ahead`."""
    if max_new_tokens < 1:
        raise InvalidInput("max_new_tokens must be at least 1")  # src/model/dense.rs:2011-2015
    if len(prompts) == 0:
        raise InvalidInput("generate needs at least one prompt")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise InvalidInput(f"prompt {i} is empty")  # "encode produced no tokens"
        limit = engine.cache.max_positions
        if len(p) + max_new_tokens > limit:
            raise ContextOverflow(len(p) + max_new_tokens, limit)
    stops = set(int(s) for s in stop_token_ids)
    stats = stats if stats is not None else GenerationStats()
    outputs: List[List[int]] = [[] for _ in prompts]
    max_batch = max(1, min(max_batch, engine.cache.max_slots))
    check_errors = getattr(engine, "check_errors", lambda: None)
    ahead = pick_async is not None and hasattr(engine, "step_decode")
    # the loop picks from a step's logits before it runs the next step, so it can
    # do without the copy that makes logits outlive later steps
    kw = {"borrow": True} if getattr(engine, "lends_logits", False) else {}
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, engine.cache.max_tokens, max_batch):
        stats.batches += 1
        live = list(batch)
        seqs = {}
        try:
            for i in live:  # inside the try: a slot taken before an open() fails is given back
                seqs[i] = engine.open()
            entries = [(seqs[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live]
            stats.prefill_tokens += sum(len(prompts[i]) for i in live)
            if ahead:
                _decode_ahead(engine, entries, live, seqs, outputs, max_new_tokens, stops, pick_async,
                              on_token, stats, check_errors, kw)
                continue
            first = True
            while live:
                logits = engine.step(entries, **kw)
                ids = pick(logits, live, [len(outputs[i]) for i in live])  # (the device's error word comes with them)
                if not first:
                    stats.decode_steps += 1
                    stats.decode_tokens += len(live)
                first = False
                still = []
                for i, tok in zip(live, ids):
                    tok = int(tok)
                    outputs[i].append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if len(outputs[i]) >= max_new_tokens or tok in stops:
                        engine.close(seqs.pop(i))
                    else:
                        still.append(i)
                live = still
                entries = [(seqs[i], [outputs[i][-1]], [0]) for i in live]
            check_errors()
        finally:
            for s in seqs.values():
                engine.close(s)
    return outputs


def _decode_ahead(engine, entries, live, seqs, outputs, max_new_tokens, stops, pick_async, on_token,
                  stats, check_errors, kw) -> None:
    """One batch, the device kept one step ahead of the host.

    The ids a step picks stay on the device and feed the next step at once; the
    host reads them, an event behind, while that next step already runs.  So
    when a request picks a stop token the host learns of it one step late: that
    step carried the request's row for nothing, its pick is dropped, and its
    slot is given back only after the step has finished with its pages.
    Requests that end by count are known in time and never ride along.  The
    tokens returned are the same as the loop that waits for every step gives."""
    logits = engine.step(entries, **kw)
    pending = pick_async(logits, live, [len(outputs[i]) for i in live])
    ended: set = set()  # picked a stop token; their row may still be in flight
    first = True
    while live:
        # who goes on, as far as the host knows: not ended, and not at its count
        # once the pending token has arrived
        goes_on = [i for i in live if i not in ended and len(outputs[i]) + 1 < max_new_tokens]
        next_pending = None
        if goes_on:
            if len(goes_on) == len(live):
                tokens_dev = pending.dev
            else:
                at = {i: r for r, i in enumerate(live)}
                tokens_dev = pending.dev[[at[i] for i in goes_on]]
            logits = engine.step_decode([seqs[i] for i in goes_on], tokens_dev, **kw)
            next_pending = pick_async(logits, goes_on, [len(outputs[i]) + 1 for i in goes_on])
        # the step that picked them is over: the rows it carried are free (the device's
        # error word comes with the ids: no wait of its own inside the loop)
        ids = pending.wait()
        if not first and any(i not in ended for i in live):
            stats.decode_steps += 1  # a step that carried only ended requests is not counted
        first = False
        for i, tok in zip(live, ids):
            if i in ended:  # rode along after its stop token: give the slot back now
                engine.close(seqs.pop(i))
                continue
            tok = int(tok)
            outputs[i].append(tok)
            stats.decode_tokens += 0 if len(outputs[i]) == 1 else 1
            if on_token is not None:
                on_token(i, tok)
            if len(outputs[i]) >= max_new_tokens or tok in stops:
                if i in goes_on:
                    ended.add(i)  # its row is in the step now running
                else:
                    engine.close(seqs.pop(i))
        live = goes_on
        pending = next_pending
    check_errors()
