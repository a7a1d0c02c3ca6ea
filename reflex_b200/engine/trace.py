"""Trace replay: given token ids fed through the engine step by step, logits
written out.  Nothing is sampled.  It drives the same model, step function,
cache and kernels that generation uses.

Input, one JSON object per line:
  {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: each request's next tokens and the places among them whose logits
are wanted; a request seen for the first time starts a sequence.  `end`:
requests finished after this step; their slots and pages go back to the cache.
For a step that wants something, `<out>/<step>.f32` holds the logits at the
wanted places in the order of the entries and of `want`, little-endian
float32 [wanted, vocab].  After every step a line `done <step>` is printed and
flushed.
"""

from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import torch

from ..errors import InvalidInput
from .step import Engine


class TraceRunner:
    def __init__(self, engine: Engine, out_dir: str):
        self.engine = engine
        self.out_dir = out_dir
        self.live: Dict[str, int] = {}
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, rec: dict) -> None:
        step = rec["step"]
        entries = rec.get("entries", [])
        step_entries = []
        opened = []
        try:
            for e in entries:
                rid = str(e["id"])
                if rid not in self.live:
                    self.live[rid] = self.engine.open()
                    opened.append(rid)
                step_entries.append((self.live[rid], e["tokens"], e.get("want", [])))
            if step_entries:
                logits = self.engine.step(step_entries)
                if logits.shape[0] > 0:
                    host = logits.detach().to("cpu", torch.float32).contiguous()
                    path = os.path.join(self.out_dir, f"{step}.f32")
                    with open(path, "wb") as f:
                        f.write(host.numpy().astype("<f4", copy=False).tobytes())
                self.engine.check_errors()
        except Exception:
            for rid in opened:
                self.engine.close(self.live.pop(rid))
            raise
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid not in self.live:
                raise InvalidInput(f"step {step}: request {rid!r} ends but is not live")
            self.engine.close(self.live.pop(rid))

    def run(self, lines: IO[str], out: IO[str] = sys.stdout) -> None:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            self.run_step(rec)
            out.write(f"done {rec['step']}\n")
            out.flush()
