"""Host-to-device upload of a checkpoint's tensors through pinned staging.

A checkpoint is memory-mapped; copying a mapped tensor straight to the device
is a pageable copy, which the driver stages through its own small buffer and
which blocks the host.  Here the host side is pipelined instead, as the
reference's loader does (src/model/loading.rs:1239-1378: pinned 64 MiB staging
buffers, a copy stream, reader threads): a few pinned buffers take turns; host
threads fill one from the mapping (which is what pages the file in) while the
copy engine drains another on its own stream.

Tensors keep their stored element type; the parts widen or narrow on the
device when they bind.  Each tensor gets its own device allocation: parts
re-lay some matrices when they bind (gate and up rows woven into one matrix)
and then drop the originals, which one arena for everything could not give
back.
"""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

import torch

STAGING_BYTES = 64 << 20
STAGING_BUFFERS = 3
READER_THREADS = 4


class Uploader:
    def __init__(self, device, staging_bytes: int = STAGING_BYTES, buffers: int = STAGING_BUFFERS,
                 threads: int = READER_THREADS):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("the uploader copies to a CUDA device")
        if staging_bytes < 1 or buffers < 2 or threads < 1:
            raise ValueError("staging_bytes >= 1, buffers >= 2, threads >= 1")
        self.staging_bytes = int(staging_bytes)
        self.pinned: List[torch.Tensor] = [
            torch.empty(self.staging_bytes, dtype=torch.uint8).pin_memory() for _ in range(buffers)]
        self.drained: List[Optional[torch.cuda.Event]] = [None] * buffers
        self.stream = torch.cuda.Stream(self.device)
        self.pool = ThreadPoolExecutor(max_workers=threads) if threads > 1 else None
        self.threads = threads
        self.turn = 0
        self.bytes_copied = 0

    def _fill(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        """Host copy of `src` into the pinned `dst`, cut among the reader threads."""
        n = src.numel()
        if self.pool is None or n < (4 << 20):
            dst.copy_(src)
            return
        step = (n + self.threads - 1) // self.threads
        step = (step + 4095) // 4096 * 4096
        jobs = [self.pool.submit(dst[o:o + step].copy_, src[o:o + step]) for o in range(0, n, step)]
        for j in jobs:
            j.result()

    def upload(self, host: torch.Tensor) -> torch.Tensor:
        """A device tensor of `host`'s shape and element type; the copy may still
        be in flight on the uploader's stream until `finish`."""
        out = torch.empty(host.shape, dtype=host.dtype, device=self.device)
        if host.numel() == 0:
            return out
        src = host.contiguous().reshape(-1).view(torch.uint8)
        dst = out.reshape(-1).view(torch.uint8)
        n = src.numel()
        # the allocation belongs to the current stream; the copies run on ours
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        for off in range(0, n, self.staging_bytes):
            m = min(self.staging_bytes, n - off)
            i = self.turn % len(self.pinned)
            self.turn += 1
            if self.drained[i] is not None:
                self.drained[i].synchronize()  # the buffer's last copy has left it
            stage = self.pinned[i][:m]
            self._fill(stage, src[off:off + m])
            with torch.cuda.stream(self.stream):
                dst[off:off + m].copy_(stage, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.drained[i] = ev
        self.bytes_copied += n
        return out

    def finish(self) -> None:
        """Every copy has landed, and the current stream may read the tensors."""
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        self.stream.synchronize()
        if self.pool is not None:
            self.pool.shutdown(wait=True)
            self.pool = None


def upload_all(tensors: Dict[str, torch.Tensor], device, **kw) -> Dict[str, torch.Tensor]:
    """Every tensor of `tensors` on `device`, element types kept."""
    up = Uploader(device, **kw)
    try:
        out = {name: up.upload(t) for name, t in tensors.items()}
    finally:
        up.finish()
    return out
