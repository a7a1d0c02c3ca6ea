"""Reading and writing safetensors files, by tensor name.

The file is an 8-byte little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` and the raw
little-endian tensor bytes; offsets count from the first byte after the header.
The reader maps the file and hands out one tensor at a time, so a model larger
than host memory's free part can still be uploaded; it plays the role the
reference's mmap'd GGUF reader has (src/gguf.rs:201-340).  A folder may hold one
`model.safetensors` or shards listed by `model.safetensors.index.json`.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

from ..errors import CheckpointError, IoError

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped file: `keys()`, `info(name) -> (dtype, shape)`, `tensor(name)`."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise IoError(f"{path}: cannot open: {e.strerror}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise CheckpointError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise CheckpointError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not valid JSON: {e}") from e
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.metadata = header.pop("__metadata__", {}) or {}
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, ent in header.items():
            try:
                dtype = _DTYPES[ent["dtype"]]
                shape = tuple(int(s) for s in ent["shape"])
                b, e = (int(x) for x in ent["data_offsets"])
            except (KeyError, TypeError, ValueError) as err:
                raise CheckpointError(
                    f"{path}: bad header entry for tensor {name!r}: {ent!r}"
                ) from err
            count = 1
            for s in shape:
                count *= s
            nbytes = count * torch.empty((), dtype=dtype).element_size()
            if e - b != nbytes or b < 0 or self._base + e > size:
                raise CheckpointError(
                    f"{path}: tensor {name!r} of shape {list(shape)} needs {nbytes} "
                    f"bytes but its offsets [{b}, {e}) give {e - b}"
                )
            self._entries[name] = (dtype, shape, b, e)

    def keys(self) -> List[str]:
        return list(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self._entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A host tensor that views the mapped bytes (read-only: copy or upload
        before writing to it)."""
        dtype, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dtype)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._base + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.from_numpy(raw)
        return t.view(dtype).reshape(shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass  # a tensor still views the map; the map dies with it
        self._f.close()


class Checkpoint:
    """All tensors of a model folder, whichever file holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
            except (OSError, KeyError, json.JSONDecodeError) as e:
                raise CheckpointError(f"{index}: unreadable shard index: {e}") from e
            for fname in sorted(set(weight_map.values())):
                self._files[fname] = SafetensorsFile(os.path.join(model_dir, fname))
            for fname, st in self._files.items():
                for k in st.keys():
                    self._where[k] = fname
        elif os.path.exists(single):
            st = SafetensorsFile(single)
            self._files["model.safetensors"] = st
            for k in st.keys():
                self._where[k] = "model.safetensors"
        else:
            raise IoError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found"
            )

    def keys(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        return self._files[self._where[name]].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write `(name, tensor)` pairs in the given order; tensors are taken one
    at a time so only one needs to be alive."""
    tensors = list(tensors)
    header: Dict[str, dict] = {}
    offset = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise CheckpointError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in tensors:
            c = t.detach().contiguous().cpu()
            if c.numel():
                f.write(c.reshape(-1).view(torch.uint8).numpy().tobytes())
