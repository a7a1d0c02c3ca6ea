"""Ahead-of-time build of the CUDA kernels into one shared library.

Every `*.cu` beside this file is compiled by nvcc for sm_100a only
(`-gencode arch=compute_100a,code=sm_100a`) and linked into
`_build/libreflex_b200.so`; nothing is compiled by a JIT at run time, which is
the reference's rule for its kernels too (build.rs:1-21, src/aot.rs:61-105).
The library is rebuilt when a source or a flag changes (a stamp of their
hashes lies beside it).  The first call in a fresh checkout therefore compiles;
it prints a line per file and a heartbeat meanwhile.  Where the package folder
cannot be written, the build goes to `$REFLEX_B200_BUILD_DIR` or a per-user
folder under the system's temporary directory.
"""

from __future__ import annotations

import concurrent.futures
import fcntl
import glob
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libreflex_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _log(msg: str) -> None:
    print(f"[reflex_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (
        os.environ.get("REFLEX_B200_NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise RuntimeError(
        "nvcc not found (looked at $REFLEX_B200_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
        "the kernels cannot be built"
    )


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def _headers() -> List[str]:
    return sorted(glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "*.h")))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("REFLEX_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(HERE, "_build")
    if _writable_dir(local):
        return local
    fallback = os.path.join(tempfile.gettempdir(), f"reflex_b200_build_{os.getuid()}")
    os.makedirs(fallback, exist_ok=True)
    return fallback


def _up_to_date(bdir: str, digest: str) -> bool:
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "stamp.json")
    if not (os.path.exists(lib) and os.path.exists(stamp)):
        return False
    try:
        with open(stamp) as f:
            return json.load(f).get("digest") == digest
    except (OSError, ValueError):
        return False


def ensure_built(force: bool = False, verbose: Optional[bool] = None) -> str:
    """Build if needed; return the path of the shared library."""
    digest = _digest()
    # a library shipped beside the sources (built earlier in this tree) wins
    local = os.path.join(HERE, "_build")
    if not force and not os.environ.get("REFLEX_B200_BUILD_DIR") and _up_to_date(local, digest):
        return os.path.join(local, LIB_NAME)
    bdir = build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    if not force and _up_to_date(bdir, digest):
        return lib
    lock_path = os.path.join(bdir, ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and _up_to_date(bdir, digest):
                return lib
            _compile_all(bdir, lib, digest)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def _compile_all(bdir: str, lib: str, digest: str) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    _log(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {bdir}")
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            _log(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    objs = []

    def one(src: str) -> str:
        obj = os.path.join(bdir, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", src, "-o", obj]
        t = time.time()
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
        _log(f"  {os.path.basename(src)} done in {time.time() - t:.1f} s")
        return obj

    try:
        workers = max(1, min(len(srcs), os.cpu_count() or 2, 8))
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            objs = list(pool.map(one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-o", tmp] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        os.replace(tmp, lib)
        with open(os.path.join(bdir, "stamp.json"), "w") as f:
            json.dump({"digest": digest, "flags": NVCC_FLAGS}, f)
    finally:
        done.set()
    _log(f"built {lib} in {time.time() - t0:.1f} s")


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv))
