"""Builds the C interface of the engine, `libreflex_b200_engine.so`, with the
host compiler, against the interpreter that runs this script (its path is
compiled in so that a C caller gets the same environment; `$REFLEX_B200_PYTHON`
overrides it at run time)."""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libreflex_b200_engine.so"
HEADER = os.path.join(HERE, "reflex_b200.h")


def _command(out: str):
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise RuntimeError("no C++ compiler found (g++ or $CXX)")
    include = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    version = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", f"-I{include}", f"-I{HERE}",
           f'-DRFX_PYTHON_EXECUTABLE="{sys.executable}"', os.path.join(HERE, "engine_abi.cpp"), "-o", out]
    if libdir:
        cmd += [f"-L{libdir}", f"-Wl,-rpath,{libdir}"]
    cmd += [f"-lpython{version}", "-ldl", "-lpthread"]
    return cmd


def _digest() -> str:
    h = hashlib.sha256()
    h.update(sys.executable.encode())
    for name in ("engine_abi.cpp", "reflex_b200.h"):
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def ensure_built(force: bool = False) -> str:
    from ..csrc.build import build_dir

    bdir = build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "engine_abi_stamp.json")
    digest = _digest()
    if not force and os.path.exists(lib) and os.path.exists(stamp):
        try:
            with open(stamp) as f:
                if json.load(f).get("digest") == digest:
                    return lib
        except (OSError, ValueError):
            pass
    tmp = lib + f".tmp{os.getpid()}"
    res = subprocess.run(_command(tmp), capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {LIB_NAME} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        json.dump({"digest": digest}, f)
    return lib


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv))
