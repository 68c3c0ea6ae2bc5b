"""Compile the CUDA sources of this folder into one shared library with nvcc.

The library has a C interface only (no PyTorch headers), so a cold build takes
well under a minute per file and the files are compiled in parallel.  It is
built in-tree (``csrc/_build/``) when that folder can be written, else in a
per-user temporary folder; a stamp with the hash of the sources and flags makes
the first call after a change rebuild and every other call a no-op.  There is
no fallback: without ``nvcc`` or with a failing compile this raises.

The reference builds its kernels for sm_86 through CMake
(CMakeLists.txt:35-37); here the only target is sm_100a.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libmini_infer_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    cand = [os.environ.get("MINI_INFER_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.exists(c):
            return c
    raise RuntimeError("mini_infer_b200: nvcc not found (set MINI_INFER_NVCC); the CUDA kernels cannot be built "
                       "and there is no fallback path")


def _stamp() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.environ.get("MINI_INFER_BUILD_DIR")
    if d:
        os.makedirs(d, exist_ok=True)
        return d
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"mini_infer_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[mini_infer_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, extra: List[str]) -> None:
    cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    t0 = time.time()
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"mini_infer_b200: nvcc failed on {src}:\n{p.stdout}")
    _say(f"compiled {src} in {time.time() - t0:.0f}s")
    if extra and p.stdout.strip():
        _say(p.stdout.strip())


def build(verbose_ptxas: bool = False, force: bool = False) -> str:
    """Build if needed and return the path of the shared library."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp_file = os.path.join(bdir, "stamp.txt")
    stamp = _stamp()
    if not force and os.path.exists(lib) and os.path.exists(stamp_file):
        with open(stamp_file) as f:
            if f.read().strip() == stamp:
                return lib
    nvcc = _find_nvcc()
    srcs = sources()
    _say(f"building {LIB_NAME} for sm_100a from {len(srcs)} CUDA files in {bdir} (first call only)")
    done = threading.Event()

    def heartbeat():
        t0 = time.time()
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f}s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        extra = ["-Xptxas", "-v"] if verbose_ptxas else []
        tag = f"{os.getpid()}"
        objs = [os.path.join(bdir, s[:-3] + f".{tag}.o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, extra) for s, o in zip(srcs, objs)]
            for f in futs:
                f.result()
        tmp_lib = lib + f".{tag}.tmp"
        cmd = [nvcc, "-shared", "-o", tmp_lib] + objs + ["-lcudart"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"mini_infer_b200: linking failed:\n{p.stdout}")
        os.replace(tmp_lib, lib)  # atomic: a concurrent process sees the old or the new library
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
        with open(stamp_file + f".{tag}", "w") as f:
            f.write(stamp)
        os.replace(stamp_file + f".{tag}", stamp_file)
    finally:
        done.set()
    _say("build finished")
    return lib


if __name__ == "__main__":
    print(build(verbose_ptxas="-v" in sys.argv, force="--force" in sys.argv))
