"""Compiles the CUDA sources of this folder into one shared library.

The library is built for sm_100a with nvcc alone (no Python headers: the
kernels are reached through a C interface) the first time it is needed and
whenever a source changes.  It is placed next to the sources
(``_build/libagave_b200.so``) when that folder can be written, else under
the system's temporary folder, so a fresh checkout owned by another user and
an empty HOME both work.  Progress goes to standard error, one line per file.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libagave_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _say(msg: str) -> None:
    print(f"[agave_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("AGAVE_B200_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc was not found (looked at $AGAVE_B200_NVCC, PATH and "
                       "/usr/local/cuda/bin); the CUDA kernels cannot be built")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"agave_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed: bool = True, verbose: bool = True) -> str:
    """Path of an up-to-date library, compiling first if it is missing or stale."""
    d = _build_dir()
    lib = os.path.join(d, LIB_NAME)
    stamp = os.path.join(d, "stamp.txt")
    want = _digest()
    if os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return lib
    if not build_if_needed:
        raise RuntimeError(f"{lib} is missing or older than its sources")
    build(d, verbose)
    with open(stamp, "w") as f:
        f.write(want)
    return lib


def build(build_dir: Optional[str] = None, verbose: bool = True) -> str:
    d = build_dir or _build_dir()
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {d} (first use or sources "
             "changed; this takes a minute or two)")

    def one(src: str) -> str:
        obj = os.path.join(d, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    workers = max(1, min(len(srcs), (os.cpu_count() or 2)))
    with ThreadPoolExecutor(workers) as ex:
        objs = list(ex.map(one, srcs))
    lib = os.path.join(d, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    if verbose:
        _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    print(library_path())
