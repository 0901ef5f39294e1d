"""Builds the CUDA library of this package for sm_100a with nvcc and loads it.

The sources are `csrc/*.cu`; every file becomes one object, the objects are
linked into `csrc/_build/libhymt2sharp_b200.so`.  A stamp beside the library
holds a hash of the sources and flags: the library is rebuilt when they
change and only then, so a built library that travels with the checkout is
used as it is.  When the package folder cannot be written to, the build goes
to a per-user folder under the system's temporary directory.

There is no fallback: without nvcc or with a failing build, `load_library`
raises, and nothing of the engine runs.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libhymt2sharp_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_lock = threading.Lock()
_library = None


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[hymt2sharp_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("HYMT2_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $HYMT2_NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of hymt2sharp_b200 cannot be built")


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _build_dir() -> str:
    local = os.path.join(CSRC, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"hymt2sharp_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compiles what is stale and returns the library's path."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp_path = os.path.join(bdir, "stamp.json")
    digest = _source_hash()
    if not force and os.path.exists(lib) and os.path.exists(stamp_path):
        try:
            with open(stamp_path) as f:
                if json.load(f).get("hash") == digest:
                    return lib
        except (OSError, ValueError):
            pass
    nvcc = find_nvcc()
    srcs = sources()
    t0 = time.time()
    if verbose:
        _say(f"building {len(srcs)} CUDA sources for sm_100a into {bdir} (first call only)")
    done = [0]

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        with _lock:
            done[0] += 1
            if verbose:
                _say(f"  compiled {src} ({done[0]}/{len(srcs)}, {time.time() - t0:.0f} s)")
        return obj

    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with ThreadPoolExecutor(workers) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = lib + f".{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp_path, "w") as f:
        json.dump({"hash": digest, "flags": NVCC_FLAGS, "sources": srcs}, f)
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib


def load_library() -> ctypes.CDLL:
    """The loaded CUDA library; builds it first if it is missing or stale."""
    global _library
    with _lock:
        if _library is not None:
            return _library
    path = build()
    lib = ctypes.CDLL(path)
    lib.hymt2_last_error.restype = ctypes.c_char_p
    with _lock:
        _library = lib
    return lib
