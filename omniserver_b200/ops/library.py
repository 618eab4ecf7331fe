"""Builds and loads the CUDA kernel library (sm_100a) and exposes its C entry points.

The kernels are plain ``extern "C"`` launch functions compiled by nvcc into one
shared library inside the package (``omniserver_b200/_build``), loaded with
ctypes and called with raw device pointers and the current CUDA stream.  The
first call compiles what is missing and prints a line per file meanwhile; a
build is reused as long as the sources and flags are unchanged.  There is no
fallback: when the library cannot be built or loaded, every op raises.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
_PKG = os.path.dirname(_CSRC)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


class KernelLibraryError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[omniserver_b200] {msg}", file=sys.stderr, flush=True)


def _find_nvcc() -> str:
    cands = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            cands.append(os.path.join(os.environ[env], "bin", "nvcc"))
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    cands.append("/usr/local/cuda/bin/nvcc")
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelLibraryError("nvcc not found (looked at CUDA_HOME, PATH and /usr/local/cuda/bin)")


def source_files() -> List[str]:
    return sorted(f for f in os.listdir(_CSRC) if f.endswith(".cu"))


def _source_hash() -> str:
    h = hashlib.sha256()
    for fn in sorted(os.listdir(_CSRC)):
        if fn.endswith((".cu", ".cuh", ".h")):
            h.update(fn.encode())
            with open(os.path.join(_CSRC, fn), "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    env = os.environ.get("OMNISERVER_B200_BUILD_DIR")
    cands = [env] if env else []
    cands.append(os.path.join(_PKG, "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"omniserver_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelLibraryError("no writable directory to build the kernel library in: " + ", ".join(map(str, cands)))


def library_path(create_dir: bool = True) -> str:
    tag = _source_hash()
    in_tree = os.path.join(_PKG, "_build", f"libosb_kernels_{tag}.so")
    if os.path.isfile(in_tree):
        return in_tree
    return os.path.join(_build_dir(), f"libosb_kernels_{tag}.so")


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library; returns its path."""
    out = library_path()
    if os.path.isfile(out) and not force:
        return out
    nvcc = _find_nvcc()
    bdir = os.path.dirname(out)
    tag = _source_hash()
    objdir = os.path.join(bdir, f"obj_{tag}")
    os.makedirs(objdir, exist_ok=True)
    srcs = source_files()
    t0 = time.time()
    if verbose:
        _say(f"building the CUDA kernels for sm_100a ({len(srcs)} files) in {bdir}")
    lock = threading.Lock()
    done = [0]

    def compile_one(fn: str) -> str:
        obj = os.path.join(objdir, fn[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", _CSRC, "-c", os.path.join(_CSRC, fn), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise KernelLibraryError(f"nvcc failed on {fn}:\n{p.stdout}")
        with lock:
            done[0] += 1
            if verbose:
                _say(f"compiled {fn} ({done[0]}/{len(srcs)}, {time.time() - t0:.0f}s)")
        return obj

    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = out + f".tmp{os.getpid()}"
    p = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise KernelLibraryError(f"linking the kernel library failed:\n{p.stdout}")
    os.replace(tmp, out)
    shutil.rmtree(objdir, ignore_errors=True)
    # drop libraries of older sources from the same directory
    for fn in os.listdir(bdir):
        if fn.startswith("libosb_kernels_") and fn.endswith(".so") and fn != os.path.basename(out):
            try:
                os.remove(os.path.join(bdir, fn))
            except OSError:
                pass
    if verbose:
        _say(f"kernel library ready after {time.time() - t0:.0f}s: {out}")
    return out


_LIB: Optional[ctypes.CDLL] = None
_LIB_LOCK = threading.Lock()


def load() -> ctypes.CDLL:
    """The loaded kernel library; built first if needed. Raises if that is impossible."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LIB_LOCK:
        if _LIB is None:
            path = build(verbose=True)
            try:
                _LIB = ctypes.CDLL(path)
            except OSError as e:
                raise KernelLibraryError(f"cannot load {path}: {e}") from e
    return _LIB


def is_loaded() -> bool:
    return _LIB is not None
