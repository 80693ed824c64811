"""Builds and loads the native library (hand-written CUDA for sm_100a, C ABI).

The sources under ``freetoken_b200/csrc`` are compiled with ``nvcc`` straight to one
shared object that is loaded with ``ctypes``; there is no CPU fallback and no second
backend: if the library cannot be built or loaded, every op raises
:class:`KernelError`.  The object is kept in-tree (``freetoken_b200/csrc/_build``) when
that folder can be written, else under the temporary directory, and is rebuilt when a
source file changes.  The first build prints a line per compiled file so that a caller
waiting on it sees progress.

The reference compiles its own CUDA files at first use too, through tvm-ffi
(python/freetoken/kernel/utils.py:188-284).
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
from typing import List, Optional

from ..errors import KernelError

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_BASENAME = "libfreetoken_b200"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# No --use_fast_math: the 32-bit path needs IEEE division, expf and rsqrtf; the bfloat16
# kernels ask for the approximate forms (ex2.approx and friends) by name where they want them.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None


def _sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in _sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(cand):
        raise KernelError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                          "the CUDA kernels cannot be compiled")
    return cand


def _build_dir() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"freetoken_b200-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[freetoken_b200] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile (if stale) and return the path of the shared object."""
    tag = source_hash()
    bdir = _build_dir()
    out = os.path.join(bdir, f"{LIB_BASENAME}-{tag}.so")
    if os.path.isfile(out) and not force:
        return out
    nvcc = _nvcc()
    srcs = _sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)")
    t0 = time.time()
    objs = []

    def one(src: str) -> str:
        obj = os.path.join(bdir, f"{os.path.splitext(src)[0]}-{tag}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if p.returncode != 0:
            raise KernelError(f"nvcc failed on {src}:\n{p.stdout}")
        if verbose:
            _say(f"  compiled {src} ({time.time() - t0:.0f} s)")
        return obj

    workers = max(1, min(len(srcs), os.cpu_count() or 1))
    with ThreadPoolExecutor(max_workers=workers) as ex:
        objs = list(ex.map(one, srcs))
    tmp = out + f".{os.getpid()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart"]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise KernelError(f"linking {LIB_BASENAME} failed:\n{p.stdout}")
    os.replace(tmp, out)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    # drop stale builds of other source versions
    for f in os.listdir(bdir):
        if f.startswith(LIB_BASENAME + "-") and f.endswith(".so") and f != os.path.basename(out):
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    if verbose:
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.0f} s")
    return out


def load() -> ctypes.CDLL:
    """The loaded library; builds it first when needed.  Raises :class:`KernelError`."""
    global _lib, _lib_path
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from e
        lib.ftk_last_error.restype = ctypes.c_char_p
        lib.ftk_last_error.argtypes = []
        _lib, _lib_path = lib, path
        return lib


def library_path() -> Optional[str]:
    return _lib_path
