"""Compiles the sources of this folder (CUDA for sm_100a with nvcc, host C++ with g++) and loads them with ctypes.

Every `.cu` or `.cpp` file becomes one shared library with a C ABI, built the first time one of its
functions is asked for and cached under `_build/` next to the sources (or under the
system's temporary folder if that is not writable).  The cache key is a hash of the
source, the shared headers and the flags, so an edited file is rebuilt and a stale
library is never loaded.  There is no fallback: a missing compiler or a failed build
raises.
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
from typing import Dict, Iterable, Tuple

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]

_loaded: Dict[Tuple[str, Tuple[str, ...]], ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def _gxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++); the host runtime of lmsf_b200 cannot be built")


def _nvcc() -> str:
    for cand in (os.environ.get("LMSF_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $LMSF_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of lmsf_b200 cannot be built and there is no other path")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("LMSF_BUILD_DIR")
    if env and _writable_dir(env):
        return env
    in_tree = os.path.join(CSRC_DIR, "_build")
    if _writable_dir(in_tree):
        return in_tree
    tmp = os.path.join(tempfile.gettempdir(), f"lmsf_b200_build_{os.getuid()}")
    if _writable_dir(tmp):
        return tmp
    raise BuildError(f"no writable folder for built kernels (tried {in_tree} and {tmp})")


def _headers() -> Iterable[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _key(source: str, defines: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for name in [source, *_headers()]:
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    flags = HOST_FLAGS if source.endswith(".cpp") else [*ARCH_FLAGS, *BASE_FLAGS]
    h.update(" ".join([*flags, *defines]).encode())
    return h.hexdigest()[:16]


def library_path(source: str, defines: Tuple[str, ...] = ()) -> str:
    stem = os.path.splitext(source)[0]
    return os.path.join(build_dir(), f"liblmsf_{stem}_{_key(source, defines)}.so")


def compile_source(source: str, defines: Tuple[str, ...] = (), verbose: bool = True,
                   extra_flags: Tuple[str, ...] = ()) -> str:
    """Builds `source` if its library is not cached; returns the library's path."""
    out = library_path(source, defines)
    if os.path.isfile(out):
        return out
    if source.endswith(".cpp"):      # host code: the C++ compiler alone
        cmd = [_gxx(), *HOST_FLAGS, *extra_flags, *[f"-D{d}" for d in defines], "-I", CSRC_DIR,
               os.path.join(CSRC_DIR, source), "-o", out + f".tmp{os.getpid()}"]
    else:
        cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *extra_flags, *[f"-D{d}" for d in defines], "-I", CSRC_DIR,
               os.path.join(CSRC_DIR, source), "-o", out + f".tmp{os.getpid()}", "-lcudart"]
    if verbose:
        what = "for the host" if source.endswith(".cpp") else "for sm_100a"
        print(f"[lmsf_b200] compiling {source} {' '.join(defines)} {what} ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[lmsf_b200]   still compiling {source} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.remove(out + f".tmp{os.getpid()}")
        except OSError:
            pass
        raise BuildError(f"the compiler failed on {source}:\n{' '.join(cmd)}\n{log}")
    os.replace(out + f".tmp{os.getpid()}", out)
    if verbose:
        print(f"[lmsf_b200]   built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(source: str, defines: Tuple[str, ...] = ()) -> ctypes.CDLL:
    """The ctypes handle of `source` built with `defines` (compiled on first use)."""
    key = (source, tuple(defines))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_source(source, tuple(defines)))
            _loaded[key] = lib
        return lib


def all_sources() -> Iterable[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cu", ".cpp")))
