"""Compiles the CUDA sources under ``csrc/`` for sm_100a with nvcc and loads the
result with ctypes.  Nothing is compiled at import: a library is built the
first time one of its kernels is asked for, and only the libraries that the
running model needs are built.  Built files are kept under ``csrc/_build/``
(or, if the package folder cannot be written, under the system's temporary
folder) and are named by a hash of their sources and flags, so a stale build
is never loaded.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

# library name -> sources.  ``core`` holds what every model and both dtypes
# need; the tensor-core libraries serve bfloat16 only.
LIBRARIES: Dict[str, List[str]] = {
    "core": ["elementwise.cu", "gemm_simt.cu", "shortconv.cu", "attention.cu", "attention_decode.cu",
             "sampling.cu"],
    "bf16": ["gemm_small_m.cu", "gemm_tc.cu", "gemm_tc_pair.cu", "gemm_tc_swap.cu", "attention_prefill.cu",
             "attention_prefill_tc.cu", "attention_decode_tc.cu"],
}

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# MIVI_DEBUG_CHECKS=1: a build of its own whose kernels check page and slot indices against declared bounds
# (see common.cuh); it lives beside the ordinary build under another name.
DEBUG_CHECKS = os.environ.get("MIVI_DEBUG_CHECKS", "0") == "1"


def nvcc_flags(debug_checks: bool = None) -> List[str]:
    debug_checks = DEBUG_CHECKS if debug_checks is None else debug_checks
    return NVCC_FLAGS + (["-DMIVI_DEBUG_CHECKS"] if debug_checks else [])


_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[mivi_v4_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("MIVI_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $MIVI_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the kernels of this library have to be compiled for sm_100a")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    env = os.environ.get("MIVI_BUILD_DIR")
    if env and _writable_dir(env):
        return env
    in_tree = os.path.join(CSRC, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"mivi_v4_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"no writable folder for compiled kernels (tried {in_tree} and {fallback})")


def _digest(name: str, debug_checks: bool = None) -> str:
    h = hashlib.sha256()
    h.update(" ".join(nvcc_flags(debug_checks)).encode())
    files = sorted(set(LIBRARIES[name]) | {f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))})
    for f in files:
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _stem(name: str, debug_checks: bool = None) -> str:
    debug_checks = DEBUG_CHECKS if debug_checks is None else debug_checks
    return f"libmivi_{name}{'dbg' if debug_checks else ''}_"


def library_path(name: str, debug_checks: bool = None) -> str:
    return os.path.join(build_dir(), f"{_stem(name, debug_checks)}{_digest(name, debug_checks)}.so")


def _run(cmd: List[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{proc.stdout}")


def compile_library(name: str, verbose: bool = True, debug_checks: bool = None) -> str:
    """Build ``name`` if its file is not there yet; returns the path of the .so."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {', '.join(sorted(LIBRARIES))}")
    out = library_path(name, debug_checks)
    flags = nvcc_flags(debug_checks)
    stem = _stem(name, debug_checks)
    if os.path.isfile(out):
        return out
    bdir = os.path.dirname(out)
    with open(os.path.join(bdir, f".lock_{stem}"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)        # another process may be building the same file
        try:
            if os.path.isfile(out):
                return out
            nvcc = find_nvcc()
            srcs = LIBRARIES[name]
            t0 = time.time()
            if verbose:
                _say(f"compiling the {name} kernels for sm_100a ({len(srcs)} files, first call only"
                     f"{', with index checks' if '-DMIVI_DEBUG_CHECKS' in flags else ''}) ...")
            stop = threading.Event()

            def ticker():
                while not stop.wait(10.0):
                    _say(f"  still compiling {name} ... {time.time() - t0:.0f} s")
            tick = threading.Thread(target=ticker, daemon=True)
            if verbose:
                tick.start()
            try:
                tmp = tempfile.mkdtemp(prefix=f"{name}_", dir=bdir)
                objs = []

                def one(src: str) -> str:
                    obj = os.path.join(tmp, src.replace(".cu", ".o"))
                    _run([nvcc, *flags, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj], src)
                    return obj
                with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
                    objs = list(pool.map(one, srcs))
                part = out + f".part{os.getpid()}"
                _run([nvcc, "-shared", "-o", part, *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                     f"link of {name}")
                os.replace(part, out)
                shutil.rmtree(tmp, ignore_errors=True)
                for old in os.listdir(bdir):              # builds of older sources
                    if old.startswith(stem) and old.endswith(".so") and \
                            os.path.join(bdir, old) != out:
                        try:
                            os.remove(os.path.join(bdir, old))
                        except OSError:
                            pass
            finally:
                stop.set()
            if verbose:
                _say(f"  {name} kernels ready in {time.time() - t0:.0f} s: {out}")
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(compile_library(name))
        return _loaded[name]


def build_all(verbose: bool = True, debug_checks: bool = None) -> Dict[str, str]:
    return {name: compile_library(name, verbose, debug_checks) for name in LIBRARIES}
