"""Compiling the kernel library for sm_100a and loading it.

The sources under this folder are compiled with nvcc into one shared library,
``_build/libcitlali_b200.so`` beside them (or, if that folder cannot be written, under the
system's temporary folder).  The library is rebuilt when a source, a header or a flag
changed.  Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import CitlaliError

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libcitlali_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
_lock = threading.Lock()
_lib = None


def _say(message):
    print(f"[citlali_b200 build] {message}", file=sys.stderr, flush=True)


def sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(path):
        raise CitlaliError("nvcc was not found (PATH and /usr/local/cuda/bin): the kernel library cannot be "
                           "compiled, and there is no other way to run a model")
    return path


def _digest():
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _build_dir():
    preferred = os.path.join(_HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"citlali_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def library_path():
    return os.path.join(_build_dir(), LIB_NAME)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile what is stale; return the library's path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "sources.sha256")
    digest = _digest()
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == digest:
                return lib_path
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} (first use, or the sources changed)")
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise CitlaliError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        return src, obj

    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        futures = [pool.submit(compile_one, s) for s in srcs]
        pending = set(futures)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=10.0)
            for f in done:
                src, obj = f.result()
                objs.append(obj)
                if verbose:
                    _say(f"  compiled {src} ({len(objs)}/{len(srcs)}, {time.time() - t0:.0f} s)")
            if pending and not done and verbose:
                _say(f"  still compiling ({len(objs)}/{len(srcs)} done, {time.time() - t0:.0f} s)")
    tmp = lib_path + f".{os.getpid()}.tmp"
    r = subprocess.run([nvcc, "-shared", "-o", tmp] + sorted(objs), capture_output=True, text=True)
    if r.returncode != 0:
        raise CitlaliError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib_path)
    with open(stamp_path, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"built {lib_path} in {time.time() - t0:.0f} s")
    return lib_path


def load() -> ctypes.CDLL:
    """The loaded library; compiled first if it is missing or stale.  There is no other
    implementation of the kernels: a failure here is an error, never a fallback."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise CitlaliError(f"the kernel library {path} could not be loaded: {e}") from None
        return _lib
