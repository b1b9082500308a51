"""Builds and loads the CUDA library of this package.

The kernels are plain `.cu` files with `extern "C"` entry points; they are compiled by
nvcc for sm_100a into one shared library beside the sources (`_build/libcatena_b200.so`,
or a per-user folder under the system temp directory when the source tree is read-only)
and loaded with ctypes.  The library is rebuilt when a source file changes.  Nothing here
imports torch, so the build also runs on a machine without a GPU.
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

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libcatena_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_lib = None


class BuildError(RuntimeError):
    pass


def _say(msg):
    print(f"[catena_models_b200 build] {msg}", file=sys.stderr, flush=True)


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def find_nvcc():
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.exists(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc not found (looked in CUDA_HOME, /usr/local/cuda and PATH)")


def _digest():
    h = hashlib.sha256()
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir():
    """In-tree `_build/` when it can be written, else a per-user temp folder."""
    local = os.path.join(CSRC, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"catena_models_b200_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _compile_one(nvcc, src, obj):
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{proc.stdout}\n{proc.stderr}")
    return src


def build(force=False, verbose=True):
    """Compile every `.cu` file for sm_100a and link the library; returns its path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "digest.txt")
    digest = _digest()
    if not force and os.path.exists(lib_path) and os.path.exists(stamp_path):
        with open(stamp_path) as fh:
            if fh.read().strip() == digest:
                return lib_path
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    objs = [os.path.join(out_dir, s[:-3] + f".{os.getpid()}.o") for s in srcs]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        futs = {pool.submit(_compile_one, nvcc, s, o): s for s, o in zip(srcs, objs)}
        done = 0
        pending = set(futs)
        while pending:
            finished, pending = concurrent.futures.wait(pending, timeout=10.0)
            for f in finished:
                f.result()
                done += 1
                if verbose:
                    _say(f"  [{done}/{len(srcs)}] {futs[f]} ({time.time() - t0:.0f}s)")
            if pending and not finished and verbose:
                _say(f"  still compiling, {len(pending)} file(s) left ({time.time() - t0:.0f}s)")
    tmp_lib = lib_path + f".{os.getpid()}.tmp"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *objs, "-lcudart"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib_path)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    with open(stamp_path, "w") as fh:
        fh.write(digest)
    if verbose:
        _say(f"built {lib_path} in {time.time() - t0:.0f}s")
    return lib_path


def load():
    """The loaded library (built on first use).  Raises if it cannot be built or loaded:
    there is no fallback path."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as exc:
                raise BuildError(f"cannot load {path}: {exc}") from exc
        return _lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
