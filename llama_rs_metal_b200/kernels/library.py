"""Builds the CUDA sources under csrc/ for sm_100a and loads them through ctypes.

There is no CPU fallback and no second backend: if the shared object cannot be
built or loaded, KernelUnavailableError is raised with the compiler's output.
The object is built in-tree at first use (a line is printed per file, and one
now and then while nvcc runs), and rebuilt when a source file or a flag changes.
The entry points are plain C symbols (`lrm_*`); callers pass device pointers
and a stream handle.
"""
from __future__ import annotations

import concurrent.futures
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
from typing import List, Optional

from ..errors import KernelUnavailableError

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "libllama_b200_kernels.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_library: Optional[ctypes.CDLL] = None


def _say(message: str) -> None:
    print(f"[llama_rs_metal_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelUnavailableError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin)")


def source_files() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _fingerprint() -> str:
    digest = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            digest.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as handle:
                digest.update(handle.read())
    return digest.hexdigest()


def _build_dir() -> str:
    """In-tree build folder, or a private temporary one when the tree is read-only."""
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        path = os.path.join(tempfile.gettempdir(), f"llama_rs_metal_b200_build_{os.getuid()}")
        os.makedirs(path, exist_ok=True)
        return path


def library_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)


def _run_with_heartbeat(cmd: List[str], label: str) -> None:
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        while not done.wait(20.0):
            _say(f"still compiling {label} ({time.time() - start:.0f} s)")

    watcher = threading.Thread(target=beat, daemon=True)
    watcher.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise KernelUnavailableError(f"{label} failed to compile:\n{' '.join(cmd)}\n{output}")


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every .cu under csrc/ for sm_100a and link one shared object. Returns its path."""
    out_dir = _build_dir()
    target = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "stamp.json")
    fingerprint = _fingerprint()
    if not force and os.path.isfile(target) and os.path.isfile(stamp_path):
        try:
            with open(stamp_path) as handle:
                if json.load(handle).get("fingerprint") == fingerprint:
                    return target
        except (OSError, ValueError):
            pass
    nvcc = find_nvcc()
    sources = source_files()
    if not sources:
        raise KernelUnavailableError(f"no CUDA sources under {CSRC}")
    if verbose:
        _say(f"building {len(sources)} CUDA sources for sm_100a into {out_dir}")
    objects = []

    def compile_one(name: str) -> str:
        obj = os.path.join(out_dir, name[:-3] + ".o")
        _run_with_heartbeat([nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj], name)
        if verbose:
            _say(f"compiled {name}")
        return obj

    workers = max(1, min(len(sources), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        objects = list(pool.map(compile_one, sources))
    scratch = target + f".tmp{os.getpid()}"
    _run_with_heartbeat([nvcc, "-shared", "-o", scratch, *objects, "-cudart", "static"], "link")
    os.replace(scratch, target)
    with open(stamp_path, "w") as handle:
        json.dump({"fingerprint": fingerprint, "sources": sources}, handle)
    if verbose:
        _say(f"built {target}")
    return target


def load() -> ctypes.CDLL:
    """The loaded library (built first if needed). Raises KernelUnavailableError on failure."""
    global _library
    with _lock:
        if _library is None:
            path = build()
            try:
                _library = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelUnavailableError(f"cannot load {path}: {exc}") from None
            # Kernels are launched with programmatic dependent launch: a kernel may be scheduled
            # while its predecessor drains and prefetch what does not depend on it. Small kernels
            # let their successor start at once, large ones after their main loop (letting every
            # kernel do so at once made the whole step slower). LRM_PDL=0 switches it off.
            _library.lrm_set_pdl(0 if os.environ.get("LRM_PDL", "1") == "0" else 1)
            from . import profile
            if profile.enabled:  # LRM_PROFILE=1: every launch is timed (see profile.py)
                _library = profile.ProfiledLibrary(_library)
        return _library
