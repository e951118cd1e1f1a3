"""Compiling the native sources and loading the result.

Each *library* is a set of files from ``moe_b200/csrc`` linked into one shared
object with plain C entry points, loaded with ``ctypes``: ``.cu`` files are
compiled by ``nvcc`` for sm_100a, ``.cpp`` files (the host runtime, which needs
no CUDA and is tested on machines without a GPU) by the host C++ compiler.  A library is
compiled the first time it is asked for (one ``nvcc`` per file, in parallel, a
progress line every few seconds) and afterwards only when a source, a header or
a flag changed.  The objects live beside the sources in ``csrc/_build``; when
that folder cannot be written they go to a per-user folder under the system's
temporary directory.
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
from typing import Dict, List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# library name -> sources; what a model needs is decided by the caller
LIBRARIES: Dict[str, List[str]] = {
    "core": ["embed_norm.cu", "gemm_generic.cu", "rope_cache.cu", "attention_generic.cu", "attention_tiled.cu",
             "attention_decode.cu", "moe.cu", "sampling.cu"],
    # tcgen05 / TMA kernels of the bfloat16 path; a float32 model never builds or loads them
    "tc": ["gemm_tc.cu", "attention_prefill.cu", "attention_prefill_tc.cu"],
    # host side of a step (cache ledger, step packing): plain C++, no CUDA
    "host": ["host_runtime.cpp"],
}
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); the kernels cannot be built")


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++); the host runtime cannot be built")


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"moe_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(files: List[str], extra: List[str]) -> str:
    h = hashlib.sha256()
    for f in files + _headers():
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra).encode())
    return h.hexdigest()[:16]


def _say(msg: str) -> None:
    print(f"[moe_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(compiler: str, src: str, obj: str, extra: List[str]) -> None:
    if src.endswith(".cpp"):
        cmd = [compiler, *CXX_FLAGS, *extra, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    else:
        cmd = [compiler, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"{os.path.basename(compiler)} failed on {src}:\n{r.stdout}\n{r.stderr}")


def build(name: str, verbose: bool = True) -> str:
    """Compile library ``name`` if needed; return the path of its shared object."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'")
    sources = LIBRARIES[name]
    extra: List[str] = []
    out_dir = _build_dir()
    so = os.path.join(out_dir, f"libmoe_b200_{name}.so")
    stamp = so + ".stamp"
    want = _digest(sources, extra)
    if os.path.isfile(so) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return so
    host_only = all(s.endswith(".cpp") for s in sources)
    nvcc = find_cxx() if host_only else find_nvcc()
    if verbose and not host_only:
        _say(f"compiling kernel library '{name}' ({len(sources)} files) for sm_100a ...")
    t0 = time.time()
    objs = [os.path.join(out_dir, f"{name}_{os.path.splitext(s)[0]}.{want}.o") for s in sources]
    done = [0]

    def work(pair):
        _compile_one(nvcc, pair[0], pair[1], extra)
        done[0] += 1

    with ThreadPoolExecutor(max_workers=min(len(sources), max(1, (os.cpu_count() or 2)))) as pool:
        futures = [pool.submit(work, p) for p in zip(sources, objs)]
        last = t0
        while any(not f.done() for f in futures):
            time.sleep(0.25)
            if verbose and time.time() - last >= 5.0:
                last = time.time()
                _say(f"  ... {done[0]}/{len(sources)} files compiled, {last - t0:.0f} s")
        for f in futures:
            f.result()
    tmp = so + f".{os.getpid()}.tmp"
    link = [nvcc, "-shared", "-o", tmp, *objs] if host_only else [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {name} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, so)
    with open(stamp, "w") as f:
        f.write(want)
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    if verbose and not host_only:
        _say(f"kernel library '{name}' ready in {time.time() - t0:.0f} s")
    return so


def load(name: str) -> ctypes.CDLL:
    """The loaded library; built first if needed.  Raises if it cannot be had."""
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(build(name))
        return _loaded[name]


def build_all(verbose: bool = True) -> List[str]:
    return [build(n, verbose) for n in LIBRARIES]
