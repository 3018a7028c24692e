"""Builds the CUDA sources of csrc/ into shared libraries and loads them with ctypes.

Each .cu file becomes one library with plain C entry points, compiled for sm_100a by nvcc when it
is first needed (a model builds what its parts need, nothing else) and kept under csrc/_build/,
named by a hash of the source, the headers and the flags.  A library exists in two flavours: the
default one, whose 16-bit type is bfloat16, and "f16" (compiled with -DTNX_F16), whose 16-bit type is
float16; a library name may carry the flavour as a suffix ("gemm_tc.f16").  When that folder cannot be written,
a per-user folder under the system's temporary directory is used.  There is no fallback: a
library that cannot be built or loaded raises.
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
from typing import Dict, Iterable, List, Optional

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc")
CSRC = os.path.normpath(CSRC)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# library name -> source file (relative to csrc/)
SOURCES: Dict[str, str] = {
    "embedding": "embedding.cu",
    "layernorm": "layernorm.cu",
    "gemm_simt": "gemm_simt.cu",
    "kv_cache": "kv_cache.cu",
    "attention_simt": "attention_simt.cu",
    "sampling": "sampling.cu",
    "gemm_tc": "gemm_tc.cu",
    "gemv": "gemv.cu",
    "attention_decode": "attention_decode.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_build_locks: Dict[str, threading.Lock] = {}


class KernelBuildError(RuntimeError):
    pass


def register_source(name: str, filename: str) -> None:
    SOURCES[name] = filename


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found: the engine's kernels are compiled from source at first use")


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(src: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in [src] + _headers():
        with open(p, "rb") as fp:
            h.update(fp.read())
    return h.hexdigest()[:16]


_build_dir_cached: Optional[str] = None


def _build_dir() -> str:
    global _build_dir_cached
    with _lock:
        if _build_dir_cached is not None:
            return _build_dir_cached
        first = os.path.join(CSRC, "_build")
        try:
            os.makedirs(first, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=first)
            os.close(fd)
            os.remove(probe)
            _build_dir_cached = first
        except OSError:
            alt = os.path.join(tempfile.gettempdir(), f"tnx_b200_build_{os.getuid()}")
            os.makedirs(alt, exist_ok=True)
            _build_dir_cached = alt
        return _build_dir_cached


FLAVOURS = {"": [], "f16": ["-DTNX_F16"]}


def split_name(name: str):
    """'gemm_tc.f16' -> ('gemm_tc', 'f16'); 'gemm_tc' -> ('gemm_tc', '')."""
    base, _, flavour = name.partition(".")
    if base not in SOURCES:
        raise KernelBuildError(f"no kernel source registered under {base!r}")
    if flavour not in FLAVOURS:
        raise KernelBuildError(f"unknown flavour {flavour!r} of {base!r}; known: {sorted(FLAVOURS)}")
    return base, flavour


def flavour_of(dtype) -> str:
    """The flavour whose 16-bit type is `dtype` (a torch dtype or its name); '' for bfloat16 and float32."""
    return "f16" if str(dtype).replace("torch.", "") in ("float16", "half") else ""


def with_flavour(names: Iterable[str], dtype) -> List[str]:
    f = flavour_of(dtype)
    return [n if (not f or "." in n) else f"{n}.{f}" for n in names]


def library_path(name: str) -> str:
    base, flavour = split_name(name)
    src = os.path.join(CSRC, SOURCES[base])
    return os.path.join(_build_dir(), f"{name}.{_digest(src)}.so")


def _say(msg: str) -> None:
    print(f"[tnx-b200 build] {msg}", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> str:
    """Compiles one library if its up-to-date binary is not there yet; returns its path."""
    base, flavour = split_name(name)
    out = library_path(name)
    with _lock:
        lk = _build_locks.setdefault(name, threading.Lock())
    with lk:
        src = os.path.join(CSRC, SOURCES[base])
        if os.path.isfile(out):
            return out
        tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
        cmd = [_nvcc()] + NVCC_FLAGS + FLAVOURS[flavour] + ["-I", CSRC, "-o", tmp, src]
        what = SOURCES[base] + (f" ({flavour})" if flavour else "")
        if verbose:
            _say(f"compiling {what} for sm_100a ...")
        t0 = time.time()
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        while True:                      # a line now and then while a long compile runs
            try:
                log, _ = proc.communicate(timeout=20)
                break
            except subprocess.TimeoutExpired:
                if verbose:
                    _say(f"  still compiling {what} ({time.time() - t0:.0f} s)")
        if proc.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise KernelBuildError(f"nvcc failed on {src}:\n{log}")
        os.replace(tmp, out)
        _drop_older_builds(out)
        if verbose:
            _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
        return out


def _drop_older_builds(current: str) -> None:
    """Removes the binaries of earlier versions of the same source and flavour (a process that has one
    loaded keeps its mapping).  Best effort: a folder that is not ours to write is left as it is."""
    folder, keep = os.path.dirname(current), os.path.basename(current)
    stem = keep.rsplit(".", 2)[0]                      # "gemm_tc" or "gemm_tc.f16"
    try:
        for f in os.listdir(folder):
            if f != keep and f.endswith(".so") and f.rsplit(".", 2)[0] == stem and len(f.rsplit(".", 2)) == 3:
                os.remove(os.path.join(folder, f))
    except OSError:
        pass


def export_libraries(names: Iterable[str], directory: str) -> List[str]:
    """Copies the compiled libraries of `names` (building what is missing) into `directory`, under
    the names that carry their source's digest; returns the paths written."""
    os.makedirs(directory, exist_ok=True)
    out = []
    for n in dict.fromkeys(names):
        path = build(n)
        dst = os.path.join(directory, os.path.basename(path))
        if not os.path.isfile(dst):
            tmp = f"{dst}.{os.getpid()}.tmp"
            shutil.copyfile(path, tmp)
            os.replace(tmp, dst)
        out.append(dst)
    return out


def import_libraries(directory: str) -> List[str]:
    """Takes from `directory` every library whose name carries the digest of today's source (a
    library of another source version, or of a file that is not ours, is left alone), so that
    build() finds it instead of compiling; returns the kernel names taken."""
    taken = []
    if not os.path.isdir(directory):
        raise KernelBuildError(f"{directory!r} is not a folder of compiled kernels")
    for n in [b if not f else f"{b}.{f}" for b in SOURCES for f in FLAVOURS]:
        want = library_path(n)
        src = os.path.join(directory, os.path.basename(want))
        if os.path.isfile(src) and not os.path.isfile(want):
            tmp = f"{want}.{os.getpid()}.tmp"
            shutil.copyfile(src, tmp)
            os.replace(tmp, want)
        if os.path.isfile(src):
            taken.append(n)
    return taken


def build_many(names: Iterable[str], verbose: bool = True) -> None:
    names = [n for n in dict.fromkeys(names) if n not in _loaded]
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as ex:
        list(ex.map(lambda n: build(n, verbose), todo))


def build_all(verbose: bool = True) -> None:
    """Every library in every flavour."""
    build_many([b if not f else f"{b}.{f}" for f in FLAVOURS for b in SOURCES], verbose)


def load(name: str, dtype=None) -> ctypes.CDLL:
    """The library `name`; with `dtype` given, in the flavour whose 16-bit type it is."""
    if dtype is not None and "." not in name:
        f = flavour_of(dtype)
        if f:
            name = f"{name}.{f}"
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    path = build(name)
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise KernelBuildError(f"cannot load {path}: {e}") from e
    _loaded[name] = lib
    return lib
