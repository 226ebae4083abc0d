"""Building and loading the kernel library.

The ``.cu`` files beside this module are compiled with ``nvcc`` for sm_100a into one shared
library (``kernels``) that is loaded with ``ctypes``.  The library's file name carries a hash
of its sources and flags, so an edited source is never served by a stale build.  Libraries are looked for, and built at first need, in ``_build/`` beside the
sources; if that folder cannot be written (a read-only installation) a per-user folder under
the system's temporary directory is used instead.  While compiling, a line is printed to
stderr for every file so that a first call does not look hung.
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
import time
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
_NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
               "--expt-relaxed-constexpr", "-Xptxas", "-v"]

_OPTIONAL: dict = {}       # group -> sources of a library of its own; the rest is "kernels"
_libs: dict = {}
_lib_paths: dict = {}


class KernelBuildError(RuntimeError):
    """The kernel library could not be built or loaded."""


def groups() -> List[str]:
    return ["kernels"] + sorted(_OPTIONAL)


def sources(group: str = "kernels") -> List[str]:
    if group in _OPTIONAL:
        return sorted(_OPTIONAL[group])
    if group != "kernels":
        raise KeyError(f"no kernel library {group!r}; there are {groups()}")
    taken = {f for fs in _OPTIONAL.values() for f in fs}
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu") and f not in taken)


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".h", ".cuh")))


def _find_nvcc() -> str:
    for cand in (os.environ.get("CRETIF_NVCC"), shutil.which("nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $CRETIF_NVCC, PATH and "
                           "/usr/local/cuda/bin); the kernels cannot be compiled")


def source_hash(group: str = "kernels") -> str:
    h = hashlib.sha256()
    for name in sources(group) + _headers():
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(_ARCH_FLAGS + _NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> List[str]:
    dirs = []
    env = os.environ.get("CRETIF_BUILD_DIR")
    if env:
        dirs.append(env)
    dirs.append(os.path.join(_HERE, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"cretif_b200_build_{os.getuid()}"))
    return dirs


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


def library_path(build: bool = True, verbose: bool = True, group: str = "kernels") -> str:
    """Path of the built library for the present sources; builds it if it is missing."""
    name = f"libcretif_{group}_{source_hash(group)}.so"
    for d in _build_dirs():
        p = os.path.join(d, name)
        if os.path.isfile(p):
            return p
    if not build:
        raise KernelBuildError(f"{name} has not been built")
    for d in _build_dirs():
        if _writable_dir(d):
            return _compile(d, name, verbose, group)
    raise KernelBuildError("no writable folder to build the kernel library in; "
                           f"tried {_build_dirs()}")


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[cretif_b200] {msg}", file=sys.stderr, flush=True)


def _compile(build_dir: str, name: str, verbose: bool, group: str) -> str:
    nvcc = _find_nvcc()
    srcs = sources(group)
    tag = name[len("libcretif_"):-3]
    obj_dir = os.path.join(build_dir, f"obj_{tag}")
    os.makedirs(obj_dir, exist_ok=True)
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {build_dir} (first use only)",
         verbose)
    t0 = time.time()

    def one(src: str):
        obj = os.path.join(obj_dir, src[:-3] + ".o")
        cmd = [nvcc, *_ARCH_FLAGS, *_NVCC_FLAGS, "-I", _HERE, "-c",
               os.path.join(_HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        with open(os.path.join(obj_dir, src[:-3] + ".ptxas.txt"), "w") as f:
            f.write(r.stderr)
        return src, obj

    objs = []
    workers = max(1, min(len(srcs), os.cpu_count() or 1, 8))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        for src, obj in pool.map(one, srcs):
            objs.append(obj)
            _say(f"  compiled {src} ({time.time() - t0:.0f} s)", verbose)
    tmp = os.path.join(build_dir, f".{name}.{os.getpid()}.tmp")
    cmd = [nvcc, *_ARCH_FLAGS, "-shared", "-o", tmp, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"linking the kernel library failed:\n{r.stdout}\n{r.stderr}")
    out = os.path.join(build_dir, name)
    os.replace(tmp, out)
    for old in os.listdir(build_dir):          # builds of earlier sources are of no use
        path = os.path.join(build_dir, old)
        if old.startswith(f"libcretif_{group}_") and old.endswith(".so") and old != name:
            os.remove(path)
        elif old.startswith(f"obj_{group}_") and old != f"obj_{tag}":
            shutil.rmtree(path, ignore_errors=True)
    _say(f"built {name} in {time.time() - t0:.0f} s", verbose)
    return out


def load_library(verbose: bool = True, group: str = "kernels") -> ctypes.CDLL:
    """A kernel library, built on first use.  Raises KernelBuildError if that fails.  An
    optional library uses host functions of ``kernels``, which is therefore loaded first and
    with its symbols visible to later loads."""
    if group not in _libs:
        if group != "kernels":
            load_library(verbose, "kernels")
        path = library_path(build=True, verbose=verbose, group=group)
        try:
            _libs[group] = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        _lib_paths[group] = path
    return _libs[group]


def loaded_library_path(group: str = "kernels") -> Optional[str]:
    return _lib_paths.get(group)
