"""Compile the CUDA sources under csrc/ for sm_100a into one shared library and load it; and the host-only C++
sources under csrc/host/ (the cache's bookkeeping) into a second one that needs no CUDA.

The library is plain CUDA with C entry points (no Python or torch headers), so a build takes
seconds per file.  It is built at the first call that needs it, in `_build/` inside the package
when that is writable, else under the temporary directory; a line is printed now and then while
the compiler runs.  The file name carries a hash of the sources and flags, so an edit rebuilds.
"""
from __future__ import annotations

import ctypes
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

_PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC_DIR = os.path.join(_PACKAGE_DIR, "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"),
                      os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                      shutil.which("nvcc")):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError("nvcc not found (set NVCC or CUDA_HOME); the CUDA kernels cannot be built")


def sources() -> list:
    return sorted(glob.glob(os.path.join(CSRC_DIR, "*.cu")))


def _digest() -> str:
    h = hashlib.sha256()
    headers = sorted(glob.glob(os.path.join(CSRC_DIR, "*.cuh")) + glob.glob(os.path.join(CSRC_DIR, "*.h")))
    for path in sources() + headers:
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    preferred = os.path.join(_PACKAGE_DIR, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"lia_rs_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def library_path() -> str:
    return os.path.join(_build_dir(), f"liblia_b200_{_digest()}.so")


def build(verbose: bool = True) -> str:
    """Compile if needed; return the path of the shared library."""
    target = library_path()
    if os.path.exists(target):
        return target
    nvcc = _nvcc()
    out_dir = os.path.dirname(target)
    work = tempfile.mkdtemp(prefix="obj_", dir=out_dir)
    log = (lambda msg: print(f"[lia_rs_b200] {msg}", file=sys.stderr, flush=True)) if verbose else (lambda msg: None)
    files = sources()
    log(f"compiling {len(files)} CUDA sources for sm_100a into {out_dir} (first call only)")
    started = time.time()
    jobs = []
    for src in files:
        obj = os.path.join(work, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC_DIR, "-c", src, "-o", obj]
        jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    pending = list(jobs)
    last = time.time()
    while pending:
        pending = [j for j in pending if j[2].poll() is None]
        if pending and time.time() - last > 5:
            log(f"still compiling: {len(pending)} of {len(jobs)} files left, {time.time() - started:.0f} s")
            last = time.time()
        time.sleep(0.05)
    failures = []
    for src, obj, proc in jobs:
        output = proc.stdout.read()
        if proc.returncode != 0:
            failures.append(f"{os.path.basename(src)}:\n{output}")
    if failures:
        shutil.rmtree(work, ignore_errors=True)
        raise KernelBuildError("nvcc failed:\n" + "\n".join(failures))
    partial = target + f".tmp{os.getpid()}"
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", partial,
            *[obj for _, obj, _ in jobs], "-lcudart"]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    shutil.rmtree(work, ignore_errors=True)
    if done.returncode != 0:
        raise KernelBuildError("link failed:\n" + done.stdout)
    os.replace(partial, target)
    for stale in glob.glob(os.path.join(out_dir, "liblia_b200_*.so")):
        if stale != target:
            try:
                os.remove(stale)
            except OSError:
                pass
    log(f"built {os.path.basename(target)} in {time.time() - started:.0f} s")
    return target


_LIBRARY = None


def load() -> ctypes.CDLL:
    """The loaded kernel library; builds it first if needed.  Raises if it cannot be had: the
    engine has no fallback."""
    global _LIBRARY
    if _LIBRARY is None:
        path = build()
        try:
            _LIBRARY = ctypes.CDLL(path)
        except OSError as error:
            raise KernelBuildError(f"cannot load {path}: {error}") from error
    return _LIBRARY


# ---- the host-only library (csrc/host/*.cpp): plain C++, no CUDA, so it also serves the CPU-only tests ----
HOST_DIR = os.path.join(CSRC_DIR, "host")
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]
_HOST_LIBRARY = None


def _host_compiler() -> str:
    for candidate in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if candidate and (os.path.exists(candidate) or shutil.which(candidate)):
            return candidate
    raise KernelBuildError("no C++ compiler found (set CXX); the cache's host library cannot be built")


def host_sources() -> list:
    return sorted(glob.glob(os.path.join(HOST_DIR, "*.cpp")))


def host_library_path() -> str:
    h = hashlib.sha256()
    for path in host_sources() + sorted(glob.glob(os.path.join(HOST_DIR, "*.h"))):
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    return os.path.join(_build_dir(), f"liblia_host_{h.hexdigest()[:16]}.so")


def build_host(verbose: bool = True) -> str:
    target = host_library_path()
    if os.path.exists(target):
        return target
    partial = target + f".tmp{os.getpid()}"
    if verbose:
        print(f"[lia_rs_b200] compiling the host library into {os.path.dirname(target)} (first call only)", file=sys.stderr, flush=True)
    done = subprocess.run([_host_compiler(), *HOST_FLAGS, "-o", partial, *host_sources()],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise KernelBuildError("the host library failed to compile:\n" + done.stdout)
    os.replace(partial, target)
    for stale in glob.glob(os.path.join(os.path.dirname(target), "liblia_host_*.so")):
        if stale != target:
            try:
                os.remove(stale)
            except OSError:
                pass
    return target


def load_host() -> ctypes.CDLL:
    """The loaded host library (the cache's native bookkeeping); builds it first if needed."""
    global _HOST_LIBRARY
    if _HOST_LIBRARY is None:
        path = build_host()
        try:
            _HOST_LIBRARY = ctypes.CDLL(path)
        except OSError as error:
            raise KernelBuildError(f"cannot load {path}: {error}") from error
        _HOST_LIBRARY.lia_host_error.restype = ctypes.c_char_p
        for name in ("lia_pool_create", "lia_cache_create"):
            getattr(_HOST_LIBRARY, name).restype = ctypes.c_void_p
    return _HOST_LIBRARY
