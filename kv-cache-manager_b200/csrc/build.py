"""Builds the two native libraries of the package at first use and loads them.

* ``kvcm_core``  : the CPU core (C++17 + pybind11): allocator, prefix cache, cache managers,
                   state slots, scheduler, batch builder.  Compiled with g++.
* ``libkvcm_cuda``: every CUDA kernel, compiled by nvcc for sm_100a only
                   (``-gencode arch=compute_100a,code=sm_100a``), exported with a C ABI and
                   loaded through ctypes.  nvcc cross-compiles without a GPU.

Objects live in ``<package>/_build`` (or, when the package folder is read-only, in a per-user
folder under the system temp dir).  A library is rebuilt when the hash of its sources and flags
changes.  While compiling, a line is printed to stderr for every finished object so that a first
call never sits silent.  There is no fallback: a failed build raises with the compiler's output.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.dirname(_HERE)

CORE_SOURCES = ["core/block_allocator.cpp", "core/prefix_cache.cpp", "core/kv_manager.cpp",
                "core/paged_manager.cpp", "core/scheduler.cpp", "core/batch.cpp",
                "core/safetensors.cpp", "core/native_engine.cpp", "core/bindings.cpp"]
CUDA_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[kvcm build] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    """``<package>/_build`` when it can be written, else a per-user temp folder."""
    override = os.environ.get("KVCM_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(_PKG, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"kvcm_build_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise BuildError("no writable build folder (tried: " + ", ".join(candidates) + ")")


def cuda_sources() -> List[str]:
    d = os.path.join(_HERE, "cuda")
    return sorted(os.path.join("cuda", f) for f in os.listdir(d) if f.endswith(".cu"))


def _digest(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    h.update("\0".join(flags).encode())
    dirs = sorted({os.path.dirname(os.path.join(_HERE, p)) for p in paths} | {os.path.join(_HERE, "include")})
    files = set(os.path.join(_HERE, p) for p in paths)
    for d in dirs:                                  # headers count too
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                files.add(os.path.join(d, f))
    for f in sorted(files):
        h.update(os.path.relpath(f, _HERE).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed (exit {p.returncode}):\n$ {' '.join(cmd)}\n{p.stdout}")


class _Lock:
    def __init__(self, path: str):
        self.path = path

    def __enter__(self):
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *a):
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _compile_all(compiler: str, flags: List[str], sources: List[str], objdir: str,
                 tag: str) -> List[str]:
    os.makedirs(objdir, exist_ok=True)
    objs, jobs = [], []
    for s in sources:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        jobs.append((s, [compiler, *flags, "-c", os.path.join(_HERE, s), "-o", o]))
    t0 = time.time()
    workers = max(1, min(len(jobs), os.cpu_count() or 1, 8))
    with ThreadPoolExecutor(workers) as ex:
        futs = {ex.submit(_run, cmd, f"compiling {s}"): s for s, cmd in jobs}
        done = 0
        for f in as_completed(futs):
            f.result()
            done += 1
            _log(f"{tag}: compiled {futs[f]} ({done}/{len(jobs)}, {time.time() - t0:.0f}s)")
    return objs


def _build(lib_name: str, sources: List[str], compiler: str, flags: List[str],
           link: List[str], tag: str) -> str:
    bd = build_dir()
    digest = _digest(sources, [compiler, *flags, *link])
    lib = os.path.join(bd, lib_name)
    stamp = lib + ".stamp"
    with _Lock(os.path.join(bd, f".{tag}.lock")):
        if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == digest:
            return lib
        if shutil.which(compiler) is None:
            raise BuildError(f"'{compiler}' not found on PATH; cannot build {lib_name}")
        _log(f"{tag}: building {lib_name} in {bd} ({len(sources)} sources; first call only)")
        objs = _compile_all(compiler, flags, sources, os.path.join(bd, f"obj_{tag}_{digest}"), tag)
        tmp = lib + f".tmp{os.getpid()}"
        _run([compiler, "-shared", "-o", tmp, *objs, *link], f"linking {lib_name}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(digest)
        shutil.rmtree(os.path.join(bd, f"obj_{tag}_{digest}"), ignore_errors=True)
        _log(f"{tag}: {lib_name} ready")
    return lib


_core_module = None
_cuda_lib: Optional[ctypes.CDLL] = None


def build_core() -> str:
    import pybind11
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    flags = CXX_FLAGS + ["-I" + sysconfig.get_paths()["include"], "-I" + pybind11.get_include()]
    return _build("kvcm_core" + suffix, CORE_SOURCES, "g++", flags, [], "core")


def load_core():
    """The ``kvcm_core`` extension module (built on first call)."""
    global _core_module
    if _core_module is None:
        path = build_core()
        spec = importlib.util.spec_from_file_location("kvcm_core", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules.setdefault("kvcm_core", mod)
        _core_module = mod
    return _core_module


def build_cuda() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    flags = NVCC_FLAGS + CUDA_ARCH_FLAGS
    return _build("libkvcm_cuda.so", cuda_sources(), nvcc, flags, ["-lcudart", "-lcuda", "-lcublas"], "cuda")


def load_cuda() -> ctypes.CDLL:
    """``libkvcm_cuda.so`` through ctypes (built on first call).  Raises if it cannot be built
    or loaded: there is no other implementation of the kernels to fall back to."""
    global _cuda_lib
    if _cuda_lib is None:
        path = build_cuda()
        try:
            _cuda_lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
    return _cuda_lib
