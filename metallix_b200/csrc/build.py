"""Builds and loads the native code: the CUDA kernels (one shared library,
called through ctypes) and the host runtime (a pybind11 module).

Both are compiled at first use into ``metallix_b200/_build`` (or, when that
folder cannot be written, into a per-user folder under the system's temporary
directory), keyed by a hash of their sources so that an edit rebuilds them.
nvcc targets sm_100a only. While a compile runs a line is printed to stderr
every few seconds.
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
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
_KERNEL_DIR = os.path.join(_HERE, "kernels")
_HOST_DIR = os.path.join(_HERE, "host")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]

_kernels: Optional[ctypes.CDLL] = None
_host = None
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[metallix_b200] {message}", file=sys.stderr, flush=True)


def build_dir() -> str:
    preferred = os.path.join(os.path.dirname(_HERE), "_build")
    override = os.environ.get("METALLIX_B200_BUILD_DIR")
    for candidate in ([override] if override else []) + [preferred]:
        try:
            os.makedirs(candidate, exist_ok=True)
            probe = os.path.join(candidate, f".write_probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return candidate
        except OSError:
            continue
    fallback = os.path.join(tempfile.gettempdir(), f"metallix_b200_build_{os.getuid()}")
    os.makedirs(fallback, exist_ok=True)
    return fallback


def _sources(folder: str, suffixes) -> List[str]:
    return sorted(os.path.join(folder, name) for name in os.listdir(folder)
                  if name.endswith(tuple(suffixes)))


def _digest(paths: List[str], flags: List[str]) -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(flags).encode())
    for path in paths:
        digest.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            digest.update(handle.read())
    return digest.hexdigest()


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no fallback")


def _run(command: List[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    result = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=env)
    if result.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(command)}\n{result.stdout}")


class _Heartbeat:
    """Prints a line now and then while a compile runs."""

    def __init__(self, what: str):
        self.what, self.started = what, time.time()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._beat, daemon=True)

    def _beat(self) -> None:
        while not self._stop.wait(5.0):
            _say(f"still compiling {self.what} ({time.time() - self.started:.0f} s)")

    def __enter__(self):
        _say(f"compiling {self.what} (first use; sm_100a)")
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join()
        if exc[0] is None:
            _say(f"compiled {self.what} in {time.time() - self.started:.0f} s")


def _locked(path: str):
    handle = open(path + ".lock", "w")
    fcntl.flock(handle, fcntl.LOCK_EX)
    return handle


def _build_kernels(out_dir: str) -> str:
    sources = _sources(_KERNEL_DIR, (".cu",))
    headers = _sources(_KERNEL_DIR, (".cuh", ".h"))
    timeline = os.environ.get("METALLIX_B200_TIMELINE", "") not in ("", "0")
    flags = NVCC_FLAGS + (["-DMXB_TIMELINE"] if timeline else [])
    tag = _digest(sources + headers, flags)
    # the build that records the kernels' timeline is a library of its own
    library = os.path.join(out_dir, "_mxb_kernels_timeline.so" if timeline else "_mxb_kernels.so")
    stamp = library + ".stamp"
    lock = _locked(library)
    try:
        if os.path.exists(library) and os.path.exists(stamp) and open(stamp).read() == tag:
            return library
        nvcc = _nvcc()
        object_dir = os.path.join(out_dir, "obj_timeline" if timeline else "obj")
        os.makedirs(object_dir, exist_ok=True)
        with _Heartbeat(f"{len(sources)} CUDA kernel files"):
            def compile_one(source: str) -> str:
                # Objects are keyed by their own source, so an edit of one
                # file recompiles one file.
                own = _digest([source] + headers, flags)[:16]
                target = os.path.join(object_dir,
                                      os.path.basename(source)[:-3] + f".{own}.o")
                if not os.path.exists(target):
                    partial = target + f".{os.getpid()}.tmp"
                    _run([nvcc, *flags, "-I", _KERNEL_DIR, "-c", source, "-o", partial],
                         os.path.basename(source))
                    os.replace(partial, target)
                return target
            with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
                objects = list(pool.map(compile_one, sources))
            partial = library + f".{os.getpid()}.tmp"
            _run([nvcc, "-shared", "-o", partial, *objects, "-gencode",
                  "arch=compute_100a,code=sm_100a"], "kernel library")
            os.replace(partial, library)
            with open(stamp, "w") as handle:
                handle.write(tag)
            # Objects of earlier versions of the sources are of no use any more.
            kept = {os.path.basename(path) for path in objects}
            for name in os.listdir(object_dir):
                if name.endswith(".o") and name not in kept:
                    try:
                        os.remove(os.path.join(object_dir, name))
                    except OSError:
                        pass
        return library
    finally:
        lock.close()


def _build_host(out_dir: str) -> str:
    sources = _sources(_HOST_DIR, (".cpp",))
    headers = _sources(_HOST_DIR, (".hpp", ".h"))
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    tag = _digest(sources + headers, HOST_FLAGS + [suffix])
    library = os.path.join(out_dir, "_mxb_host" + suffix)
    stamp = library + ".stamp"
    lock = _locked(library)
    try:
        if os.path.exists(library) and os.path.exists(stamp) and open(stamp).read() == tag:
            return library
        try:
            import pybind11
        except ImportError as error:
            raise BuildError(f"pybind11 is needed to build the host runtime: {error}") from None
        compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not compiler:
            raise BuildError("no C++ compiler (g++) was found for the host runtime")
        with _Heartbeat("the host runtime (cache manager, scheduler)"):
            partial = library + f".{os.getpid()}.tmp"
            _run([compiler, *HOST_FLAGS, "-I", sysconfig.get_paths()["include"], "-I",
                  pybind11.get_include(), "-I", _HOST_DIR, *sources, "-o", partial],
                 "host runtime")
            os.replace(partial, library)
            with open(stamp, "w") as handle:
                handle.write(tag)
        return library
    finally:
        lock.close()


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library, built if needed. Raises ``BuildError`` if it
    cannot be built: there is no other implementation to fall back to."""
    global _kernels
    with _lock:
        if _kernels is None:
            _kernels = ctypes.CDLL(_build_kernels(build_dir()))
        return _kernels


def host():
    """The pybind11 module with ``CacheManager`` and ``Scheduler``."""
    global _host
    with _lock:
        if _host is None:
            path = _build_host(build_dir())
            spec = importlib.util.spec_from_file_location("_mxb_host", path)
            module = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(module)
            _host = module
        return _host


def build_all() -> None:
    """Compiles everything (used by the build check)."""
    out_dir = build_dir()
    _build_host(out_dir)
    _build_kernels(out_dir)
