"""Builds the CUDA sources of this folder into one shared library for sm_100a and loads it.

The library has a C interface (see the ``PB_EXPORT`` functions of each ``.cu``) and is
loaded with ``ctypes``; it does not link against PyTorch, so a source file compiles in
seconds and the same symbols serve callers that have no PyTorch at all.  The build is
kept beside the sources (``_build/``); when that folder cannot be written, a folder
under the system's temporary directory is used.  A build is reused while the hash of
sources and flags matches.

The reference compiles for whatever GPU is in the build box
(pulsar-core/xmake.lua:28, add_cugencodes("native")); this library is sm_100a only.
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
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
# PULSAR_CHECK_BOUNDS=1: the debug build, in a library of its own beside the ordinary one.  Its kernels check every
# page id and slot they take from an index array against the pool's size, record a bad one in an error word and skip
# the access (common.cuh: PoolBounds).
CHECK_BOUNDS = os.environ.get("PULSAR_CHECK_BOUNDS", "0") not in ("", "0")
LIB_NAME = "libpulsar_b200_checked.so" if CHECK_BOUNDS else "libpulsar_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
] + (["-DPB_CHECK_BOUNDS"] if CHECK_BOUNDS else [])   # precise math: never -use_fast_math

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def find_nvcc() -> str:
    for cand in (os.environ.get("PULSAR_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found (set PULSAR_NVCC or put nvcc on PATH): the CUDA extension cannot be built, "
                     "and this engine has no other execution path")


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        path = os.path.join(tempfile.gettempdir(), f"pulsar_b200_build_{os.getuid()}")
        os.makedirs(path, exist_ok=True)
        return path


def _say(msg: str) -> None:
    print(f"[pulsar_b200 build] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False, extra_flags: Optional[List[str]] = None) -> str:
    """Compile what is stale and return the library's path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "stamp_checked.txt" if CHECK_BOUNDS else "stamp.txt")
    digest = _digest()
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == digest:
                return lib_path
    nvcc = find_nvcc()
    srcs = sources()
    flags = NVCC_FLAGS + (extra_flags or [])
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    procs, logs = [], {}
    for name in srcs:
        obj = os.path.join(out_dir, name[:-3] + (".checked.o" if CHECK_BOUNDS else ".o"))
        cmd = [nvcc, *flags, "-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
        # the compiler's messages go to a file: a pipe that nobody reads until the process ends blocks a compiler
        # that has more to say than the pipe holds
        log = open(obj + ".log", "w+")
        logs[name] = log
        procs.append((name, obj, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL)))
    pending = {name for name, _, _ in procs}
    last = time.time()
    outputs = {}
    while pending:
        for name, _, p in procs:
            if name in pending and p.poll() is not None:
                logs[name].seek(0)
                outputs[name] = logs[name].read()
                logs[name].close()
                pending.discard(name)
                if verbose:
                    _say(f"  {name} done ({time.time() - t0:.0f}s, {len(pending)} left)")
        if pending:
            time.sleep(0.2)
            if verbose and time.time() - last > 10:
                _say(f"  still compiling: {', '.join(sorted(pending))} ({time.time() - t0:.0f}s)")
                last = time.time()
    failed = [(n, outputs[n]) for n, _, p in procs if p.returncode != 0]
    if failed:
        raise BuildError("nvcc failed:\n" + "\n".join(f"--- {n} ---\n{o}" for n, o in failed))
    if extra_flags and verbose:
        for n in srcs:
            if outputs[n].strip():
                print(outputs[n], file=sys.stderr)
    tmp_lib = lib_path + f".tmp{os.getpid()}"
    link = [nvcc, "-shared", "-o", tmp_lib, *[o for _, o, _ in procs], "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError("link failed:\n" + r.stdout)
    os.replace(tmp_lib, lib_path)
    with open(stamp_path, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
    return lib_path


def library() -> ctypes.CDLL:
    """The loaded library; builds it on first use.  Raises if it cannot be had: there
    is no fallback path."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                _lib = ctypes.CDLL(build())
    return _lib


# ------------------------------------------------------------------ the host runtime (plain C++, no CUDA)
HOST_DIR = os.path.join(HERE, "host")
HOST_LIB_NAME = "libpulsar_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall"]
_host_lib: Optional[ctypes.CDLL] = None


def find_cxx() -> str:
    for cand in (os.environ.get("PULSAR_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                 shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (set PULSAR_CXX or put g++ on PATH): the host runtime cannot be built")


def build_host(verbose: bool = True, force: bool = False) -> str:
    """Compile the sources of ``host/`` into one shared library (cache accounting, step packer, scheduler:
    see the ``PH_EXPORT`` functions) and return its path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, HOST_LIB_NAME)
    stamp_path = os.path.join(out_dir, "host_stamp.txt")
    names = sorted(f for f in os.listdir(HOST_DIR) if f.endswith((".cpp", ".h")))
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    for name in names:
        h.update(name.encode())
        with open(os.path.join(HOST_DIR, name), "rb") as f:
            h.update(f.read())
    digest = h.hexdigest()[:16]
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == digest:
                return lib_path
    cxx = find_cxx()
    if verbose:
        _say(f"compiling the host runtime ({len([n for n in names if n.endswith('.cpp')])} C++ sources) into {out_dir}")
    t0 = time.time()
    tmp_lib = lib_path + f".tmp{os.getpid()}"
    cmd = [cxx, *HOST_FLAGS, "-I", HOST_DIR, "-o", tmp_lib, *[os.path.join(HOST_DIR, n) for n in names if n.endswith(".cpp")]]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError(f"{cxx} failed:\n" + r.stdout)
    os.replace(tmp_lib, lib_path)
    with open(stamp_path, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"built {HOST_LIB_NAME} in {time.time() - t0:.0f}s")
    return lib_path


def host_library() -> ctypes.CDLL:
    """The loaded host runtime; builds it on first use."""
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                _host_lib = ctypes.CDLL(build_host())
    return _host_lib


if __name__ == "__main__":
    print(build_host(force="--force" in sys.argv))
    print(build(force="--force" in sys.argv, extra_flags=["-Xptxas", "-v"] if "-v" in sys.argv else None))
