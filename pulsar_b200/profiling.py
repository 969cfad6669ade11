"""Where a step's time goes: device time per kernel class and host time per phase.

``PULSAR_PROF=1`` turns it on.  Every launch of this library's kernels (and the library products beside them) is
then bracketed by two CUDA events on the launching stream, host phases (plan, pack, launch, read) by wall-clock
scopes, and a table of both is printed to standard error when the process exits (or by ``report()``).  Steps are
not captured into CUDA graphs while profiling, since events inside a captured graph time nothing; the figures are
therefore those of eager launches, kernel by kernel (without the overlap that programmatic dependent launch gives
inside a graph: compare shares, not sums).  Off, none of this costs anything: the wrappers are not installed.

The reference has opt-in host phase timers only, compiled in with its ``prof`` option and printed at exit
(pulsar-core/inc/pulsar/profiling.hpp:21-107, hooked at pulsar-core/src/runtime/engine.cpp:732), and explicitly no
device timers (:8-10).
"""
from __future__ import annotations

import atexit
import os
import sys
import time
from contextlib import contextmanager
from typing import Dict, List, Tuple

ENABLED = os.environ.get("PULSAR_PROF", "0") not in ("", "0")

_kernel_events: List[Tuple[str, object, object]] = []
_kernel_totals: Dict[str, List[float]] = {}        # class -> [launches, milliseconds]
_host_totals: Dict[str, List[float]] = {}          # phase -> [entries, seconds]
_MAX_PENDING = 20000


def _drain() -> None:
    """Turn recorded event pairs into totals (waits for the device)."""
    if not _kernel_events:
        return
    import torch
    torch.cuda.synchronize()
    for name, e0, e1 in _kernel_events:
        slot = _kernel_totals.setdefault(name, [0, 0.0])
        slot[0] += 1
        slot[1] += e0.elapsed_time(e1)
    _kernel_events.clear()


@contextmanager
def kernel(name: str):
    """Device time of what is launched inside, under the class ``name``."""
    if not ENABLED:
        yield
        return
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    try:
        yield
    finally:
        e1.record()
        _kernel_events.append((name, e0, e1))
        if len(_kernel_events) >= _MAX_PENDING:
            _drain()


def timed_launcher(name: str, f):
    """``f`` (a launcher of the CUDA library) bracketed by events, under its own name."""
    label = name[3:] if name.startswith("pb_") else name

    def call(*args):
        with kernel(label):
            return f(*args)
    return call


@contextmanager
def scope(name: str):
    """Host wall-clock time of a phase."""
    if not ENABLED:
        yield
        return
    t0 = time.perf_counter()
    try:
        yield
    finally:
        slot = _host_totals.setdefault(name, [0, 0.0])
        slot[0] += 1
        slot[1] += time.perf_counter() - t0


def reset() -> None:
    _drain()
    _kernel_totals.clear()
    _host_totals.clear()


def totals() -> Tuple[Dict[str, List[float]], Dict[str, List[float]]]:
    _drain()
    return dict(_kernel_totals), dict(_host_totals)


def report(file=None) -> None:
    if not ENABLED:
        return
    file = file or sys.stderr
    try:
        kernels, host = totals()
    except Exception as exc:                      # the device may be gone at exit
        print(f"[pulsar_b200 prof] no device figures: {exc}", file=file)
        kernels, host = dict(_kernel_totals), dict(_host_totals)
    if kernels:
        whole = sum(ms for _, ms in kernels.values()) or 1.0
        print("[pulsar_b200 prof] device time per kernel class (CUDA events, eager launches)", file=file)
        print(f"  {'class':44s} {'launches':>9s} {'ms':>10s} {'us each':>9s} {'share':>7s}", file=file)
        for name, (n, ms) in sorted(kernels.items(), key=lambda kv: -kv[1][1]):
            print(f"  {name:44s} {int(n):9d} {ms:10.3f} {ms / n * 1e3:9.1f} {ms / whole:7.1%}", file=file)
    if host:
        print("[pulsar_b200 prof] host time per phase (wall clock)", file=file)
        print(f"  {'phase':44s} {'entries':>9s} {'ms':>10s} {'us each':>9s}", file=file)
        for name, (n, sec) in sorted(host.items(), key=lambda kv: -kv[1][1]):
            print(f"  {name:44s} {int(n):9d} {sec * 1e3:10.3f} {sec / n * 1e6:9.1f}", file=file)


if ENABLED:
    atexit.register(report)
