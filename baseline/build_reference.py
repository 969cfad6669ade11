#!/usr/bin/env python3
"""Builds the unmodified reference (cosmonomic/pulsar) into ``baseline/_ref`` without xmake.

    python baseline/build_reference.py --src <checkout of cosmonomic/pulsar>

The reference's own build is a wheel hook that runs xmake (pulsar/hatch_build.py:12-36):
a static library of every ``pulsar-core/src/**.cu`` and ``**.cpp`` (one digest source)
with ``pulsar-core/inc`` on the include path (pulsar-core/xmake.lua:26-47), linked with
``pulsar/ext/*.cpp`` against libtorch into one shared object named ``pulsar_core.so``
(pulsar/xmake.lua:16-26) that lands at the top of the ``pulsar`` package
(pulsar/src/pulsar/core/__init__.py:12-33).  This script follows that description with plain
nvcc and g++: the same sources, unchanged, the same include path, the same output name and
place.  Two flags differ from xmake.lua because the local toolchain has no equivalent:
nvcc 12.9 knows no ``-std=c++23`` (the CUDA sources are compiled as C++20, which they are
within), and the code is generated for sm_100a instead of "native" (there may be no GPU in
the build box).  The Python package is copied as it is; nothing of this repository is on
the reference's path.

The result is loaded with ``sys.path.insert(0, "baseline/_ref"); import pulsar.core``, which
registers ``torch.classes.pulsar.Engine`` and ``torch.ops.pulsar.*``.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("PULSAR_REFERENCE_SRC"), help="checkout of cosmonomic/pulsar")
    ap.add_argument("--jobs", type=int, default=max(1, (os.cpu_count() or 4) // 2))
    args = ap.parse_args()
    if not args.src or not os.path.isdir(os.path.join(args.src, "pulsar-core", "src")):
        print("build_reference: --src (or PULSAR_REFERENCE_SRC) must name a checkout of cosmonomic/pulsar", file=sys.stderr)
        return 2
    import torch
    src = os.path.abspath(args.src)
    core = os.path.join(src, "pulsar-core")
    torch_dir = os.path.dirname(torch.__file__)
    import sysconfig
    includes = ["-I" + os.path.join(core, "inc"), "-I" + os.path.join(torch_dir, "include"),
                "-I" + os.path.join(torch_dir, "include", "torch", "csrc", "api", "include"),
                "-I" + sysconfig.get_paths()["include"], "-I/usr/local/cuda/include"]
    obj_dir = os.path.join(OUT, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    cuda = sorted(glob.glob(os.path.join(core, "src", "**", "*.cu"), recursive=True))
    cpp = sorted(f for f in glob.glob(os.path.join(core, "src", "**", "*.cpp"), recursive=True)
                 if not os.path.basename(f).startswith("digest_"))
    cpp.append(os.path.join(core, "src", "digest_sha256.cpp"))          # xmake.lua's default option digest=sha256
    cpp += sorted(glob.glob(os.path.join(src, "pulsar", "ext", "*.cpp")))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    jobs = []
    for f in cuda:
        obj = os.path.join(obj_dir, os.path.relpath(f, src).replace(os.sep, "_") + ".o")
        jobs.append((f, obj, [nvcc, "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-DNDEBUG",
                              "-Xcompiler=-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda", *includes,
                              "-c", f, "-o", obj]))
    for f in cpp:
        obj = os.path.join(obj_dir, os.path.relpath(f, src).replace(os.sep, "_") + ".o")
        jobs.append((f, obj, ["g++", "-std=c++23", "-O3", "-DNDEBUG", "-fPIC", *includes, "-c", f, "-o", obj]))
    t0 = time.time()
    log = []

    def run(job):
        f, obj, cmd = job
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        print(f"[build_reference] {os.path.relpath(f, src)}: {'ok' if r.returncode == 0 else 'FAILED'} "
              f"({time.time() - t0:.0f}s)", flush=True)
        return f, r.returncode, r.stdout

    with ThreadPoolExecutor(args.jobs) as pool:
        results = list(pool.map(run, jobs))
    failed = [(f, out) for f, rc, out in results if rc != 0]
    if failed:
        for f, out in failed:
            first = next((ln for ln in out.splitlines() if "error" in ln), out[:400])
            print(f"[build_reference] first error in {os.path.relpath(f, src)}: {first}", file=sys.stderr)
        return 1
    package = os.path.join(OUT, "pulsar")
    if os.path.isdir(package):
        shutil.rmtree(package)
    shutil.copytree(os.path.join(src, "pulsar", "src", "pulsar"), package)
    for folder, _, names in os.walk(package):            # a read-only checkout gives read-only copies
        os.chmod(folder, 0o755)
        for n in names:
            os.chmod(os.path.join(folder, n), 0o644)
    lib = os.path.join(package, "pulsar_core.so")
    link = ["g++", "-shared", "-o", lib, *[obj for _, obj, _ in jobs], "-L" + os.path.join(torch_dir, "lib"),
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-L/usr/local/cuda/lib64", "-lcudart", "-lcrypto"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        print("[build_reference] link failed:\n" + r.stdout, file=sys.stderr)
        return 1
    with open(os.path.join(OUT, "BUILD.txt"), "w") as f:
        f.write(f"built from {len(cuda)} CUDA and {len(cpp)} C++ sources of the reference, unchanged, in "
                f"{time.time() - t0:.0f}s; torch {torch.__version__}; nvcc -std=c++20 sm_100a, g++ -std=c++23\n")
    print(f"[build_reference] {lib} ({os.path.getsize(lib) >> 10} KiB, {time.time() - t0:.0f}s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
