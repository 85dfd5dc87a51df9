"""Compile the CUDA sources of this package into ``libdartkv_b200.so`` (sm_100a only).

``python dartkv_b200/build.py [--force] [-v]``; ``-v`` prints ptxas resource usage.  Extra nvcc flags can be
passed in ``DARTKV_NVCC_FLAGS`` (the decode kernels have build-time knobs for timing experiments: unroll factors
``-DPEROP_QK_UNROLL=`` / ``-DFUSED_PV_UNROLL=`` ..., and parts that can be compiled out, ``-DFUSED_SKIP_QK``,
``-DFUSED_SKIP_PV``, ``-DFUSED_SKIP_SETUP``, ``-DDENSE_SKIP``; a library built with the latter computes garbage).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PACKAGE_DIR, "csrc")
LIB_PATH = os.path.join(PACKAGE_DIR, "libdartkv_b200.so")
SOURCES = ("quantize.cu", "cache_append.cu", "append_fast.cu", "decode_attention.cu", "decode_fast.cu", "decode_fused32.cu",
           "decode_wide.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
)


def _nvcc() -> str:
    for candidate in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; the dartkv_b200 kernels need the CUDA toolkit to build")


def _stale(sources) -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    headers = [os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith(".cuh")]
    deps = list(sources) + headers + [os.path.join(PACKAGE_DIR, "..", "include", "dartkv_b200.h")]
    return any(os.path.exists(p) and os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the shared library in-tree and return its path (no-op when up to date)."""

    sources = [os.path.join(CSRC, name) for name in SOURCES if os.path.exists(os.path.join(CSRC, name))]
    if not force and not _stale(sources):
        return LIB_PATH
    objects = []
    build_dir = os.path.join(PACKAGE_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in sources:
        obj = os.path.join(build_dir, os.path.basename(src) + ".o")
        objects.append(obj)
        cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("DARTKV_NVCC_FLAGS", "").split(), "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if out.strip() and (verbose or proc.returncode):
            print(out, file=sys.stderr)
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the compiler output above")
    link = [_nvcc(), "-shared", "-o", LIB_PATH, *objects, "-lcudart"]
    subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
