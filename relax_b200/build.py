"""Builds ``librelax_b200.so`` in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: ``python relax_b200/build.py [--force]``.  Objects go to ``relax_b200/build/``; a source
is recompiled only when it, or any header next to it, is newer than its object.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_PKG, "csrc")
_OBJ = os.path.join(_PKG, "build")
LIB_PATH = os.path.join(_PKG, "librelax_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _host_compiler_flags() -> list:
    # a wrapper gcc earlier on PATH lacks some runtime specs; prefer the system compiler
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def sources() -> list:
    return sorted(glob.glob(os.path.join(_SRC, "*.cu")) + glob.glob(os.path.join(_SRC, "*.cc")))


def _stale(src: str, obj: str, headers_mtime: float) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return os.path.getmtime(src) > t or headers_mtime > t


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(_OBJ, exist_ok=True)
    headers = glob.glob(os.path.join(_SRC, "*.h")) + glob.glob(os.path.join(_SRC, "*.cuh")) + \
        glob.glob(os.path.join(_PKG, "..", "include", "*.h"))
    hm = max([os.path.getmtime(h) for h in headers] + [0.0])
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(_OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hm):
            cmd = [nvcc] + NVCC_FLAGS + _host_compiler_flags() + ["-x", "cu", "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose and (r.stdout or r.stderr):
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if jobs or not os.path.exists(LIB_PATH):
        link = [nvcc, "-shared", "-o", LIB_PATH] + objs + _host_compiler_flags() + \
            ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s\n%s" % (" ".join(link), r.stdout, r.stderr))
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
