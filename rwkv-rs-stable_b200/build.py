"""Builds ``librwkv7_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

Run as ``python build.py`` from this directory or call :func:`build_library`.
Objects go to ``build/`` next to this file; the shared library is written beside
this file so that it is found by :mod:`ctypes` without installation.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "librwkv7_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    # The explicit -gencode form: plain -arch=sm_100a also emits a compute_100
    # target for which ptxas rejects tcgen05.
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build librwkv7_b200.so")
    return nvcc


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


# Named variants of the library: the same sources with extra preprocessor flags, built into their own object
# directory and written beside the product library as librwkv7_b200_<variant>.so.
VARIANTS = {
    "checked": ["-DRWKV7_CHECKED", "-DRWKV7_NVTX"],   # device-side index checks + NVTX ranges (tests only)
}


def build_variant(name: str, force: bool = False) -> str:
    return build_library(force=force, extra_flags=VARIANTS[name], variant=name)


def build_library(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
                  variant: str | None = None) -> str:
    BUILD = os.path.join(HERE, "build", variant) if variant else os.path.join(HERE, "build")
    LIB = os.path.join(HERE, f"librwkv7_b200_{variant}.so") if variant else os.path.join(HERE, "librwkv7_b200.so")
    os.makedirs(BUILD, exist_ok=True)
    nvcc = _nvcc()
    # nvcc's host compiler: the environment's CC/CXX may point at a compiler
    # without the usual runtime pieces, so name the system one explicitly.
    host = ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    flags = NVCC_FLAGS + (extra_flags or [])
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(BUILD, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc, *host, *flags, "-x", "cu", "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, res

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for cmd, res in ex.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    if force or jobs or _newer(LIB, objs):
        cmd = [nvcc, *host, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
