"""Compiles the CUDA sources for sm_100a into in-tree shared libraries.

    python -m opennn_b200._build            # build what is out of date
    python -m opennn_b200._build --force

libonn_b200.so       kernels + C ABI (include/onn_b200.h)
libonn_b200_host.so  C++ host mirror of the OpenNN interfaces + its driver ABI (include/onn_b200_host.h)

nvcc cross-compiles without a GPU; the libraries are git-ignored build products.
"""

from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "lib")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]


def _nccl_dirs():
    site = sysconfig.get_paths()["purelib"]
    base = os.path.join(site, "nvidia", "nccl")
    return os.path.join(base, "include"), os.path.join(base, "lib")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + result.stdout + result.stderr)
    return result.stdout + result.stderr


def _headers(directory):
    found = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    for f in os.listdir(directory):
        if f.endswith((".h", ".cuh", ".hpp")):
            found.append(os.path.join(directory, f))
    return found


def _compile_all(directory, suffixes, extra, tag, force, verbose):
    sources = sorted(f for f in os.listdir(directory) if f.endswith(suffixes))
    headers = _headers(directory)
    jobs, objects = [], []
    for name in sources:
        src = os.path.join(directory, name)
        obj = os.path.join(OBJ, tag + "_" + os.path.splitext(name)[0] + ".o")
        objects.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append([NVCC] + ARCH + COMMON + extra + ["-c", src, "-o", obj])
    if jobs:
        if verbose:
            print(f"[opennn_b200] compiling {len(jobs)} file(s) for sm_100a ({tag})", file=sys.stderr)
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    return objects, bool(jobs)


def build(force: bool = False, verbose: bool = True) -> dict:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    nccl_inc, nccl_lib = _nccl_dirs()

    kernels = os.path.join(LIB, "libonn_b200.so")
    objects, changed = _compile_all(CSRC, (".cu",), ["-I", nccl_inc], "k", force, verbose)
    if changed or not os.path.exists(kernels):
        _run([NVCC] + ARCH + ["-shared", "-o", kernels] + objects +
             ["-L", nccl_lib, "-l:libnccl.so.2", "-Xlinker", "-rpath", "-Xlinker", nccl_lib])

    host = os.path.join(LIB, "libonn_b200_host.so")
    if os.path.isdir(HOST) and any(f.endswith(".cpp") for f in os.listdir(HOST)):
        objects, host_changed = _compile_all(HOST, (".cpp",), ["-x", "cu"], "h", force, verbose)
        if host_changed or changed or not os.path.exists(host):
            _run([NVCC] + ARCH + ["-shared", "-o", host] + objects +
                 ["-L", LIB, "-lonn_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"])
    return {"kernels": kernels, "host": host if os.path.exists(host) else None}


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
