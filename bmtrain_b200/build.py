"""Build the in-tree native libraries.

``python -m bmtrain_b200.build`` compiles every ``csrc/*.cu`` for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) into ``bmtrain_b200/_C.so`` and the
host sources into ``bmtrain_b200/_cpu.so``.  nvcc cross-compiles without a GPU.
(The reference builds one pybind module with CMake for sm_61..sm_86:
``CMakeLists.txt``, ``setup.py:9-112``.)
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-mavx2", "-mfma", "-mf16c"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, log_path=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + res.stdout)
    return res.stdout


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    target = os.path.join(HERE, "_C.so")
    objs, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(obj)
        full = os.path.join(CSRC, src)
        if force or _stale(obj, [full] + headers):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-I", CSRC, "-c", full, "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            outs = list(pool.map(lambda c: _run(c, c[-1] + ".log"), jobs))
        if verbose:
            print("\n".join(outs))
    if jobs or force or _stale(target, objs):
        _run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", target, *objs, "-Xcompiler", "-fPIC"])
    return target


def build_cpu(force: bool = False) -> str:
    target = os.path.join(HERE, "_cpu.so")
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cpp")]
    if sources and (force or _stale(target, sources)):
        _run([os.environ.get("CXX", "g++"), *CXX_FLAGS, "-I", CSRC, "-o", target, *sources, "-lrt"])
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cpu(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", os.path.join(HERE, "_C.so"), "and", os.path.join(HERE, "_cpu.so"))
