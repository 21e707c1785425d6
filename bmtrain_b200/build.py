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
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cpp") and f not in _OWN_LIBRARY]
    if sources and (force or _stale(target, sources)):
        _run([os.environ.get("CXX", "g++"), *CXX_FLAGS, "-I", CSRC, "-o", target, *sources, "-lrt"])
    return target


_OWN_LIBRARY = {"nccl_comm.cpp"}  # sources that are linked into a library of their own


def _nccl_paths():
    """(include dir, library file) of the NCCL this process would load: the pip package next to torch when present (the
    one torch itself links), else the system install."""
    try:
        import importlib.util

        spec = importlib.util.find_spec("nvidia.nccl")
        for root in (spec.submodule_search_locations if spec else []):
            inc, lib = os.path.join(root, "include"), os.path.join(root, "lib", "libnccl.so.2")
            if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(lib):
                return inc, lib
    except Exception:
        pass
    for inc, lib in (("/usr/include", "/usr/lib/x86_64-linux-gnu/libnccl.so.2"), ("/usr/local/cuda/include", "/usr/local/cuda/lib64/libnccl.so.2")):
        if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(lib):
            return inc, lib
    return None, None


def build_nccl(force: bool = False) -> str:
    """``_nccl.so``: the C++ communicator wrapper (``csrc/nccl_comm.cpp``), linked against the NCCL shared library."""
    target = os.path.join(HERE, "_nccl.so")
    src = os.path.join(CSRC, "nccl_comm.cpp")
    inc, lib = _nccl_paths()
    if inc is None:
        return ""   # no NCCL on this machine: the wrapper is optional (torch.distributed carries the collectives)
    if force or _stale(target, [src]):
        cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include") if os.path.sep in _nvcc() else "/usr/local/cuda/include"
        _run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", inc, "-I", cuda_inc,
              "-o", target, src, lib, "-Wl,-rpath," + os.path.dirname(lib)])
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cpu(force)
    build_nccl(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", os.path.join(HERE, "_C.so"), "and", os.path.join(HERE, "_cpu.so"))
