"""Packaging: ``pip install .`` (or ``python setup.py build_ext --inplace``) compiles the native libraries with
``bmtrain_b200/build.py`` -- nvcc for sm_100a only, g++ for the host library -- and ships them inside the package.

Environment switches: ``NVCC`` / ``CXX`` pick the compilers, ``BMT_BUILD_FORCE=1`` rebuilds everything,
``BMT_SKIP_NATIVE=1`` packages the Python sources alone (CPU-only development installs).
(The reference drives CMake from ``setup.py:9-112`` for sm_61..sm_86 and links NCCL at build time.)
"""
import importlib.util
import os

from setuptools import Extension, find_packages, setup
from setuptools.command.build_ext import build_ext

ROOT = os.path.dirname(os.path.abspath(__file__))


def _load_builder():
    # load build.py by path: importing the package would pull in torch before the install has finished
    spec = importlib.util.spec_from_file_location("_bmt_build", os.path.join(ROOT, "bmtrain_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class NativeBuild(build_ext):
    """Runs the in-tree build script; the two shared objects are package data, not setuptools extensions."""

    def run(self):
        if os.environ.get("BMT_SKIP_NATIVE") == "1":
            return
        builder = _load_builder()
        builder.build_all(force=os.environ.get("BMT_BUILD_FORCE") == "1")
        if not self.inplace:
            dst = os.path.join(self.build_lib, "bmtrain_b200")
            os.makedirs(dst, exist_ok=True)
            for name in ("_C.so", "_cpu.so"):
                src = os.path.join(ROOT, "bmtrain_b200", name)
                if os.path.exists(src):
                    self.copy_file(src, os.path.join(dst, name))


setup(
    name="bmtrain_b200",
    version="0.2.0",
    description="ZeRO / tensor / pipeline parallel training toolkit with hand-written sm_100a kernels",
    packages=find_packages(include=["bmtrain_b200", "bmtrain_b200.*"]),
    package_data={"bmtrain_b200": ["csrc/*", "_C.so", "_cpu.so"]},
    python_requires=">=3.10",
    install_requires=[],  # torch (built for CUDA 12.8+) is expected to be present; it is never fetched from an index
    ext_modules=[Extension("bmtrain_b200._native_placeholder", sources=[])],
    cmdclass={"build_ext": NativeBuild},
    zip_safe=False,
)
