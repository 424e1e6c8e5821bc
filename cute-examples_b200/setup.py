"""Builds gemm_kernels for sm_100a (B200) only: `pip install ./cute-examples_b200 --no-build-isolation`
or `python setup.py build_ext --inplace`.

Same package / module names as the reference's kernels/setup.py:10-15 (`gemm_kernels._C`), but
the CUDA code is compiled by nvcc into gemm_kernels/libgemm_sm100.so without torch headers and
the extension is a plain C++ shim over its C ABI (see build_native.py)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.extension import Extension

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import build_native  # noqa: E402


class BuildNative(build_ext):
    def run(self):
        build_native.build_all(force=False, verbose=bool(self.verbose))

    def get_outputs(self):
        return [str(build_native.LIB), str(build_native.ext_path())]


setup(
    name="gemm_kernels",
    version="0.1.0",
    packages=["gemm_kernels"],
    package_data={"gemm_kernels": ["*.so"]},
    ext_modules=[Extension("gemm_kernels._C", sources=[])],
    cmdclass={"build_ext": BuildNative},
)
