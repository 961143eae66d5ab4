"""Builds the native library (CUDA kernels for sm_100a + the C++ host runtime) into the package before the Python
files are collected, so that a wheel carries ``fms_acceleration_b200/lib/libfmsb200.so``.  ``nvcc`` cross-compiles
without a GPU; set ``FMSB_SKIP_NATIVE=1`` to package the Python layer only (CPU paths, tests of the host logic)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class build_py_with_native(build_py):
    def run(self):
        if os.environ.get("FMSB_SKIP_NATIVE") != "1":
            sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
            from fms_acceleration_b200.build import build

            print("building", build(verbose=False))
        super().run()


setup(cmdclass={"build_py": build_py_with_native})
