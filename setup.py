"""Builds the native library in-tree before packaging (`pip install .` / `python setup.py build_py`).

The CUDA sources are compiled for sm_100a only, with nvcc (no GPU needed at build time). Set
PSGD_B200_SKIP_NATIVE=1 to package the pure-PyTorch path alone (CPU / gloo machines).
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithNative(build_py):
    def run(self):
        if os.environ.get("PSGD_B200_SKIP_NATIVE", "0") != "1":
            sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
            try:
                from powersgd_b200.csrc import build as native_build

                native_build.build()
            except Exception as exc:  # no nvcc: the package still works on CPU
                print(f"warning: native library not built ({exc})", file=sys.stderr)
        super().run()


setup(cmdclass={"build_py": BuildWithNative})
