"""Builds libpippy_b200.so with nvcc before the package is installed (reference setup.py writes a version file and
has nothing to compile; here the CUDA library is the build step).  `PIPPY_B200_SKIP_BUILD=1` skips it, e.g. on a
machine without nvcc that only needs the CPU paths."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithCuda(build_py):
    def run(self):
        if os.environ.get("PIPPY_B200_SKIP_BUILD") != "1":
            sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
            from pippy_b200.csrc.build import build_all

            print("building", build_all(verbose=True))
        super().run()


setup(cmdclass={"build_py": BuildWithCuda})
