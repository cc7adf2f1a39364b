"""``pip install .`` builds the sm_100a kernel library in-tree (needs nvcc >= 12.8) before the package is collected.

Set ``KSA_SKIP_KERNEL_BUILD=1`` to install the Python side only (CPU paths; the library can be built later with
``python -m ksa_b200.csrc.build``)."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("KSA_SKIP_KERNEL_BUILD") != "1":
            sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
            from ksa_b200.csrc.build import build
            print(f"built {build()}")
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
