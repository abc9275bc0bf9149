"""Builds the two native libraries in-tree before the package is collected: ``libb200ops.so`` (the sm_100a kernels, nvcc) and
``libb200host.so`` + ``devquery`` (the C++ host helpers, g++).  ``pip install .`` on a machine with CUDA 12.8+ is the whole
install; the metadata lives in pyproject.toml."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from ollama_b200.kernels.build import build
        build(verbose=False)
        super().run()


setup(cmdclass={"build_py": BuildNative})
