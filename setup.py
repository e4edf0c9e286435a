"""Build and install: compiles libfp6_b200.so for sm_100a in-tree (fp6_llm_b200/_lib) and installs the package together
with the reference's module names (`fp6_llm`, `fp6_llm_cuda`).  Counterpart of the reference's setup.py, which builds
the `fp6_llm_cuda` torch extension for sm_80.

    python setup.py build_ext --inplace      # compile only
    pip install --no-build-isolation .       # compile and install
"""
import os
import sys

from setuptools import Command, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _compile():
    from fp6_llm_b200 import _native
    print("built", _native.build())


class BuildNative(Command):
    description = "compile libfp6_b200.so with nvcc (sm_100a)"
    user_options = [("inplace", "i", "accepted for compatibility: the library is always built in-tree")]

    def initialize_options(self):
        self.inplace = False

    def finalize_options(self):
        pass

    def run(self):
        _compile()


class BuildPy(build_py):
    def run(self):
        _compile()
        super().run()


setup(
    name="fp6_llm_b200",
    version="0.2.0",
    description="FP6/FP5 x FP16 linear layer of FP6-LLM for NVIDIA B200 (sm_100a), behind the reference's operator names",
    packages=["fp6_llm_b200", "fp6_llm"],
    py_modules=["fp6_llm_cuda"],
    package_data={"fp6_llm_b200": ["_lib/*.so", "csrc/*"]},
    cmdclass={"build_ext": BuildNative, "build_py": BuildPy},
)
