"""Wheel build: the CUDA sources travel inside the package, and when ``nvcc`` is on the build machine the kernel
library is compiled for sm_100a first so that the wheel also carries ``_C/libringattn_b200.so``. A wheel built
without ``nvcc`` still works: the library is built on first use from the packaged sources
(``ringattention_b200.ops._lib.lib``)."""
import os
import sys

from setuptools import Distribution, setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        here = os.path.dirname(os.path.abspath(__file__))
        sys.path.insert(0, here)
        try:
            from ringattention_b200 import _build

            try:
                _build.build()
            except _build.NvccMissing as e:
                print(f"warning: {e}; the wheel ships sources only")
        finally:
            sys.path.pop(0)
        super().run()


class BinaryWhenBuilt(Distribution):
    """The wheel is platform-specific once it carries the compiled library."""

    def has_ext_modules(self):
        here = os.path.dirname(os.path.abspath(__file__))
        return os.path.exists(os.path.join(here, "ringattention_b200", "_C", "libringattn_b200.so"))


setup(cmdclass={"build_py": BuildWithKernels}, distclass=BinaryWhenBuilt)
