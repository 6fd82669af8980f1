"""Wheel build: compiles the ahead-of-time sm_100a kernels (kermac_b200/csrc, nvcc, no GPU needed)
into kermac_b200/libkermac_b200.so and ships that file inside the package, so an installed
kermac_b200 needs neither nvcc nor a JIT cache at run time.

    python -m pip wheel --no-deps --no-build-isolation -w dist .
"""
import os
import subprocess

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildKernelsThenPython(build_py):
    def run(self):
        jobs = str(os.cpu_count() or 4)
        subprocess.check_call(["make", "-C", os.path.join(HERE, "kermac_b200", "csrc"), "-j", jobs])
        super().run()


try:
    from wheel.bdist_wheel import bdist_wheel

    class PlatformWheel(bdist_wheel):
        """The wheel carries a native library: tag it for this platform, any Python 3."""

        def finalize_options(self):
            super().finalize_options()
            self.root_is_pure = False

        def get_tag(self):
            _, _, plat = super().get_tag()
            return "py3", "none", plat

    cmdclass = {"build_py": BuildKernelsThenPython, "bdist_wheel": PlatformWheel}
except ImportError:      # sdist-only environments
    cmdclass = {"build_py": BuildKernelsThenPython}

setup(cmdclass=cmdclass)
