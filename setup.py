"""``pip install -e .`` compiles the CUDA library in-tree first (nvcc, sm_100a only)."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        from siirl_b200.build_ext import build
        build()
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
