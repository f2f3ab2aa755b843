"""Builds the sm_100a kernel library in-tree before packaging (``pip install -e .`` or ``python setup.py build_py``)."""
from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        from flame_b200.ops import _build
        _build.build_library()
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
