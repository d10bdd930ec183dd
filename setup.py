"""Editable / in-tree install: `pip install --no-build-isolation -e .` builds the three native
libraries with nvcc and g++ (heterofusedkernels_b200/build.py) before the package is installed, the way
the reference's setup.py drives its native build (pcieThrough/setup.py:107-176)."""
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.command.develop import develop

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _build_native():
    from heterofusedkernels_b200 import build

    build.build_all(verbose=True)


class BuildPy(build_py):
    def run(self):
        _build_native()
        super().run()


class Develop(develop):
    def run(self):
        _build_native()
        super().run()


setup(cmdclass={"build_py": BuildPy, "develop": Develop})
