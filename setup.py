"""Packaging of the B200 attention library.

Installs two packages: ``acctransformer_b200`` (the implementation, with ``libacct_b200.so`` built
by nvcc for sm_100a during the build step) and ``acctransformer`` (the reference's import paths,
re-exporting the former), so that ``pip install .`` gives a user of the reference the same
``from acctransformer... import FlashAttention`` statements (the reference's own packaging:
train/setup.py:22-31, a pure-Python package of the same name).

    python setup.py build_ext --inplace      # just (re)build the shared library in-tree
    pip install --no-build-isolation .       # build and install
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _build_library():
    from acctransformer_b200 import build as libbuild
    return libbuild.build()


class BuildSharedLibrary(Command):
    """`build_ext`: compiles csrc/*.cu into acctransformer_b200/libacct_b200.so (always in-tree)."""
    description = "build libacct_b200.so with nvcc for sm_100a"
    user_options = [("inplace", "i", "accepted for familiarity; the library is always built in-tree")]

    def initialize_options(self):
        self.inplace = 0

    def finalize_options(self):
        pass

    def run(self):
        print("built", _build_library())


class BuildPyWithLibrary(build_py):
    def run(self):
        _build_library()
        super().run()


setup(
    name="acctransformer-b200",
    version="0.2.0",
    description="FlashAttention2 / TriangleAttention / inference attention of acctransformer as hand-written CUDA for NVIDIA B200",
    packages=find_packages(where=".", include=["acctransformer", "acctransformer.*", "acctransformer_b200", "acctransformer_b200.*"]),
    package_data={"acctransformer_b200": ["libacct_b200.so", "csrc/*.cu", "csrc/*.cuh"]},
    data_files=[("include", ["include/acct_b200.h"])],
    python_requires=">=3.9",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildSharedLibrary, "build_py": BuildPyWithLibrary},
    zip_safe=False,
)
