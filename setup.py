"""Packaging.  The native extension is built by ``pccl_b200._build`` (g++ for the host sources, ``nvcc -gencode
arch=compute_100a,code=sm_100a`` for the kernels) into ``pccl_b200/_C.so`` and shipped as package data; nothing is
compiled through setuptools' own extension machinery, which knows no GPU architecture (the reference's setup.py built a
``CppExtension`` without one, setup.py:74-76,105).  ``PCCL_DEBUG=1`` in the environment adds ``-DPCCL_DEBUG`` (the
reference's ``debug=True``, setup.py:78-81).  The version carries the git revision like the reference's (setup.py:84-92).

    python setup.py build_ext --inplace        # same as python -m pccl_b200._build
    python -m pip install --no-build-isolation -e .
"""
import os
import subprocess
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def version() -> str:
    base = "0.1.0"
    try:
        sha = subprocess.run(["git", "rev-parse", "--short", "HEAD"], cwd=ROOT, capture_output=True, text=True, timeout=10).stdout.strip()
        return f"{base}+{sha}" if sha else base
    except (OSError, subprocess.SubprocessError):
        return base


def build_native():
    from pccl_b200 import _build
    return _build.build(verbose=True)


class BuildExt(Command):
    """``build_ext`` (with or without ``--inplace``): compile whatever changed and link pccl_b200/_C.so in the tree."""
    description = "build the sm_100a extension in-tree"
    user_options = [("inplace", "i", "accepted for familiarity; the build is always in-tree")]
    boolean_options = ["inplace"]

    def initialize_options(self):
        self.inplace = False

    def finalize_options(self):
        pass

    def run(self):
        print("built", build_native())


class BuildPy(build_py):
    def run(self):
        build_native()
        super().run()


setup(
    name="pccl_b200",
    version=version(),
    description="Programmable collective communication and communication/computation overlap for B200 (sm_100a)",
    packages=find_packages(include=["pccl_b200", "pccl_b200.*", "pccl", "pccl.*"]),
    package_data={"pccl_b200": ["_C.so"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy", "scipy", "pybind11"],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
    zip_safe=False,
)
