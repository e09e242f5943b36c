"""Packaging: ``python setup.py build_ext --inplace`` (or ``pip install -e . --no-build-isolation``) compiles the
native module in-tree with nvcc for sm_100a; the build itself lives in ``parameter_server_b200/_build.py``."""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class build_ext(_build_ext):
    def run(self):
        from parameter_server_b200 import _build
        _build.build()


class build_native(Command):
    description = "compile the CUDA / C++ sources into parameter_server_b200/_C*.so"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        from parameter_server_b200 import _build
        _build.build()


setup(
    name="parameter_server_b200",
    version="0.1.0",
    description="Blackwell-native (sm_100a) parameter server: fused NVLink sparse / dense paths, RPC service layer",
    packages=find_packages(include=["parameter_server_b200", "parameter_server_b200.*"]),
    package_data={"parameter_server_b200": ["_C*.so", "csrc/**/*"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    cmdclass={"build_ext": build_ext, "build_native": build_native},
)
