"""Editable / wheel install of the Python layer; the native library is built in-tree by cann_hccl_b200/build.py.

    pip install --no-build-isolation -e .      # keeps the package and lib/libhccl_b200.so where they are
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    """g++ + nvcc (sm_100a) over csrc/ into cann_hccl_b200/lib before the Python files are collected."""

    def run(self):
        sys.path.insert(0, HERE)
        from cann_hccl_b200 import build as native
        native.build()
        super().run()


setup(
    name="cann-hccl-b200",
    version="0.2.0",
    description="HCCL-compatible collective communication library for NVIDIA B200 (sm_100a kernels, NVLink / NVSwitch)",
    packages=find_packages(include=["cann_hccl_b200", "cann_hccl_b200.*"]),
    package_data={"cann_hccl_b200": ["lib/*.so", "include/hccl/*.h"]},
    cmdclass={"build_py": BuildNative},
    python_requires=">=3.10",
)
