"""Packaging: ``pip install .`` compiles the sm_100a kernels in-tree (``fastfold_b200/lib/libffb200.so``, nvcc from
``CUDA_HOME``; no GPU needed to build) and installs ``fastfold_b200`` plus the ``fastfold`` compatibility namespace."""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        from fastfold_b200 import _build
        _build.build(verbose=True)
        super().run()


setup(
    name="fastfold-b200",
    version="0.2.0",
    description="AlphaFold training and inference on NVIDIA B200: tcgen05 / TMA kernels, NVLink symmetric-heap collectives, Dynamic Axial Parallelism",
    packages=find_packages(include=["fastfold_b200", "fastfold_b200.*", "fastfold", "fastfold.*"]),
    package_data={"fastfold_b200": ["lib/*.so", "csrc/*", "common/data/*.json"]},
    python_requires=">=3.9",
    install_requires=["numpy", "einops", "scipy"],
    cmdclass={"build_py": BuildWithKernels},
)
