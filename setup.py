"""Builds the two in-tree native libraries (CUDA kernels for sm_100a, C++ compiler/runtime) and
installs the package. ``pip install -e .`` keeps the libraries inside the source tree, where the
package loads them from."""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildNative(build_py):
    def run(self):
        from multimesh_jax_b200.csrc import build as native
        native.build_kernels(force=False)
        native.build_host(force=False)
        super().run()


setup(
    name="multimesh_jax_b200",
    version="0.1.0",
    description="Blackwell-native MPMD parallelism runtime for PyTorch (tasks on sub-meshes, automatic resharding, "
                "pipeline schedules, hand-written sm_100a kernels)",
    packages=find_packages(include=["multimesh_jax_b200", "multimesh_jax_b200.*"]),
    package_data={"multimesh_jax_b200": ["*.so", "csrc/**/*"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pybind11"],
    cmdclass={"build_py": BuildNative},
)
