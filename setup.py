"""Packaging for flextrain_b200.

Capability parity: setup.py / requirements.txt / version.txt of the reference.
The native libraries are built in-tree by ``flextrain_b200.ops.op_builder``
(g++ for the host library, nvcc ``-gencode arch=compute_100a,code=sm_100a`` for
the CUDA library) - at install time when the compilers are present, otherwise on
first use.
"""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithNative(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        try:
            from flextrain_b200.ops.op_builder import build_all
            build_all()
        except Exception as exc:                      # compilers missing: built lazily later
            print(f"[flextrain_b200] native build skipped: {exc}")
        super().run()


setup(
    name="flextrain_b200",
    version="0.1.0",
    description="Blackwell-native memory-tiering LLM training engine with the FlexTrain API",
    packages=find_packages(include=["flextrain_b200", "flextrain_b200.*"]),
    package_data={"flextrain_b200": ["_native/*.so", "_native/*.sig"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.4", "numpy", "psutil"],
    extras_require={"planner": ["scipy"], "test": ["pytest", "hypothesis"]},
    cmdclass={"build_py": BuildWithNative},
)
