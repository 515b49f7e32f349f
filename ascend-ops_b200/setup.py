"""Packaging of the B200 decode operator set: `pip install [-e] .` in this directory.

Counterpart of the reference's setup.py (setup.py:122-176 there builds the CANN op library and
the pybind module with CMake and copies the results next to the Python package, also for
editable installs).  Here the native part is two compiler invocations driven by build.py
(nvcc for sm_100a, g++ for the torch extension); this file only runs them before the Python
files are collected and ships the two shared objects as package data, so that
`import ascend910a_extras.ops` works from site-packages, or from this tree after `-e`, with no
path edits.  The decode-layer modules that sit beside the package are installed as top-level
modules.
"""
import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = Path(__file__).resolve().parent


def build_native():
    spec = importlib.util.spec_from_file_location("b200ops_build", HERE / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all()


class BuildPyWithNative(build_py):
    """Compile libb200ops.so and the torch extension in-tree, then collect the package."""

    def run(self):
        build_native()
        super().run()


setup(
    packages=["ascend910a_extras"],
    package_data={"ascend910a_extras": ["*.so", "lib/*.so"]},
    py_modules=["moe_decode_layer", "moe_parallel", "decode_workloads"],
    cmdclass={"build_py": BuildPyWithNative},
    zip_safe=False,
)
