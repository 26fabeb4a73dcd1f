"""Packaging: ``pip install -e .`` (or ``python setup.py build_ext --inplace``)
compiles the native extension in-tree with horovod_b200/build_ext.py (g++ for
the runtime, nvcc for the sm_100a kernels, linked against the installed
PyTorch) and installs the ``horovodrun`` launcher.

Build-time switches (environment):
  HOROVOD_B200_BUILD_JOBS   parallel compile jobs for ninja (default: all cores)
  HOROVOD_B200_SKIP_BUILD   "1": install the Python sources only (the extension
                            must then be built separately before import)

Parity: setup.py:30-210 and CMakeLists.txt of the reference drive one CMake
build per framework; here there is one framework (PyTorch) and one target
architecture, so the build is a generated ninja file.
"""
import os
import subprocess
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_ext import build_ext as _build_ext
from setuptools.command.build_py import build_py as _build_py

HERE = os.path.dirname(os.path.abspath(__file__))


def _build_native():
    if os.environ.get("HOROVOD_B200_SKIP_BUILD") == "1":
        return
    cmd = [sys.executable, os.path.join(HERE, "horovod_b200", "build_ext.py")]
    subprocess.check_call(cmd, cwd=HERE)


class build_ext(_build_ext):
    def run(self):
        _build_native()


class build_py(_build_py):
    def run(self):
        _build_native()
        super().run()


class build_native(Command):
    description = "compile horovod_b200/_C.so in the source tree"
    user_options = []

    def initialize_options(self):
        pass

    def finalize_options(self):
        pass

    def run(self):
        _build_native()


setup(
    name="horovod_b200",
    version="0.1.0",
    description="Blackwell-native data-parallel training library with Horovod's PyTorch API",
    packages=find_packages(include=["horovod_b200", "horovod_b200.*"]),
    package_data={"horovod_b200": ["_C.so", "csrc/**/*"]},
    python_requires=">=3.9",
    install_requires=["torch", "cloudpickle", "psutil", "pyyaml"],
    extras_require={"ray": ["ray"], "spark": ["pyspark>=3.0", "pyarrow", "pandas", "numpy"]},
    entry_points={"console_scripts": ["horovodrun = horovod_b200.runner.launch:run_commandline"]},
    cmdclass={"build_ext": build_ext, "build_py": build_py, "build_native": build_native},
)
