"""Builds the native parts in-tree before packaging (``pip install .`` or ``python setup.py build_py``):
the C++ core, the sm_100a kernel library (when nvcc is present), the torch glue, the command-line tools
and the circuit simulator. The reference's packaging is maturin over a Rust workspace
(``pyproject.toml`` of the reference); here the build driver is ``nangila/_build.py``."""
import shutil
import sys
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


class BuildNative(build_py):
    def run(self):
        sys.path.insert(0, str(ROOT))
        from nangila import _build

        _build.build_core()
        _build.build_cli()
        _build.build_spice()
        if shutil.which("nvcc") or Path("/usr/local/cuda/bin/nvcc").exists():
            _build.build_kernels()
            _build.build_glue()
        else:
            print("nvcc not found: the CUDA kernel library and the torch glue are not built (CPU / gloo paths only)")
        super().run()


setup(cmdclass={"build_py": BuildNative})
