"""``pip install .`` entry point: metadata lives in ``pyproject.toml``; this file only adds the step that compiles
``csrc/`` for sm_100a into ``mcore_bridge_b200/lib/libmcb200.so`` when ``nvcc`` is available (a CPU-only install
skips it and the package runs on its PyTorch reference paths)."""
import shutil
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):

    def run(self):
        if shutil.which('nvcc') or shutil.which('/usr/local/cuda/bin/nvcc'):
            sys.path.insert(0, '.')
            from mcore_bridge_b200.build_ext import build
            build(verbose=True)
        else:
            print('nvcc not found: installing without the CUDA library (CPU reference paths only)')
        super().run()


setup(cmdclass={'build_py': BuildWithKernels})
