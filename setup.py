"""Packaging entry: compiles the sm_100a kernel library in-tree (nvcc, no GPU needed) before the Python files are
collected, so that the wheel / editable install carries ``openrlhf_b200/libopenrlhf_b200.so``."""
import os
import subprocess
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("OPENRLHF_B200_SKIP_NVCC") != "1":
            subprocess.check_call([sys.executable, "-m", "openrlhf_b200.csrc.build"],
                                  cwd=os.path.dirname(os.path.abspath(__file__)))
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
