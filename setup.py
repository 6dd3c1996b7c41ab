"""Packaging of atex_b200: the Python host layer plus libnvnorms.so, built in-tree by nvcc.

Takes the place of the reference's setup.py (atex setup.py:21-160: a CMake extension per
sub-package, TensorFlow as a requirement).  This library needs neither CMake nor
TensorFlow: `build_ext` calls atex_b200.build.build(), which runs one nvcc process per
translation unit for sm_100a and links atex_b200/libnvnorms.so, and the wheel carries that
file as package data next to atex_b200/_lib.py, which is where the loader looks for it
(the reference's loader looks beside nv_norm_ops.py the same way, nv_norm_ops.py:19-21).

    python setup.py build_ext --inplace        # compile in-tree
    pip install --no-build-isolation .         # build + install
"""
import os
import sys

from setuptools import Extension, find_packages, setup
from setuptools.command.build_ext import build_ext

HERE = os.path.dirname(os.path.abspath(__file__))


class NvccBuild(build_ext):
    """Builds libnvnorms.so with atex_b200/build.py instead of a compiler driven by setuptools."""

    def run(self):
        sys.path.insert(0, HERE)
        from atex_b200 import build as nvn_build
        lib = nvn_build.build(verbose=bool(self.verbose))
        if not self.inplace:
            dst = os.path.join(self.build_lib, "atex_b200")
            os.makedirs(dst, exist_ok=True)
            self.copy_file(lib, os.path.join(dst, os.path.basename(lib)))


setup(
    name="atex_b200",
    version="0.2.0",
    description="Fused LayerNorm / InstanceNorm for NVIDIA B200 (sm_100a) behind a C ABI",
    packages=find_packages(include=["atex_b200", "atex_b200.*"]),
    package_data={"atex_b200": ["libnvnorms.so", "csrc/*.cu", "csrc/*.cuh", "csrc/*.h", "csrc/tf/*"]},
    data_files=[("include", ["include/nvnorms.h"])],
    # a placeholder extension so that build_ext runs; the real work is in NvccBuild.run
    ext_modules=[Extension("atex_b200._nvcc_placeholder", sources=[])],
    cmdclass={"build_ext": NvccBuild},
    python_requires=">=3.9",
    install_requires=["torch", "numpy"],
)
