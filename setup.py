"""Packaging for `tensorflow_allreduce_b200`.

`python setup.py build_ext --inplace` (or `pip install -e . --no-build-isolation`) compiles the
native library in-tree with `tensorflow_allreduce_b200/build.py` (nvcc for sm_100a + g++); the
shared object stays next to the package, where `_lib.py` loads it from. The reference ships its
op library through Bazel (`tensorflow/contrib/mpi_collectives/BUILD:38-46`).
"""
import os
import sys

from setuptools import Command, find_packages, setup

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(Command):
    description = "compile tensorflow_allreduce_b200/lib/libbcoll.so in-tree"
    user_options = [("inplace", "i", "accepted for compatibility; the build is always in-tree"),
                    ("debug-kernels", None, "also build the bounds-checked variant (libbcoll_debug.so)")]
    boolean_options = ["inplace", "debug-kernels"]

    def initialize_options(self):
        self.inplace = True
        self.debug_kernels = False

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, ROOT)
        from tensorflow_allreduce_b200 import build

        print(build.build())
        if self.debug_kernels:
            print(build.build(debug=True))


setup(
    name="tensorflow-allreduce-b200",
    version="0.1.0",
    description="B200-native data-parallel collectives for PyTorch with the API of tensorflow/contrib/mpi_collectives",
    packages=find_packages(include=["tensorflow_allreduce_b200", "tensorflow_allreduce_b200.*"]),
    package_data={"tensorflow_allreduce_b200": ["csrc/*", "csrc/*/*", "lib/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_ext": BuildNative},
)
