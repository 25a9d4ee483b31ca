"""Builds and installs xattn_b200 for Blackwell (sm_100a) only.

The reference's setup.py compiles a torch C++ extension for several architectures, with a CUTLASS
checkout and generated instantiation files (setup.py:40,93-310,497-504 of ifm-ai/xattn).  Here the
native part is one plain-C-ABI shared library built by nvcc with a single
``-gencode arch=compute_100a,code=sm_100a`` (xattn_b200/build.py); it needs no torch headers, no
CUTLASS and no host-compiler extension step, so the build is a pre-step of ``build_py`` that drops
``libxattn_b200.so`` next to the Python sources.  Three packages are installed: ``xattn_b200`` (the
implementation), ``xattn`` (the reference's package name for the same API) and ``xattn_cuda`` (the
reference's native-op module name over the C ABI).

    pip install --no-build-isolation .        # needs nvcc on PATH or under /usr/local/cuda
"""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildWithLibrary(build_py):
    def run(self):
        sys.path.insert(0, HERE)
        from xattn_b200.build import build
        build()                              # nvcc -gencode arch=compute_100a,code=sm_100a
        super().run()


setup(
    name="xattn_b200",
    version="0.2.0",
    description="xattn attention ops (causal, sliding-window, sliding-chunk, SoftDelta) for NVIDIA B200 (sm_100a)",
    packages=["xattn_b200", "xattn_b200.ops", "xattn", "xattn_cuda"],
    package_data={"xattn_b200": ["libxattn_b200.so", "csrc/*.cu", "csrc/*.cuh"]},
    data_files=[("include", ["include/xattn_b200.h"])],
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_py": BuildWithLibrary},
    zip_safe=False,
)
