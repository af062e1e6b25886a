"""Builds the ``TAB_CUDA`` PyTorch extension for NVIDIA B200 (sm_100a) only.

    python Setup_CUDA.py build_ext --inplace

Counterpart of the reference's ``Setup_CUDA.py:1-15`` (same module name, same exported functions).  The
CUDA kernels are compiled by nvcc into ``tab_b200/libtab_b200.so`` (the C ABI in ``include/tab_b200.h``)
with ``-gencode arch=compute_100a,code=sm_100a`` and nothing else; the extension module itself is the
thin torch/pybind11 binding ``tab_b200/csrc/tab_api.cpp`` linked against that library.
"""
import os
import sys

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CppExtension, CUDA_HOME

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from tab_b200 import build as tab_build  # noqa: E402

tab_build.build_library()

cuda_home = CUDA_HOME or "/usr/local/cuda"
setup(
    name="TAB_CUDA",
    version="1.0",
    description="TAB ternary/binary quantise + popcount convolution for sm_100a",
    ext_modules=[
        CppExtension(
            name="TAB_CUDA",
            sources=[os.path.join("tab_b200", "csrc", "tab_api.cpp")],
            include_dirs=[os.path.join(cuda_home, "include")],
            library_dirs=[os.path.join(ROOT, "tab_b200"), os.path.join(cuda_home, "lib64")],
            libraries=["tab_b200", "c10_cuda", "torch_cuda", "cudart"],
            extra_compile_args=["-O2", "-std=c++17"],
            extra_link_args=["-Wl,-rpath,$ORIGIN/tab_b200"],
        ),
    ],
    cmdclass={"build_ext": BuildExtension},
)
