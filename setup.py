"""Builds the `neoGEMM` PyTorch extension, as the reference's setup.py does (setup.py:4-24), for
B200:  python setup.py build_ext --inplace   (or `install`).

Two steps instead of the reference's single torch-header .cu: nvcc compiles the kernels and the
C-ABI launcher into gemm_b200/libneogemm.so for compute_100a/sm_100a (the reference targets
compute_90a, setup.py:15), then the host compiler builds the thin binding and links it to that
library.  cuBLAS is not linked (the reference links it without using it, setup.py:17).
"""
import os
import sys

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from gemm_b200.build import build_library  # noqa: E402

build_library()

setup(
    name="neoGEMM",
    version="1.0.0",
    packages=["gemm_b200"],
    ext_modules=[
        CUDAExtension(
            name="neoGEMM",
            sources=["gemm_b200/csrc/binding.cpp"],
            include_dirs=[os.path.join(ROOT, "include")],
            library_dirs=[os.path.join(ROOT, "gemm_b200")],
            libraries=["neogemm"],
            extra_compile_args={"cxx": ["-O2", "-std=c++17"]},
            extra_link_args=["-Wl,-rpath,$ORIGIN/gemm_b200"],
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=False)},
)
