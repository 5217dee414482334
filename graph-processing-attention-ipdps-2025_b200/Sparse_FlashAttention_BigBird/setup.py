"""Build `spfa_bigbird` in place:  python setup.py build_ext --inplace

Targets sm_100a only. The CUDA kernels live in the shared C-ABI library (../lib/libspfa_b200.so, built by
../build.py with `nvcc -gencode arch=compute_100a,code=sm_100a`); this extension is the torch binding that
is an additive module (the reference has no such folder) and links against that library.
"""
import os
import sys

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CppExtension

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, PKG)
import build as spfa_build  # noqa: E402  (../build.py)

spfa_build.build_lib()  # nvcc, sm_100a; no-op when up to date

setup(
    name="spfa_bigbird",
    ext_modules=[
        CppExtension(
            "spfa_bigbird",
            ["sp_flatt_bigbird.cpp"],
            include_dirs=[os.path.join(PKG, "bindings"), os.path.join(os.path.dirname(PKG), "include")],
            library_dirs=[spfa_build.LIBDIR],
            libraries=["spfa_b200", "c10_cuda", "torch_cuda"],
            runtime_library_dirs=[spfa_build.LIBDIR],
            extra_compile_args=["-O2", "-std=c++17"],
        )
    ],
    cmdclass={"build_ext": BuildExtension},
)
